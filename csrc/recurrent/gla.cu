// Gated linear attention as a recurrence over a per-sequence state, for ragged batches (portions of prompts next to
// single decoded tokens), bf16 or fp32 projections.
//
// Per head, with q_t, k_t (d numbers), v_t (e numbers) and a decay per key channel a_t in (0, 1):
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T            S: [d, e], fp32, zero before a sequence's first token
//     o_t = S_t^T q_t
//     a_t = sigmoid(z_t + bias)^(1/tau) = exp(logsigmoid(z_t + bias) / tau)
//
//   llmctl_gla_scan   : first, fully parallel, the scaled queries, keys and decays (minus one) of the step's tokens in
//       fp32.  Then a CTA owns (portion, head, block of 32 value columns); lane = column, warp = block of RPT key
//       rows, whose state lives in registers for the whole portion.  The portion is walked in chunks of 16 tokens: the
//       CTA stages a chunk's prepared numbers and values in shared memory while the previous chunk's steps run on
//       what was staged before; a step reads its rows' numbers as broadcast float4s.  The warps' partial outputs of a chunk meet in shared memory: two barriers per chunk, none per token.
//       A portion that starts at position 0 starts from zeros whatever its slot holds; otherwise from the slot.
//   llmctl_gla_output : per (token, head), o / sqrt(mean(o^2) + eps) * w (w shared by the heads) times silu(gate).
// Decay, state, outputs and the norm are fp32; q, k, v, z and the gate are read in the projections' type.
// Reference: none (the reference has no model code).
#include "../common/dtype.cuh"

namespace llmctl {

struct GlaParams {
  const void* q;       // [T, *]: head h at column h * d (row stride ldq), likewise k (d per head) and v (e per head)
  const void* k;
  const void* v;
  const void* z;       // decay logits [T, H * d] (row stride ldz)
  long long ldq, ldk, ldv, ldz;
  const float* z_bias; // [H * d] or null
  const int* portions; // [n, 4] = (first token row, tokens, position of the first token, state slot)
  float* state;        // [slots, H, d, e]
  float* out;          // [T, H * e]
  int H, d, e;
  float q_scale, inv_tau;
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

constexpr int kGlaTC = 16;      // tokens staged per chunk

// work[t] = [scaled queries | keys | decay minus one] of token t in fp32, 3 * H * d numbers: everything the serial scan
// would otherwise evaluate (the decay's three transcendentals above all) happens here, fully parallel.
template <typename T>
__global__ void __launch_bounds__(256)
gla_prepare_kernel(const GlaParams p, float* __restrict__ work, int tokens) {
  const int nk = p.H * p.d;
  const long long total = static_cast<long long>(tokens) * nk;
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* z = static_cast<const T*>(p.z);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / nk;
    const int c = static_cast<int>(i % nk);
    float* w = work + t * 3 * nk + c;
    w[0] = to_f32(q[t * p.ldq + c]) * p.q_scale;
    w[nk] = to_f32(k[t * p.ldk + c]);
    // the decay minus one: a is close to 1 for slow channels, and S + (a - 1) S keeps it exact to ~1e-10 instead of the
    // ulp of 1 that a rounded factor carries (a state with a memory of thousands of tokens would accumulate that)
    w[2 * nk] = expm1f(log_sigmoid(to_f32(z[t * p.ldz + c]) + (p.z_bias ? p.z_bias[c] : 0.f)) * p.inv_tau);
  }
}

template <typename T, int RPT>
__global__ void __launch_bounds__(256)
gla_scan_kernel(const GlaParams p, const float* __restrict__ work) {
  constexpr int TC = kGlaTC, NTR = RPT / 2;      // (q, k, decay) triples a thread stages per chunk: TC * dpad / threads
  constexpr int TSTEP = 32 / RPT;                // tokens between a thread's staging elements
  extern __shared__ __align__(16) float gla_smem[];
  const int H = p.H, d = p.d, e = p.e, nk = H * d;
  const int* pt = p.portions + blockIdx.x * 4;
  const int t0 = pt[0], n = pt[1], pos0 = pt[2], slot = pt[3];
  if (n <= 0) return;
  const int h = blockIdx.y, col = blockIdx.z * 32 + (threadIdx.x & 31);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5, nthreads = blockDim.x;
  const int dpad = nwarps * RPT, row0 = warp * RPT;
  const bool colok = col < e;
  float* sq = gla_smem;                  // [TC][dpad] scaled queries
  float* sk = sq + TC * dpad;            // [TC][dpad] keys
  float* sa = sk + TC * dpad;            // [TC][dpad] decay minus one
  float* sv = sa + TC * dpad;            // [TC][32] values of this CTA's columns
  float* part = sv + TC * 32;            // [TC][nwarps][32] partial outputs of the warps

  float S[RPT];
#pragma unroll
  for (int j = 0; j < RPT; ++j) S[j] = 0.f;
  float* st = slot >= 0 ? p.state + ((static_cast<long long>(slot) * H + h) * d) * e : nullptr;
  if (st && pos0 > 0 && colok) {
#pragma unroll
    for (int j = 0; j < RPT; ++j)
      if (row0 + j < d) S[j] = st[static_cast<long long>(row0 + j) * e + col];
  }
  const T* v = static_cast<const T*>(p.v);

  // staging: this thread's element i of a chunk is (token stok + i * TSTEP, key row srow); nthreads is a multiple of dpad
  const int srow = tid % dpad, stok = tid / dpad;
  const bool srow_ok = srow < d;
  const float* wbase = work + static_cast<long long>(t0) * 3 * nk + h * d + srow;
  // values: element (token tid / 32 + j * nwarps, column lane)
  float rq[NTR], rk[NTR], ra[NTR], rv[TC];
  auto fetch = [&](int c0) {
#pragma unroll
    for (int i = 0; i < NTR; ++i) {
      const int tok = c0 + stok + i * TSTEP;
      const bool ok = srow_ok && tok < n;
      const float* w = wbase + static_cast<long long>(tok) * 3 * nk;
      rq[i] = ok ? w[0] : 0.f;
      rk[i] = ok ? w[nk] : 0.f;
      ra[i] = ok ? w[2 * nk] : -1.f;               // rows beyond d keep a zero state
    }
#pragma unroll
    for (int j = 0; j < TC; ++j) {
      const int tok = warp + j * nwarps;
      if (tok < TC) rv[j] = (colok && c0 + tok < n) ? to_f32(v[static_cast<long long>(t0 + c0 + tok) * p.ldv + h * e + col]) : 0.f;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int i = 0; i < NTR; ++i) {
      const int idx = (stok + i * TSTEP) * dpad + srow;
      sq[idx] = rq[i];
      sk[idx] = rk[i];
      sa[idx] = ra[i];
    }
#pragma unroll
    for (int j = 0; j < TC; ++j) {
      const int tok = warp + j * nwarps;
      if (tok < TC) sv[tok * 32 + lane] = rv[j];
    }
  };
  fetch(0);
  stash();
  __syncthreads();
  for (int c0 = 0; c0 < n; c0 += TC) {
    const bool more = c0 + TC < n;
    if (more) fetch(c0 + TC);                       // the next chunk's loads fly during this chunk's steps
    const int cnt = min(TC, n - c0);
    for (int tok = 0; tok < cnt; ++tok) {
      const float* aq = sq + tok * dpad + row0;
      const float* ak = sk + tok * dpad + row0;
      const float* aa = sa + tok * dpad + row0;
      const float vv = sv[tok * 32 + lane];
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int j = 0; j < RPT; j += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(aa + j), k4 = *reinterpret_cast<const float4*>(ak + j);
        const float4 q4 = *reinterpret_cast<const float4*>(aq + j);
        S[j] = fmaf(a4.x, S[j], fmaf(k4.x, vv, S[j]));
        S[j + 1] = fmaf(a4.y, S[j + 1], fmaf(k4.y, vv, S[j + 1]));
        S[j + 2] = fmaf(a4.z, S[j + 2], fmaf(k4.z, vv, S[j + 2]));
        S[j + 3] = fmaf(a4.w, S[j + 3], fmaf(k4.w, vv, S[j + 3]));
        o0 += q4.x * S[j] + q4.z * S[j + 2];
        o1 += q4.y * S[j + 1] + q4.w * S[j + 3];
      }
      part[(tok * nwarps + warp) * 32 + lane] = o0 + o1;
    }
    __syncthreads();                                // the chunk's partial outputs are complete, its staged rows read
    for (int idx = tid; idx < cnt * 32; idx += nthreads) {
      const int tok = idx >> 5, c = idx & 31;
      if (blockIdx.z * 32 + c < e) {
        float s = 0.f;
        for (int w = 0; w < nwarps; ++w) s += part[(tok * nwarps + w) * 32 + c];
        p.out[(static_cast<long long>(t0 + c0 + tok) * H + h) * e + blockIdx.z * 32 + c] = s;
      }
    }
    if (more) stash();
    __syncthreads();
  }
  if (st && colok) {
#pragma unroll
    for (int j = 0; j < RPT; ++j)
      if (row0 + j < d) st[static_cast<long long>(row0 + j) * e + col] = S[j];
  }
}

// one warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(256)
gla_output_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ gate, long long ldg,
                  T* __restrict__ out, long long rows, int H, int e, float eps) {
  const long long r = blockIdx.x * static_cast<long long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = r / H;
  const int h = static_cast<int>(r % H);
  const float* orow = o + r * e;
  float ss = 0.f;
  for (int c = lane; c < e; c += 32) ss += orow[c] * orow[c];
  ss = warp_sum(ss);
  const float f = 1.f / sqrtf(ss / e + eps);
  for (int c = lane; c < e; c += 32) {
    const float g = to_f32(gate[t * ldg + h * e + c]);
    out[r * e + c] = from_f32<T>(orow[c] * f * w[c] * (g / (1.f + expf(-g))));
  }
}

}  // namespace llmctl

using namespace llmctl;

// work: fp32 [tokens, 3 * H * d] scratch (the prepared queries, keys and decays of the step's tokens).
LLMCTL_API int llmctl_gla_scan(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv, const void* z,
                               long long ldz, const float* z_bias, const int* portions, int nportions, int tokens, float* state,
                               float* out, float* work, int H, int d, int e, float q_scale, float tau, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && d > 0 && d <= 256 && e > 0 && tau > 0.f && work != nullptr);
  if (nportions == 0 || tokens == 0) return 0;
  GlaParams p{q, k, v, z, ldq, ldk, ldv, ldz, z_bias, portions, state, out, H, d, e, q_scale, 1.f / tau};
  const dim3 grid(nportions, H, (e + 31) / 32);
  cudaStream_t s = (cudaStream_t)stream;
  const int rpt = d <= 64 ? 8 : d <= 128 ? 16 : 32;
  const int warps = (d + rpt - 1) / rpt, threads = 32 * warps;
  const size_t smem = sizeof(float) * kGlaTC * (3 * static_cast<size_t>(warps) * rpt + 32 + warps * 32);       // <= 42 KB
  const long long total = static_cast<long long>(tokens) * H * d;
  const int pgrid = static_cast<int>(total / 256 + 1 < kNumSMs * 16 ? total / 256 + 1 : kNumSMs * 16);
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, {
    gla_prepare_kernel<T><<<pgrid, 256, 0, s>>>(p, work, tokens);
    if (rpt == 8) gla_scan_kernel<T, 8><<<grid, threads, smem, s>>>(p, work);
    else if (rpt == 16) gla_scan_kernel<T, 16><<<grid, threads, smem, s>>>(p, work);
    else gla_scan_kernel<T, 32><<<grid, threads, smem, s>>>(p, work);
  });
  LLMCTL_RETURN_LAST();
}

// o: fp32 [T, H * e]; w: fp32 [e]; gate: [T, H * e] (row stride ldg) pre-activation; out: [T, H * e] in the activation type.
LLMCTL_API int llmctl_gla_output(const float* o, const float* w, const void* gate, long long ldg, void* out, int tokens, int H, int e,
                                 float eps, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  if (tokens == 0) return 0;
  const long long rows = static_cast<long long>(tokens) * H;
  const int grid = static_cast<int>((rows + 7) / 8);
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (gla_output_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(o, w, (const T*)gate, ldg, (T*)out, rows,
                                                                                                H, e, eps)));
  LLMCTL_RETURN_LAST();
}
