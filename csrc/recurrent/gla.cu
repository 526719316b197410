// Gated linear attention as a recurrence over a per-sequence state, for ragged batches (portions of prompts next to
// single decoded tokens), bf16 or fp32 projections.
//
// Per head, with q_t, k_t (d numbers), v_t (e numbers) and a decay per key channel a_t in (0, 1):
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T            S: [d, e], fp32, zero before a sequence's first token
//     o_t = S_t^T q_t
//     a_t = sigmoid(z_t + bias)^(1/tau) = exp(logsigmoid(z_t + bias) / tau)
//
//   llmctl_gla_scan   : a CTA owns (portion, head, block of 32 value columns); lane = column, warp = block of RPT key
//       rows, whose state lives in registers for the whole portion.  Each warp loads its rows' q, k and decay logits
//       of the next token while it works on the current one (no block-wide staging); the per-row numbers reach the
//       lanes by shuffles; the warps' partial outputs meet in shared memory (one barrier per token, two buffers).
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

template <typename T, int RPT>
__global__ void __launch_bounds__(256)
gla_scan_kernel(const GlaParams p) {
  __shared__ float part[2][8][32];
  const int H = p.H, d = p.d, e = p.e;
  const int* pt = p.portions + blockIdx.x * 4;
  const int t0 = pt[0], n = pt[1], pos0 = pt[2], slot = pt[3];
  if (n <= 0) return;
  const int h = blockIdx.y, col = blockIdx.z * 32 + (threadIdx.x & 31);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int row0 = warp * RPT;
  const bool colok = col < e;
  const int myrow = row0 + lane;                         // the key row whose q / k / decay this lane fetches
  const bool rowok = lane < RPT && myrow < d;

  float S[RPT];
#pragma unroll
  for (int j = 0; j < RPT; ++j) S[j] = 0.f;
  float* st = slot >= 0 ? p.state + ((static_cast<long long>(slot) * H + h) * d) * e : nullptr;
  if (st && pos0 > 0 && colok) {
#pragma unroll
    for (int j = 0; j < RPT; ++j)
      if (row0 + j < d) S[j] = st[static_cast<long long>(row0 + j) * e + col];
  }
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const T* z = static_cast<const T*>(p.z);
  const float zb = (rowok && p.z_bias) ? p.z_bias[h * d + myrow] : 0.f;

  float nq = 0.f, nk = 0.f, nz = 0.f, nv = 0.f;
  auto fetch = [&](long long t) {
    if (rowok) {
      nq = to_f32(q[t * p.ldq + h * d + myrow]);
      nk = to_f32(k[t * p.ldk + h * d + myrow]);
      nz = to_f32(z[t * p.ldz + h * d + myrow]);
    }
    nv = colok ? to_f32(v[t * p.ldv + h * e + col]) : 0.f;
  };
  fetch(t0);
  for (int i = 0; i < n; ++i) {
    const float cq = rowok ? nq * p.q_scale : 0.f, ck = rowok ? nk : 0.f;
    // the decay minus one: a is close to 1 for slow channels, and S + (a - 1) S keeps it exact to ~1e-10 instead of the
    // ulp of 1 that a rounded factor carries (a state with a memory of thousands of tokens would accumulate that)
    const float ca = rowok ? expm1f(log_sigmoid(nz + zb) * p.inv_tau) : -1.f;
    const float cv = nv;
    if (i + 1 < n) fetch(t0 + i + 1);
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const float aj = __shfl_sync(0xffffffffu, ca, j), kj = __shfl_sync(0xffffffffu, ck, j), qj = __shfl_sync(0xffffffffu, cq, j);
      S[j] = fmaf(aj, S[j], fmaf(kj, cv, S[j]));
      o += qj * S[j];
    }
    part[i & 1][warp][lane] = o;
    __syncthreads();
    if (warp == 0 && colok) {
      float s = 0.f;
      for (int w = 0; w < nwarps; ++w) s += part[i & 1][w][lane];
      p.out[(static_cast<long long>(t0 + i) * H + h) * e + col] = s;
    }
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

LLMCTL_API int llmctl_gla_scan(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv, const void* z,
                               long long ldz, const float* z_bias, const int* portions, int nportions, float* state, float* out,
                               int H, int d, int e, float q_scale, float tau, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && d > 0 && d <= 256 && e > 0 && tau > 0.f);
  if (nportions == 0) return 0;
  GlaParams p{q, k, v, z, ldq, ldk, ldv, ldz, z_bias, portions, state, out, H, d, e, q_scale, 1.f / tau};
  const dim3 grid(nportions, H, (e + 31) / 32);
  cudaStream_t s = (cudaStream_t)stream;
  const int rpt = d <= 64 ? 8 : d <= 128 ? 16 : 32;
  const int threads = 32 * ((d + rpt - 1) / rpt);
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, {
    if (rpt == 8) gla_scan_kernel<T, 8><<<grid, threads, 0, s>>>(p);
    else if (rpt == 16) gla_scan_kernel<T, 16><<<grid, threads, 0, s>>>(p);
    else gla_scan_kernel<T, 32><<<grid, threads, 0, s>>>(p);
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
