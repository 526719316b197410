// Selective state-space scan (Mamba) with its short causal convolution, for ragged batches (portions of prompts next
// to single decoded tokens), bf16 or fp32 projections.
//
// Per channel c of the inner width and state index n < N, with u_t the convolved and activated input:
//
//     u_t[c]   = silu(sum_j w[c, j] x_(t - (taps-1-j))[c] + wb[c])         (inputs before the sequence are zero)
//     dt_t[c]  = softplus(dtp_t[c] + dt_bias[c])
//     S[c, n] <- exp(dt_t[c] A[c, n]) S[c, n] + dt_t[c] u_t[c] B_t[n]      (S fp32, zero before the first token)
//     y_t[c]   = (sum_n S[c, n] C_t[n] + D[c] u_t[c]) * silu(z_t[c])
//
// A sequence's state is S and the last taps-1 raw inputs x of every channel.
//
//   llmctl_causal_conv_silu : one thread per (token, channel); inputs before the portion come from the slot's stored
//       inputs (zeros when the portion starts the sequence).  Reads the stored inputs only.
//   llmctl_selective_scan   : 4 or 16 lanes per channel share its N states (interleaved), a CTA owns 32 or 8 channels of
//       one portion and walks its tokens in chunks of 16: a chunk's step sizes (softplus evaluated once per number), inputs,
//       gates, B and C are staged in shared memory while the previous chunk's steps run; the lanes' partial sums meet
//       by shuffles.  At the end the CTA stores S and the portion's last taps-1 raw inputs (shifting in stored ones when
//       the portion is shorter).  A portion at position 0 starts from zeros whatever its slot holds.
// The decay is applied as S + expm1(dt A) S.  Step sizes, exponentials, state and sums are fp32; x, z, B, C and dtp are
// read in the projections' type.
// Reference: none (the reference has no model code).
#include "../common/dtype.cuh"

namespace llmctl {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

// x: [T, *] raw inputs (row stride ldx); conv_state: fp32 [slots, taps-1, C]; out: [T, C]
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ w, const float* __restrict__ wb,
                        const int* __restrict__ portions, const int* __restrict__ seq_rows, const float* __restrict__ conv_state,
                        T* __restrict__ out, int C, int taps) {
  const long long t = blockIdx.x;
  const int* pt = portions + seq_rows[t] * 4;
  const int t0 = pt[0], pos0 = pt[2], slot = pt[3];
  const float* st = (slot >= 0 && pos0 > 0) ? conv_state + static_cast<long long>(slot) * (taps - 1) * C : nullptr;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float a = wb ? wb[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const long long src = t - (taps - 1 - j);                    // token row of this tap's input
      float v = 0.f;
      if (src >= t0) v = to_f32(x[src * ldx + c]);
      else if (st) v = st[static_cast<long long>(taps - 1 - (t0 - src)) * C + c];
      a += w[c * taps + j] * v;
    }
    out[t * C + c] = from_f32<T>(silu_f(a));
  }
}

struct ScanParams {
  const void* u;        // [T, C] convolved inputs
  const void* bc;       // [T, *]: B at column off_b, C at column off_c (row stride ldbc)
  long long ldbc;
  int off_b, off_c;
  const void* dtp;      // [T, C] (row stride lddt)
  long long lddt;
  const float* dt_bias; // [C]
  const float* A;       // [C, N] (negative)
  const float* D;       // [C]
  const void* z;        // [T, *] gate pre-activation, channel c at column c (row stride ldz)
  long long ldz;
  const void* x;        // raw inputs of the convolution (row stride ldx), for the stored inputs
  long long ldx;
  const int* portions;
  float* state;         // [slots, C, N]
  float* conv_state;    // [slots, taps-1, C]
  void* out;            // [T, C]
  int C, N, taps;
};

constexpr int kScanTC = 16;     // tokens staged per chunk

// exp(x) - 1 for x <= 0: the series where the result is small (relative error < 1e-8 there), exp2-based elsewhere, where
// the decay 1 + result is at most 0.94 and its 2-ulp error dies out within a few tokens
__device__ __forceinline__ float expm1_neg(float x) {
  const float series = x * (1.f + x * (0.5f + x * (0.16666667f + x * (0.041666668f + x * 0.0083333338f))));
  return x > -0.0625f ? series : __expf(x) - 1.f;
}

// LPC lanes share a channel's N states (state s of lane `sub` and register k is sub + LPC * k); a CTA of 128 threads owns
// 128 / LPC channels of one portion.
template <typename T, int SPT, int LPC>
__global__ void __launch_bounds__(128)
selective_scan_kernel(const ScanParams p) {
  constexpr int TC = kScanTC, NP = LPC * SPT;        // NP: padded state count
  constexpr int CPB = 128 / LPC;                     // channels per CTA
  constexpr int NST = TC * CPB / 128;                // (dt, u, z) staging elements per thread and chunk
  constexpr int NBC = (TC * 2 * NP + 127) / 128;     // B / C staging elements per thread and chunk
  __shared__ float sdt[TC][CPB], su[TC][CPB], sz[TC][CPB];
  __shared__ float sBC[TC][2 * NP];                  // [B | C] of a token
  const int C = p.C, N = p.N;
  const int* pt = p.portions + blockIdx.x * 4;
  const int t0 = pt[0], n = pt[1], pos0 = pt[2], slot = pt[3];
  if (n <= 0) return;
  const int tid = threadIdx.x, sub = tid % LPC, chl = tid / LPC;
  const int c = blockIdx.y * CPB + chl;
  const bool cok = c < C;
  const T* u = static_cast<const T*>(p.u);
  const T* bc = static_cast<const T*>(p.bc);
  const T* dtp = static_cast<const T*>(p.dtp);
  const T* z = static_cast<const T*>(p.z);
  float S[SPT], A[SPT];
  float* st = (slot >= 0 && cok) ? p.state + (static_cast<long long>(slot) * C + c) * N : nullptr;
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    const int s = sub + LPC * i;
    A[i] = (cok && s < N) ? p.A[static_cast<long long>(c) * N + s] : 0.f;
    S[i] = (st && pos0 > 0 && s < N) ? st[s] : 0.f;
  }
  const float Dc = cok ? p.D[c] : 0.f;
  // staging: element j of this thread is (token stok + j * (128 / CPB), channel sch) of dt, u and z
  const int sch = tid % CPB, stok = tid / CPB;
  const int gch = blockIdx.y * CPB + sch;
  const float dtb = gch < C ? p.dt_bias[gch] : 0.f;
  // B and C: element tid + 128 i of the chunk's [TC][2 N] numbers -> (token, source column, slot in sBC)
  int bc_tok[NBC], bc_col[NBC], bc_dst[NBC];
#pragma unroll
  for (int i = 0; i < NBC; ++i) {
    const int idx = tid + 128 * i, tok = idx / (2 * N), r = idx % (2 * N);
    bc_tok[i] = tok < TC ? tok : -1;
    bc_col[i] = r < N ? p.off_b + r : p.off_c + r - N;
    bc_dst[i] = tok * 2 * NP + (r < N ? r : NP + r - N);
  }
  float rdt[NST], ru[NST], rz[NST], rbc[NBC];
  auto fetch = [&](int c0) {
#pragma unroll
    for (int j = 0; j < NST; ++j) {
      const int tok = stok + j * (128 / CPB);
      const bool ok = c0 + tok < n && gch < C;
      const long long t = t0 + c0 + tok;
      rdt[j] = ok ? to_f32(dtp[t * p.lddt + gch]) : 0.f;
      ru[j] = ok ? to_f32(u[t * C + gch]) : 0.f;
      rz[j] = ok ? to_f32(z[t * p.ldz + gch]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NBC; ++i)
      rbc[i] = (bc_tok[i] >= 0 && c0 + bc_tok[i] < n) ? to_f32(bc[static_cast<long long>(t0 + c0 + bc_tok[i]) * p.ldbc + bc_col[i]]) : 0.f;
  };
  auto stash = [&]() {
#pragma unroll
    for (int j = 0; j < NST; ++j) {
      const int tok = stok + j * (128 / CPB);
      sdt[tok][sch] = softplus_f(rdt[j] + dtb);
      su[tok][sch] = ru[j];
      sz[tok][sch] = rz[j];
    }
#pragma unroll
    for (int i = 0; i < NBC; ++i)
      if (bc_tok[i] >= 0) (&sBC[0][0])[bc_dst[i]] = rbc[i];
  };
  for (int i = tid; i < TC * 2 * NP; i += 128) (&sBC[0][0])[i] = 0.f;          // states beyond N stay zero
  __syncthreads();
  fetch(0);
  stash();
  __syncthreads();
  for (int c0 = 0; c0 < n; c0 += TC) {
    const bool more = c0 + TC < n;
    if (more) fetch(c0 + TC);                         // the next chunk's loads fly during this chunk's steps
    const int cnt = min(TC, n - c0);
    for (int tok = 0; tok < cnt; ++tok) {
      const float dt = sdt[tok][chl], uu = su[tok][chl];
      const float du = dt * uu;
      float y = 0.f;
#pragma unroll
      for (int k = 0; k < SPT; ++k) {
        // exp(dt A) is close to 1 for slow channels: S + expm1(dt A) S keeps the decay exact to ~1e-8 instead of the
        // ulp of 1 that a rounded factor carries, which a state with a memory of thousands of tokens would accumulate
        S[k] = fmaf(expm1_neg(dt * A[k]), S[k], fmaf(du, sBC[tok][sub + LPC * k], S[k]));
        y += S[k] * sBC[tok][NP + sub + LPC * k];
      }
#pragma unroll
      for (int o = 1; o < LPC; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (sub == 0 && cok) static_cast<T*>(p.out)[static_cast<long long>(t0 + c0 + tok) * C + c] = from_f32<T>((y + Dc * uu) * silu_f(sz[tok][chl]));
    }
    __syncthreads();                                  // the staged chunk has been read
    if (more) stash();
    __syncthreads();
  }
  if (st) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      const int s = sub + LPC * i;
      if (s < N) st[s] = S[i];
    }
  }
  // the stored inputs of the convolution: entry i is the raw input (taps-1-i) tokens before the next one.  Ascending i
  // reads stored entries above i only, so the shift is safe in place.
  if (sub == 0 && cok && slot >= 0) {
    const int keep = p.taps - 1;
    float* cs = p.conv_state + static_cast<long long>(slot) * keep * C + c;
    const T* x = static_cast<const T*>(p.x);
    for (int i = 0; i < keep; ++i) {
      const int idx = n - keep + i;                     // index within the portion
      float v = 0.f;
      if (idx >= 0) v = to_f32(x[static_cast<long long>(t0 + idx) * p.ldx + c]);
      else if (pos0 > 0) v = cs[static_cast<long long>(keep + idx) * C];
      cs[static_cast<long long>(i) * C] = v;
    }
  }
}

}  // namespace llmctl

using namespace llmctl;

// seq_rows: int32 [tokens], the row of `portions` each token belongs to.  w: fp32 [C, taps], wb: fp32 [C] or null.
LLMCTL_API int llmctl_causal_conv_silu(const void* x, long long ldx, const float* w, const float* wb, const int* portions,
                                       const int* seq_rows, const float* conv_state, void* out, int tokens, int C, int taps,
                                       int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(C > 0 && taps >= 1 && ldx >= C);
  if (tokens == 0) return 0;
  const dim3 grid(tokens, (C + 1023) / 1024);
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (causal_conv_silu_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
                                        (const T*)x, ldx, w, wb, portions, seq_rows, conv_state, (T*)out, C, taps)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_selective_scan(const void* u, const void* bc, long long ldbc, int off_b, int off_c, const void* dtp, long long lddt,
                                     const float* dt_bias, const float* A, const float* D, const void* z, long long ldz, const void* x,
                                     long long ldx, const int* portions, int nportions, float* state, float* conv_state, void* out,
                                     int C, int N, int taps, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(C > 0 && N > 0 && N <= 128 && taps >= 1);
  if (nportions == 0) return 0;
  ScanParams p{u, bc, ldbc, off_b, off_c, dtp, lddt, dt_bias, A, D, z, ldz, x, ldx, portions, state, conv_state, out, C, N, taps};
  cudaStream_t s = (cudaStream_t)stream;
  // 4 lanes per channel and 32 channels per CTA when that already fills the GPU (many portions) or the states are few:
  // fewest instructions per (token, channel).  Otherwise 16 lanes per channel and 8 channels per CTA: a step is one or
  // two exponentials per thread and a portion spreads over four times as many CTAs (long prompts, few sequences).
  const dim3 grid4(nportions, (C + 31) / 32), grid16(nportions, (C + 7) / 8);
  const bool wide = N > 8 && static_cast<long long>(nportions) * ((C + 31) / 32) < 2 * kNumSMs;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, {
    if (wide) {
      if (N <= 16) selective_scan_kernel<T, 1, 16><<<grid16, 128, 0, s>>>(p);
      else if (N <= 32) selective_scan_kernel<T, 2, 16><<<grid16, 128, 0, s>>>(p);
      else if (N <= 64) selective_scan_kernel<T, 4, 16><<<grid16, 128, 0, s>>>(p);
      else selective_scan_kernel<T, 8, 16><<<grid16, 128, 0, s>>>(p);
    } else {
      if (N <= 4) selective_scan_kernel<T, 1, 4><<<grid4, 128, 0, s>>>(p);
      else if (N <= 8) selective_scan_kernel<T, 2, 4><<<grid4, 128, 0, s>>>(p);
      else if (N <= 16) selective_scan_kernel<T, 4, 4><<<grid4, 128, 0, s>>>(p);
      else if (N <= 32) selective_scan_kernel<T, 8, 4><<<grid4, 128, 0, s>>>(p);
      else if (N <= 64) selective_scan_kernel<T, 16, 4><<<grid4, 128, 0, s>>>(p);
      else selective_scan_kernel<T, 32, 4><<<grid4, 128, 0, s>>>(p);
    }
  });
  LLMCTL_RETURN_LAST();
}
