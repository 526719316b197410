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
//   llmctl_selective_scan   : four lanes per channel share its N states (interleaved), a CTA owns 32 channels of one
//       portion and walks its tokens with the next token's operands in flight; the lanes' partial sums meet by two
//       shuffles.  At the end the CTA stores S and the portion's last taps-1 raw inputs (shifting in stored ones when
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

template <typename T, int SPT>
__global__ void __launch_bounds__(128)
selective_scan_kernel(const ScanParams p) {
  const int C = p.C, N = p.N;
  const int* pt = p.portions + blockIdx.x * 4;
  const int t0 = pt[0], n = pt[1], pos0 = pt[2], slot = pt[3];
  if (n <= 0) return;
  const int sub = threadIdx.x & 3;
  const int c = blockIdx.y * 32 + (threadIdx.x >> 2);
  const bool cok = c < C;
  const T* u = static_cast<const T*>(p.u);
  const T* bc = static_cast<const T*>(p.bc);
  const T* dtp = static_cast<const T*>(p.dtp);
  const T* z = static_cast<const T*>(p.z);
  float S[SPT], A[SPT];
  float* st = (slot >= 0 && cok) ? p.state + (static_cast<long long>(slot) * C + c) * N : nullptr;
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    const int s = sub + 4 * i;
    A[i] = (cok && s < N) ? p.A[static_cast<long long>(c) * N + s] : 0.f;
    S[i] = (st && pos0 > 0 && s < N) ? st[s] : 0.f;
  }
  const float dtb = cok ? p.dt_bias[c] : 0.f, Dc = cok ? p.D[c] : 0.f;
  float nB[SPT], nC[SPT], ndt = 0.f, nu = 0.f, nz = 0.f;
  auto fetch = [&](long long t) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      const int s = sub + 4 * i;
      nB[i] = s < N ? to_f32(bc[t * p.ldbc + p.off_b + s]) : 0.f;
      nC[i] = s < N ? to_f32(bc[t * p.ldbc + p.off_c + s]) : 0.f;
    }
    if (cok) {
      ndt = to_f32(dtp[t * p.lddt + c]);
      nu = to_f32(u[t * C + c]);
      nz = to_f32(z[t * p.ldz + c]);
    }
  };
  fetch(t0);
  for (int i = 0; i < n; ++i) {
    float B[SPT], Cc[SPT];
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
      B[k] = nB[k];
      Cc[k] = nC[k];
    }
    const float dt = softplus_f(ndt + dtb), uu = nu, zz = nz;
    if (i + 1 < n) fetch(t0 + i + 1);
    const float du = dt * uu;
    float y = 0.f;
#pragma unroll
    for (int k = 0; k < SPT; ++k) {
      // exp(dt A) is close to 1 for slow channels: S + expm1(dt A) S keeps the decay exact to ~1e-10 instead of the
      // ulp of 1 that a rounded factor carries, which a state with a memory of thousands of tokens would accumulate
      S[k] = fmaf(expm1f(dt * A[k]), S[k], fmaf(du, B[k], S[k]));
      y += S[k] * Cc[k];
    }
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    y += __shfl_xor_sync(0xffffffffu, y, 2);
    if (sub == 0 && cok) static_cast<T*>(p.out)[static_cast<long long>(t0 + i) * C + c] = from_f32<T>((y + Dc * uu) * silu_f(zz));
  }
  if (st) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      const int s = sub + 4 * i;
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
  const dim3 grid(nportions, (C + 31) / 32);
  cudaStream_t s = (cudaStream_t)stream;
  const int spt = (N + 3) / 4;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, {
    if (spt <= 4) selective_scan_kernel<T, 4><<<grid, 128, 0, s>>>(p);
    else if (spt <= 8) selective_scan_kernel<T, 8><<<grid, 128, 0, s>>>(p);
    else if (spt <= 16) selective_scan_kernel<T, 16><<<grid, 128, 0, s>>>(p);
    else selective_scan_kernel<T, 32><<<grid, 128, 0, s>>>(p);
  });
  LLMCTL_RETURN_LAST();
}
