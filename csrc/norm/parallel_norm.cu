// Parallel residual layout on an fp32 stream: one layer norm (weight and bias) feeds the mixer AND the feed-forward,
// and both outputs join the stream in one step:
//
//     h = (x - mean(x)) / sqrt(var(x) + eps) * w + b          var = mean of squared deviations
//     x <- x + m * (mixer(h) + ff(h))
//
//   llmctl_layernorm_rows     : optional x[row] += add[:] in place (a per-pass vector), then the norm of all rows or
//                               of selected rows, in the activation type and optionally also unrounded in fp32 (a
//                               router reads the latter).
//   llmctl_parallel_residual  : x += m * (a + f) in place (a: mixer output, bf16 or fp32; f: fp32 feed-forward output
//                               or null), optionally x += add, and optionally, from the same pass over the row, the
//                               layer norm of the new row with the NEXT layer's weights.
// One CTA per row; mean, variance, sums and the stream are fp32.  The row is held in registers between the passes
// (two-pass variance: no cancellation).
// Reference: none (the reference has no model code).
#include "../common/dtype.cuh"

namespace llmctl {

constexpr int kPnThreads = 256;
constexpr int kPnMaxPer = 16;      // row elements per thread held in registers: W <= 4096; wider rows re-read x

template <typename TO>
__device__ __forceinline__ void layernorm_row(const float* vals, int n_held, const float* __restrict__ xrow, int W,
                                              const float* __restrict__ w, const float* __restrict__ b, float eps,
                                              TO* __restrict__ out, float* __restrict__ out32, float* red) {
  const bool held = W <= kPnThreads * kPnMaxPer;
  float s = 0.f;
  if (held) {
#pragma unroll
    for (int i = 0; i < kPnMaxPer; ++i)
      if (i < n_held) s += vals[i];
  } else {
    for (int c = threadIdx.x; c < W; c += kPnThreads) s += xrow[c];
  }
  const float mean = block_sum(s, red) / W;
  float q = 0.f;
  if (held) {
#pragma unroll
    for (int i = 0; i < kPnMaxPer; ++i)
      if (i < n_held) {
        const float dlt = vals[i] - mean;
        q += dlt * dlt;
      }
  } else {
    for (int c = threadIdx.x; c < W; c += kPnThreads) {
      const float dlt = xrow[c] - mean;
      q += dlt * dlt;
    }
  }
  const float rstd = 1.f / sqrtf(block_sum(q, red) / W + eps);
  if (held) {
#pragma unroll
    for (int i = 0; i < kPnMaxPer; ++i)
      if (i < n_held) {
        const int c = threadIdx.x + i * kPnThreads;
        const float y = (vals[i] - mean) * rstd * w[c] + b[c];
        out[c] = from_f32<TO>(y);
        if (out32) out32[c] = y;
      }
  } else {
    for (int c = threadIdx.x; c < W; c += kPnThreads) {
      const float y = (xrow[c] - mean) * rstd * w[c] + b[c];
      out[c] = from_f32<TO>(y);
      if (out32) out32[c] = y;
    }
  }
}

template <typename TO>
__global__ void __launch_bounds__(kPnThreads)
layernorm_rows_kernel(float* __restrict__ x, const long long* __restrict__ rows, const float* __restrict__ add,
                      const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ out,
                      float* __restrict__ out32, int W, float eps) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  float* xrow = x + (rows ? rows[r] : r) * W;
  float vals[kPnMaxPer];
  int n = 0;
  const bool held = W <= kPnThreads * kPnMaxPer;
#pragma unroll
  for (int i = 0; i < kPnMaxPer; ++i) {
    const int c = threadIdx.x + i * kPnThreads;
    if (held && c < W) {
      float v = xrow[c];
      if (add) xrow[c] = v = v + add[c];
      vals[i] = v;
      n = i + 1;
    }
  }
  if (!held && add) {
    for (int c = threadIdx.x; c < W; c += kPnThreads) xrow[c] += add[c];
    __syncthreads();
  }
  layernorm_row<TO>(vals, n, xrow, W, w, b, eps, out + r * W, out32 ? out32 + r * W : nullptr, red);
}

template <typename TA, typename TO>
__global__ void __launch_bounds__(kPnThreads)
parallel_residual_kernel(const TA* __restrict__ a, long long lda, const float* __restrict__ f, float* __restrict__ x, float mult,
                         const float* __restrict__ add, const float* __restrict__ w, const float* __restrict__ b,
                         TO* __restrict__ out, float* __restrict__ out32, int W, float eps) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  float* xrow = x + r * W;
  const TA* arow = a + r * lda;
  const float* frow = f ? f + r * W : nullptr;
  float vals[kPnMaxPer];
  int n = 0;
  const bool held = W <= kPnThreads * kPnMaxPer;
  if (held) {
#pragma unroll
    for (int i = 0; i < kPnMaxPer; ++i) {
      const int c = threadIdx.x + i * kPnThreads;
      if (c < W) {
        float v = xrow[c] + mult * (to_f32(arow[c]) + (frow ? frow[c] : 0.f));
        if (add) v += add[c];
        xrow[c] = v;
        vals[i] = v;
        n = i + 1;
      }
    }
  } else {
    for (int c = threadIdx.x; c < W; c += kPnThreads) {
      float v = xrow[c] + mult * (to_f32(arow[c]) + (frow ? frow[c] : 0.f));
      if (add) v += add[c];
      xrow[c] = v;
    }
    __syncthreads();
  }
  if (w) layernorm_row<TO>(vals, n, xrow, W, w, b, eps, out + r * W, out32 ? out32 + r * W : nullptr, red);
}

}  // namespace llmctl

using namespace llmctl;

// x: fp32 [*, W] (modified when `add` is given, which needs rows == null); out: [n, W] bf16 or fp32; out32: fp32 or null.
LLMCTL_API int llmctl_layernorm_rows(float* x, const long long* rows, const float* add, const float* w, const float* b, void* out,
                                     int out_fp32, float* out32, int n, int W, float eps, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(W > 0 && !(add && rows));
  if (n == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(out_fp32, TO, (layernorm_rows_kernel<TO><<<n, kPnThreads, 0, (cudaStream_t)stream>>>(
                                          x, rows, add, w, b, (TO*)out, out32, W, eps)));
  LLMCTL_RETURN_LAST();
}

// a: [T, W] (row stride lda) bf16 or fp32; f: fp32 [T, W] or null; x: fp32 [T, W] in place; w/b null = no following norm.
LLMCTL_API int llmctl_parallel_residual(const void* a, int a_fp32, long long lda, const float* f, float* x, float mult,
                                        const float* add, const float* w, const float* b, void* out, int out_fp32, float* out32,
                                        int T, int W, float eps, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(W > 0 && lda >= W && (w == nullptr || (b != nullptr && out != nullptr)));
  if (T == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (a_fp32) {
    LLMCTL_DISPATCH_DTYPE(out_fp32, TO, (parallel_residual_kernel<float, TO><<<T, kPnThreads, 0, s>>>(
                                            (const float*)a, lda, f, x, mult, add, w, b, (TO*)out, out32, W, eps)));
  } else {
    LLMCTL_DISPATCH_DTYPE(out_fp32, TO, (parallel_residual_kernel<__nv_bfloat16, TO><<<T, kPnThreads, 0, s>>>(
                                            (const __nv_bfloat16*)a, lda, f, x, mult, add, w, b, (TO*)out, out32, W, eps)));
  }
  LLMCTL_RETURN_LAST();
}
