// Pre-norm with a short causal convolution on the normed stream ("canon" input convolution), for ragged batches whose
// sequences keep the last taps - 1 normed rows in a state slot.
//
// The residual stream x is fp32.  A layer's sublayers all read the same normed stream n = x / sqrt(mean(x^2) + eps), each
// through its own norm weight w_s and its own depthwise convolution c_s over time:
//
//     h_s[t]   = w_s * n[t]
//     out_s[t] = h_s[t] + sum_j c_s[:, j] * h_s[t - taps + 1 + j]        j = 0 .. taps - 1, zeros before position 0
//
//   llmctl_residual_rms : x[t] += a[t] + f[t] (each optional, bf16 or fp32) and r[t] = 1 / sqrt(mean(x[t]^2) + eps): the
//       residual update of a layer with the statistics of the next layer's norm, one pass over the row.
//   llmctl_norm_canon   : out_s for up to two sublayers from x and r; rows before a portion's first token come from the
//       sequence's state slot ([slots, taps - 1, W] fp32, the unweighted n of the last taps - 1 positions, oldest first;
//       a portion that starts at position 0 reads zeros whatever the slot holds).  A second launch then stores the new
//       last rows: the first one only reads the state, so no block can see a row of the step it is in.
// Everything is fp32 up to the rounding of out_s to the activation type.
// Reference: none (the reference has no model code).
#include "../common/dtype.cuh"

namespace llmctl {

__device__ __forceinline__ float load_any(const void* p, int is32, long long i) {
  return is32 ? static_cast<const float*>(p)[i] : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__global__ void __launch_bounds__(256)
residual_rms_kernel(const void* __restrict__ a, int a32, long long lda, const void* __restrict__ f, int f32, long long ldf,
                    float* __restrict__ x, float* __restrict__ r, int W, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float* row = x + t * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = row[c];
    if (a != nullptr || f != nullptr) {
      float s = 0.f;
      if (a != nullptr) s = load_any(a, a32, t * lda + c);
      if (f != nullptr) s += load_any(f, f32, t * ldf + c);
      v += s;
      row[c] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) r[t] = 1.f / sqrtf(ss / static_cast<float>(W) + eps);
}

constexpr int kCanonMaxTaps = 8;

struct CanonParams {
  const float* x;            // [T, W]
  const float* r;            // [T]
  const float* norm_w[2];    // [W] each
  const float* conv_w[2];    // [W, taps] each
  void* out[2];              // [T, W] each, activation type
  const int* portions;       // [B, 4] = (first token row, tokens, position of the first token, state slot)
  const int* seq_rows;       // [T] portion of every token
  float* state;              // [slots, taps - 1, W]
  int S, W, taps;
};

template <typename T>
__global__ void __launch_bounds__(256)
norm_canon_kernel(const CanonParams p) {
  const long long t = blockIdx.x;
  const int W = p.W, taps = p.taps, keep = taps - 1;
  const int* pr = p.portions + 4 * p.seq_rows[t];
  const int i = static_cast<int>(t) - pr[0];                  // offset of the token within its portion
  const bool has_state = pr[2] > 0 && pr[3] >= 0;
  const float* st = has_state ? p.state + static_cast<long long>(pr[3]) * keep * W : nullptr;
  // source of tap j: row t - keep + j of the step, or row i + j of the state
  const float* src[kCanonMaxTaps];
  float mul[kCanonMaxTaps];
#pragma unroll
  for (int j = 0; j < kCanonMaxTaps; ++j) {
    src[j] = nullptr;
    mul[j] = 0.f;
    if (j < taps) {
      const int off = i - keep + j;
      if (off >= 0) {
        src[j] = p.x + (t - keep + j) * W;
        mul[j] = p.r[t - keep + j];
      } else if (st != nullptr) {
        src[j] = st + static_cast<long long>(i + j) * W;
        mul[j] = 1.f;
      }
    }
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float n[kCanonMaxTaps];
#pragma unroll
    for (int j = 0; j < kCanonMaxTaps; ++j) n[j] = (j < taps && src[j] != nullptr) ? src[j][c] * mul[j] : 0.f;
    for (int s = 0; s < p.S; ++s) {
      const float* cw = p.conv_w[s] + static_cast<long long>(c) * taps;
      float acc = 0.f, cur = 0.f;
#pragma unroll
      for (int j = 0; j < kCanonMaxTaps; ++j)
        if (j < taps) {
          acc += cw[j] * n[j];
          if (j == keep) cur = n[j];
        }
      static_cast<T*>(p.out[s])[t * W + c] = from_f32<T>((cur + acc) * p.norm_w[s][c]);
    }
  }
}

// One block per portion: the slot's new rows are the last taps - 1 normed rows of the sequence, taken from the step's
// rows and, for portions shorter than that, from the slot's own later rows.
__global__ void __launch_bounds__(256)
canon_state_store_kernel(const CanonParams p) {
  const int* pr = p.portions + 4 * blockIdx.x;
  const int t0 = pr[0], n = pr[1], pos0 = pr[2], slot = pr[3];
  const int W = p.W, keep = p.taps - 1;
  if (slot < 0 || n <= 0 || keep <= 0) return;
  float* st = p.state + static_cast<long long>(slot) * keep * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v[kCanonMaxTaps];
#pragma unroll
    for (int k = 0; k < kCanonMaxTaps - 1; ++k) {
      v[k] = 0.f;
      if (k < keep) {
        const int off = n - keep + k;
        if (off >= 0) v[k] = p.x[static_cast<long long>(t0 + off) * W + c] * p.r[t0 + off];
        else if (pos0 > 0) v[k] = st[static_cast<long long>(k + n) * W + c];
      }
    }
#pragma unroll
    for (int k = 0; k < kCanonMaxTaps - 1; ++k)
      if (k < keep) st[static_cast<long long>(k) * W + c] = v[k];
  }
}

}  // namespace llmctl

using namespace llmctl;

LLMCTL_API int llmctl_residual_rms(const void* a, int a_is_fp32, long long lda, const void* f, int f_is_fp32, long long ldf, float* x,
                                   float* r, int tokens, int W, float eps, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(x != nullptr && r != nullptr && W > 0);
  if (tokens == 0) return 0;
  residual_rms_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>(a, a_is_fp32, lda, f, f_is_fp32, ldf, x, r, W, eps);
  LLMCTL_RETURN_LAST();
}

// S = 1 or 2 sublayers; norm_w1 / conv_w1 / out1 are ignored for S = 1.  state may be null when taps == 1.
LLMCTL_API int llmctl_norm_canon(const float* x, const float* r, int S, const float* norm_w0, const float* conv_w0, void* out0,
                                 const float* norm_w1, const float* conv_w1, void* out1, const int* portions, int nportions,
                                 const int* seq_rows, float* state, int tokens, int W, int taps, int out_is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE((S == 1 || S == 2) && taps >= 1 && taps <= kCanonMaxTaps && W > 0 && (taps == 1 || state != nullptr));
  if (tokens == 0) return 0;
  CanonParams p{x, r, {norm_w0, norm_w1}, {conv_w0, conv_w1}, {out0, out1}, portions, seq_rows, state, S, W, taps};
  cudaStream_t s = (cudaStream_t)stream;
  LLMCTL_DISPATCH_DTYPE(out_is_fp32, T, (norm_canon_kernel<T><<<tokens, 256, 0, s>>>(p)));
  if (taps > 1 && nportions > 0) canon_state_store_kernel<<<nportions, 256, 0, s>>>(p);
  LLMCTL_RETURN_LAST();
}
