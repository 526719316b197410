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
//   llmctl_residual_norm_canon_small : all of it in one launch, one block per portion, for batches of short portions
//       (decoding: a step is bound by its launches, not by bytes).
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

// four neighbouring elements of a bf16 or fp32 row (the address a multiple of 8 or 16 bytes)
__device__ __forceinline__ float4 load4_any(const void* p, int is32, long long i) {
  if (is32) return *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
  const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p) + i);
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                     __uint_as_float(u.y & 0xffff0000u));
}

// The same with 16-byte accesses (W and the strides multiples of 4, aligned rows): a thread owns four neighbouring columns.
__global__ void __launch_bounds__(256)
residual_rms_vec_kernel(const void* __restrict__ a, int a32, long long lda, const void* __restrict__ f, int f32, long long ldf,
                        float* __restrict__ x, float* __restrict__ r, int W, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float* row = x + t * W;
  float ss = 0.f;
  for (int c = threadIdx.x << 2; c < W; c += blockDim.x << 2) {
    float4 v = *reinterpret_cast<const float4*>(row + c);
    if (a != nullptr || f != nullptr) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a != nullptr) s = load4_any(a, a32, t * lda + c);
      if (f != nullptr) {
        const float4 g = load4_any(f, f32, t * ldf + c);
        s.x += g.x, s.y += g.y, s.z += g.z, s.w += g.w;
      }
      v.x += s.x, v.y += s.y, v.z += s.z, v.w += s.w;
      *reinterpret_cast<float4*>(row + c) = v;
    }
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) r[t] = 1.f / sqrtf(ss / static_cast<float>(W) + eps);
}

constexpr int kCanonMaxTaps = 8;
constexpr int kCanonChunk = 8;      // most consecutive tokens a thread of the vector kernel walks

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

// Vector path (W a multiple of 4): a thread owns four neighbouring channels of `tokens_per_cta` consecutive tokens and
// keeps the last TAPS - 1 normed rows in registers, so every row of x is read once; the window is rebuilt from the step's
// earlier rows or from the state slot at the block's first token and wherever a portion starts.
template <typename T, int TAPS>
__global__ void __launch_bounds__(256)
norm_canon_vec_kernel(const CanonParams p, int tokens, int tokens_per_cta) {
  constexpr int KEEP = TAPS - 1;
  const int W = p.W, W4 = W >> 2;
  const int t_begin = blockIdx.x * tokens_per_cta, t_end = min(tokens, t_begin + tokens_per_cta);
  // what is the same for every thread of the block is looked up once: a token's statistics and its index within its
  // portion (0: the window starts anew).  Per-thread scalar loads of these fill the load queue of the SM.
  __shared__ float s_rr[kCanonChunk];
  __shared__ int s_within[kCanonChunk];
  if (threadIdx.x < kCanonChunk) {
    const int t = t_begin + threadIdx.x;
    s_rr[threadIdx.x] = t < t_end ? p.r[t] : 0.f;
    s_within[threadIdx.x] = t < t_end ? t - p.portions[4 * p.seq_rows[t]] : -1;
  }
  __syncthreads();
  for (int c4 = blockIdx.y * blockDim.x + threadIdx.x; c4 < W4; c4 += gridDim.y * blockDim.x) {
    const int c = c4 << 2;
    float cw[2][4 * TAPS];              // a channel's taps follow one another: [channel * TAPS + tap], 16 bytes at a time
    float4 nw[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      nw[s] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s < p.S) {
        nw[s] = *reinterpret_cast<const float4*>(p.norm_w[s] + c);
        const float4* src = reinterpret_cast<const float4*>(p.conv_w[s] + static_cast<long long>(c) * TAPS);
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
          const float4 v = src[j];
          cw[s][4 * j] = v.x, cw[s][4 * j + 1] = v.y, cw[s][4 * j + 2] = v.z, cw[s][4 * j + 3] = v.w;
        }
      }
    }
    // all rows of the chunk are requested before the first one is used
    float4 rows[kCanonChunk];
    float rr[kCanonChunk];
#pragma unroll
    for (int k = 0; k < kCanonChunk; ++k) {
      rows[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      rr[k] = s_rr[k];
      if (t_begin + k < t_end) rows[k] = *reinterpret_cast<const float4*>(p.x + static_cast<long long>(t_begin + k) * W + c);
    }
    float4 win[KEEP > 0 ? KEEP : 1];
#pragma unroll
    for (int k = 0; k < kCanonChunk; ++k) {
      const int t = t_begin + k;
      if (t >= t_end) break;
      const int i = s_within[k];
      if (k == 0 || i == 0) {
        const int* pr = p.portions + 4 * p.seq_rows[t];
        const bool has_state = pr[2] > 0 && pr[3] >= 0;
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
          const int off = i - KEEP + j;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (off >= 0) {
            v = *reinterpret_cast<const float4*>(p.x + static_cast<long long>(t - KEEP + j) * W + c);
            const float rv = p.r[t - KEEP + j];
            v.x *= rv, v.y *= rv, v.z *= rv, v.w *= rv;
          } else if (has_state) {
            v = *reinterpret_cast<const float4*>(p.state + (static_cast<long long>(pr[3]) * KEEP + i + j) * W + c);
          }
          win[j] = v;
        }
      }
      float4 cur = rows[k];
      cur.x *= rr[k], cur.y *= rr[k], cur.z *= rr[k], cur.w *= rr[k];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (s < p.S) {
          float o[4] = {cur.x * (1.f + cw[s][KEEP]), cur.y * (1.f + cw[s][TAPS + KEEP]), cur.z * (1.f + cw[s][2 * TAPS + KEEP]),
                        cur.w * (1.f + cw[s][3 * TAPS + KEEP])};
#pragma unroll
          for (int j = 0; j < KEEP; ++j) {
            o[0] += cw[s][j] * win[j].x;
            o[1] += cw[s][TAPS + j] * win[j].y;
            o[2] += cw[s][2 * TAPS + j] * win[j].z;
            o[3] += cw[s][3 * TAPS + j] * win[j].w;
          }
          o[0] *= nw[s].x, o[1] *= nw[s].y, o[2] *= nw[s].z, o[3] *= nw[s].w;
          T* dst = static_cast<T*>(p.out[s]) + static_cast<long long>(t) * W + c;
          if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
          } else {
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
          }
        }
      }
#pragma unroll
      for (int j = 0; j + 1 < KEEP; ++j) win[j] = win[j + 1];
      if (KEEP > 0) win[KEEP > 0 ? KEEP - 1 : 0] = cur;
    }
  }
}

template <typename T>
static void launch_norm_canon_vec(const CanonParams& p, int tokens, cudaStream_t s) {
  // about two waves of blocks; long chunks amortise the window's rebuild, short ones keep small batches parallel
  const int per = max(1, min(kCanonChunk, tokens / (2 * kNumSMs)));
  const int W4 = p.W >> 2;
  const dim3 grid((tokens + per - 1) / per, (W4 + 255) / 256);
  const int threads = W4 >= 256 ? 256 : ((W4 + 31) / 32) * 32;
  switch (p.taps) {
#define LLMCTL_CANON_CASE(N) case N: norm_canon_vec_kernel<T, N><<<grid, threads, 0, s>>>(p, tokens, per); break;
    LLMCTL_CANON_CASE(1) LLMCTL_CANON_CASE(2) LLMCTL_CANON_CASE(3) LLMCTL_CANON_CASE(4)
    LLMCTL_CANON_CASE(5) LLMCTL_CANON_CASE(6) LLMCTL_CANON_CASE(7) LLMCTL_CANON_CASE(8)
#undef LLMCTL_CANON_CASE
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

// One token per portion and the whole row in one pass of the block (W / 4 <= threads): a thread owns four neighbouring
// channels, asks for the slot's rows and the weights before the row's statistics are known, and finishes from registers.
template <typename T, int TAPS>
__device__ __forceinline__ void residual_norm_canon_one_token(const void* __restrict__ a, int a32, long long lda, const void* __restrict__ f,
                                                              int f32, long long ldf, float* __restrict__ x, float eps, const CanonParams& p,
                                                              long long t, int pos0, int slot, float* red) {
  constexpr int KEEP = TAPS - 1;
  const int W = p.W, c = threadIdx.x << 2;
  const bool active = c < W;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 win[KEEP > 0 ? KEEP : 1];
  float4 nw[2];
  float* st = slot >= 0 && KEEP > 0 ? p.state + static_cast<long long>(slot) * KEEP * W : nullptr;
  if (active) {
    v = *reinterpret_cast<const float4*>(x + t * W + c);
    float add[4] = {0.f, 0.f, 0.f, 0.f};
    if (a != nullptr)
#pragma unroll
      for (int k = 0; k < 4; ++k) add[k] = load_any(a, a32, t * lda + c + k);
    if (f != nullptr)
#pragma unroll
      for (int k = 0; k < 4; ++k) add[k] += load_any(f, f32, t * ldf + c + k);
#pragma unroll
    for (int j = 0; j < KEEP; ++j)
      win[j] = (st != nullptr && pos0 > 0) ? *reinterpret_cast<const float4*>(st + static_cast<long long>(j) * W + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 2; ++s)
      if (s < p.S) nw[s] = *reinterpret_cast<const float4*>(p.norm_w[s] + c);
    if (a != nullptr || f != nullptr) {
      v.x += add[0], v.y += add[1], v.z += add[2], v.w += add[3];
      *reinterpret_cast<float4*>(x + t * W + c) = v;
    }
  }
  const float ss = block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, red);
  if (!active) return;
  const float r = 1.f / sqrtf(ss / static_cast<float>(W) + eps);
  const float4 cur = make_float4(v.x * r, v.y * r, v.z * r, v.w * r);
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    if (s < p.S) {
      float cw[4][TAPS];          // the same few kilobytes for every block: they come from the cache
#pragma unroll
      for (int ch = 0; ch < 4; ++ch)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) cw[ch][j] = p.conv_w[s][static_cast<long long>(c + ch) * TAPS + j];
      float o[4] = {cur.x * (1.f + cw[0][KEEP]), cur.y * (1.f + cw[1][KEEP]), cur.z * (1.f + cw[2][KEEP]), cur.w * (1.f + cw[3][KEEP])};
#pragma unroll
      for (int j = 0; j < KEEP; ++j) {
        o[0] += cw[0][j] * win[j].x;
        o[1] += cw[1][j] * win[j].y;
        o[2] += cw[2][j] * win[j].z;
        o[3] += cw[3][j] * win[j].w;
      }
      o[0] *= nw[s].x, o[1] *= nw[s].y, o[2] *= nw[s].z, o[3] *= nw[s].w;
      T* dst = static_cast<T*>(p.out[s]) + t * W + c;
      if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
      } else {
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
      }
    }
  }
  if (st != nullptr) {
#pragma unroll
    for (int j = 0; j + 1 < KEEP; ++j) *reinterpret_cast<float4*>(st + static_cast<long long>(j) * W + c) = win[j + 1];
    *reinterpret_cast<float4*>(st + static_cast<long long>(KEEP > 0 ? KEEP - 1 : 0) * W + c) = cur;
  }
}

// Small portions (each at most kCanonChunk tokens: a decoding batch): one block per portion does the residual update, the
// statistics, the sublayers' inputs and the slot's new rows in a single launch.  A thread owns the channels c, c + 256, ...
// through all phases, so it only ever rereads what it wrote itself; the rows' statistics cross the block once.  A portion of
// one token whose row fits one pass of the block takes the register path above.
template <typename T>
__global__ void __launch_bounds__(1024)
residual_norm_canon_small_kernel(const void* __restrict__ a, int a32, long long lda, const void* __restrict__ f, int f32, long long ldf,
                                 float* __restrict__ x, float eps, const CanonParams p, int vec_ok) {
  __shared__ float red[32];
  __shared__ float rr[kCanonChunk];
  const int* pr = p.portions + 4 * blockIdx.x;
  const int t0 = pr[0], n = min(pr[1], kCanonChunk), pos0 = pr[2], slot = pr[3];
  if (n <= 0) return;
  const int W = p.W, taps = p.taps, keep = taps - 1;
  if (n == 1 && vec_ok && (W >> 2) <= static_cast<int>(blockDim.x)) {       // uniform over the block
    switch (taps) {
#define LLMCTL_CANON_ONE(N) case N: residual_norm_canon_one_token<T, N>(a, a32, lda, f, f32, ldf, x, eps, p, t0, pos0, slot, red); return;
      LLMCTL_CANON_ONE(1) LLMCTL_CANON_ONE(2) LLMCTL_CANON_ONE(3) LLMCTL_CANON_ONE(4)
      LLMCTL_CANON_ONE(5) LLMCTL_CANON_ONE(6) LLMCTL_CANON_ONE(7) LLMCTL_CANON_ONE(8)
#undef LLMCTL_CANON_ONE
    }
  }
  for (int k = 0; k < n; ++k) {
    const long long t = t0 + k;
    float* row = x + t * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
      float v = row[c];
      if (a != nullptr || f != nullptr) {
        float sum = 0.f;
        if (a != nullptr) sum = load_any(a, a32, t * lda + c);
        if (f != nullptr) sum += load_any(f, f32, t * ldf + c);
        v += sum;
        row[c] = v;
      }
      ss += v * v;
    }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) rr[k] = 1.f / sqrtf(ss / static_cast<float>(W) + eps);
  }
  __syncthreads();
  const bool has_state = pos0 > 0 && slot >= 0;
  float* st = slot >= 0 && keep > 0 ? p.state + static_cast<long long>(slot) * keep * W : nullptr;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float nb[kCanonMaxTaps - 1 + kCanonChunk];          // normed values at offsets -keep .. n - 1 of the portion
    for (int m = 0; m < keep; ++m) nb[m] = has_state ? st[static_cast<long long>(m) * W + c] : 0.f;
    for (int k = 0; k < n; ++k) nb[keep + k] = x[static_cast<long long>(t0 + k) * W + c] * rr[k];
    for (int s = 0; s < p.S; ++s) {
      const float* cw = p.conv_w[s] + static_cast<long long>(c) * taps;
      const float nw = p.norm_w[s][c];
      for (int k = 0; k < n; ++k) {
        float acc = nb[keep + k];
        for (int j = 0; j < taps; ++j) acc += cw[j] * nb[k + j];
        static_cast<T*>(p.out[s])[static_cast<long long>(t0 + k) * W + c] = from_f32<T>(acc * nw);
      }
    }
    if (st != nullptr)
      for (int m = 0; m < keep; ++m) st[static_cast<long long>(m) * W + c] = nb[n + m];
  }
}

}  // namespace llmctl

using namespace llmctl;

LLMCTL_API int llmctl_residual_rms(const void* a, int a_is_fp32, long long lda, const void* f, int f_is_fp32, long long ldf, float* x,
                                   float* r, int tokens, int W, float eps, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(x != nullptr && r != nullptr && W > 0);
  if (tokens == 0) return 0;
  auto ok4 = [](const void* p, int is32, long long ld) {
    return p == nullptr || ((reinterpret_cast<uintptr_t>(p) & (is32 ? 15 : 7)) == 0 && ld % 4 == 0);
  };
  if (W % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ok4(a, a_is_fp32, lda) && ok4(f, f_is_fp32, ldf))
    residual_rms_vec_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>(a, a_is_fp32, lda, f, f_is_fp32, ldf, x, r, W, eps);
  else
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
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out0) | reinterpret_cast<uintptr_t>(out1) |
                         reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(norm_w0) | reinterpret_cast<uintptr_t>(norm_w1) |
                         reinterpret_cast<uintptr_t>(conv_w0) | reinterpret_cast<uintptr_t>(conv_w1)) & 15) == 0;
  if (W % 4 == 0 && aligned) {
    LLMCTL_DISPATCH_DTYPE(out_is_fp32, T, (launch_norm_canon_vec<T>(p, tokens, s)));
  } else {
    LLMCTL_DISPATCH_DTYPE(out_is_fp32, T, (norm_canon_kernel<T><<<tokens, 256, 0, s>>>(p)));
  }
  if (taps > 1 && nportions > 0) canon_state_store_kernel<<<nportions, 256, 0, s>>>(p);
  LLMCTL_RETURN_LAST();
}

// The three steps above in one launch for batches whose portions have at most 8 tokens each (decoding): x += a + f, the
// statistics, out_s and the state's new rows; one block per portion.
LLMCTL_API int llmctl_residual_norm_canon_small(const void* a, int a_is_fp32, long long lda, const void* f, int f_is_fp32, long long ldf,
                                                float* x, float eps, int S, const float* norm_w0, const float* conv_w0, void* out0,
                                                const float* norm_w1, const float* conv_w1, void* out1, const int* portions,
                                                int nportions, float* state, int W, int taps, int out_is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE((S == 1 || S == 2) && taps >= 1 && taps <= kCanonMaxTaps && W > 0 && (taps == 1 || state != nullptr) && x != nullptr);
  if (nportions == 0) return 0;
  CanonParams p{x, nullptr, {norm_w0, norm_w1}, {conv_w0, conv_w1}, {out0, out1}, portions, nullptr, state, S, W, taps};
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out0) | reinterpret_cast<uintptr_t>(out1) |
                         reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(norm_w0) | reinterpret_cast<uintptr_t>(norm_w1)) & 15) == 0;
  const int vec_ok = (W % 4 == 0 && aligned) ? 1 : 0;
  const int threads = vec_ok ? min(1024, max(128, ((W / 4 + 31) / 32) * 32)) : 256;
  LLMCTL_DISPATCH_DTYPE(out_is_fp32, T, (residual_norm_canon_small_kernel<T><<<nportions, threads, 0, (cudaStream_t)stream>>>(
                                            a, a_is_fp32, lda, f, f_is_fp32, ldf, x, eps, p, vec_ok)));
  LLMCTL_RETURN_LAST();
}
