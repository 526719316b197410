// Mixture-of-experts feed-forward: routing, token permutation, grouped expert GEMMs and the weighted combine, with no
// host synchronisation anywhere (expert loads stay on the device).  bf16 or fp32 activations / weights; router
// arithmetic, accumulators and the combine are fp32.
//
//   llmctl_moe_route   : per token, logits = Wr x (fp32), score = sigmoid or softmax over experts, the `top` largest
//                        (ties: lowest index), optionally renormalised to sum 1; optional per-token gate
//                        sigmoid(wg . x) of a shared expert; counts tokens per expert.  Optionally the CHOICE is made on
//                        score + correction[e] (the weights stay the plain scores) and restricted to the
//                        `keep_groups` of `n_groups` equal groups of neighbouring experts whose best choice score is
//                        largest (the others count as minus infinity).  Expert ids >= the number of experts with
//                        weights (`E` of plan / permute) are identity experts: they get no rows in the permuted
//                        buffer and the combine adds weight * (the token's input) for them.
//   llmctl_moe_plan    : one CTA: per-expert row offsets in the permuted buffer, every expert's segment padded to a
//                        multiple of the GEMM's row tile, and the tile -> expert map.
//   llmctl_moe_permute : copies every (token, choice) pair's input row into its expert's segment, multiplied by the
//                        routing weight when the weight applies to the expert's INPUT (scale_input), and records
//                        where it went.
//   llmctl_grouped_gemm: out[row, :] = A[row, :] W[expert(row)]^T over the permuted rows; a CTA computes a 64 x 64 tile
//                        of one expert (row tiles never straddle experts thanks to the padding).  bf16 with K and N
//                        multiples of 8 runs 64 x 128 tiles on the tensor cores (mma.sync m16n8k16, fp32 accumulation,
//                        next k-slice prefetched into registers); fp32 and odd sizes run the FMA kernel.
//                        bf16 on 128-row tiles can instead run on the tcgen05 GEMM's grouped mode (llmctl_gemm_bf16_grouped,
//                        csrc/gemm/gemm_tcgen05.cu), which reads the same plan.
//   llmctl_moe_combine : y[t] = sum_k (w_k if the weight applies to the OUTPUT) * expert_out[row(t, k)]
//                               + gate[t] * shared_out[t], in a fixed order (deterministic), fp32.
// Reference: none (the reference has no model code).
#include "../common/dtype.cuh"
#include "../common/mma_sync.cuh"

namespace llmctl {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

// x: fp32 [tokens, W] (the residual stream); wr: [E, W]; wg: [W] or null.
template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ x, const T* __restrict__ wr, const T* __restrict__ wg, int W, int E, int top,
                 int softmax_scores, int renormalise, const float* __restrict__ correction, int n_groups, int keep_groups,
                 int* __restrict__ ids, float* __restrict__ weights, float* __restrict__ gate, int* __restrict__ counts) {
  extern __shared__ float score[];   // [E] scores, then [E] choice scores
  float* choice = score + E;
  const long long tok = blockIdx.x;
  const float* xr = x + tok * W;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int e = warp; e < E + (wg ? 1 : 0); e += nwarp) {
    const T* w = e < E ? wr + static_cast<long long>(e) * W : wg;
    // four independent partial sums per lane: the loads of a row are in flight together (a decode step routes a
    // handful of tokens, so the kernel is pure latency); the order of the sum is fixed by W alone
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int c = lane;
    for (; c + 96 < W; c += 128) {
      s0 += xr[c] * to_f32(w[c]);
      s1 += xr[c + 32] * to_f32(w[c + 32]);
      s2 += xr[c + 64] * to_f32(w[c + 64]);
      s3 += xr[c + 96] * to_f32(w[c + 96]);
    }
    for (; c < W; c += 32) s0 += xr[c] * to_f32(w[c]);
    float s = (s0 + s1) + (s2 + s3);
    s = warp_sum(s);
    if (lane == 0) {
      if (e < E) score[e] = s;
      else gate[tok] = 1.f / (1.f + expf(-s));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (softmax_scores == 2) {
      // raw logits decide the choice; the weights are a softmax over the chosen logits only (below)
    } else if (softmax_scores) {
      float m = -INFINITY, z = 0.f;
      for (int e = 0; e < E; ++e) m = fmaxf(m, score[e]);
      for (int e = 0; e < E; ++e) z += (score[e] = expf(score[e] - m));
      for (int e = 0; e < E; ++e) score[e] /= z;
    } else {
      for (int e = 0; e < E; ++e) score[e] = 1.f / (1.f + expf(-score[e]));
    }
    for (int e = 0; e < E; ++e) choice[e] = score[e] + (correction ? correction[e] : 0.f);
    if (n_groups > 1 && keep_groups < n_groups) {
      // a group's score is its largest choice score; groups outside the best `keep_groups` cannot be chosen
      const int gs = E / n_groups;
      unsigned long long kept = 0ull;                  // n_groups <= 64
      for (int r = 0; r < keep_groups; ++r) {
        int bg = -1;
        float bgv = -INFINITY;
        for (int gi = 0; gi < n_groups; ++gi) {
          if (kept >> gi & 1ull) continue;
          float gv = -INFINITY;
          for (int e = gi * gs; e < (gi + 1) * gs; ++e) gv = fmaxf(gv, choice[e]);
          if (bg < 0 || gv > bgv) {
            bgv = gv;
            bg = gi;
          }
        }
        kept |= 1ull << bg;
      }
      for (int e = 0; e < E; ++e)
        if (!(kept >> (e / gs) & 1ull)) choice[e] = -INFINITY;
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e)
        if (choice[e] > bv || (best < 0 && choice[e] > -INFINITY)) {
          bv = choice[e];
          best = e;
        }
      if (best < 0) {                                  // fewer choosable experts than `top` (NaN scores): first unchosen one
        for (int e = 0; e < E && best < 0; ++e) {
          bool taken = false;
          for (int kk = 0; kk < k; ++kk) taken |= ids[tok * top + kk] == e;
          if (!taken) best = e;
        }
      }
      ids[tok * top + k] = best;
      weights[tok * top + k] = score[best];
      total += score[best];
      choice[best] = -INFINITY;
      atomicAdd(&counts[best], 1);
    }
    if (softmax_scores == 2) {
      const float m = weights[tok * top];        // the first choice is the largest logit
      float z = 0.f;
      for (int k = 0; k < top; ++k) z += (weights[tok * top + k] = expf(weights[tok * top + k] - m));
      for (int k = 0; k < top; ++k) weights[tok * top + k] /= z;
    } else if (renormalise)
      for (int k = 0; k < top; ++k) weights[tok * top + k] /= total + 1e-20f;
  }
}

// meta: int32 [2 * E + 2 + max_tiles] = { offsets[E] | cursor[E] | num_tiles | padded rows | tile_expert[max_tiles] }
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ meta, int max_tiles, int tile_m) {
  if (threadIdx.x != 0) return;
  int* offsets = meta;
  int* cursor = meta + E;
  int* tile_expert = meta + 2 * E + 2;
  int row = 0, tile = 0;
  for (int e = 0; e < E; ++e) {
    offsets[e] = row;
    cursor[e] = 0;
    const int nt = (counts[e] + tile_m - 1) / tile_m;
    for (int i = 0; i < nt && tile < max_tiles; ++i) tile_expert[tile++] = e;
    row += nt * tile_m;
  }
  meta[2 * E] = tile;
  meta[2 * E + 1] = row;
}

// One CTA per (token, choice).  dst rows of a segment beyond the expert's count are never read back.
template <typename T>
__global__ void __launch_bounds__(128)
moe_permute_kernel(const float* __restrict__ x, int W, const int* __restrict__ ids, const float* __restrict__ weights,
                   int scale_input, int* __restrict__ meta, int E, int top, int* __restrict__ pair_row, T* __restrict__ xs) {
  __shared__ int s_row;
  const long long pair = blockIdx.x;
  if (threadIdx.x == 0) {
    const int e = ids[pair];
    s_row = e < E ? meta[e] + atomicAdd(&meta[E + e], 1) : -1;       // ids >= E: identity experts, no row
    pair_row[pair] = s_row;
  }
  __syncthreads();
  if (s_row < 0) return;
  const long long tok = pair / top;
  const float w = scale_input ? weights[pair] : 1.f;
  const float* src = x + tok * W;
  T* dst = xs + static_cast<long long>(s_row) * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) dst[c] = from_f32<T>(w * src[c]);
}

// A: [padded rows, K] (row stride lda); Wt: [E, N, K] contiguous; out: [padded rows, N].
// 256 threads, each a 4 x 4 block of the 64 x 64 tile; fp32 accumulation whatever T.
template <typename T>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const T* __restrict__ A, long long lda, const T* __restrict__ Wt, T* __restrict__ out, long long ldo,
                    int N, int K, const int* __restrict__ meta, int E) {
  const int tile = blockIdx.x;
  if (tile >= meta[2 * E]) return;
  const int e = meta[2 * E + 2 + tile];
  const long long row0 = static_cast<long long>(tile) * kTileM;
  const int n0 = blockIdx.y * kTileN;
  const T* Bw = Wt + static_cast<long long>(e) * N * K;
  __shared__ float As[kTileK][kTileM + 4];
  __shared__ float Bs[kTileK][kTileN + 4];
  const int tid = threadIdx.x;
  const int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += kTileK) {
    for (int idx = tid; idx < kTileM * kTileK; idx += 256) {
      const int r = idx / kTileK, k = idx % kTileK;
      As[k][r] = (k0 + k < K) ? to_f32(A[(row0 + r) * lda + k0 + k]) : 0.f;
      const int n = n0 + r;
      Bs[k][r] = (k0 + k < K && n < N) ? to_f32(Bw[static_cast<long long>(n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTileK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[k][tr + i];
        b[i] = Bs[k][tc + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (n0 + tc + j < N) out[(row0 + tr + i) * ldo + n0 + tc + j] = from_f32<T>(acc[i][j]);
}

// bf16 tensor-core variant: 64 x 128 tile, 8 warps as 2 (rows) x 4 (columns), each 32 x 32.
constexpr int kTcN = 128, kTcK = 32, kTcLd = kTcK + 8;

__global__ void __launch_bounds__(256)
grouped_gemm_tc_kernel(const __nv_bfloat16* __restrict__ A, long long lda, const __nv_bfloat16* __restrict__ Wt,
                       __nv_bfloat16* __restrict__ out, long long ldo, int N, int K, const int* __restrict__ meta, int E) {
  const int tile = blockIdx.x;
  if (tile >= meta[2 * E]) return;
  const int e = meta[2 * E + 2 + tile];
  const long long row0 = static_cast<long long>(tile) * kTileM;
  const int n0 = blockIdx.y * kTcN;
  const __nv_bfloat16* Bw = Wt + static_cast<long long>(e) * N * K;
  __shared__ __align__(16) __nv_bfloat16 As[kTileM * kTcLd];
  __shared__ __align__(16) __nv_bfloat16 Bs[kTcN * kTcLd];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;
  const int lr = tid >> 2, lv = tid & 3;          // this thread's row and 8-element slice within a k-slice
  float acc[2][4][4] = {};
  uint4 ra, rb[2];
  auto fetch = [&](int k0) {
    const int k = k0 + lv * 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    ra = k < K ? *reinterpret_cast<const uint4*>(A + (row0 + lr) * lda + k) : zero;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int n = n0 + lr + 64 * i;
      rb[i] = (k < K && n < N) ? *reinterpret_cast<const uint4*>(Bw + static_cast<long long>(n) * K + k) : zero;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += kTcK) {
    *reinterpret_cast<uint4*>(As + lr * kTcLd + lv * 8) = ra;
    *reinterpret_cast<uint4*>(Bs + lr * kTcLd + lv * 8) = rb[0];
    *reinterpret_cast<uint4*>(Bs + (lr + 64) * kTcLd + lv * 8) = rb[1];
    __syncthreads();
    if (k0 + kTcK < K) fetch(k0 + kTcK);
#pragma unroll
    for (int kk = 0; kk < kTcK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) load_a_frag(a[mi], As, kTcLd, 32 * wm + 16 * mi, kk, lane);
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        uint32_t b[2];
        load_b_frag_nk(b, Bs, kTcLd, 32 * wn + 8 * ni, kk, lane);
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) mma_bf16_16816(acc[mi][ni], a[mi], b);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) {
      const int col = n0 + 32 * wn + 8 * ni + 2 * t;
      if (col < N) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const long long row = row0 + 32 * wm + 16 * mi + g + 8 * half;
          *reinterpret_cast<__nv_bfloat162*>(out + row * ldo + col) =
              __floats2bfloat162_rn(acc[mi][ni][2 * half], acc[mi][ni][2 * half + 1]);
        }
      }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* __restrict__ expert_out, int W, const int* __restrict__ pair_row,
                   const float* __restrict__ weights, int top, int scale_output, const T* __restrict__ shared_out,
                   const float* __restrict__ gate, const float* __restrict__ identity_in, float* __restrict__ y) {
  const long long tok = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = pair_row[tok * top + k];
      if (row < 0) {                                   // an identity expert: weight times the token's input
        a += weights[tok * top + k] * identity_in[tok * W + c];
        continue;
      }
      const float v = to_f32(expert_out[static_cast<long long>(row) * W + c]);
      a += scale_output ? weights[tok * top + k] * v : v;
    }
    if (shared_out) a += (gate ? gate[tok] : 1.f) * to_f32(shared_out[tok * W + c]);
    y[tok * W + c] = a;
  }
}

}  // namespace llmctl

using namespace llmctl;

LLMCTL_API int llmctl_moe_tile_rows() { return kTileM; }

LLMCTL_API int llmctl_moe_route(const float* x, const void* wr, const void* wg, int is_fp32, int tokens, int W, int E, int top,
                                int softmax_scores, int renormalise, const float* correction, int n_groups, int keep_groups,
                                int* ids, float* weights, float* gate, int* counts, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(E >= 1 && top >= 1 && top <= E && E <= 4096 && (wg == nullptr || gate != nullptr));
  LLMCTL_REQUIRE(n_groups <= 1 || (n_groups <= 64 && E % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups &&
                                   keep_groups * (E / n_groups) >= top));
  cudaStream_t s = (cudaStream_t)stream;
  LLMCTL_CHECK(cudaMemsetAsync(counts, 0, sizeof(int) * E, s));
  if (tokens == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (moe_route_kernel<T><<<tokens, 256, 2 * E * sizeof(float), s>>>(
                                        x, (const T*)wr, (const T*)wg, W, E, top, softmax_scores, renormalise, correction, n_groups,
                                        keep_groups, ids, weights, gate, counts)));
  LLMCTL_RETURN_LAST();
}

// tile_rows: the row tile of the grouped GEMM that will read the plan: llmctl_moe_tile_rows() for llmctl_grouped_gemm,
// 128 for llmctl_gemm_bf16_grouped (which takes tile_expert = meta + 2 E + 2 and num_tiles = meta + 2 E).
LLMCTL_API int llmctl_moe_plan(const int* counts, int E, int* meta, int max_tiles, int tile_rows, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(tile_rows == kTileM || tile_rows == 128);
  moe_plan_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(counts, E, meta, max_tiles, tile_rows);
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_moe_permute(const float* x, int W, const int* ids, const float* weights, int scale_input, int* meta,
                                  int E, int* pair_row, void* xs, int is_fp32, int tokens, int top, void* stream) {
  LLMCTL_BEGIN();
  if (tokens == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (moe_permute_kernel<T><<<tokens * top, 128, 0, (cudaStream_t)stream>>>(
                                        x, W, ids, weights, scale_input, meta, E, top, pair_row, (T*)xs)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_grouped_gemm(const void* A, long long lda, const void* Wt, void* out, long long ldo, int N, int K,
                                   const int* meta, int E, int max_tiles, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(N > 0 && K > 0 && lda >= K && ldo >= N);
  if (max_tiles == 0) return 0;
  if (!is_fp32 && K % 8 == 0 && N % 8 == 0 && lda % 8 == 0 && ldo % 2 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(Wt) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0) {
    grouped_gemm_tc_kernel<<<dim3(max_tiles, (N + kTcN - 1) / kTcN), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)Wt, (__nv_bfloat16*)out, ldo, N, K, meta, E);
    LLMCTL_RETURN_LAST();
  }
  dim3 grid(max_tiles, (N + kTileN - 1) / kTileN);
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (grouped_gemm_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
                                        (const T*)A, lda, (const T*)Wt, (T*)out, ldo, N, K, meta, E)));
  LLMCTL_RETURN_LAST();
}

LLMCTL_API int llmctl_moe_combine(const void* expert_out, int W, const int* pair_row, const float* weights, int top,
                                  int scale_output, const void* shared_out, const float* gate, const float* identity_in,
                                  float* y, int tokens, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  if (tokens == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (moe_combine_kernel<T><<<tokens, 256, 0, (cudaStream_t)stream>>>(
                                        (const T*)expert_out, W, pair_row, weights, top, scale_output, (const T*)shared_out, gate, identity_in, y)));
  LLMCTL_RETURN_LAST();
}
