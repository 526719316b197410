// Latent (low-rank joint key/value) attention over a paged cache, for prompts, portions of prompts and decoded
// tokens in one ragged batch; bf16 or fp32 activations and cache, all attention arithmetic in fp32.
//
// What is cached per token is ONE row shared by all heads: [ c (R numbers: the RMS-normed latent) | kr (dr numbers:
// the rotated key part) ].  The per-head keys and values are linear images of c (k_h = Uk_h c, v_h = Uv_h c), so
//
//     score(i, j, h) = (Uk_h^T qn_ih) . c_j  +  qr_ih . kr_j          out_ih = Uv_h * sum_j p_ij c_j
//
// The caller folds Uk_h into the query ("absorbed" query ql = Uk_h^T qn, R numbers) and applies Uv_h to the
// kernel's output; the kernel therefore is multi-query attention with key width R + dr and value width R read
// straight from the cache rows, and nothing per head is ever materialised for past tokens.
//
//   llmctl_latent_kv_write  : per token, RMS norm (vector weight) of the query latent; RMS norm of the key/value
//                             latent and interleaved-pair rotation of the shared key part, written to the token's
//                             cache slot (fused norm + rotation + append).
//   llmctl_latent_attention : a CTA owns up to 16 query rows = (token, head) pairs of ONE sequence, so a key tile
//                             is loaded once for 16 tokens of a prompt portion (one head) or for 16 heads of a
//                             decoded token.  Keys stream through shared memory in tiles of 32 with an online
//                             softmax; the rotated query part is rotated on load.  Causal: a row at position p
//                             sees cache positions 0..p of its sequence.  Long contexts are split over CTAs
//                             (`splits` > 1) and merged by a second kernel, as the decode kernel in
//                             csrc/serve/paged_attention.cu does.  bf16 with R + dr a multiple of 16 runs both
//                             products on the tensor cores (mma.sync m16n8k16, fp32 accumulation; softmax, masks
//                             and the running maximum / sum stay fp32); other sizes and fp32 run the FMA kernel.
// Reference: none (the reference re-runs the HF model over the whole sequence, reference llmctl/serve/server.py:199-204).
#include "../common/dtype.cuh"
#include "../common/mma_sync.cuh"
#include "../rope/rope_interleaved.cuh"

namespace llmctl {

// d: [tokens, ld] = [ q latent raw (Q) | kv latent raw (R) | key rope part raw (dr) ] (R = dr = 0 columns absent for
// a layer that reads another layer's cache).
template <typename T>
__global__ void __launch_bounds__(128)
latent_kv_write_kernel(const T* __restrict__ d, long long ld, int Q, int R, int dr, const T* __restrict__ wq,
                       const T* __restrict__ wkv, T* __restrict__ cq, T* __restrict__ cache,
                       const long long* __restrict__ slots, const int* __restrict__ positions,
                       const float* __restrict__ freq, float mult, float eps) {
  __shared__ float red[32];
  const long long tok = blockIdx.x;
  const T* row = d + tok * ld;
  float ss = 0.f;
  for (int c = threadIdx.x; c < Q; c += blockDim.x) {
    const float v = to_f32(row[c]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float rq = 1.f / sqrtf(ss / static_cast<float>(Q) + eps);
  for (int c = threadIdx.x; c < Q; c += blockDim.x) cq[tok * Q + c] = from_f32<T>(to_f32(row[c]) * rq * to_f32(wq[c]));
  if (R == 0) return;
  const long long slot = slots[tok];
  if (slot < 0) return;  // padded token: uniform over the block, nobody waits below
  float sk = 0.f;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    const float v = to_f32(row[Q + c]);
    sk += v * v;
  }
  sk = block_sum(sk, red);
  const float rk = 1.f / sqrtf(sk / static_cast<float>(R) + eps);
  T* dst = cache + slot * (R + dr);
  for (int c = threadIdx.x; c < R; c += blockDim.x) dst[c] = from_f32<T>(to_f32(row[Q + c]) * rk * to_f32(wkv[c]));
  const T* kr = row + Q + R;
  const int pos = positions[tok];
  for (int c = threadIdx.x; c < dr; c += blockDim.x)
    dst[R + c] = from_f32<T>(rope_interleaved_coord([&](int k) { return to_f32(kr[k]); }, c, pos, freq, mult));
}

constexpr int kRows = 16;      // query rows per CTA
constexpr int kKeys = 32;      // keys per tile
constexpr int kAttnThreads = 128;

// tiles: int32 [ntiles, 4] = {first token row, token count, sequence row (block table), unused}
// ql: fp32 [tokens, H, R] absorbed queries;  q: [tokens, ldq] raw queries, head h at h * (dn + dr), rope part last
// out: [tokens, H, R] (T) if gridDim.z == 1, else partial fp32 [tokens, H, splits, R + 2] = {acc, max, sum}
template <typename T, int NC>
__global__ void __launch_bounds__(kAttnThreads)
latent_attention_kernel(const float* __restrict__ ql, long long ql_st, long long ql_sh, const T* __restrict__ q, long long ldq, int dn,
                        const T* __restrict__ cache, const int* __restrict__ block_tables, int max_blocks,
                        int block_size, const int* __restrict__ tiles, const int* __restrict__ positions,
                        const float* __restrict__ freq, float mult, float scale, int H, int R, int dr, int heads_per_tile,
                        int keys_per_split, T* __restrict__ out, float* __restrict__ partial, const float* __restrict__ sinks) {
  extern __shared__ float smem[];
  const int D = R + dr, Dp = D + 1;
  float* qs = smem;                      // [kRows][Dp]
  float* ks = qs + kRows * Dp;           // [kKeys][Dp]
  float* ps = ks + kKeys * Dp;           // [kRows][kKeys]
  float* row_m = ps + kRows * kKeys;     // [kRows]
  float* row_l = row_m + kRows;
  float* row_c = row_l + kRows;
  int* row_pos = reinterpret_cast<int*>(row_c + kRows);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* tile = tiles + 4 * blockIdx.x;
  const int tok0 = tile[0], ntok = tile[1], seq = tile[2];
  const int h0 = blockIdx.y * heads_per_tile;
  const int nh = min(heads_per_tile, H - h0);
  const int nrows = ntok * nh;           // row r -> token tok0 + r / nh, head h0 + r % nh
  const int split = blockIdx.z, nsplit = gridDim.z;
  const int* bt = block_tables + static_cast<long long>(seq) * max_blocks;

  if (tid < kRows) {
    // a sink is a key without a value: it is the row's initial (maximum, sum) in the first slice of the keys
    const bool sink = sinks != nullptr && split == 0 && tid < nrows;
    row_m[tid] = sink ? sinks[h0 + tid % nh] : -INFINITY;
    row_l[tid] = sink ? 1.f : 0.f;
    row_c[tid] = 1.f;
    row_pos[tid] = tid < nrows ? positions[tok0 + tid / nh] : -1;
  }
  __syncthreads();
  for (int idx = tid; idx < kRows * D; idx += kAttnThreads) {
    const int r = idx / D, c = idx % D;
    float v = 0.f;
    if (r < nrows) {
      const int tok = tok0 + r / nh, h = h0 + r % nh;
      if (c < R) {
        v = ql[tok * ql_st + h * ql_sh + c];
      } else {
        const T* qr = q + tok * ldq + static_cast<long long>(h) * (dn + dr) + dn;
        v = rope_interleaved_coord([&](int k) { return to_f32(qr[k]); }, c - R, row_pos[r], freq, mult);
      }
    }
    qs[r * Dp + c] = v * scale;
  }
  float acc[kRows][NC];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int i = 0; i < NC; ++i) acc[r][i] = 0.f;

  const int last = row_pos[nrows - 1];                     // positions grow with the token index
  const int k_begin = split * keys_per_split;
  const int k_end = min(last + 1, k_begin + keys_per_split);
  for (int j0 = k_begin; j0 < k_end; j0 += kKeys) {
    __syncthreads();                                       // previous tile fully consumed (and qs written)
    for (int idx = tid; idx < kKeys * D; idx += kAttnThreads) {
      const int jj = idx / D, c = idx % D, j = j0 + jj;
      float v = 0.f;
      if (j < k_end) {
        const long long slot = static_cast<long long>(bt[j / block_size]) * block_size + (j % block_size);
        v = to_f32(cache[slot * D + c]);
      }
      ks[jj * Dp + c] = v;
    }
    __syncthreads();
    {   // scores: thread -> row tid % 16, keys tid / 16 + 8 * i
      const int r = tid & 15;
      const float* qr = qs + r * Dp;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int jj = (tid >> 4) + 8 * i;
        const float* kr = ks + jj * Dp;
        float s = 0.f;
        for (int c = 0; c < D; ++c) s += qr[c] * kr[c];
        const int j = j0 + jj;
        ps[r * kKeys + jj] = (j < k_end && j <= row_pos[r]) ? s : -INFINITY;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kRows / 4; ++i) {   // online softmax: warp w owns rows 4w .. 4w+3, one key per lane
      const int r = warp * (kRows / 4) + i;
      const float s = ps[r * kKeys + lane];
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float p = (m_new == -INFINITY) ? 0.f : expf(s - m_new);
      const float corr = (m_new == -INFINITY) ? 1.f : expf(m_old - m_new);
      const float sum = warp_sum(p);
      ps[r * kKeys + lane] = p;
      if (lane == 0) {
        row_m[r] = m_new;
        row_l[r] = row_l[r] * corr + sum;
        row_c[r] = corr;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int c = tid + i * kAttnThreads;
      if (c < R) {
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc[r][i] *= row_c[r];
        for (int jj = 0; jj < kKeys; ++jj) {
          const float kv = ks[jj * Dp + c];
#pragma unroll
          for (int r = 0; r < kRows; ++r) acc[r][i] += ps[r * kKeys + jj] * kv;
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    if (r >= nrows) continue;
    const int tok = tok0 + r / nh, h = h0 + r % nh;
    const long long base = static_cast<long long>(tok) * H + h;
    if (nsplit == 1) {
      const float inv = row_l[r] > 0.f ? 1.f / row_l[r] : 0.f;
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = tid + i * kAttnThreads;
        if (c < R) out[base * R + c] = from_f32<T>(acc[r][i] * inv);
      }
    } else {
      float* dst = partial + (base * nsplit + split) * (R + 2);
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = tid + i * kAttnThreads;
        if (c < R) dst[c] = acc[r][i];
      }
      if (tid == 0) {
        dst[R] = row_m[r];
        dst[R + 1] = row_l[r];
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, int R, int nsplit) {
  const long long base = blockIdx.x;   // token * H + head
  const float* p = partial + base * nsplit * (R + 2);
  extern __shared__ float wsplit[];    // [nsplit]: exp(m_s - max m) / sum, 0 for empty splits
  __shared__ float s_inv;
  if (threadIdx.x < 32) {              // one warp: the maximum and the normaliser, in a fixed order
    float gm = -INFINITY;
    for (int s = threadIdx.x; s < nsplit; s += 32) gm = fmaxf(gm, p[s * (R + 2) + R]);
    gm = warp_max(gm);
    for (int s = threadIdx.x; s < nsplit; s += 32) {
      const float ms = p[s * (R + 2) + R];
      wsplit[s] = ms != -INFINITY ? expf(ms - gm) : 0.f;
    }
    __syncwarp();
    if (threadIdx.x == 0) {
      float gl = 0.f;
      for (int s = 0; s < nsplit; ++s) gl += p[s * (R + 2) + R + 1] * wsplit[s];
      s_inv = gl > 0.f ? 1.f / gl : 0.f;
    }
  }
  __syncthreads();
  const float inv = s_inv;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < nsplit; ++s) a += p[s * (R + 2) + c] * wsplit[s];
    out[base * R + c] = from_f32<T>(a * inv);
  }
}

// Used by the tcgen05 kernel's launcher (latent_attention_t5.cu) for split contexts.
int launch_latent_attention_merge_bf16(const float* partial, void* out, int R, int splits, int rows, cudaStream_t s) {
  latent_attention_merge_kernel<__nv_bfloat16><<<rows, 128, splits * sizeof(float), s>>>(partial, (__nv_bfloat16*)out, R, splits);
  return 0;
}

template <typename T>
static int launch_latent_attention(const float* ql, long long ql_st, long long ql_sh, const void* q, long long ldq, int dn, const void* cache,
                                   const int* block_tables, int max_blocks, int block_size, const int* tiles, int ntiles,
                                   const int* positions, const float* freq, float mult, float scale, int H, int R, int dr,
                                   int heads_per_tile, int splits, int keys_per_split, void* out, float* partial,
                                   int tokens, const float* sinks, cudaStream_t s) {
  const int D = R + dr;
  const size_t smem = (static_cast<size_t>(kRows + kKeys) * (D + 1) + kRows * kKeys + 4 * kRows) * sizeof(float);
  if (smem > 227 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  const int nc = (R + kAttnThreads - 1) / kAttnThreads;
  dim3 grid(ntiles, (H + heads_per_tile - 1) / heads_per_tile, splits);
#define LAUNCH(NC)                                                                                                   \
  do {                                                                                                               \
    auto kern = latent_attention_kernel<T, NC>;                                                                      \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    if (e != cudaSuccess) return static_cast<int>(e);                                                                \
    kern<<<grid, kAttnThreads, smem, s>>>(ql, ql_st, ql_sh, (const T*)q, ldq, dn, (const T*)cache, block_tables, max_blocks, \
                                          block_size, tiles, positions, freq, mult, scale, H, R, dr, heads_per_tile, \
                                          keys_per_split, (T*)out, partial, sinks);                                  \
  } while (0)
  if (nc <= 1) LAUNCH(1);
  else if (nc <= 2) LAUNCH(2);
  else if (nc <= 4) LAUNCH(4);
  else if (nc <= 8) LAUNCH(8);
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  if (splits > 1)
    latent_attention_merge_kernel<T><<<tokens * H, 128, splits * sizeof(float), s>>>(partial, (T*)out, R, splits);
  return 0;
}

// ---- bf16 tensor-core variant ------------------------------------------------------------------------------------
// Same tiling of the queries (16 rows per CTA, 8 warps); keys in tiles of 64 copied from the cache rows as they are
// (cp.async, double-buffered where shared memory allows).  Warp w
// computes the scores of keys 8w..8w+7 (S = Q K^T over all R + dr columns), the softmax runs on S in shared memory,
// P goes back as bf16 and warp w accumulates the columns [w * 8 NT, (w + 1) * 8 NT) of O += P C, where C is the first
// R columns of the very same key tile (ldmatrix with transposition).
constexpr int kTcKeys = 64;
constexpr int kSsLd = kTcKeys + 4, kPsLd = kTcKeys + 8;

// MT row tiles of 16 query rows per CTA and 8 MT warps: warp (wm, wn) = (warp / 8, warp % 8) owns row tile wm, the
// scores of keys 8 wn .. 8 wn + 7 and the output columns [8 NT wn, 8 NT (wn + 1)).  MT = 2 halves the key traffic
// per query row (prompt portions: 32 tokens per tile; decoding with more than 16 heads: 32 heads per tile).
template <int NT, int MT, typename TQ>
__global__ void __launch_bounds__(256 * MT)
latent_attention_tc_kernel(const TQ* __restrict__ ql, long long ql_st, long long ql_sh, const __nv_bfloat16* __restrict__ q, long long ldq, int dn,
                           const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_tables, int max_blocks,
                           int block_size, const int* __restrict__ tiles, const int* __restrict__ positions,
                           const float* __restrict__ freq, float mult, float scale, int H, int R, int dr, int heads_per_tile,
                           int keys_per_split, int stages, __nv_bfloat16* __restrict__ out, float* __restrict__ partial,
                           const float* __restrict__ sinks) {
  constexpr int kR = 16 * MT, kWarps = 8 * MT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = R + dr, Dp = D + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [kR][Dp]
  __nv_bfloat16* Ks0 = Qs + kR * Dp;                                    // [stages][kTcKeys][Dp]
  float* Ss = reinterpret_cast<float*>(Ks0 + stages * kTcKeys * Dp);    // [kR][kSsLd]
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(Ss + kR * kSsLd);      // [kR][kPsLd]
  float* row_m = reinterpret_cast<float*>(Ps + kR * kPsLd);
  float* row_l = row_m + kR;
  float* row_c = row_l + kR;
  int* row_pos = reinterpret_cast<int*>(row_c + kR);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int wm = warp >> 3, wn = warp & 7;
  const int* tile = tiles + 4 * blockIdx.x;
  const int tok0 = tile[0], ntok = tile[1], seq = tile[2];
  const int h0 = blockIdx.y * heads_per_tile;
  const int nh = min(heads_per_tile, H - h0);
  const int nrows = ntok * nh;
  const int split = blockIdx.z, nsplit = gridDim.z;
  const int* bt = block_tables + static_cast<long long>(seq) * max_blocks;

  if (tid < kR) {
    // a sink is a key without a value: it is the row's initial (maximum, sum) in the first slice of the keys
    const bool sink = sinks != nullptr && split == 0 && tid < nrows;
    row_m[tid] = sink ? sinks[h0 + tid % nh] : -INFINITY;
    row_l[tid] = sink ? 1.f : 0.f;
    row_c[tid] = 1.f;
    row_pos[tid] = tid < nrows ? positions[tok0 + tid / nh] : -1;
  }
  __syncthreads();
  for (int r = warp; r < kR; r += kWarps) {     // a warp per query row
    __nv_bfloat16* dst = Qs + r * Dp;
    if (r < nrows) {
      const int tok = tok0 + r / nh, h = h0 + r % nh;
      const TQ* src = ql + tok * ql_st + h * ql_sh;
      for (int c = lane; c < R; c += 32) dst[c] = __float2bfloat16(to_f32(src[c]));
      const __nv_bfloat16* qr = q + tok * ldq + static_cast<long long>(h) * (dn + dr) + dn;
      const int pos = row_pos[r];
      for (int c = lane; c < dr; c += 32)
        dst[R + c] = __float2bfloat16(rope_interleaved_coord([&](int k) { return to_f32(qr[k]); }, c, pos, freq, mult));
    } else {
      for (int c = lane; c < D; c += 32) dst[c] = __float2bfloat16(0.f);
    }
  }
  float oacc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) oacc[i][j] = 0.f;

  const int last = row_pos[nrows - 1];
  const int k_begin = split * keys_per_split;
  const int k_end = min(last + 1, k_begin + keys_per_split);
  const int vec_per_row = D >> 3;
  // a warp per key row, asynchronous 16-byte copies of the cache rows as they are
  auto load_tile = [&](int j0, __nv_bfloat16* Kd) {
    for (int jj = warp; jj < kTcKeys; jj += kWarps) {
      const int j = j0 + jj;
      __nv_bfloat16* dst = Kd + jj * Dp;
      if (j < k_end) {
        const long long slot = static_cast<long long>(bt[j / block_size]) * block_size + (j % block_size);
        const __nv_bfloat16* src = cache + slot * D;
        for (int v = lane; v < vec_per_row; v += 32) cp_async_16(dst + v * 8, src + v * 8);
      } else {
        for (int v = lane; v < vec_per_row; v += 32) *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    cp_async_commit();
  };
  // With two stages the copy of tile i + 1 is in flight while tile i is multiplied.
  int buf = 0;
  if (stages == 2 && k_begin < k_end) load_tile(k_begin, Ks0);
  for (int j0 = k_begin; j0 < k_end; j0 += kTcKeys) {
    __nv_bfloat16* Ks = Ks0 + buf * kTcKeys * Dp;
    __syncthreads();                       // the previous tile's products are done: its buffer may be overwritten
    if (stages == 2) {
      if (j0 + kTcKeys < k_end) {
        load_tile(j0 + kTcKeys, Ks0 + (buf ^ 1) * kTcKeys * Dp);
        cp_async_wait_prior();
      } else {
        cp_async_wait_all();
      }
      buf ^= 1;
    } else {
      load_tile(j0, Ks);
      cp_async_wait_all();
    }
    __syncthreads();
    {
      float sacc[2][4] = {};                   // two independent accumulation chains over alternate k-steps
      int k0 = 0;
      for (; k0 + 32 <= D; k0 += 32) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          uint32_t a[4], b[2];
          load_a_frag(a, Qs, Dp, 16 * wm, k0 + 16 * u, lane);
          load_b_frag_nk(b, Ks, Dp, 8 * wn, k0 + 16 * u, lane);
          mma_bf16_16816(sacc[u], a, b);
        }
      }
      if (k0 < D) {
        uint32_t a[4], b[2];
        load_a_frag(a, Qs, Dp, 16 * wm, k0, lane);
        load_b_frag_nk(b, Ks, Dp, 8 * wn, k0, lane);
        mma_bf16_16816(sacc[0], a, b);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = 16 * wm + g + (e >> 1) * 8, col = 8 * wn + 2 * t + (e & 1), j = j0 + col;
        Ss[r * kSsLd + col] = (j < k_end && j <= row_pos[r]) ? (sacc[0][e] + sacc[1][e]) * scale : -INFINITY;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kR / kWarps; ++i) {
      const int r = warp * (kR / kWarps) + i;
      const float s0 = Ss[r * kSsLd + lane], s1 = Ss[r * kSsLd + lane + 32];
      const float m_old = row_m[r];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
      const bool none = m_new == -INFINITY;
      const float p0 = none ? 0.f : expf(s0 - m_new), p1 = none ? 0.f : expf(s1 - m_new);
      const float corr = none ? 1.f : expf(m_old - m_new);
      const float sum = warp_sum(p0 + p1);
      Ps[r * kPsLd + lane] = __float2bfloat16(p0);
      Ps[r * kPsLd + lane + 32] = __float2bfloat16(p1);
      if (lane == 0) {
        row_m[r] = m_new;
        row_l[r] = row_l[r] * corr + sum;
        row_c[r] = corr;
      }
    }
    __syncthreads();
    {
      const float c_lo = row_c[16 * wm + g], c_hi = row_c[16 * wm + g + 8];
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        oacc[i][0] *= c_lo;
        oacc[i][1] *= c_lo;
        oacc[i][2] *= c_hi;
        oacc[i][3] *= c_hi;
      }
#pragma unroll
      for (int kk = 0; kk < kTcKeys / 16; ++kk) {
        uint32_t a[4];
        load_a_frag(a, Ps, kPsLd, 16 * wm, 16 * kk, lane);
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          const int n0 = 8 * (wn * NT + i);
          if (n0 < R) {      // uniform over the warp
            uint32_t b[2];
            load_b_frag_kn(b, Ks, Dp, 16 * kk, n0, lane);
            mma_bf16_16816(oacc[i], a, b);
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = 16 * wm + g + 8 * half;
    if (r >= nrows) continue;
    const int tok = tok0 + r / nh, h = h0 + r % nh;
    const long long base = static_cast<long long>(tok) * H + h;
    const float inv = row_l[r] > 0.f ? 1.f / row_l[r] : 0.f;
    float* dst = nsplit > 1 ? partial + (base * nsplit + split) * (R + 2) : nullptr;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int c = 8 * (wn * NT + i) + 2 * t;
      if (c < R) {
        const float v0 = oacc[i][2 * half], v1 = oacc[i][2 * half + 1];
        if (dst) {
          dst[c] = v0;
          dst[c + 1] = v1;
        } else {
          *reinterpret_cast<__nv_bfloat162*>(out + base * R + c) = __floats2bfloat162_rn(v0 * inv, v1 * inv);
        }
      }
    }
    if (dst && wn == 0 && t == 0) {
      dst[R] = row_m[r];
      dst[R + 1] = row_l[r];
    }
  }
}

static size_t latent_attention_tc_smem(int R, int dr, int rows, int stages = 1) {
  return static_cast<size_t>(rows + stages * kTcKeys) * (R + dr + 8) * 2 + static_cast<size_t>(rows) * (kSsLd * 4 + kPsLd * 2 + 16);
}

static bool latent_attention_tc_ok(int R, int dr, int rows = kRows) {
  const int D = R + dr;
  return D % 16 == 0 && R % 8 == 0 && R <= 512 && (rows == 16 || rows == 32) && latent_attention_tc_smem(R, dr, rows) <= 227 * 1024;
}

template <typename TQ>
static int launch_latent_attention_tc(const TQ* ql, long long ql_st, long long ql_sh, const void* q, long long ldq, int dn, const void* cache,
                                      const int* block_tables, int max_blocks, int block_size, const int* tiles, int ntiles,
                                      const int* positions, const float* freq, float mult, float scale, int H, int R, int dr,
                                      int heads_per_tile, int splits, int keys_per_split, void* out, float* partial,
                                      int tokens, int rows, const float* sinks, cudaStream_t s) {
  // A second key-tile stage overlaps the copy of the next tile with the products of this one.  16-row tiles take it
  // only while two CTAs still share an SM (they overlap each other's copies anyway); 32-row tiles whenever it fits
  // (up to R + dr = 576 it does).
  const size_t smem2 = latent_attention_tc_smem(R, dr, rows, 2);
  const int stages = (rows == 32 ? smem2 <= 227 * 1024 : smem2 <= 113 * 1024) ? 2 : 1;
  const size_t smem = latent_attention_tc_smem(R, dr, rows, stages);
  const int nt = (R + 63) / 64;
  dim3 grid(ntiles, (H + heads_per_tile - 1) / heads_per_tile, splits);
#define LAUNCH_TC(NT, MT)                                                                                            \
  do {                                                                                                               \
    auto kern = latent_attention_tc_kernel<NT, MT, TQ>;                                                              \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    if (e != cudaSuccess) return static_cast<int>(e);                                                                \
    kern<<<grid, 256 * MT, smem, s>>>(ql, ql_st, ql_sh, (const __nv_bfloat16*)q, ldq, dn, (const __nv_bfloat16*)cache, \
                                      block_tables, max_blocks, block_size, tiles, positions, freq, mult, scale,     \
                                      H, R, dr, heads_per_tile, keys_per_split, stages, (__nv_bfloat16*)out, partial, sinks); \
  } while (0)
#define LAUNCH_TC_NT(MT)          \
  do {                            \
    if (nt <= 1) LAUNCH_TC(1, MT); \
    else if (nt <= 2) LAUNCH_TC(2, MT); \
    else if (nt <= 4) LAUNCH_TC(4, MT); \
    else LAUNCH_TC(8, MT);        \
  } while (0)
  if (rows == 32) LAUNCH_TC_NT(2);
  else LAUNCH_TC_NT(1);
#undef LAUNCH_TC_NT
#undef LAUNCH_TC
  if (splits > 1)
    latent_attention_merge_kernel<__nv_bfloat16><<<tokens * H, 128, splits * sizeof(float), s>>>(partial, (__nv_bfloat16*)out, R, splits);
  return 0;
}

}  // namespace llmctl

using namespace llmctl;

LLMCTL_API int llmctl_latent_kv_write(const void* d, long long ld, int Q, int R, int dr, const void* wq, const void* wkv,
                                      void* cq, void* cache, const long long* slots, const int* positions,
                                      const float* freq, float mult, float eps, int tokens, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(Q > 0 && R >= 0 && dr >= 0 && dr % 2 == 0 && ld >= Q + R + dr);
  if (tokens == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (latent_kv_write_kernel<T><<<tokens, 128, 0, (cudaStream_t)stream>>>(
                                        (const T*)d, ld, Q, R, dr, (const T*)wq, (const T*)wkv, (T*)cq, (T*)cache, slots,
                                        positions, freq, mult, eps)));
  LLMCTL_RETURN_LAST();
}

// partial: fp32 scratch of tokens * H * splits * (R + 2) numbers when splits > 1 (may be null otherwise).
// sinks: fp32 [H] or null; exp(sinks[h]) (not scaled) joins the softmax denominator of head h.
// ql: absorbed queries, element (token, head, c) at ql[token * ql_st + head * ql_sh + c]; fp32, or bf16 (ql_bf16) on the
// tensor-core path only (llmctl_latent_attention_uses_tensor_cores).
LLMCTL_API int llmctl_latent_attention_uses_tensor_cores(int is_fp32, int R, int dr, int rows_per_tile) {
  return (!is_fp32 && latent_attention_tc_ok(R, dr, rows_per_tile)) ? 1 : 0;
}

LLMCTL_API int llmctl_latent_attention(const void* ql, int ql_bf16, long long ql_st, long long ql_sh, const void* q, long long ldq, int dn, const void* cache,
                                       const int* block_tables, int max_blocks, int block_size, const int* tiles,
                                       int ntiles, int tokens, const int* positions, const float* freq, float mult,
                                       float scale, int H, int R, int dr, int heads_per_tile, int splits,
                                       int keys_per_split, void* out, float* partial, int is_fp32, int tensor_cores,
                                       int rows_per_tile, const float* sinks, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && R > 0 && dr >= 0 && dr % 2 == 0 && block_size > 0 && heads_per_tile >= 1 &&
                 heads_per_tile <= rows_per_tile && (rows_per_tile == 16 || rows_per_tile == 32) && splits >= 1 && keys_per_split > 0 && (splits == 1 || partial != nullptr));
  if (ntiles == 0) return 0;
  int rc;
  if (!is_fp32 && tensor_cores && latent_attention_tc_ok(R, dr, rows_per_tile) && keys_per_split % kTcKeys == 0) {
    if (ql_bf16)
      rc = launch_latent_attention_tc<__nv_bfloat16>((const __nv_bfloat16*)ql, ql_st, ql_sh, q, ldq, dn, cache, block_tables, max_blocks,
                                                     block_size, tiles, ntiles, positions, freq, mult, scale, H, R, dr, heads_per_tile,
                                                     splits, keys_per_split, out, partial, tokens, rows_per_tile, sinks, (cudaStream_t)stream);
    else
    rc = launch_latent_attention_tc<float>((const float*)ql, ql_st, ql_sh, q, ldq, dn, cache, block_tables, max_blocks, block_size, tiles, ntiles, positions, freq,
                                    mult, scale, H, R, dr, heads_per_tile, splits, keys_per_split, out, partial, tokens,
                                    rows_per_tile, sinks, (cudaStream_t)stream);
    if (rc != 0) LLMCTL_FAIL(rc, "latent attention launch");
    LLMCTL_RETURN_LAST();
  }
  LLMCTL_REQUIRE(!ql_bf16 && rows_per_tile == kRows);
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (rc = launch_latent_attention<T>((const float*)ql, ql_st, ql_sh, q, ldq, dn, cache, block_tables, max_blocks, block_size,
                                                                     tiles, ntiles, positions, freq, mult, scale, H, R, dr,
                                                                     heads_per_tile, splits, keys_per_split, out, partial,
                                                                     tokens, sinks, (cudaStream_t)stream)));
  if (rc != 0) LLMCTL_FAIL(rc, "latent attention launch");
  LLMCTL_RETURN_LAST();
}
