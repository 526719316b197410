// Soft-capped sliding-window attention with kept first tokens, a distance bias and a sink, over a paged cache, for ragged
// batches (portions of prompts next to single decoded tokens), bf16 or fp32.
//
// H query heads use G key/value heads (head h reads head h / (H/G)).  For query position i and key position j <= i:
//
//     visible(i, j) = window == 0  or  i - j < window  or  j < keep_first
//     s_ij = q_i . k_j * scale;   cap > 0:  s_ij <- cap * tanh(s_ij / cap);   s_ij <- s_ij - slope_h * (i - j)
//     p_ij = exp(s_ij) / (sum_visible exp(s_ij') + exp(sink_h))            sinks == null: no sink term
//     o_i  = sum_j p_ij v_j,  times sigmoid(gate[i, h, :]) where a gate is given
//
// slopes and sinks are fp32 arrays of H numbers (null: no bias / no sink); a sink has no value, so it only enlarges the
// denominator.  Cache of a layer: [pages, bs, G*d + G*e]; a token's row holds the keys of all key/value heads and then
// their values.
//
//   llmctl_window_kv_append : per token, from a packed projection [q | k | v | ...]: fp32 biases (optional), unit-RMS
//       norm of every value head (optional: v / sqrt(mean(v^2) + eps), no weight); q leaves in fp32, k and v go to the
//       token's cache row.
//   llmctl_softcap_window_attention : key tiles run over the kept first tokens and then over the window of the tile's
//       queries only; everything else is never read.  FMA kernel (fp32 caches, any sizes): a CTA owns up to 16
//       consecutive tokens x HB heads of one key/value head as <= 32 softmax rows, a warp owns four rows through all
//       phases.  bf16 caches with d a multiple of 16 and e a multiple of 8 up to 128 run on the tensor cores (mma.sync
//       m16n8k16): a CTA owns up to 128 consecutive tokens of one head (8 warps x 16 rows; prompt portions) or one
//       token's heads of one key/value head (one warp; decoded tokens).  Key/value tiles of 32 keys come by 16-byte
//       cp.async into two stages; the fp32 queries and the softmax weights enter the products as bf16 pairs hi + lo
//       (exact to ~2^-17); scores, cap, bias, maxima, sums and accumulators are fp32.
//       With splits > 1 a tile's key tiles are dealt to several CTAs (few tiles, long windows: decoding) and merged.
//       The sink is the initial (maximum, sum) = (sink_h, 1) of a row's running softmax, in the first slice only.
// Reference: none (the reference has no attention code; reference llmctl/serve/server.py:199-204 calls HF).
#include "../common/dtype.cuh"
#include "../common/mma_sync.cuh"

namespace llmctl {

// ---------------------------------------------------------------------------------------------------------------
// bias + value norm + cache append: one CTA per token
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
window_kv_append_kernel(const T* __restrict__ proj, long long ld, const float* __restrict__ bias, int H, int G, int d, int e,
                        int value_norm, float eps, const long long* __restrict__ slots, float* __restrict__ q_out,
                        T* __restrict__ cache) {
  const long long t = blockIdx.x;
  const int Nq = H * d, Nk = G * d, Wc = Nk + G * e;
  const T* row = proj + t * ld;
  const long long slot = slots[t];
  T* crow = slot >= 0 ? cache + slot * Wc : nullptr;
  for (int c = threadIdx.x; c < Nq + Nk; c += blockDim.x) {
    const float v = to_f32(row[c]) + (bias ? bias[c] : 0.f);
    if (c < Nq) q_out[t * Nq + c] = v;
    else if (crow) crow[c - Nq] = from_f32<T>(v);
  }
  if (!crow) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int g = warp; g < G; g += nwarp) {
    const int base = Nq + Nk + g * e;
    float ss = 0.f;
    for (int c = lane; c < e; c += 32) {
      const float v = to_f32(row[base + c]) + (bias ? bias[base + c] : 0.f);
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float f = value_norm ? 1.f / sqrtf(ss / static_cast<float>(e) + eps) : 1.f;
    for (int c = lane; c < e; c += 32)
      crow[Nk + g * e + c] = from_f32<T>((to_f32(row[base + c]) + (bias ? bias[base + c] : 0.f)) * f);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------------------------
constexpr int kSwKT = 32;         // keys per tile
constexpr int kSwRows = 32;       // softmax rows per CTA of the FMA kernel: (token, head)
constexpr int kSwThreads = 256;   // 8 warps x 4 rows

struct SoftcapAttnParams {
  const float* q;            // [T, H*d]
  const void* cache;
  const int* block_tables;
  int max_blocks;
  const int* tiles;          // [n, 4] = (first token row, tokens, block-table row, 0)
  const int* positions;
  const void* gate;          // [T, >= H*e] pre-sigmoid gates (row stride gate_ld); null = no gate
  long long gate_ld;
  const float* slopes;       // [H] or null
  const float* sinks;        // [H] or null
  float scale, cap;
  int window, keep_first;
  int H, G, d, e, bs;
  int HB;                    // heads per CTA
  void* out;                 // [T, H*e]
  int splits;                // slices of a tile's key tiles (1 = whole)
  float* part_ml;            // [tiles * H/HB * splits, 32, 2]
  float* part_o;             // [tiles * H/HB * splits, 32, e]
};

// The key tiles of a query tile whose positions are p_first .. p_last: tiles 0 .. nA-1 cover the kept first tokens
// [0, endA), tiles nA .. nA+nB-1 the window [wb, p_last + 1).
struct KeyTiles {
  int endA, wb, nkeys, nA, nB;
  __device__ KeyTiles(int p_first, int p_last, int window, int keep_first) {
    nkeys = p_last + 1;
    wb = window > 0 ? max(p_first - window + 1, 0) : 0;
    endA = window > 0 ? min(keep_first, wb) : 0;
    nA = (endA + kSwKT - 1) / kSwKT;
    nB = (nkeys - wb + kSwKT - 1) / kSwKT;
  }
  __device__ int first(int it) const { return it < nA ? it * kSwKT : wb + (it - nA) * kSwKT; }
  __device__ int limit(int it) const { return it < nA ? endA : nkeys; }
};

__device__ __forceinline__ bool sw_visible(int qpos, int key, int window, int keep_first) {
  return key <= qpos && (window <= 0 || qpos - key < window || key < keep_first);
}

// NC: output columns per lane (e <= 32 * NC)
template <typename T, int NC, bool SPLIT>
__global__ void __launch_bounds__(kSwThreads)
softcap_attention_kernel(const SoftcapAttnParams p) {
  extern __shared__ float sm[];
  const int H = p.H, G = p.G, d = p.d, e = p.e, bs = p.bs, HB = p.HB;
  const int rep = H / G, Wc = G * (d + e), ldk = d + 1;
  const int tile = blockIdx.x / p.splits, split = blockIdx.x % p.splits;
  const int t0 = p.tiles[tile * 4], nq = p.tiles[tile * 4 + 1];
  if (nq <= 0) return;
  const int* table = p.block_tables + static_cast<long long>(p.tiles[tile * 4 + 2]) * p.max_blocks;
  const int h0 = blockIdx.y * HB, g = h0 / rep;
  const int p_first = p.positions[t0], p_last = p_first + nq - 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nrows = nq * HB;                     // row r = tq * HB + hb

  float* Qs = sm;                                // [32][d]
  float* Ks = Qs + kSwRows * d;                  // [KT][d + 1]
  float* Vs = Ks + kSwKT * ldk;                  // [KT][e]
  float* Ps = Vs + kSwKT * e;                    // [32][KT]

  const T* cache = static_cast<const T*>(p.cache);
  for (int i = tid; i < kSwRows * d; i += kSwThreads) {
    const int r = i / d, c = i % d;
    float v = 0.f;
    if (r < nrows) v = p.q[(static_cast<long long>(t0 + r / HB) * H + h0 + r % HB) * d + c] * p.scale;
    Qs[i] = v;
  }

  float m[4], l[4], acc[4][NC], slope[4];
  int qpos[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp * 4 + i;
    const int h = h0 + (r < nrows ? r % HB : 0);
    qpos[i] = r < nrows ? p_first + r / HB : -1;
    slope[i] = p.slopes ? p.slopes[h] : 0.f;
    const bool sink = p.sinks != nullptr && split == 0;
    m[i] = sink ? p.sinks[h] : -INFINITY;
    l[i] = sink ? 1.f : 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
  }
  const int warp_rows = min(max(nrows - warp * 4, 0), 4);

  const KeyTiles kt(p_first, p_last, p.window, p.keep_first);
  int it_begin = 0, it_end = kt.nA + kt.nB;
  if (SPLIT) {
    const int per = (it_end + p.splits - 1) / p.splits;
    it_begin = min(split * per, it_end);
    it_end = min(it_begin + per, it_end);
  }
  for (int it = it_begin; it < it_end; ++it) {
    const int k0 = kt.first(it), k_lim = kt.limit(it);
    __syncthreads();                             // the previous tile's readers are done (and Qs is written)
    const int nk = min(kSwKT, k_lim - k0);
    for (int i = tid; i < kSwKT * d; i += kSwThreads) {
      const int kk = i / d, c = i % d;
      float v = 0.f;
      if (kk < nk) {
        const int j = k0 + kk;
        v = to_f32(cache[(static_cast<long long>(table[j / bs]) * bs + j % bs) * Wc + g * d + c]);
      }
      Ks[kk * ldk + c] = v;
    }
    for (int i = tid; i < kSwKT * e; i += kSwThreads) {
      const int kk = i / e, c = i % e;
      float v = 0.f;
      if (kk < nk) {
        const int j = k0 + kk;
        v = to_f32(cache[(static_cast<long long>(table[j / bs]) * bs + j % bs) * Wc + G * d + g * e + c]);
      }
      Vs[i] = v;
    }
    __syncthreads();
    if (warp_rows > 0) {
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      const float* kr = Ks + lane * ldk;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (i < warp_rows) {
          const float* qr = Qs + (warp * 4 + i) * d;
          float a0 = 0.f, a1 = 0.f;
          int c = 0;
          for (; c + 1 < d; c += 2) {
            a0 += qr[c] * kr[c];
            a1 += qr[c + 1] * kr[c + 1];
          }
          if (c < d) a0 += qr[c] * kr[c];
          s[i] = a0 + a1;
        }
      }
      const int j = k0 + lane;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (i < warp_rows) {
          const bool seen = lane < nk && sw_visible(qpos[i], j, p.window, p.keep_first);
          float sv = -INFINITY;
          if (seen) {
            sv = p.cap > 0.f ? p.cap * tanhf(s[i] / p.cap) : s[i];
            sv -= slope[i] * static_cast<float>(qpos[i] - j);
          }
          const float mn = fmaxf(m[i], warp_max(sv));
          float pw = 0.f, corr = 1.f;
          if (mn > -INFINITY) {
            pw = seen ? expf(sv - mn) : 0.f;
            corr = m[i] > -INFINITY ? expf(m[i] - mn) : 0.f;
          }
          l[i] = l[i] * corr + warp_sum(pw);
          m[i] = mn;
#pragma unroll
          for (int c = 0; c < NC; ++c) acc[i][c] *= corr;
          Ps[(warp * 4 + i) * kSwKT + lane] = pw;
        }
      }
      __syncwarp();
      for (int kk = 0; kk < nk; ++kk) {
        float v[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) v[c] = lane + 32 * c < e ? Vs[kk * e + lane + 32 * c] : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (i < warp_rows) {
            const float pw = Ps[(warp * 4 + i) * kSwKT + kk];
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[i][c] += pw * v[c];
          }
        }
      }
      __syncwarp();
    }
  }
  if (warp_rows == 0) return;
  if (SPLIT) {
    const long long base = (static_cast<long long>(tile) * gridDim.y + blockIdx.y) * p.splits + split;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < warp_rows) {
        const int r = warp * 4 + i;
        if (lane == 0) {
          p.part_ml[(base * kSwRows + r) * 2] = m[i];
          p.part_ml[(base * kSwRows + r) * 2 + 1] = l[i];
        }
#pragma unroll
        for (int c = 0; c < NC; ++c)
          if (lane + 32 * c < e) p.part_o[(base * kSwRows + r) * e + lane + 32 * c] = acc[i][c];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i < warp_rows) {
      const int r = warp * 4 + i;
      const long long t = t0 + r / HB;
      const int h = h0 + r % HB;
      const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
      T* orow = static_cast<T*>(p.out) + (t * H + h) * e;
      const T* grow = p.gate ? static_cast<const T*>(p.gate) + t * p.gate_ld + static_cast<long long>(h) * e : nullptr;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int col = lane + 32 * c;
        if (col < e) {
          float o = acc[i][c] * inv;
          if (grow) o *= 1.f / (1.f + expf(-to_f32(grow[col])));
          orow[col] = from_f32<T>(o);
        }
      }
    }
  }
}

// One warp per (tile, head block, row): merges the slices and finishes like the unsplit kernels.  rows_are_heads: the
// partial rows of a unit are the HB heads of the tile's single token (tensor-core decode) instead of (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
softcap_attention_merge_kernel(const SoftcapAttnParams p, int head_blocks) {
  const int H = p.H, e = p.e, HB = p.HB;
  const int lane = threadIdx.x & 31;
  const long long unit = blockIdx.x;                        // (tile, head block)
  const int tile = static_cast<int>(unit / head_blocks), hblk = static_cast<int>(unit % head_blocks);
  const int t0 = p.tiles[tile * 4], nq = p.tiles[tile * 4 + 1];
  const int nrows = nq * HB;
  for (int r = threadIdx.x >> 5; r < nrows; r += blockDim.x >> 5) {
    const long long t = t0 + r / HB;
    const int h = hblk * HB + r % HB;
    float mx = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mx = fmaxf(mx, p.part_ml[((unit * p.splits + s) * kSwRows + r) * 2]);
    float ls = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float* ml = p.part_ml + ((unit * p.splits + s) * kSwRows + r) * 2;
      if (ml[0] > -INFINITY) ls += ml[1] * expf(ml[0] - mx);
    }
    const float inv = ls > 0.f ? 1.f / ls : 0.f;
    T* orow = static_cast<T*>(p.out) + (t * H + h) * e;
    const T* grow = p.gate ? static_cast<const T*>(p.gate) + t * p.gate_ld + static_cast<long long>(h) * e : nullptr;
    for (int c = lane; c < e; c += 32) {
      float a = 0.f;
      for (int s = 0; s < p.splits; ++s) {
        const long long row = (unit * p.splits + s) * kSwRows + r;
        const float mv = p.part_ml[row * 2];
        if (mv > -INFINITY) a += p.part_o[row * e + c] * expf(mv - mx);
      }
      float o = a * inv;
      if (grow) o *= 1.f / (1.f + expf(-to_f32(grow[c])));
      orow[c] = from_f32<T>(o);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// tensor-core attention (bf16 cache)
// ---------------------------------------------------------------------------------------------------------------
constexpr float kSwLog2e = 1.4426950408889634f, kSwLn2 = 0.6931471805599453f;

__device__ __forceinline__ float sw_quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}
__device__ __forceinline__ float sw_quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
// bf16 pair hi + lo of two fp32 numbers, packed for an A fragment
__device__ __forceinline__ void sw_split_pack(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 ah = __float2bfloat16(a), bh = __float2bfloat16(b);
  hi = pack_bf16x2(__bfloat162float(ah), __bfloat162float(bh));
  lo = pack_bf16x2(a - __bfloat162float(ah), b - __bfloat162float(bh));
}
// tanh(x) = 1 - 2 / (1 + e^(2x)): absolute error of a few 1e-7
__device__ __forceinline__ float sw_tanh(float x) {
  return 1.f - __fdividef(2.f, 1.f + exp2f(2.f * kSwLog2e * x));
}

// NT: n-tiles of 8 output columns (e <= 8 NT).  decode = 0: rows of the CTA are the tile's tokens (head blockIdx.y);
// decode = 1: rows are HB heads of the tile's single token.
template <int NT, bool SPLIT>
__global__ void __launch_bounds__(256, SPLIT ? 1 : 2)
softcap_attention_mma_kernel(const SoftcapAttnParams p, int decode) {
  extern __shared__ __align__(16) unsigned char sw_smem[];
  const int H = p.H, G = p.G, d = p.d, e = p.e, bs = p.bs;
  const int rep = H / G, Wc = G * (d + e);
  const int tile = blockIdx.x / p.splits, split = blockIdx.x % p.splits;
  const int t0 = p.tiles[tile * 4], nq = p.tiles[tile * 4 + 1];
  if (nq <= 0) return;
  const int* table = p.block_tables + static_cast<long long>(p.tiles[tile * 4 + 2]) * p.max_blocks;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
  const int rows_cta = (nthreads >> 5) * 16;
  const int h0 = decode ? blockIdx.y * p.HB : blockIdx.y, g = h0 / rep;
  const int nvalid = decode ? p.HB : nq;
  const int p_first = p.positions[t0], p_last = decode ? p_first : p_first + nq - 1;
  const int ldq = d + 8, ldk = d + 8, ldv = e + 8;
  __nv_bfloat16* Qhi = reinterpret_cast<__nv_bfloat16*>(sw_smem);       // [rows][ldq]
  __nv_bfloat16* Qlo = Qhi + rows_cta * ldq;
  __nv_bfloat16* Ks = Qlo + rows_cta * ldq;                              // [2][KT][ldk]
  __nv_bfloat16* Vs = Ks + 2 * kSwKT * ldk;                              // [2][KT][ldv]
  const __nv_bfloat16* cache = static_cast<const __nv_bfloat16*>(p.cache);

  {
    const int per_row = d >> 2;
    for (int i = tid; i < nvalid * per_row; i += nthreads) {
      const int r = i / per_row, c = (i % per_row) << 2;
      const long long tok = decode ? t0 : t0 + r;
      const int head = decode ? h0 + r : h0;
      float4 v = *reinterpret_cast<const float4*>(p.q + (tok * H + head) * d + c);
      v.x *= p.scale, v.y *= p.scale, v.z *= p.scale, v.w *= p.scale;
      uint32_t h01, l01, h23, l23;
      sw_split_pack(v.x, v.y, h01, l01);
      sw_split_pack(v.z, v.w, h23, l23);
      *reinterpret_cast<uint2*>(Qhi + r * ldq + c) = make_uint2(h01, h23);
      *reinterpret_cast<uint2*>(Qlo + r * ldq + c) = make_uint2(l01, l23);
    }
    const int per_row8 = d >> 3;                 // rows without a query: zeros (16 bytes at a time; ldq is a multiple of 8)
    for (int i = tid; i < (rows_cta - nvalid) * per_row8; i += nthreads) {
      const int r = nvalid + i / per_row8, c = (i % per_row8) << 3;
      *reinterpret_cast<uint4*>(Qhi + r * ldq + c) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(Qlo + r * ldq + c) = make_uint4(0u, 0u, 0u, 0u);
    }
  }

  const KeyTiles kt(p_first, p_last, p.window, p.keep_first);
  int it_begin = 0, it_end = kt.nA + kt.nB;
  if (SPLIT) {
    const int per = (it_end + p.splits - 1) / p.splits;
    it_begin = min(split * per, it_end);
    it_end = min(it_begin + per, it_end);
  }
  const int kch = d >> 3, vch = e >> 3, chunks = kch + vch;
  // cache offsets of a tile's keys are looked up (page table) one tile ahead of the copies that use them
  __shared__ long long rowoff[2][kSwKT];
  auto index_tile = [&](int stage, int it) {
    if (tid < kSwKT) {
      const int j = kt.first(it) + tid;
      rowoff[stage][tid] = j < kt.limit(it) ? (static_cast<long long>(table[j / bs]) * bs + j % bs) * Wc : -1;
    }
  };
  auto load_tile = [&](int stage) {
    for (int i = tid; i < kSwKT * chunks; i += nthreads) {
      const int kk = i / chunks, ch = i % chunks;
      const long long off = rowoff[stage][kk];
      __nv_bfloat16* dst = ch < kch ? Ks + (stage * kSwKT + kk) * ldk + ch * 8 : Vs + (stage * kSwKT + kk) * ldv + (ch - kch) * 8;
      if (off >= 0) {
        const __nv_bfloat16* row = cache + off;
        cp_async_16(dst, ch < kch ? row + g * d + ch * 8 : row + G * d + g * e + (ch - kch) * 8);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);      // a weight of 0 times stale bits could be a NaN
      }
    }
  };

  const int grow = lane >> 2, tq = lane & 3;
  const int r_lo = warp * 16 + grow, r_hi = r_lo + 8;
  const int qpos_lo = r_lo < nvalid ? (decode ? p_first : p_first + r_lo) : -1;
  const int qpos_hi = r_hi < nvalid ? (decode ? p_first : p_first + r_hi) : -1;
  const int head_lo = decode ? h0 + min(r_lo, nvalid - 1) : h0, head_hi = decode ? h0 + min(r_hi, nvalid - 1) : h0;
  const float slope_lo = p.slopes ? p.slopes[head_lo] : 0.f, slope_hi = p.slopes ? p.slopes[head_hi] : 0.f;
  const bool warp_active = warp * 16 < nvalid;
  // keys this warp's rows can see: the kept first tokens and [warp_wb, warp_last]
  const int warp_first = decode ? p_first : p_first + warp * 16;
  const int warp_last = decode ? p_first : p_first + min(warp * 16 + 15, nvalid - 1);
  const int warp_wb = p.window > 0 ? warp_first - p.window + 1 : 0;

  float O[NT][4];
  float mrow[2], lrow[2];                 // lo / hi row; maxima in units of ln 2
  {
    const bool sink = p.sinks != nullptr && split == 0;
    mrow[0] = sink ? p.sinks[head_lo] * kSwLog2e : -INFINITY;
    mrow[1] = sink ? p.sinks[head_hi] * kSwLog2e : -INFINITY;
    // the quad adds its four partial sums up at the end: the sink's 1 sits in one of them
    lrow[0] = lrow[1] = (sink && tq == 0) ? 1.f : 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) O[nt][j] = 0.f;
  }

  const int ntile = it_end - it_begin;
  if (ntile > 0) index_tile(0, it_begin);
  if (ntile > 1) index_tile(1, it_begin + 1);
  __syncthreads();
  if (ntile > 0) load_tile(0);
  cp_async_commit();
  for (int n = 0; n < ntile; ++n) {
    cp_async_wait_all();
    __syncthreads();                       // tile n has landed (and Q); everyone is done with the other stage
    if (n + 1 < ntile) load_tile((n + 1) & 1);
    cp_async_commit();
    if (n + 2 < ntile) index_tile(n & 1, it_begin + n + 2);     // its last readers ran before the barrier
    const int it = it_begin + n, st = n & 1;
    const int k0 = kt.first(it), k_lim = kt.limit(it);
    if (!warp_active || k0 > warp_last) continue;
    if (it >= kt.nA && k0 + kSwKT <= warp_wb && k0 >= p.keep_first) continue;      // wholly before this warp's window
    const __nv_bfloat16* Kt = Ks + st * kSwKT * ldk;
    const __nv_bfloat16* Vt = Vs + st * kSwKT * ldv;
    float S[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) S[nt][j] = 0.f;
    for (int ks = 0; ks < d; ks += 16) {
      uint32_t ah[4], al[4];
      load_a_frag(ah, Qhi, ldq, warp * 16, ks, lane);
      load_a_frag(al, Qlo, ldq, warp * 16, ks, lane);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        uint32_t b[2];
        load_b_frag_nk(b, Kt, ldk, nt * 8, ks, lane);
        mma_bf16_16816(S[nt], ah, b);
        mma_bf16_16816(S[nt], al, b);
      }
    }
    // cap, distance bias, mask; running maximum and sum per row (scores in units of ln 2 from here on)
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int key = k0 + nt * 8 + 2 * tq + j;
        const bool in = key < k_lim;
        float s_lo = S[nt][j], s_hi = S[nt][2 + j];
        if (p.cap > 0.f) {
          s_lo = p.cap * sw_tanh(s_lo / p.cap);
          s_hi = p.cap * sw_tanh(s_hi / p.cap);
        }
        s_lo = (s_lo - slope_lo * static_cast<float>(qpos_lo - key)) * kSwLog2e;
        s_hi = (s_hi - slope_hi * static_cast<float>(qpos_hi - key)) * kSwLog2e;
        S[nt][j] = (in && sw_visible(qpos_lo, key, p.window, p.keep_first)) ? s_lo : -INFINITY;
        S[nt][2 + j] = (in && sw_visible(qpos_hi, key, p.window, p.keep_first)) ? s_hi : -INFINITY;
        mx_lo = fmaxf(mx_lo, S[nt][j]);
        mx_hi = fmaxf(mx_hi, S[nt][2 + j]);
      }
    mx_lo = fmaxf(mrow[0], sw_quad_max(mx_lo));
    mx_hi = fmaxf(mrow[1], sw_quad_max(mx_hi));
    const float c_lo = mx_lo > -INFINITY ? exp2f(mrow[0] - mx_lo) : 1.f;      // exp2f(-inf) = 0 for a first tile
    const float c_hi = mx_hi > -INFINITY ? exp2f(mrow[1] - mx_hi) : 1.f;
    const float b_lo = mx_lo > -INFINITY ? mx_lo : 0.f, b_hi = mx_hi > -INFINITY ? mx_hi : 0.f;
    mrow[0] = mx_lo;
    mrow[1] = mx_hi;
    float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        S[nt][j] = exp2f(S[nt][j] - b_lo);               // masked scores are -inf: weight 0
        S[nt][2 + j] = exp2f(S[nt][2 + j] - b_hi);
        s_lo += S[nt][j];
        s_hi += S[nt][2 + j];
      }
    lrow[0] = lrow[0] * c_lo + s_lo;                     // per-thread partial sums; the quad adds up at the end
    lrow[1] = lrow[1] * c_hi + s_hi;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      O[nt][0] *= c_lo;
      O[nt][1] *= c_lo;
      O[nt][2] *= c_hi;
      O[nt][3] *= c_hi;
    }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {                     // 16 keys per step
      uint32_t ph[4], pl[4];
      sw_split_pack(S[2 * kk][0], S[2 * kk][1], ph[0], pl[0]);
      sw_split_pack(S[2 * kk][2], S[2 * kk][3], ph[1], pl[1]);
      sw_split_pack(S[2 * kk + 1][0], S[2 * kk + 1][1], ph[2], pl[2]);
      sw_split_pack(S[2 * kk + 1][2], S[2 * kk + 1][3], ph[3], pl[3]);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (nt * 8 < e) {
          uint32_t b[2];
          load_b_frag_kn(b, Vt, ldv, kk * 16, nt * 8, lane);
          mma_bf16_16816(O[nt], ph, b);
          mma_bf16_16816(O[nt], pl, b);
        }
      }
    }
  }
  if (!warp_active) return;
  lrow[0] = sw_quad_sum(lrow[0]);
  lrow[1] = sw_quad_sum(lrow[1]);
  if (SPLIT) {          // decode only: row r of the CTA is head h0 + r; slices use the FMA kernel's partial layout
    const long long base = (static_cast<long long>(tile) * gridDim.y + blockIdx.y) * p.splits + split;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? r_hi : r_lo;
      if (r >= nvalid) continue;
      const long long prow = base * kSwRows + r;
      if (tq == 0) {
        p.part_ml[prow * 2] = mrow[half] > -INFINITY ? mrow[half] * kSwLn2 : -INFINITY;
        p.part_ml[prow * 2 + 1] = lrow[half];
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        if (nt * 8 < e) {
          p.part_o[prow * e + nt * 8 + 2 * tq] = O[nt][2 * half];
          p.part_o[prow * e + nt * 8 + 2 * tq + 1] = O[nt][2 * half + 1];
        }
    }
    return;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r_hi : r_lo;
    if (r >= nvalid) continue;
    const float inv = lrow[half] > 0.f ? 1.f / lrow[half] : 0.f;
    const long long tok = decode ? t0 : t0 + r;
    const int head = decode ? h0 + r : h0;
    __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(p.out) + (tok * H + head) * e;
    const __nv_bfloat16* gr = p.gate ? static_cast<const __nv_bfloat16*>(p.gate) + tok * p.gate_ld + static_cast<long long>(head) * e : nullptr;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      if (nt * 8 < e) {
        float o0 = O[nt][2 * half] * inv, o1 = O[nt][2 * half + 1] * inv;
        if (gr) {
          o0 *= 1.f / (1.f + expf(-__bfloat162float(gr[nt * 8 + 2 * tq])));
          o1 *= 1.f / (1.f + expf(-__bfloat162float(gr[nt * 8 + 2 * tq + 1])));
        }
        *reinterpret_cast<__nv_bfloat162*>(orow + nt * 8 + 2 * tq) = __floats2bfloat162_rn(o0, o1);
      }
  }
}

}  // namespace llmctl

using namespace llmctl;

// proj: [tokens, >= H*d + G*d + G*e] (row stride ld) = [q | k | v | ...]; bias: fp32 [H*d + G*d + G*e] or null; cache rows
// have G*d + G*e numbers; slots = page * bs + offset, negative = not cached.
LLMCTL_API int llmctl_window_kv_append(const void* proj, long long ld, const float* bias, int H, int G, int d, int e, int value_norm,
                                       float eps, const long long* slots, float* q_out, void* cache, int tokens, int is_fp32,
                                       void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && G > 0 && d > 0 && e > 0 && ld >= static_cast<long long>(H + G) * d + static_cast<long long>(G) * e);
  if (tokens == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (window_kv_append_kernel<T><<<tokens, 256, 0, (cudaStream_t)stream>>>(
                                        (const T*)proj, ld, bias, H, G, d, e, value_norm, eps, slots, q_out, (T*)cache)));
  LLMCTL_RETURN_LAST();
}

// Largest number of heads a CTA takes for tiles of `tile_tokens` tokens: a divisor of H/G with tile_tokens * heads <= rows
// (32 on the FMA kernel, 16 on the tensor-core kernel's single-token tiles).
static int softcap_heads_per_cta(int H, int G, int tile_tokens, int rows) {
  const int rep = H / G;
  int hb = 1;
  for (int c = 1; c <= rep; ++c)
    if (rep % c == 0 && tile_tokens * c <= rows) hb = c;
  return hb;
}

LLMCTL_API int llmctl_softcap_attention_heads_per_cta(int H, int G, int tile_tokens, int use_mma) {
  if (H <= 0 || G <= 0 || H % G || tile_tokens < 1) return 0;
  if (use_mma) return tile_tokens == 1 ? softcap_heads_per_cta(H, G, 1, 16) : 1;
  if (tile_tokens > 16) return 0;
  return softcap_heads_per_cta(H, G, tile_tokens, kSwRows);
}

static size_t softcap_attention_mma_smem(int d, int e, int warps) {
  return sizeof(__nv_bfloat16) * (2 * static_cast<size_t>(warps) * 16 * (d + 8) + 2 * kSwKT * (d + 8) + 2 * kSwKT * (e + 8));
}

// 1 when bf16 caches of these sizes run on the tensor-core kernel (tile_tokens 1: decoded tokens; otherwise tiles of up
// to 128 tokens).
LLMCTL_API int llmctl_softcap_attention_mma_ok(int H, int G, int d, int e, int tile_tokens) {
  if (H <= 0 || G <= 0 || H % G || d % 16 || e % 8 || e > 128 || d > 512 || tile_tokens < 1 || tile_tokens > 128) return 0;
  return softcap_attention_mma_smem(d, e, tile_tokens == 1 ? 1 : 8) <= 200 * 1024 ? 1 : 0;
}

template <bool SPLIT>
static int launch_softcap_attention_mma(const SoftcapAttnParams& p, int ntiles, int decode, cudaStream_t s) {
  const int warps = decode ? 1 : 8;
  const size_t smem = softcap_attention_mma_smem(p.d, p.e, warps);
  const dim3 grid(ntiles * p.splits, decode ? p.H / p.HB : p.H);
#define LLMCTL_SW_LAUNCH(NT)                                                                                                     \
  do {                                                                                                                           \
    auto kern = softcap_attention_mma_kernel<NT, SPLIT>;                                                                         \
    if (smem > 48 * 1024) LLMCTL_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))); \
    kern<<<grid, warps * 32, smem, s>>>(p, decode);                                                                              \
  } while (0)
  if (p.e <= 32) LLMCTL_SW_LAUNCH(4);
  else if (p.e <= 64) LLMCTL_SW_LAUNCH(8);
  else if (p.e <= 96) LLMCTL_SW_LAUNCH(12);
  else LLMCTL_SW_LAUNCH(16);
#undef LLMCTL_SW_LAUNCH
  return 0;
}

template <typename T, bool SPLIT>
static int launch_softcap_attention(const SoftcapAttnParams& p, int ntiles, size_t smem, cudaStream_t s) {
  const dim3 grid(ntiles * p.splits, p.H / p.HB);
#define LLMCTL_SF_LAUNCH(NC)                                                                                                     \
  do {                                                                                                                           \
    auto kern = softcap_attention_kernel<T, NC, SPLIT>;                                                                          \
    if (smem > 48 * 1024) LLMCTL_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))); \
    kern<<<grid, kSwThreads, smem, s>>>(p);                                                                                      \
  } while (0)
  if (p.e <= 32) LLMCTL_SF_LAUNCH(1);
  else if (p.e <= 64) LLMCTL_SF_LAUNCH(2);
  else if (p.e <= 128) LLMCTL_SF_LAUNCH(4);
  else if (p.e <= 256) LLMCTL_SF_LAUNCH(8);
  else LLMCTL_SF_LAUNCH(16);
#undef LLMCTL_SF_LAUNCH
  return 0;
}

// tile_tokens: most tokens in a tile (<= 16; the tensor-core kernel, use_mma, takes 1 or up to 128); splits > 1 needs
// part_ml [ntiles * H/HB * splits * 64] and part_o [ntiles * H/HB * splits * 32 * e] (fp32) and, on the tensor-core
// kernel, tile_tokens 1.  window 0: every earlier key is seen.  cap 0: no soft cap.
LLMCTL_API int llmctl_softcap_window_attention(const float* q, const void* cache, const int* block_tables, int max_blocks,
                                               const int* tiles, int ntiles, int tile_tokens, const int* positions, const void* gate,
                                               long long gate_ld, const float* slopes, const float* sinks, float scale, float cap,
                                               int window, int keep_first, int H, int G, int d, int e, int bs, void* out, int splits,
                                               float* part_ml, float* part_o, int is_fp32, int use_mma, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0 && e <= 512 && bs > 0 && tile_tokens >= 1 && window >= 0 &&
                 keep_first >= 0 && cap >= 0.f);
  LLMCTL_REQUIRE(splits >= 1 && (splits == 1 || (part_ml != nullptr && part_o != nullptr)));
  if (ntiles == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  SoftcapAttnParams p{q, cache, block_tables, max_blocks, tiles, positions, gate, gate_ld, slopes, sinks, scale, cap, window, keep_first,
                      H, G, d, e, bs, llmctl_softcap_attention_heads_per_cta(H, G, tile_tokens, use_mma), out, splits, part_ml, part_o};
  LLMCTL_REQUIRE(p.HB >= 1);
  const int head_blocks = H / p.HB;
  if (use_mma) {
    LLMCTL_REQUIRE(!is_fp32 && llmctl_softcap_attention_mma_ok(H, G, d, e, tile_tokens) && (splits == 1 || tile_tokens == 1));
    LLMCTL_REQUIRE((reinterpret_cast<uintptr_t>(cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0);
    const int decode = tile_tokens == 1;
    int rcm = splits == 1 ? launch_softcap_attention_mma<false>(p, ntiles, decode, s) : launch_softcap_attention_mma<true>(p, ntiles, decode, s);
    if (rcm) return rcm;
    if (splits > 1) softcap_attention_merge_kernel<__nv_bfloat16><<<ntiles * head_blocks, 128, 0, s>>>(p, head_blocks);
    LLMCTL_RETURN_LAST();
  }
  LLMCTL_REQUIRE(tile_tokens <= 16);
  const size_t smem = sizeof(float) * (static_cast<size_t>(kSwRows) * d + kSwKT * (d + 1) + kSwKT * e + kSwRows * kSwKT);
  LLMCTL_REQUIRE(smem <= 200 * 1024);
  int rc;
  if (splits == 1) {
    LLMCTL_DISPATCH_DTYPE(is_fp32, T, (rc = launch_softcap_attention<T, false>(p, ntiles, smem, s)));
    if (rc) return rc;
    LLMCTL_RETURN_LAST();
  }
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (rc = launch_softcap_attention<T, true>(p, ntiles, smem, s)));
  if (rc) return rc;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (softcap_attention_merge_kernel<T><<<ntiles * head_blocks, 128, 0, s>>>(p, head_blocks)));
  LLMCTL_RETURN_LAST();
}
