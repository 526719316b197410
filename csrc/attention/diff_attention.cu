// Differential attention over a paged cache, for ragged batches (portions of prompts next to single decoded tokens),
// bf16 or fp32.
//
// Every query head carries TWO score maps over the same values.  With q1, q2 the head's two query vectors, k1, k2 the
// two key vectors of its key/value head (H query heads use G key/value heads, head h reads head h / (H/G)) and v that
// head's values:
//
//     a_m = softmax_j<=i (q_m . k_m,j * scale) v_j             m = 1, 2, causal, ordinary softmax
//     o   = a_1 - lambda * a_2
//     o   <- o / sqrt(mean(o^2) + eps) * post_scale * sigmoid(gate[t, h])       (gate optional)
//
// lambda, post_scale and eps are numbers of the layer.  Cache of a layer: [pages, bs, G*2*d + G*e]; a token's row holds
// the keys of all heads (head by head as [map 1 | map 2]) and then the values of all heads.
//
//   llmctl_rotary_kv_append : per token, from a packed projection [q | k | v | ...]: rotation of the first `rot`
//       numbers of every d-sized query and key vector as interleaved pairs at the token's position; q leaves in fp32,
//       k and v go to the token's cache row.  Not specific to two maps: it sees `nq` query and `nk` key vectors.
//   llmctl_diff_attention : a CTA owns up to 16 consecutive tokens of a sequence x HB heads of one key/value head
//       (HB = 1 for prompt portions, up to 16 heads for single decoded tokens) as 2 * tokens * HB <= 32 softmax rows;
//       a warp owns four rows through all phases (scores, online softmax, weights x values), so only the key/value tile
//       loads synchronise the CTA.  Scores, softmax, sums, the difference and the norm are fp32 (FMA).
//       With splits > 1 every tile's keys are cut into slices over several CTAs (few tiles, long contexts: decoding);
//       the slices' (max, sum, weighted values) are merged before the difference.
//   bf16 caches with d a multiple of 16 and e a multiple of 8 up to 128 run on the tensor cores (mma.sync m16n8k16, fp32
//       accumulation) instead: a CTA owns up to 128 consecutive tokens of a sequence for one head (8 warps x 16 rows;
//       prompt portions) or one token's heads of one key/value head (one warp; decoded tokens, keys cut into slices).
//       Key/value tiles of 32 keys come straight from the paged cache by 16-byte cp.async into two stages.  The fp32
//       queries (scaled, in units of ln 2) are held as a bf16 pair hi + lo and so are the softmax weights, so that both
//       products are exact to ~2^-17; maxima, sums and the output accumulators are fp32 registers.  A warp runs map 1
//       and map 2 of a key tile one after the other against the same value tile.
// Reference: none (the reference has no attention code; reference llmctl/serve/server.py:199-204 calls HF).
#include "../common/dtype.cuh"
#include "../common/mma_sync.cuh"
#include "../rope/rope_interleaved.cuh"

namespace llmctl {

// ---------------------------------------------------------------------------------------------------------------
// rotation + cache append: one CTA per token
// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
rotary_kv_append_kernel(const T* __restrict__ proj, long long ld, int nq, int nk, int d, int nv, int rot,
                        const float* __restrict__ freq, float mult, const int* __restrict__ positions,
                        const long long* __restrict__ slots, float* __restrict__ q_out, T* __restrict__ cache) {
  const long long t = blockIdx.x;
  const int Nq = nq * d, Nk = nk * d, Wc = Nk + nv;
  const T* row = proj + t * ld;
  const int pos = positions[t];
  const long long slot = slots[t];
  T* crow = slot >= 0 ? cache + slot * Wc : nullptr;
  for (int c = threadIdx.x; c < Nq + Nk; c += blockDim.x) {
    const int dd = c % d, base = c - dd;
    float v = to_f32(row[c]);
    if (dd < rot) v = rope_interleaved_coord([&](int k) { return to_f32(row[base + k]); }, dd, pos, freq, mult);
    if (c < Nq) q_out[t * Nq + c] = v;
    else if (crow) crow[c - Nq] = from_f32<T>(v);
  }
  if (crow)
    for (int c = threadIdx.x; c < nv; c += blockDim.x) crow[Nk + c] = row[Nq + Nk + c];
}

// ---------------------------------------------------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------------------------------------------------
constexpr int kDaKT = 32;         // keys per tile
constexpr int kDaRows = 32;       // softmax rows per CTA: (token, head, map)
constexpr int kDaThreads = 256;   // 8 warps x 4 rows

struct DiffAttnParams {
  const float* q;            // [T, H*2*d]
  const void* cache;
  const int* block_tables;
  int max_blocks;
  const int* tiles;          // [n, 4] = (first token row, tokens, block-table row, 0)
  const int* positions;
  const void* gate;          // [T, *] pre-sigmoid gates, column h of row t (row stride gate_ld); null = no gate
  long long gate_ld;
  float scale, lambda, post_scale, eps;
  int H, G, d, e, bs;
  int HB;                    // heads per CTA
  void* out;                 // [T, H*e]
  int splits;                // key slices per tile (1 = whole)
  float* part_ml;            // [tiles * H/HB * splits, 32, 2]
  float* part_o;             // [tiles * H/HB * splits, 32, e]
};

// NC: output columns per lane (e <= 32 * NC)
template <typename T, int NC, bool SPLIT>
__global__ void __launch_bounds__(kDaThreads)
diff_attention_kernel(const DiffAttnParams p) {
  extern __shared__ float sm[];
  const int H = p.H, G = p.G, d = p.d, e = p.e, bs = p.bs, HB = p.HB;
  const int rep = H / G, Wc = G * (2 * d + e), ldk = 2 * d + 1;
  const int tile = blockIdx.x / p.splits, split = blockIdx.x % p.splits;
  const int t0 = p.tiles[tile * 4], nq = p.tiles[tile * 4 + 1];
  if (nq <= 0) return;
  const int* table = p.block_tables + static_cast<long long>(p.tiles[tile * 4 + 2]) * p.max_blocks;
  const int h0 = blockIdx.y * HB, g = h0 / rep;
  const int p_first = p.positions[t0], p_last = p_first + nq - 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nrows = nq * HB * 2;                 // row r = (tq * HB + hb) * 2 + map

  float* Qs = sm;                                // [32][d]
  float* Ks = Qs + kDaRows * d;                  // [KT][2d + 1]
  float* Vs = Ks + kDaKT * ldk;                  // [KT][e]
  float* Ps = Vs + kDaKT * e;                    // [32][KT]

  const T* cache = static_cast<const T*>(p.cache);
  for (int i = tid; i < kDaRows * d; i += kDaThreads) {
    const int r = i / d, c = i % d;
    float v = 0.f;
    if (r < nrows) {
      const int tq = (r >> 1) / HB, hb = (r >> 1) % HB, mp = r & 1;
      v = p.q[(static_cast<long long>(t0 + tq) * H + h0 + hb) * 2 * d + mp * d + c] * p.scale;
    }
    Qs[i] = v;
  }

  float m[4], l[4], acc[4][NC];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
  }
  // position of the query of this warp's row i
  int qpos[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp * 4 + i;
    qpos[i] = r < nrows ? p_first + (r >> 1) / HB : -1;
  }
  const int warp_rows = min(max(nrows - warp * 4, 0), 4);

  const int nkeys = p_last + 1;
  int k_begin = 0, k_end = nkeys;
  if (SPLIT) {
    const int per = ((nkeys + p.splits - 1) / p.splits + kDaKT - 1) / kDaKT * kDaKT;
    k_begin = min(split * per, nkeys);
    k_end = min(k_begin + per, nkeys);
  }
  for (int k0 = k_begin; k0 < k_end; k0 += kDaKT) {
    __syncthreads();                             // the previous tile's readers are done (and Qs is written)
    const int nk = min(kDaKT, k_end - k0);
    for (int i = tid; i < kDaKT * 2 * d; i += kDaThreads) {
      const int kk = i / (2 * d), c = i % (2 * d);
      float v = 0.f;
      if (kk < nk) {
        const int j = k0 + kk;
        v = to_f32(cache[(static_cast<long long>(table[j / bs]) * bs + j % bs) * Wc + g * 2 * d + c]);
      }
      Ks[kk * ldk + c] = v;
    }
    for (int i = tid; i < kDaKT * e; i += kDaThreads) {
      const int kk = i / e, c = i % e;
      float v = 0.f;
      if (kk < nk) {
        const int j = k0 + kk;
        v = to_f32(cache[(static_cast<long long>(table[j / bs]) * bs + j % bs) * Wc + G * 2 * d + g * e + c]);
      }
      Vs[i] = v;
    }
    __syncthreads();
    if (warp_rows > 0) {
      // scores of this lane's key for the warp's rows
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      const float* kr = Ks + lane * ldk;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (i < warp_rows) {
          const int r = warp * 4 + i;
          const float* qr = Qs + r * d;
          const float* kv = kr + (r & 1) * d;
          float a0 = 0.f, a1 = 0.f;
          int c = 0;
          for (; c + 1 < d; c += 2) {
            a0 += qr[c] * kv[c];
            a1 += qr[c + 1] * kv[c + 1];
          }
          if (c < d) a0 += qr[c] * kv[c];
          s[i] = a0 + a1;
        }
      }
      const int j = k0 + lane;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (i < warp_rows) {
          const bool seen = lane < nk && j <= qpos[i];
          const float sv = seen ? s[i] : -INFINITY;
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
          Ps[(warp * 4 + i) * kDaKT + lane] = pw;
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
            const float pw = Ps[(warp * 4 + i) * kDaKT + kk];
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
          p.part_ml[(base * kDaRows + r) * 2] = m[i];
          p.part_ml[(base * kDaRows + r) * 2 + 1] = l[i];
        }
#pragma unroll
        for (int c = 0; c < NC; ++c)
          if (lane + 32 * c < e) p.part_o[(base * kDaRows + r) * e + lane + 32 * c] = acc[i][c];
      }
    }
    return;
  }
  // rows 2k and 2k+1 of the warp are the two maps of one (token, head)
#pragma unroll
  for (int pr = 0; pr < 2; ++pr) {
    if (2 * pr < warp_rows) {
      const int r = warp * 4 + 2 * pr;
      const int tq = (r >> 1) / HB, hb = (r >> 1) % HB;
      const float i1 = 1.f / l[2 * pr], i2 = 1.f / l[2 * pr + 1];
      float o[NC], ss = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        o[c] = acc[2 * pr][c] * i1 - p.lambda * (acc[2 * pr + 1][c] * i2);
        if (lane + 32 * c < e) ss += o[c] * o[c];
      }
      ss = warp_sum(ss);
      float f = p.post_scale / sqrtf(ss / e + p.eps);
      const long long t = t0 + tq;
      if (p.gate) {
        const float gz = to_f32(static_cast<const T*>(p.gate)[t * p.gate_ld + h0 + hb]);
        f *= 1.f / (1.f + expf(-gz));
      }
      T* orow = static_cast<T*>(p.out) + (t * H + h0 + hb) * e;
#pragma unroll
      for (int c = 0; c < NC; ++c)
        if (lane + 32 * c < e) orow[lane + 32 * c] = from_f32<T>(o[c] * f);
    }
  }
}

// One warp per (tile, head block, row pair): merges the slices and finishes like the unsplit kernel.
template <typename T>
__global__ void __launch_bounds__(128)
diff_attention_merge_kernel(const DiffAttnParams p, int head_blocks) {
  const int H = p.H, e = p.e, HB = p.HB;
  const int lane = threadIdx.x & 31;
  const long long unit = blockIdx.x;                        // (tile, head block)
  const int tile = static_cast<int>(unit / head_blocks), hblk = static_cast<int>(unit % head_blocks);
  const int t0 = p.tiles[tile * 4], nq = p.tiles[tile * 4 + 1];
  const int nrows = nq * HB * 2;
  for (int pair = threadIdx.x >> 5; 2 * pair < nrows; pair += blockDim.x >> 5) {
    const int tq = pair / HB, hb = pair % HB, h = hblk * HB + hb;
    const long long t = t0 + tq;
    float ss = 0.f;
    // two passes over the columns in chunks of 32: the difference is staged in the output's fp32 partial buffer row
    float* stage = p.part_o + ((unit * p.splits) * kDaRows + 2 * pair) * e;      // slice 0, map 1 row: reused as staging
    float mx[2] = {-INFINITY, -INFINITY};
    for (int s = 0; s < p.splits; ++s)
      for (int mp = 0; mp < 2; ++mp) mx[mp] = fmaxf(mx[mp], p.part_ml[((unit * p.splits + s) * kDaRows + 2 * pair + mp) * 2]);
    float ls[2] = {0.f, 0.f};
    for (int s = 0; s < p.splits; ++s)
      for (int mp = 0; mp < 2; ++mp) {
        const float* ml = p.part_ml + ((unit * p.splits + s) * kDaRows + 2 * pair + mp) * 2;
        if (ml[0] > -INFINITY) ls[mp] += ml[1] * expf(ml[0] - mx[mp]);
      }
    for (int c = lane; c < e; c += 32) {
      float a[2] = {0.f, 0.f};
      for (int s = 0; s < p.splits; ++s)
        for (int mp = 0; mp < 2; ++mp) {
          const long long row = (unit * p.splits + s) * kDaRows + 2 * pair + mp;
          const float mv = p.part_ml[row * 2];
          if (mv > -INFINITY) a[mp] += p.part_o[row * e + c] * expf(mv - mx[mp]);
        }
      const float o = a[0] / ls[0] - p.lambda * (a[1] / ls[1]);
      ss += o * o;
      stage[c] = o;                                           // this lane wrote and will read column c only
    }
    ss = warp_sum(ss);
    float f = p.post_scale / sqrtf(ss / e + p.eps);
    if (p.gate) {
      const float gz = to_f32(static_cast<const T*>(p.gate)[t * p.gate_ld + h]);
      f *= 1.f / (1.f + expf(-gz));
    }
    T* orow = static_cast<T*>(p.out) + (t * H + h) * e;
    for (int c = lane; c < e; c += 32) orow[c] = from_f32<T>(stage[c] * f);
  }
}


// ---------------------------------------------------------------------------------------------------------------
// tensor-core attention (bf16 cache)
// ---------------------------------------------------------------------------------------------------------------
constexpr int kDmKT = 32;          // keys per tile
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
// bf16 pair hi + lo of two fp32 numbers, packed for an A fragment
__device__ __forceinline__ void split_pack(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 ah = __float2bfloat16(a), bh = __float2bfloat16(b);
  hi = pack_bf16x2(__bfloat162float(ah), __bfloat162float(bh));
  lo = pack_bf16x2(a - __bfloat162float(ah), b - __bfloat162float(bh));
}

// NT: n-tiles of 8 output columns held per map (e <= 8 NT).  decode = 0: rows of the CTA are the tile's tokens (head
// blockIdx.y); decode = 1: rows are HB heads of the tile's single token.
template <int NT, bool SPLIT>
__global__ void __launch_bounds__(256)
diff_attention_mma_kernel(const DiffAttnParams p, int decode) {
  extern __shared__ __align__(16) unsigned char dm_smem[];
  const int H = p.H, G = p.G, d = p.d, e = p.e, bs = p.bs;
  const int rep = H / G, Wc = G * (2 * d + e);
  const int tile = blockIdx.x / p.splits, split = blockIdx.x % p.splits;
  const int t0 = p.tiles[tile * 4], nq = p.tiles[tile * 4 + 1];
  if (nq <= 0) return;
  const int* table = p.block_tables + static_cast<long long>(p.tiles[tile * 4 + 2]) * p.max_blocks;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
  const int rows_cta = (nthreads >> 5) * 16;
  const int h0 = decode ? blockIdx.y * p.HB : blockIdx.y, g = h0 / rep;
  const int nvalid = decode ? p.HB : nq;
  const int p_first = p.positions[t0], p_last = decode ? p_first : p_first + nq - 1;
  const int ldq = 2 * d + 8, ldk = 2 * d + 8, ldv = e + 8;
  __nv_bfloat16* Qhi = reinterpret_cast<__nv_bfloat16*>(dm_smem);       // [rows][ldq]
  __nv_bfloat16* Qlo = Qhi + rows_cta * ldq;
  __nv_bfloat16* Ks = Qlo + rows_cta * ldq;                              // [2][KT][ldk]
  __nv_bfloat16* Vs = Ks + 2 * kDmKT * ldk;                              // [2][KT][ldv]
  const __nv_bfloat16* cache = static_cast<const __nv_bfloat16*>(p.cache);

  {
    const float qs = p.scale * kLog2e;
    const int per_row = (2 * d) >> 2;
    for (int i = tid; i < rows_cta * per_row; i += nthreads) {
      const int r = i / per_row, c = (i % per_row) << 2;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < nvalid) {
        const long long tok = decode ? t0 : t0 + r;
        const int head = decode ? h0 + r : h0;
        v = *reinterpret_cast<const float4*>(p.q + (tok * H + head) * 2 * d + c);
        v.x *= qs, v.y *= qs, v.z *= qs, v.w *= qs;
      }
      uint32_t h01, l01, h23, l23;
      split_pack(v.x, v.y, h01, l01);
      split_pack(v.z, v.w, h23, l23);
      *reinterpret_cast<uint2*>(Qhi + r * ldq + c) = make_uint2(h01, h23);
      *reinterpret_cast<uint2*>(Qlo + r * ldq + c) = make_uint2(l01, l23);
    }
  }

  const int nkeys = p_last + 1;
  int k_begin = 0, k_end = nkeys;
  if (SPLIT) {
    const int per = ((nkeys + p.splits - 1) / p.splits + kDmKT - 1) / kDmKT * kDmKT;
    k_begin = min(split * per, nkeys);
    k_end = min(k_begin + per, nkeys);
  }
  const int kch = (2 * d) >> 3, vch = e >> 3, chunks = kch + vch;
  // cache offsets of a tile's keys are looked up (page table) one tile ahead of the copies that use them
  __shared__ long long rowoff[2][kDmKT];
  auto index_tile = [&](int stage, int k0) {
    if (tid < kDmKT) {
      const int j = k0 + tid;
      rowoff[stage][tid] = j < k_end ? (static_cast<long long>(table[j / bs]) * bs + j % bs) * Wc : -1;
    }
  };
  auto load_tile = [&](int stage) {
    for (int i = tid; i < kDmKT * chunks; i += nthreads) {
      const int kk = i / chunks, ch = i % chunks;
      const long long off = rowoff[stage][kk];
      __nv_bfloat16* dst = ch < kch ? Ks + (stage * kDmKT + kk) * ldk + ch * 8 : Vs + (stage * kDmKT + kk) * ldv + (ch - kch) * 8;
      if (off >= 0) {
        const __nv_bfloat16* row = cache + off;
        cp_async_16(dst, ch < kch ? row + g * 2 * d + ch * 8 : row + G * 2 * d + g * e + (ch - kch) * 8);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);      // a weight of 0 times stale bits could be a NaN
      }
    }
  };

  const int grow = lane >> 2, tq = lane & 3;
  const int r_lo = warp * 16 + grow, r_hi = r_lo + 8;
  const int qpos_lo = r_lo < nvalid ? (decode ? p_first : p_first + r_lo) : -1;
  const int qpos_hi = r_hi < nvalid ? (decode ? p_first : p_first + r_hi) : -1;
  const bool warp_active = warp * 16 < nvalid;
  const int warp_last = decode ? p_first : p_first + min(warp * 16 + 15, nvalid - 1);

  float O[2][NT][4];
  float mrow[2][2], lrow[2][2];           // [map][lo / hi row]
#pragma unroll
  for (int mp = 0; mp < 2; ++mp) {
    mrow[mp][0] = mrow[mp][1] = -INFINITY;
    lrow[mp][0] = lrow[mp][1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) O[mp][nt][j] = 0.f;
  }

  const int ntile = (k_end - k_begin + kDmKT - 1) / kDmKT;
  if (ntile > 0) index_tile(0, k_begin);
  if (ntile > 1) index_tile(1, k_begin + kDmKT);
  __syncthreads();
  if (ntile > 0) load_tile(0);
  cp_async_commit();
  for (int it = 0; it < ntile; ++it) {
    cp_async_wait_all();
    __syncthreads();                       // tile `it` has landed (and Q); everyone is done with the other stage
    if (it + 1 < ntile) load_tile((it + 1) & 1);
    cp_async_commit();
    if (it + 2 < ntile) index_tile(it & 1, k_begin + (it + 2) * kDmKT);     // its last readers ran before the barrier
    const int k0 = k_begin + it * kDmKT, st = it & 1;
    if (!warp_active || k0 > warp_last) continue;
    const __nv_bfloat16* Kt = Ks + st * kDmKT * ldk;
    const __nv_bfloat16* Vt = Vs + st * kDmKT * ldv;
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
      float S[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) S[nt][j] = 0.f;
      for (int ks = 0; ks < d; ks += 16) {
        uint32_t ah[4], al[4];
        load_a_frag(ah, Qhi, ldq, warp * 16, mp * d + ks, lane);
        load_a_frag(al, Qlo, ldq, warp * 16, mp * d + ks, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          uint32_t b[2];
          load_b_frag_nk(b, Kt, ldk, nt * 8, mp * d + ks, lane);
          mma_bf16_16816(S[nt], ah, b);
          mma_bf16_16816(S[nt], al, b);
        }
      }
      // causal mask, running maximum and sum per row
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int key = k0 + nt * 8 + 2 * tq + j;
          const bool in = key < k_end;
          if (!(in && key <= qpos_lo)) S[nt][j] = -INFINITY;
          if (!(in && key <= qpos_hi)) S[nt][2 + j] = -INFINITY;
          mx_lo = fmaxf(mx_lo, S[nt][j]);
          mx_hi = fmaxf(mx_hi, S[nt][2 + j]);
        }
      mx_lo = fmaxf(mrow[mp][0], quad_max(mx_lo));
      mx_hi = fmaxf(mrow[mp][1], quad_max(mx_hi));
      const float c_lo = mx_lo > -INFINITY ? exp2f(mrow[mp][0] - mx_lo) : 1.f;      // exp2f(-inf) = 0 for a first tile
      const float c_hi = mx_hi > -INFINITY ? exp2f(mrow[mp][1] - mx_hi) : 1.f;
      const float b_lo = mx_lo > -INFINITY ? mx_lo : 0.f, b_hi = mx_hi > -INFINITY ? mx_hi : 0.f;
      mrow[mp][0] = mx_lo;
      mrow[mp][1] = mx_hi;
      float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          S[nt][j] = exp2f(S[nt][j] - b_lo);             // masked scores are -inf: weight 0
          S[nt][2 + j] = exp2f(S[nt][2 + j] - b_hi);
          s_lo += S[nt][j];
          s_hi += S[nt][2 + j];
        }
      lrow[mp][0] = lrow[mp][0] * c_lo + s_lo;           // per-thread partial sums; the quad adds up at the end
      lrow[mp][1] = lrow[mp][1] * c_hi + s_hi;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        O[mp][nt][0] *= c_lo;
        O[mp][nt][1] *= c_lo;
        O[mp][nt][2] *= c_hi;
        O[mp][nt][3] *= c_hi;
      }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {                   // 16 keys per step
        uint32_t ph[4], pl[4];
        split_pack(S[2 * kk][0], S[2 * kk][1], ph[0], pl[0]);
        split_pack(S[2 * kk][2], S[2 * kk][3], ph[1], pl[1]);
        split_pack(S[2 * kk + 1][0], S[2 * kk + 1][1], ph[2], pl[2]);
        split_pack(S[2 * kk + 1][2], S[2 * kk + 1][3], ph[3], pl[3]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (nt * 8 < e) {
            uint32_t b[2];
            load_b_frag_kn(b, Vt, ldv, kk * 16, nt * 8, lane);
            mma_bf16_16816(O[mp][nt], ph, b);
            mma_bf16_16816(O[mp][nt], pl, b);
          }
        }
      }
    }
  }
  if (!warp_active) return;
#pragma unroll
  for (int mp = 0; mp < 2; ++mp) {
    lrow[mp][0] = quad_sum(lrow[mp][0]);
    lrow[mp][1] = quad_sum(lrow[mp][1]);
  }
  if (SPLIT) {          // decode only: row r of the CTA is head h0 + r; slices use the FMA kernel's partial layout
    const long long base = (static_cast<long long>(tile) * gridDim.y + blockIdx.y) * p.splits + split;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? r_hi : r_lo;
      if (r >= nvalid) continue;
#pragma unroll
      for (int mp = 0; mp < 2; ++mp) {
        const long long prow = base * kDaRows + 2 * r + mp;
        if (tq == 0) {
          p.part_ml[prow * 2] = mrow[mp][half] > -INFINITY ? mrow[mp][half] * kLn2 : -INFINITY;
          p.part_ml[prow * 2 + 1] = lrow[mp][half];
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          if (nt * 8 < e) {
            p.part_o[prow * e + nt * 8 + 2 * tq] = O[mp][nt][2 * half];
            p.part_o[prow * e + nt * 8 + 2 * tq + 1] = O[mp][nt][2 * half + 1];
          }
      }
    }
    return;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r_hi : r_lo;
    const float i1 = 1.f / lrow[0][half], i2 = 1.f / lrow[1][half];
    float ss = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float o = O[0][nt][2 * half + j] * i1 - p.lambda * (O[1][nt][2 * half + j] * i2);
        O[0][nt][2 * half + j] = o;
        if (nt * 8 < e) ss += o * o;
      }
    ss = quad_sum(ss);                                   // every lane of the quad takes part, valid row or not
    if (r >= nvalid) continue;
    const long long tok = decode ? t0 : t0 + r;
    const int head = decode ? h0 + r : h0;
    float f = p.post_scale / sqrtf(ss / e + p.eps);
    if (p.gate) {
      const float gz = __bfloat162float(static_cast<const __nv_bfloat16*>(p.gate)[tok * p.gate_ld + head]);
      f *= 1.f / (1.f + expf(-gz));
    }
    __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(p.out) + (tok * H + head) * e;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      if (nt * 8 < e)
        *reinterpret_cast<__nv_bfloat162*>(orow + nt * 8 + 2 * tq) = __floats2bfloat162_rn(O[0][nt][2 * half] * f, O[0][nt][2 * half + 1] * f);
  }
}

}  // namespace llmctl

using namespace llmctl;

// proj: [tokens, >= (nq + nk) * d + nv] (row stride ld); cache rows have nk * d + nv numbers; slots = page * bs + offset,
// negative = not cached.
LLMCTL_API int llmctl_rotary_kv_append(const void* proj, long long ld, int nq, int nk, int d, int nv, int rot, const float* freq,
                                       float mult, const int* positions, const long long* slots, float* q_out, void* cache,
                                       int tokens, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(nq > 0 && nk > 0 && d > 0 && nv >= 0 && rot >= 0 && rot <= d && rot % 2 == 0 && (rot == 0 || freq != nullptr));
  if (tokens == 0) return 0;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (rotary_kv_append_kernel<T><<<tokens, 256, 0, (cudaStream_t)stream>>>(
                                        (const T*)proj, ld, nq, nk, d, nv, rot, freq, mult, positions, slots, q_out, (T*)cache)));
  LLMCTL_RETURN_LAST();
}

// Largest number of heads a CTA of the attention kernel takes for tiles of `tile_tokens` tokens: a divisor of H/G with
// 2 * tile_tokens * heads <= 32.
LLMCTL_API int llmctl_diff_attention_heads_per_cta(int H, int G, int tile_tokens) {
  if (H <= 0 || G <= 0 || H % G || tile_tokens < 1 || tile_tokens > 16) return 0;
  const int rep = H / G;
  int hb = 1;
  for (int c = 1; c <= rep; ++c)
    if (rep % c == 0 && 2 * tile_tokens * c <= kDaRows) hb = c;
  return hb;
}

static size_t diff_attention_mma_smem(int d, int e, int warps) {
  return sizeof(__nv_bfloat16) * (2 * static_cast<size_t>(warps) * 16 * (2 * d + 8) + 2 * kDmKT * (2 * d + 8) + 2 * kDmKT * (e + 8));
}

// 1 when bf16 caches of these sizes run on the tensor-core kernel (tile_tokens 1: decoded tokens; otherwise tiles of up
// to 128 tokens).
LLMCTL_API int llmctl_diff_attention_mma_ok(int H, int G, int d, int e, int tile_tokens) {
  if (H <= 0 || G <= 0 || H % G || d % 16 || e % 8 || e > 128 || d > 256 || tile_tokens < 1 || tile_tokens > 128) return 0;
  return diff_attention_mma_smem(d, e, tile_tokens == 1 ? 1 : 8) <= 200 * 1024 ? 1 : 0;
}

template <bool SPLIT>
static int launch_diff_attention_mma(const DiffAttnParams& p, int ntiles, int decode, cudaStream_t s) {
  const int warps = decode ? 1 : 8;
  const size_t smem = diff_attention_mma_smem(p.d, p.e, warps);
  const dim3 grid(ntiles * p.splits, decode ? p.H / p.HB : p.H);
#define LLMCTL_DM_LAUNCH(NT)                                                                                                     \
  do {                                                                                                                           \
    auto kern = diff_attention_mma_kernel<NT, SPLIT>;                                                                            \
    if (smem > 48 * 1024) LLMCTL_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))); \
    kern<<<grid, warps * 32, smem, s>>>(p, decode);                                                                              \
  } while (0)
  if (p.e <= 32) LLMCTL_DM_LAUNCH(4);
  else if (p.e <= 64) LLMCTL_DM_LAUNCH(8);
  else if (p.e <= 96) LLMCTL_DM_LAUNCH(12);
  else LLMCTL_DM_LAUNCH(16);
#undef LLMCTL_DM_LAUNCH
  return 0;
}

template <typename T, bool SPLIT>
static int launch_diff_attention(const DiffAttnParams& p, int ntiles, size_t smem, cudaStream_t s) {
  const dim3 grid(ntiles * p.splits, p.H / p.HB);
#define LLMCTL_DA_LAUNCH(NC)                                                                                                     \
  do {                                                                                                                           \
    auto kern = diff_attention_kernel<T, NC, SPLIT>;                                                                             \
    if (smem > 48 * 1024) LLMCTL_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))); \
    kern<<<grid, kDaThreads, smem, s>>>(p);                                                                                      \
  } while (0)
  if (p.e <= 32) LLMCTL_DA_LAUNCH(1);
  else if (p.e <= 64) LLMCTL_DA_LAUNCH(2);
  else if (p.e <= 128) LLMCTL_DA_LAUNCH(4);
  else if (p.e <= 256) LLMCTL_DA_LAUNCH(8);
  else LLMCTL_DA_LAUNCH(16);
#undef LLMCTL_DA_LAUNCH
  return 0;
}

// tile_tokens: most tokens in a tile (<= 16; the tensor-core kernel, use_mma, takes 1 or up to 128); splits > 1 needs
// part_ml [ntiles * H/HB * splits * 64] and part_o [ntiles * H/HB * splits * 32 * e] (fp32) and, on the tensor-core
// kernel, tile_tokens 1.
LLMCTL_API int llmctl_diff_attention(const float* q, const void* cache, const int* block_tables, int max_blocks, const int* tiles,
                                     int ntiles, int tile_tokens, const int* positions, const void* gate, long long gate_ld,
                                     float scale, float lambda, float post_scale, float eps, int H, int G, int d, int e, int bs,
                                     void* out, int splits, float* part_ml, float* part_o, int is_fp32, int use_mma, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0 && e <= 512 && bs > 0 && tile_tokens >= 1);
  LLMCTL_REQUIRE(splits >= 1 && (splits == 1 || (part_ml != nullptr && part_o != nullptr)));
  if (ntiles == 0) return 0;
  if (use_mma) {
    LLMCTL_REQUIRE(!is_fp32 && llmctl_diff_attention_mma_ok(H, G, d, e, tile_tokens) && (splits == 1 || tile_tokens == 1));
    LLMCTL_REQUIRE((reinterpret_cast<uintptr_t>(cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0);
    const int decode = tile_tokens == 1;
    DiffAttnParams pm{q, cache, block_tables, max_blocks, tiles, positions, gate, gate_ld, scale, lambda, post_scale, eps,
                      H, G, d, e, bs, decode ? llmctl_diff_attention_heads_per_cta(H, G, 1) : 1, out, splits, part_ml, part_o};
    cudaStream_t sm = (cudaStream_t)stream;
    int rcm = splits == 1 ? launch_diff_attention_mma<false>(pm, ntiles, decode, sm) : launch_diff_attention_mma<true>(pm, ntiles, decode, sm);
    if (rcm) return rcm;
    if (splits > 1) {
      const int head_blocks = H / pm.HB;
      diff_attention_merge_kernel<__nv_bfloat16><<<ntiles * head_blocks, 128, 0, sm>>>(pm, head_blocks);
    }
    LLMCTL_RETURN_LAST();
  }
  LLMCTL_REQUIRE(tile_tokens <= 16);
  DiffAttnParams p{q, cache, block_tables, max_blocks, tiles, positions, gate, gate_ld, scale, lambda, post_scale, eps,
                   H, G, d, e, bs, llmctl_diff_attention_heads_per_cta(H, G, tile_tokens), out, splits, part_ml, part_o};
  const size_t smem = sizeof(float) * (static_cast<size_t>(kDaRows) * d + kDaKT * (2 * d + 1) + kDaKT * e + kDaRows * kDaKT);
  LLMCTL_REQUIRE(smem <= 200 * 1024);
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (splits == 1) {
    LLMCTL_DISPATCH_DTYPE(is_fp32, T, (rc = launch_diff_attention<T, false>(p, ntiles, smem, s)));
    if (rc) return rc;
    LLMCTL_RETURN_LAST();
  }
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (rc = launch_diff_attention<T, true>(p, ntiles, smem, s)));
  if (rc) return rc;
  const int head_blocks = H / p.HB;
  LLMCTL_DISPATCH_DTYPE(is_fp32, T, (diff_attention_merge_kernel<T><<<ntiles * head_blocks, 128, 0, s>>>(p, head_blocks)));
  LLMCTL_RETURN_LAST();
}
