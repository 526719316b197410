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
//   llmctl_diff_attention_split / _merge : the same with every tile's keys cut into slices over several CTAs (few
//       tiles, long contexts: decoding); the slices' (max, sum, weighted values) are merged before the difference.
// Reference: none (the reference has no attention code; reference llmctl/serve/server.py:199-204 calls HF).
#include "../common/dtype.cuh"
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
  else LLMCTL_DA_LAUNCH(8);
#undef LLMCTL_DA_LAUNCH
  return 0;
}

// tile_tokens: most tokens in a tile (<= 16); splits > 1 needs part_ml [ntiles * H/HB * splits * 64] and part_o
// [ntiles * H/HB * splits * 32 * e] (fp32).
LLMCTL_API int llmctl_diff_attention(const float* q, const void* cache, const int* block_tables, int max_blocks, const int* tiles,
                                     int ntiles, int tile_tokens, const int* positions, const void* gate, long long gate_ld,
                                     float scale, float lambda, float post_scale, float eps, int H, int G, int d, int e, int bs,
                                     void* out, int splits, float* part_ml, float* part_o, int is_fp32, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0 && e <= 256 && bs > 0 && tile_tokens >= 1 && tile_tokens <= 16);
  LLMCTL_REQUIRE(splits >= 1 && (splits == 1 || (part_ml != nullptr && part_o != nullptr)));
  if (ntiles == 0) return 0;
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
