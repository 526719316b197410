// Latent attention on the 5th-generation tensor cores (bf16): absorbed queries against the paged latent cache.
//
//   out[t, h, :] = softmax_j( scale * q[t, h, :] . k[j, :] ) c[j, :]      k[j] = [c[j] | kr[j]]  (one cache row, D = R + dr)
//
// A CTA owns 128 (token, head) query rows — 128 tokens of one head in batches with prompt portions, one token's heads
// when every sequence decodes — and one group of up to 256 output columns (the fp32 accumulator of 128 x R would fill
// tensor memory on its own at R = 512, so the columns are split over CTAs and each recomputes the scores).
//
//   * queries: assembled once per call as [tokens, heads, D] bf16 (absorbed part | rotated rope part), one TMA tile
//     of 128 x D per CTA (128-byte swizzle, D / 64 panels)
//   * keys: tiles of 32 cache rows fetched by TMA straight from the paged cache through the block table (a tile never
//     straddles a page: the page size is a multiple of 32), double-buffered; the same tile is the K-major B operand of
//     S = Q K^T (UMMA 128 x 32 x 16 over D) and, through its first R columns, the MN-major B operand of O += P C
//   * S double-buffered in tensor memory; the softmax warps (one thread per query row) read it with tcgen05.ld, mask by
//     position, keep a lazily updated running reference (the accumulator is rescaled only when the maximum grows by
//     more than 2^8), and write P back as bf16 into the same columns: O += P C takes its A operand from tensor memory
//   * warp roles: 0 = TMA producer, 1 = MMA issuer (+ TMEM allocation), 2..5 = softmax / epilogue
//   * every mbarrier wait is bounded; a wait that runs out raises the CTA's abort flag, which the other roles poll,
//     records itself in a device-side status word (llmctl_latent_attention_t5_status) and the CTA drains and frees
//     its tensor memory
//
// Contexts split over CTAs (decode) write unnormalised partial sums for latent_attention_merge.
// Reference: none (the reference has no model code).
#include "../common/dtype.cuh"
#include "../common/ptx.cuh"
#include "../common/tma_host.h"
#include "../common/util.cuh"
#include "../rope/rope_interleaved.cuh"

namespace llmctl {
using namespace ptx;

namespace t5 {
constexpr int kRows = 128;          // query rows per CTA (UMMA M)
constexpr int kKeys = 32;           // keys per tile (UMMA N of the score product, K of the value product)
constexpr int kColGroup = 256;      // output columns per CTA
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;      // O: [0, 256), S / P buffers: [256, 288) and [288, 320)
constexpr int kSCol = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;
constexpr long long kWaitCycles = 400000000LL;      // ~0.2 s: far beyond any wait of a healthy pipeline

__device__ unsigned int g_status = 0;      // != 0: a bounded wait ran out (which one: low byte)

// Bounded mbarrier wait.  Returns false when it gave up or another role already did.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort, int who) {
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort) return false;
      if (clock64() - t0 > kWaitCycles) break;
    }
  }
  *abort = 1;
  atomicCAS(&g_status, 0u, 0x100u | static_cast<unsigned int>(who));
  return false;
}
}  // namespace t5

// Qfull[t, h, :] = [ ql[t, h, :R] | rotate(q[t, h, dn:dn+dr]) at the token's position ], bf16.
template <typename TQ>
__global__ void __launch_bounds__(128)
latent_q_assemble_kernel(const TQ* __restrict__ ql, long long ql_st, long long ql_sh, const __nv_bfloat16* __restrict__ q,
                         long long ldq, int dn, const int* __restrict__ positions, const float* __restrict__ freq, float mult,
                         int H, int R, int dr, __nv_bfloat16* __restrict__ qfull) {
  const long long row = blockIdx.x;       // token * H + head
  const long long tok = row / H;
  const int h = static_cast<int>(row % H);
  const TQ* src = ql + tok * ql_st + h * ql_sh;
  __nv_bfloat16* dst = qfull + row * (R + dr);
  for (int c = threadIdx.x; c < R; c += blockDim.x) dst[c] = __float2bfloat16(to_f32(src[c]));
  const __nv_bfloat16* qr = q + tok * ldq + static_cast<long long>(h) * (dn + dr) + dn;
  const int pos = positions[tok];
  for (int c = threadIdx.x; c < dr; c += blockDim.x)
    dst[R + c] = __float2bfloat16(rope_interleaved_coord([&](int k) { return to_f32(qr[k]); }, c, pos, freq, mult));
}

__global__ void __launch_bounds__(t5::kThreads, 1)
latent_attention_t5_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                           const int* __restrict__ block_tables, int max_blocks, int block_size,
                           const int* __restrict__ tiles, const int* __restrict__ positions, float scale, int H, int R,
                           int dr, int heads_per_tile, int keys_per_split, int nsplit, int q_rows_are_heads,
                           __nv_bfloat16* __restrict__ out, float* __restrict__ partial, const float* __restrict__ sinks) {
  using namespace t5;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_q, bar_kfull[2], bar_kempty[2], bar_s[2], bar_p, bar_pv;
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = R + dr, panels = D >> 6;
  const uint32_t q_bytes = static_cast<uint32_t>(kRows) * D * 2, k_bytes = static_cast<uint32_t>(kKeys) * D * 2;
  constexpr uint32_t kQPanel = kRows * 128, kKPanel = kKeys * 128;      // bytes per 64-column panel

  const int* tile = tiles + 4 * blockIdx.x;
  const int tok0 = tile[0], ntok = tile[1], seq = tile[2];
  const int h0 = blockIdx.y * heads_per_tile;
  const int nh = min(heads_per_tile, H - h0);
  const int nrows = ntok * nh;
  const int ncg = (R + kColGroup - 1) / kColGroup;
  const int cg = blockIdx.z % ncg, split = blockIdx.z / ncg;
  const int col0 = cg * kColGroup, ncols = min(kColGroup, R - col0);
  const int* bt = block_tables + static_cast<long long>(seq) * max_blocks;
  const int k_begin = split * keys_per_split;
  const int k_end = min(positions[tok0 + ntok - 1] + 1, k_begin + keys_per_split);
  const int ntile = k_end > k_begin ? (k_end - k_begin + kKeys - 1) / kKeys : 0;

  __shared__ unsigned int seen_status;
  if (threadIdx.x == 0) seen_status = *reinterpret_cast<volatile unsigned int*>(&g_status);
  __syncthreads();
  if (seen_status != 0u) return;      // an earlier CTA gave up: do not queue up behind it (uniform over the CTA)
  if (ntile == 0) {        // a split past this tile's context: an empty partial (uniform over the CTA)
    if (partial != nullptr)
      for (int r = threadIdx.x; r < nrows; r += blockDim.x) {
        const long long base = static_cast<long long>(tok0 + r / nh) * H + h0 + r % nh;
        float* dst = partial + (base * nsplit + split) * (R + 2);
        for (int c = 0; c < ncols; ++c) dst[col0 + c] = 0.f;
        if (cg == 0) {
          dst[R] = -INFINITY;
          dst[R + 1] = 0.f;
        }
      }
    return;
  }

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  if (threadIdx.x == 0) {
    mbar_init(&bar_q, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_kfull[i], 1);
      mbar_init(&bar_kempty[i], 1);
      mbar_init(&bar_s[i], 1);
    }
    mbar_init(&bar_p, 128);
    mbar_init(&bar_pv, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
  }
  if (warp == 1) tmem_alloc<1>(&tmem_base_smem, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  volatile int* abort = &abort_flag;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(&bar_q, q_bytes);
      const int qcol0 = q_rows_are_heads ? 0 : h0 * D;
      const int qrow0 = q_rows_are_heads ? tok0 * H + h0 : tok0;
      for (int p = 0; p < panels; ++p) tma_load_2d(smem + p * kQPanel, &tmQ, &bar_q, qcol0 + 64 * p, qrow0);
      int issued = 0;
      auto slot_of = [&](int i) {
        const int j0 = k_begin + kKeys * i;
        return bt[j0 / block_size] * block_size + j0 % block_size;
      };
      int slot = slot_of(0);
      for (int i = 0; i < ntile; ++i) {
        const int st = i & 1;
        const int slot_next = i + 1 < ntile ? slot_of(i + 1) : 0;     // the page lookup overlaps the wait for the stage
        if (!wait_or_abort(&bar_kempty[st], ((i >> 1) & 1) ^ 1, abort, 1)) break;
        mbar_expect_tx(&bar_kfull[st], k_bytes);
        uint8_t* ks = smem + q_bytes + st * k_bytes;
        for (int p = 0; p < panels; ++p) tma_load_2d(ks + p * kKPanel, &tmK, &bar_kfull[st], 64 * p, slot);
        ++issued;
        slot = slot_next;
      }
      if (*abort) {      // let the copies in flight land before the CTA's shared memory is given back
        int none = 0;
        volatile int* never = &none;
        for (int b = 1; b <= 2 && b <= issued; ++b) wait_or_abort(&bar_kfull[(issued - b) & 1], ((issued - b) >> 1) & 1, never, 5);
        wait_or_abort(&bar_q, 0, never, 5);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(kRows, kKeys, 0u, 0u);
      const uint32_t idesc_pv = make_idesc_bf16(kRows, static_cast<uint32_t>(ncols), 0u, 1u);    // A from TMEM, B MN-major
      const uint32_t q_addr = smem_base;
      bool ok = wait_or_abort(&bar_q, 0, abort, 2);
      // Descriptors are linear in the start address (a 16-byte unit in their low bits), so the issue loop only adds:
      // one thread issues all 36 score products of a tile, and every scalar instruction between two of them is on the
      // critical path of the whole CTA.
      const uint64_t q_desc0 = make_smem_desc(q_addr, 16, 1024, 2);
      auto issue_s = [&](int i) {
        const int st = i & 1;
        tc_fence_after();
        const uint32_t d = tmem_base + kSCol + st * kKeys;
        uint64_t dq = q_desc0, dk = make_smem_desc(smem_base + q_bytes + st * k_bytes, 16, 1024, 2);
        for (int p = 0; p < panels; ++p) {
#pragma unroll
          for (int j = 0; j < 4; ++j) umma_ss<1>(d, dq + 2 * j, dk + 2 * j, idesc_s, (p | j) != 0 ? 1u : 0u);
          dq += kQPanel >> 4;
          dk += kKPanel >> 4;
        }
        umma_commit<1>(&bar_s[st]);
      };
      auto issue_pv = [&](int i) {
        tc_fence_after();
        const int st = i & 1;
        const uint32_t v_addr = smem_base + q_bytes + st * k_bytes + (col0 >> 6) * kKPanel;
        const uint32_t tP = tmem_base + kSCol + st * kKeys;
#pragma unroll
        for (int ks = 0; ks < kKeys / 16; ++ks)
          umma_ts<1>(tmem_base, tP + ks * 8, make_smem_desc(v_addr + ks * 2048, kKPanel, 1024, 2), idesc_pv,
                     (i | ks) != 0 ? 1u : 0u);
        umma_commit<1>(&bar_kempty[st]);      // the stage is free for tile i + 2 ...
        umma_commit<1>(&bar_pv);              // ... and O is complete up to tile i
      };
      // Whichever is ready goes first: the scores of the next tile (its keys have landed, and the value product that
      // last read its S / P buffer has been issued) or the value product of the oldest tile whose P is in place.
      // Issuing P V as soon as P is there frees the key stage early, so both stages' copies are in flight together.
      int next_s = 0, next_pv = 0;
      long long t0 = clock64();
      uint32_t spins = 0;
      while (ok && next_pv < ntile) {
        if (next_s < ntile && next_s <= next_pv + 1 && mbar_try_wait(&bar_kfull[next_s & 1], (next_s >> 1) & 1)) {
          issue_s(next_s++);
        } else if (next_s > next_pv && mbar_try_wait(&bar_p, next_pv & 1)) {
          issue_pv(next_pv++);
        } else {
          if ((++spins & 63u) == 0u) {
            if (*abort) break;
            if (clock64() - t0 > kWaitCycles) {
              *abort = 1;
              atomicCAS(&g_status, 0u, 0x100u | 3u);
              break;
            }
          }
          continue;
        }
        t0 = clock64();
        spins = 0;
      }
    }
  } else {
    // ------------------------------ softmax / epilogue (4 warps, a thread per query row) ------------------------------
    const int qd = warp & 3;                  // TMEM lane quadrant this warp may touch
    const int row = qd * 32 + lane;
    const bool valid = row < nrows;
    const int tok = tok0 + (valid ? row / nh : 0), h = h0 + (valid ? row % nh : 0);
    const int pos = valid ? positions[tok] : -1;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const float scale_log2 = scale * kLog2e;
    // a sink (a key without a value) is the row's initial (reference, sum) in the first slice of the keys
    const bool sink = sinks != nullptr && split == 0 && valid;
    float m_ref = sink ? sinks[h] * kLog2e : -INFINITY, l = sink ? 1.f : 0.f;
    bool ok = true;
    for (int i = 0; i < ntile; ++i) {
      const int st = i & 1;
      ok = __all_sync(0xffffffffu, wait_or_abort(&bar_s[st], (i >> 1) & 1, abort, 6));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tS = lane_base + kSCol + st * kKeys;
      uint32_t r[32];
      tmem_ld_x32(tS, r);
      tmem_ld_wait();
      const int vis = min(pos, k_end - 1) - (k_begin + kKeys * i) + 1;      // the first `vis` keys of the tile are visible
      float bm = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const float v = __uint_as_float(r[e]) * scale_log2;
        r[e] = __float_as_uint(v);
        if (e < vis) bm = fmaxf(bm, v);
      }
      // lazy reference: move it only when the tile's maximum outgrows it by more than 2^8
      const bool need = bm > m_ref + kRescaleThreshold;
      float alpha = 1.f;
      if (need) {
        alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - bm);
        m_ref = bm;
        l *= alpha;
      }
      const float neg = (m_ref == -INFINITY) ? 0.f : -m_ref;
      uint32_t pk[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        const float p0 = e < vis ? exp2f(__uint_as_float(r[e]) + neg) : 0.f;
        const float p1 = e + 1 < vis ? exp2f(__uint_as_float(r[e + 1]) + neg) : 0.f;
        l += p0 + p1;
        pk[e >> 1] = pack_bf16x2(p0, p1);
      }
      if (i > 0) {          // the previous value product is done: O may be rescaled, and is complete up to tile i - 1
        ok = __all_sync(0xffffffffu, wait_or_abort(&bar_pv, (i - 1) & 1, abort, 7));
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
          for (int c = 0; c < ncols; c += 32) {
            uint32_t o[32];
            tmem_ld_x32(lane_base + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_x16(lane_base + c, o);
            tmem_st_x16(lane_base + c + 16, o + 16);
          }
        }
      }
      tmem_st_x16(tS, pk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bar_p);
    }
    if (ok) {
      ok = __all_sync(0xffffffffu, wait_or_abort(&bar_pv, (ntile - 1) & 1, abort, 8));
      tc_fence_after();
    }
    if (ok) {
      const long long base = static_cast<long long>(tok) * H + h;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      float* pdst = partial != nullptr ? partial + (base * nsplit + split) * (R + 2) : nullptr;
#pragma unroll 1
      for (int c = 0; c < ncols; c += 32) {
        uint32_t o[32];
        tmem_ld_x32(lane_base + c, o);       // warp-collective: invalid rows read too, and store nothing
        tmem_ld_wait();
        if (!valid) continue;
        if (pdst != nullptr) {
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            *reinterpret_cast<float2*>(pdst + col0 + c + e) = make_float2(__uint_as_float(o[e]), __uint_as_float(o[e + 1]));
        } else {
          __nv_bfloat16* dst = out + base * R + col0 + c;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[g * 8 + e]) * inv;
            store8(dst + g * 8, pack8(f));
          }
        }
      }
      if (valid && pdst != nullptr && cg == 0) {
        pdst[R] = m_ref == -INFINITY ? -INFINITY : m_ref / kLog2e;
        pdst[R + 1] = l;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, t5::kTmemCols);
  }
}

// defined in latent_attention.cu: out[row, :] = sum over splits of the partial sums, renormalised
int launch_latent_attention_merge_bf16(const float* partial, void* out, int R, int splits, int rows, cudaStream_t s);

}  // namespace llmctl

using namespace llmctl;

// 1 if these sizes run on this kernel: bf16 only (the caller checks the type), D = R + dr and R multiples of 64 (whole
// 128-byte swizzle panels), query tile + two key tiles within shared memory, pages that hold whole 32-key tiles.
LLMCTL_API int llmctl_latent_attention_t5_ok(int R, int dr, int block_size) {
  const int D = R + dr;
  const size_t smem = static_cast<size_t>(t5::kRows + 2 * t5::kKeys) * D * 2 + 1024;
  return (R > 0 && R % 64 == 0 && D % 64 == 0 && block_size % t5::kKeys == 0 && smem <= 227 * 1024) ? 1 : 0;
}

// Status of the bounded waits since the last clearing call: 0 = none ran out.
LLMCTL_API int llmctl_latent_attention_t5_status(int clear) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, t5::g_status, sizeof(v)) != cudaSuccess) return -1;
  if (clear && v != 0) {
    const unsigned int zero = 0;
    (void)cudaMemcpyToSymbol(t5::g_status, &zero, sizeof(zero));
  }
  return static_cast<int>(v);
}

// tiles: int32 [ntiles, 4] = (first token row, tokens, block-table row, 0); a tile holds tokens x heads_per_tile <= 128
// query rows, and more than one head per tile only with single-token tiles.  qfull: bf16 scratch [tokens, H, R + dr].
// cache_rows: rows of the cache tensor (blocks x block_size).  partial: fp32 [tokens * H * splits * (R + 2)] when
// splits > 1.  ql as in llmctl_latent_attention.
LLMCTL_API int llmctl_latent_attention_t5(const void* ql, int ql_bf16, long long ql_st, long long ql_sh, const void* q,
                                          long long ldq, int dn, const void* cache, long long cache_rows,
                                          const int* block_tables, int max_blocks, int block_size, const int* tiles,
                                          int ntiles, int tokens, const int* positions, const float* freq, float mult,
                                          float scale, int H, int R, int dr, int heads_per_tile, int splits,
                                          int keys_per_split, void* qfull, void* out, float* partial, const float* sinks, void* stream) {
  LLMCTL_BEGIN();
  LLMCTL_REQUIRE(llmctl_latent_attention_t5_ok(R, dr, block_size) && H > 0 && heads_per_tile >= 1 &&
                 heads_per_tile <= t5::kRows && splits >= 1 && keys_per_split > 0 && keys_per_split % t5::kKeys == 0 &&
                 (splits == 1 || partial != nullptr) && qfull != nullptr && cache_rows >= block_size);
  if (ntiles == 0 || tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int D = R + dr;
  if (ql_bf16)
    latent_q_assemble_kernel<__nv_bfloat16><<<tokens * H, 128, 0, s>>>((const __nv_bfloat16*)ql, ql_st, ql_sh, (const __nv_bfloat16*)q,
                                                                        ldq, dn, positions, freq, mult, H, R, dr, (__nv_bfloat16*)qfull);
  else
    latent_q_assemble_kernel<float><<<tokens * H, 128, 0, s>>>((const float*)ql, ql_st, ql_sh, (const __nv_bfloat16*)q, ldq, dn,
                                                                positions, freq, mult, H, R, dr, (__nv_bfloat16*)qfull);
  const int rows_are_heads = heads_per_tile > 1 ? 1 : 0;
  CUtensorMap tmQ, tmK;
  int rc = rows_are_heads ? get_tmap_2d_bf16(&tmQ, qfull, static_cast<uint64_t>(tokens) * H, D, D, t5::kRows, 64, 1)
                          : get_tmap_2d_bf16(&tmQ, qfull, tokens, static_cast<uint64_t>(H) * D, static_cast<uint64_t>(H) * D, t5::kRows, 64, 1);
  if (rc) LLMCTL_FAIL(rc, "tensor map Q");
  rc = get_tmap_2d_bf16(&tmK, cache, cache_rows, D, D, t5::kKeys, 64, 1);
  if (rc) LLMCTL_FAIL(rc, "tensor map K");
  const int smem = (t5::kRows + 2 * t5::kKeys) * D * 2 + 1024;
  LLMCTL_CHECK(cudaFuncSetAttribute(latent_attention_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int ncg = (R + t5::kColGroup - 1) / t5::kColGroup;
  dim3 grid(ntiles, (H + heads_per_tile - 1) / heads_per_tile, splits * ncg);
  latent_attention_t5_kernel<<<grid, t5::kThreads, smem, s>>>(tmQ, tmK, block_tables, max_blocks, block_size, tiles, positions,
                                                               scale, H, R, dr, heads_per_tile, keys_per_split, splits,
                                                               rows_are_heads, (__nv_bfloat16*)out, splits > 1 ? partial : nullptr, sinks);
  if (splits > 1) {
    rc = launch_latent_attention_merge_bf16(partial, out, R, splits, tokens * H, s);
    if (rc) LLMCTL_FAIL(rc, "merge");
  }
  LLMCTL_RETURN_LAST();
}
