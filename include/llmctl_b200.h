/* C ABI of libllmctl_b200.so — hand-written sm_100a kernels.
 *
 * Conventions
 *   - every function returns a cudaError_t value as int (0 = success, 1 = invalid argument);
 *   - all device pointers are raw addresses, bf16 unless stated; `stream` is a cudaStream_t;
 *   - nothing here allocates device memory: outputs and scratch are passed in by the caller;
 *   - launches are asynchronous on `stream`.
 *
 * The reference repository ships no native code; the "Reference:" notes name the
 * library path the reference reaches for the same work.
 */
#ifndef LLMCTL_B200_H_
#define LLMCTL_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

/* ---- K3 norms.  Reference: ATen rms_norm/layer_norm inside HF modules (engine.py:284). ---- */
/* h = x (+ residual); y = h * rsqrt(mean(h^2) + eps) * w.  h_out/residual/rstd may be NULL. */
int llmctl_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* h_out, void* y,
                       float* rstd, int rows, int cols, float eps, void* stream);
/* dx = d(norm)/dh (+ dres); dw (fp32) (+)= sum_rows dy * xhat.
 * scratch: fp32 [scratch_rows * cols]; scratch_rows CTAs are used (1..rows). */
int llmctl_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd,
                       const void* dres, void* dx, float* dw, float* scratch, int scratch_rows,
                       int rows, int cols, int accumulate, void* stream);
/* RMSNorm backward for callers that cannot allocate device memory (a host runtime whose arena already owns the
 * whole device budget, or a latency-bound loop that must stay away from cudaMalloc's driver lock).  Same math
 * as llmctl_rmsnorm_bwd; the dw partials live in a 2 MiB array built into the library (held on every GPU that
 * loads it).  cols <= 8192 and a multiple of 8, else cudaErrorInvalidValue + llmctl_noalloc_last_error().  The
 * first call on a device resolves the array's address (do it before any stream capture).  Calls overlapping on
 * the GPU race on the shared array.  This entry point has no counterpart in the reference. */
int llmctl_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const float* rstd,
                               const void* dres, void* dx, float* dw, int rows, int cols, int accumulate,
                               void* stream);
const char* llmctl_noalloc_last_error(void);
int llmctl_layernorm_fwd(const void* x, const void* residual, const void* w, const void* b,
                         void* h_out, void* y, float* mean, float* rstd, int rows, int cols,
                         float eps, void* stream);
/* scratch: fp32 [2 * scratch_rows * cols] */
int llmctl_layernorm_bwd(const void* dy, const void* h, const void* w, const float* mean,
                         const float* rstd, const void* dres, void* dx, float* dw, float* db,
                         float* scratch, int scratch_rows, int rows, int cols, int accumulate,
                         void* stream);

/* ---- K4 RoPE (rotate-half), in place; sign=+1 forward, -1 backward.  Reference: HF rotary. ---- */
int llmctl_rope_inplace(void* x, long long row_stride, int n_tokens, int n_heads, int head_dim,
                        const float* cos_t, const float* sin_t, const int* positions, int seq_len,
                        float sign, void* stream);

/* ---- K5 SwiGLU on packed [M, 2F] gate|up.  Reference: ATen silu + mul. ---- */
int llmctl_swiglu_fwd(const void* gate_up, void* out, int M, int F, long long ld_gu, void* stream);
int llmctl_swiglu_bwd(const void* dout, const void* gate_up, void* d_gate_up, int M, int F,
                      long long ld_gu, void* stream);

/* ---- K9 fused AdamW + grad-norm pieces.  Reference: torch.optim.AdamW (engine.py:230-235),
 *      clip_grad_norm_ (engine.py:295-299). ---- */
int llmctl_adamw_step(void* master, void* m, void* v, const void* grad, int grad_is_fp32,
                      void* param_out, long long n, float lr, float beta1, float beta2, float eps,
                      float weight_decay, float bias_corr1, float bias_corr2, float host_scale,
                      const float* scale_dev, void* stream);
/* out (+)= sum(x^2); scratch: fp32 [scratch_elems] partial sums (deterministic two-stage). */
int llmctl_sumsq(const void* x, int is_fp32, long long n, float* scratch, int scratch_elems,
                 float* out, int accumulate, void* stream);

/* ---- K15 cross entropy (fused fwd+bwd, in-place gradient).  Reference: HF CrossEntropyLoss. ---- */
int llmctl_cross_entropy_fwd_bwd(void* logits, long long ld, const long long* targets,
                                 float* loss_per_row, float* lse_per_row, int rows, int V,
                                 long long ignore_index, float host_scale, const float* scale_dev,
                                 int write_grad, void* stream);
int llmctl_cross_entropy_partial(const void* logits, long long ld, const long long* targets,
                                 float* stats, int rows, int V_local, long long vocab_start,
                                 void* stream);
int llmctl_cross_entropy_finalize(void* logits, long long ld, const long long* targets,
                                  const float* lse, int rows, int V_local, long long vocab_start,
                                  long long ignore_index, float host_scale, const float* scale_dev,
                                  void* stream);

/* ---- K0 tcgen05/TMA GEMM.  Reference: cuBLAS via torch.matmul / nn.Linear. ----
 * D[M,N] = op(A) op(B) (+ D if beta).  a_mn=0: A is [M,K] row-major; a_mn=1: A stored [K,M].
 * b_mn=0: B is [N,K] row-major (Linear weight); b_mn=1: B stored [K,N].
 * out_fp32: D fp32 else bf16.  tile_n: 0 auto | 128 | 192 | 256 (single-CTA tiles) | 2 = 256x256 and 3 = 256x128 tile on a CTA pair
 * (cta_group::2); auto picks the 256x256 pair tile whenever M, N > 128.  max_ctas: 0 = all SMs. */
int llmctl_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                     long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32, int beta,
                     int tile_n, int max_ctas, void* stream);

/* ---- K13 / K12 paged KV cache.  Reference: none (server.py:199-204 recomputes the whole sequence). ----
 * caches: [num_blocks, block_size, heads, head_dim] bf16; slot = block * block_size + offset. */
int llmctl_kv_append(const void* qkv, long long row_stride, int k_off, int v_off, void* k_cache,
                     void* v_cache, const long long* slot_mapping, int num_tokens, int heads,
                     int head_dim, void* stream);
long long llmctl_paged_attn_scratch_elems(int batch, int heads, int head_dim, int num_splits);
/* scratch: fp32 [batch * heads * num_splits * (head_dim + 2)] split-K partials. */
int llmctl_paged_attn_decode(const void* q, long long q_stride, const void* k_cache,
                             const void* v_cache, const int* block_tables, int max_blocks_per_seq,
                             const int* context_lens, void* out, long long out_stride, float* scratch,
                             int batch, int heads, int head_dim, int block_size, int max_context,
                             int num_splits, float scale, void* stream);

/* ---- K14 sampling.  Reference: per-request Python loop with .item() syncs (server.py:209-235). ---- */
int llmctl_sample(const void* logits, int logits_is_fp32, long long ld, int rows, int V,
                  const float* temperature, const int* top_k, const float* top_p, const float* uniform,
                  long long* out_token, float* out_logprob, void* stream);

/* ---- K0s skinny (decode) GEMM: C[Mb,N] = X[Mb,K] W[N,K]^T, 1 <= Mb <= 32.  Swap-AB (UMMA M = 128 weight rows,
 * N = 16/32 token rows), split-K over CTAs with a deterministic in-kernel fix-up.  workspace: fp32 scratch;
 * counters: >= ceil(N/128) zeroed uint32 tickets (left zero on return); one call at a time per pair.
 * Reference: cuBLAS inside the HF model (server.py:199-204). */
int llmctl_gemm_skinny_bf16(const void* X, const void* W, void* C, int Mb, int N, int K, long long ldx,
                            long long ldw, long long ldc, float* workspace, long long workspace_elems,
                            unsigned int* counters, int n_counters, int splits, void* stream);

/* ---- K6 causal flash attention, head_dim 128, bf16.  q/k/v/o: [B,S,H,128] views with token strides in
 * elements; lse: fp32 [B,H,S] (natural log).  S % 128 == 0.  Reference: SDPA/eager inside the HF model
 * (engine.py:284); baseline cuDNN SDPA.
 * Forward: 256 queries per CTA as two tiles sharing K/V, S/P/O in TMEM, P never leaves TMEM.
 * Backward: two deterministic kernels (dK/dV on transposed scores, then dQ); scratch >= 2*B*H*S floats
 * (the single-kernel atomic variant selected by LLMCTL_FLASH_BWD_V1 needs B*S*H*129). */
int llmctl_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int H,
                          int D, long long q_tok_stride, long long k_tok_stride, long long v_tok_stride,
                          long long o_tok_stride, float scale, int causal, void* stream);
int llmctl_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                          const float* lse, void* dq, void* dk, void* dv, float* scratch, int B, int S, int H,
                          int D, long long q_tok_stride, long long k_tok_stride, long long v_tok_stride,
                          long long o_tok_stride, long long dqkv_tok_stride, float scale, int causal, void* stream);
/* In-kernel timeline of the forward's CTA 0 (only recorded when LLMCTL_FLASH_TRACE is set in the environment):
 * copies the 2048-word (clock64, event) log to host_out (synchronous); read with tools/trace_flash.py.  Returns a
 * cudaError_t value: 0 = ok, cudaErrorNotReady when tracing is off. */
int llmctl_flash_trace_read(long long* host_out);

/* ---- Peer-memory (NVLink 5 / NVSwitch) kernels.  No counterpart in the reference (llmctl/comms is empty).
 * llmctl_peer_table: base pointers of one symmetric allocation on every rank of the group (unused = NULL);
 * `pads` is the table of per-rank signal pads (uint32 flags); `epoch` must increase by one per call on every
 * rank for a given slot range.  A wait that exceeds the watchdog deadline gives up and is reported by
 * llmctl_comm_watchdog_poll instead of hanging the GPU. */
typedef struct { void* ptr[8]; } llmctl_peer_table;

/* stand-alone collectives on a symmetric bf16 workspace (pad slots [slot, slot + world)) */
int llmctl_allgather_pull(llmctl_peer_table buf, long long chunk_bytes, llmctl_peer_table pads, int slot, int rank,
                          int world, unsigned int epoch, int max_ctas, void* stream);
int llmctl_reduce_scatter_pull(llmctl_peer_table in, long long n_per_rank, void* out, llmctl_peer_table pads,
                               int slot, int rank, int world, unsigned int epoch, int max_ctas, void* stream);
int llmctl_allreduce_oneshot(llmctl_peer_table in, long long n, void* out, llmctl_peer_table pads, int slot,
                             int rank, int world, unsigned int epoch, int max_ctas, void* stream);
int llmctl_allreduce_multimem(void* mc, long long n, llmctl_peer_table pads, int slot, int rank, int world,
                              unsigned int epoch, int max_ctas, void* stream);   /* NVLS multimem.ld_reduce/st */

/* K1: sequence-parallel all-gather -> GEMM.  The owner pushes its rows into every rank's symmetric buffer
 * (llmctl_ag_push: NVLS multimem.st when mc_xg != NULL, else P2P stores) slab by slab and raises per-slab epoch flags
 * at pads[*][flag_base + row / rows_per_flag]; the consumer is the tcgen05 GEMM whose TMA producer waits per tile for
 * the flags of the rows it reads (llmctl_gemm_bf16_gated; flags = this rank's pad + flag_base). counters: >= 32
 * zeroed uint32 in local memory. */
/* K8: GEMM whose B operand (a ZeRO-3 parameter matrix inside a gather buffer that its shard owners are still filling
 * with llmctl_ag_push) is consumed as it arrives: before a tile's weight rows are loaded, the flags
 * b_flags[(b_off + element) / b_slab] must have reached `epoch`.  llmctl_signal_all / llmctl_signal_wait hand a gather
 * buffer back and forth between its readers and its next writers. */
int llmctl_gemm_bf16_bgated(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int a_mn, int b_mn, int out_fp32, int beta, int tile_n, int max_ctas,
                            const unsigned int* b_flags, unsigned int epoch, long long b_off, long long b_slab,
                            void* stream);
int llmctl_signal_all(llmctl_peer_table pads, int rank, int world, int slot, unsigned int epoch, void* stream);
int llmctl_ag_gemm(llmctl_peer_table xg, void* mc_xg, const void* W, void* Y, int M, int N, int K, long long ldw,
                   long long ldy, int w_mn, int rows_per_flag, llmctl_peer_table pads, int flag_base, int rank,
                   int world, unsigned int epoch, unsigned int* counters, int push_ctas, int tile_n,
                   void* push_stream, void* stream);   /* push (side stream) + gated GEMM in one call */
int llmctl_ag_push(const void* src, llmctl_peer_table xg, void* mc_xg, int rows, int cols, int rows_per_flag,
                   llmctl_peer_table pads, int flag_base, int rank, int world, unsigned int epoch,
                   unsigned int* counters, int src_in_xg, int max_ctas, void* stream);
int llmctl_gemm_bf16_gated(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, int b_mn, int out_fp32, int beta, int tile_n, int max_ctas,
                           const unsigned int* flags, unsigned int epoch, int rows_per_flag, int rank, int world,
                           void* stream);
/* K2: row-parallel GEMM whose epilogue pushes bf16 tiles into the owner's staging slot; finished by
 * llmctl_rs_reduce_rmsnorm (sum of the world slots + residual (+ RMSNorm)) on the sequence shard. */
int llmctl_gemm_rs(const void* X, const void* W, llmctl_peer_table stage, int M, int N, int K, long long ldx,
                   long long ldw, int w_mn /* W stored [K, N] */, llmctl_peer_table pads, unsigned int* local_flags,
                   int rank, int world, unsigned int epoch, void* stream);
int llmctl_rs_reduce_rmsnorm(const void* stage_local, llmctl_peer_table pads, int rank, int world,
                             const void* residual, const void* w, void* h_out, void* y, float* rstd, int rows,
                             int cols, float eps, unsigned int epoch, void* stream);
/* K7: ZeRO gradient reduce-scatter of this rank's slice (in-switch multimem.ld_reduce when mc_grads != NULL,
 * else rank-ordered P2P pull) + squared-norm partial; then AdamW on the shard + publication of the updated
 * parameters (NVLS multimem.st when mc_params != NULL, else P2P stores; push = 0 writes local_out only).
 * done_slot >= 0 announces "finished reading this bucket" to every rank; the bucket's next writer waits for it
 * with llmctl_signal_wait (transient ZeRO-2/3 buckets). */
int llmctl_rs_sumsq(llmctl_peer_table grads, long long bucket_off, const void* mc_grads, llmctl_peer_table pads,
                    int rank, int world, long long shard_lo, long long shard_n, float* reduced, int accumulate_out,
                    float* scratch, int scratch_elems, float* sumsq_out, int accumulate_sumsq, unsigned int epoch,
                    int done_slot, unsigned int done_epoch, int max_ctas, void* stream);
int llmctl_signal_wait(llmctl_peer_table pads, int rank, int world, int slot, unsigned int epoch, void* stream);
int llmctl_adam_allgather(llmctl_peer_table params, long long bucket_off, void* mc_params, llmctl_peer_table pads,
                          llmctl_peer_table scalars, const float* total_sq_dev, int rank, int world,
                          long long shard_lo, long long shard_n, float* master, float* m, float* v,
                          const float* reduced, void* local_out, int push, float lr, float beta1, float beta2,
                          float eps, float weight_decay, float bias_corr1, float bias_corr2, float grad_scale,
                          float max_norm, float* norm_out, unsigned int epoch_begin, int begin_barrier,
                          unsigned int epoch_end, int end_barrier, int max_ctas, void* stream);
/* K11: decode all-reduce of [rows, cols] partial sums + residual add + RMSNorm in one launch. */
int llmctl_ar_residual_rmsnorm(llmctl_peer_table x, long long x_off, const void* mc_x, llmctl_peer_table pads,
                               int slot_base, int rank, int world, const void* residual, void* h_out,
                               const void* w, void* y_out, int rows, int cols, float eps, unsigned int epoch,
                               const unsigned int* step_counter /* optional: epoch += *step_counter * calls_per_step */,
                               unsigned int calls_per_step, void* stream);
int llmctl_counter_add(unsigned int* counter, unsigned int value, void* stream);
/* watchdog: out[0] timed-out waits since the last clearing poll, out[1..6] = expected epoch, value seen,
 * blockIdx.x, flag address, ns waited, module index of the first one (out must hold 8 values). */
int llmctl_comm_watchdog_poll(unsigned long long* out, char* module_name, int name_cap, int clear);
int llmctl_comm_watchdog_set_timeout_ms(unsigned long long ms);
int llmctl_comm_watchdog_modules(void);

/* ---- Ragged-batch inference models (latent attention, post-norm residual, mixture of experts).  bf16 or fp32
 * activations (is_fp32 / *_fp32 flags); norms, scores, routing, sums and the residual stream are fp32.
 * Reference: none (the reference has no model code). ---- */
/* x += gain * rmsnorm(y) on the fp32 stream; x_act receives the stream rounded to the activation type. */
int llmctl_postnorm_residual(const void* y, int y_fp32, long long ldy, float* x, void* x_act, int act_fp32,
                             const float* gain, int rows, int cols, float eps, void* stream);
int llmctl_scalar_rmsnorm(const float* x, const long long* rows, void* out, int out_fp32, const float* gain, int n_out,
                          int cols, float eps, void* stream);
int llmctl_embed_scale(const long long* tokens, const void* table, int is_fp32, float scale, float* x, void* x_act,
                       int rows, int cols, void* stream);
int llmctl_softcap(float* v, long long n, float cap, void* stream);
int llmctl_xielu(const void* z, void* out, int is_fp32, long long n, float a_pos, float a_neg, void* stream);
int llmctl_gated_silu(const void* gate_up, long long ld, void* out, int is_fp32, int rows, int F, void* stream);
/* d: [tokens, Q + R + dr] packed down-projections.  cq = rmsnorm(d[:, :Q]) * wq; the cache row of every token (slots)
 * receives [rmsnorm(d[:, Q:Q+R]) * wkv | interleaved-pair rotation of d[:, Q+R:] at its position]. */
int llmctl_latent_kv_write(const void* d, long long ld, int Q, int R, int dr, const void* wq, const void* wkv, void* cq,
                           void* cache, const long long* slots, const int* positions, const float* freq, float mult,
                           float eps, int tokens, int is_fp32, void* stream);
int llmctl_latent_attention_uses_tensor_cores(int is_fp32, int R, int dr, int rows_per_tile);
/* Attention of absorbed queries over the paged latent cache (see csrc/attention/latent_attention.cu). */
int llmctl_latent_attention(const void* ql, int ql_bf16, long long ql_st, long long ql_sh, const void* q, long long ldq,
                            int dn, const void* cache, const int* block_tables, int max_blocks, int block_size,
                            const int* tiles, int ntiles, int tokens, const int* positions, const float* freq, float mult,
                            float scale, int H, int R, int dr, int heads_per_tile, int splits, int keys_per_split,
                            void* out, float* partial, int is_fp32, int tensor_cores, int rows_per_tile,
                            const float* sinks /* fp32 [H] or null: exp(sinks[h]) joins head h's softmax denominator */, void* stream);
/* The tcgen05 kernel (128-row query tiles): sizes that qualify, status of its bounded waits, and the launch.
 * qfull: bf16 scratch [tokens, H, R + dr]; cache_rows = blocks x block_size. */
int llmctl_latent_attention_t5_ok(int R, int dr, int block_size);
int llmctl_latent_attention_t5_status(int clear);
int llmctl_latent_attention_t5(const void* ql, int ql_bf16, long long ql_st, long long ql_sh, const void* q, long long ldq,
                               int dn, const void* cache, long long cache_rows, const int* block_tables, int max_blocks,
                               int block_size, const int* tiles, int ntiles, int tokens, const int* positions,
                               const float* freq, float mult, float scale, int H, int R, int dr, int heads_per_tile,
                               int splits, int keys_per_split, void* qfull, void* out, float* partial, const float* sinks, void* stream);
int llmctl_moe_tile_rows(void);
/* correction: fp32 [E] added to the scores for the CHOICE only, or null; n_groups > 1: only experts of the keep_groups
 * best groups (of E / n_groups neighbours each) can be chosen.  Ids >= the E given to plan / permute are identity
 * experts. */
int llmctl_moe_route(const float* x, const void* wr, const void* wg, int is_fp32, int tokens, int W, int E, int top,
                     int softmax_scores, int renormalise, const float* correction, int n_groups, int keep_groups, int* ids,
                     float* weights, float* gate, int* counts, void* stream);
/* meta: int32 [2 E + 2 + max_tiles] = { segment offsets[E] | cursors[E] | tiles | padded rows | tile -> expert }. */
int llmctl_moe_plan(const int* counts, int E, int* meta, int max_tiles, int tile_rows, void* stream);
int llmctl_moe_permute(const float* x, int W, const int* ids, const float* weights, int scale_input, int* meta, int E,
                       int* pair_row, void* xs, int is_fp32, int tokens, int top, void* stream);
int llmctl_grouped_gemm(const void* A, long long lda, const void* Wt, void* out, long long ldo, int N, int K,
                        const int* meta, int E, int max_tiles, int is_fp32, void* stream);
/* The tcgen05 GEMM over 128-row blocks of A, block i against expert tile_expert[i]'s [N, K] matrix. */
int llmctl_gemm_bf16_grouped(const void* A, const void* W, void* C, int max_tiles, int N, int K, long long lda,
                             long long ldc, const int* tile_expert, const int* num_tiles, int experts, void* stream);
/* identity_in: fp32 [tokens, W], what an identity expert (pair_row < 0) returns times its weight; null without them. */
int llmctl_moe_combine(const void* expert_out, int W, const int* pair_row, const float* weights, int top,
                       int scale_output, const void* shared_out, const float* gate, const float* identity_in, float* y,
                       int tokens, int is_fp32, void* stream);
int llmctl_gated_clamped(const void* gate_up, long long ld, void* out, int is_fp32, int rows, int F, float limit, float alpha,
                         void* stream);

/* ---- sandwich-norm layout and pooled-window attention (csrc/norm/sandwich_norm.cu, csrc/activation/xielu.cu,
 *      csrc/attention/pooled_window_attention.cu) ---- */
int llmctl_relu_squared(const void* z, void* out, int is_fp32, long long n, void* stream);
/* x[t] = table[tokens[t]] + pos_table[positions[t]] in fp32. */
int llmctl_embed_positions(const long long* tokens, const int* positions, const void* table, const void* pos_table,
                           int is_fp32, float* x, int rows, int cols, void* stream);
/* out[r] = w * x[rows[r]] / rms(x[rows[r]]); rows may be null (rows 0..n_out-1); x and w fp32. */
int llmctl_rmsnorm_rows(const float* x, const long long* rows, const float* w, void* out, int out_fp32, int n_out, int cols,
                        float eps, void* stream);
/* x += wb * y / rms(y) on the fp32 stream; with w_next also out = w_next * x / rms(x) of the new stream. */
int llmctl_sandwich_residual(const void* y, int y_fp32, long long ldy, float* x, const float* wb, const float* w_next,
                             void* out, int out_fp32, float* out32, int rows, int cols, float eps, void* stream);
/* Packed projection [q | k | v] -> fp32 queries and the token's cache row: bias, RMS norm over the whole q / k
 * projection, rotation of the first `rot` numbers of every head, value mixing (v_mode 1: publish v_first, 2: blend). */
int llmctl_window_qkv_write(const void* qkv, long long ld, const void* bias, const float* qn_w, const float* kn_w, int H,
                            int G, int d, int e, int rot, const float* freq, float mult, float eps, const int* positions,
                            const long long* slots, float* q_out, void* cache, int bs, int PS, void* v_first, int v_mode,
                            const float* lam, int tokens, int is_fp32, void* stream);
/* Pooled rows (means of P cached rows) of the blocks that the step's tokens complete. */
int llmctl_window_pool_update(void* cache, const int* positions, const long long* slots, const int* seq_rows,
                              const int* block_tables, int max_blocks, int bs, int PS, int P, int Wc, int tokens,
                              int is_fp32, void* stream);
int llmctl_pooled_window_attention_rows(int H, int d, int e, int tile_tokens);
/* Attention over a window of S tokens and the pooled rows of the blocks before it; temp / talk may be null. */
int llmctl_pooled_window_attention(const float* q, const void* cache, const int* block_tables, int max_blocks,
                                   const int* tiles, int ntiles, int tile_tokens, const int* positions, const float* temp,
                                   const float* talk, float scale, int H, int G, int d, int e, int S, int P, int bs, int PS,
                                   void* out, int is_fp32, void* stream);
/* The same on mma.sync tensor cores (bf16 cache and output); _ok says whether the sizes fit. */
int llmctl_pooled_window_attention_mma_ok(int H, int G, int d, int e, int tile_tokens);
int llmctl_pooled_window_attention_mma(const float* q, const void* cache, const int* block_tables, int max_blocks,
                                       const int* tiles, int ntiles, int tile_tokens, const int* positions,
                                       const float* temp, const float* talk, float scale, int H, int G, int d, int e, int S,
                                       int P, int bs, int PS, void* out, int splits, int tokens, float* part_ml,
                                       float* part_o, void* stream);

/* ---- parallel residual layout, differential attention, recurrent mixers (csrc/norm/parallel_norm.cu,
 *      csrc/attention/diff_attention.cu, csrc/recurrent/gla.cu, csrc/recurrent/selective_scan.cu) ---- */
/* Optional x[row] += add in place, then layer norm (weight, bias) of all rows or of `rows`; out32: unrounded copy or null. */
int llmctl_layernorm_rows(float* x, const long long* rows, const float* add, const float* w, const float* b, void* out,
                          int out_fp32, float* out32, int n, int W, float eps, void* stream);
/* x += mult * (a + f) (+ add) in place; with w/b also the layer norm of the new rows. */
int llmctl_parallel_residual(const void* a, int a_fp32, long long lda, const float* f, float* x, float mult, const float* add,
                             const float* w, const float* b, void* out, int out_fp32, float* out32, int T, int W, float eps,
                             void* stream);
/* Rotates the first `rot` numbers of each of nq query and nk key vectors of d numbers; q -> fp32, [k | v] -> cache row. */
int llmctl_rotary_kv_append(const void* proj, long long ld, int nq, int nk, int d, int nv, int rot, const float* freq,
                            float mult, const int* positions, const long long* slots, float* q_out, void* cache, int tokens,
                            int is_fp32, void* stream);
int llmctl_diff_attention_heads_per_cta(int H, int G, int tile_tokens);
/* Two softmax maps per head over shared values: o = a1 - lambda a2, unit RMS, * post_scale * sigmoid(gate). */
int llmctl_diff_attention(const float* q, const void* cache, const int* block_tables, int max_blocks, const int* tiles,
                          int ntiles, int tile_tokens, const int* positions, const void* gate, long long gate_ld, float scale,
                          float lambda, float post_scale, float eps, int H, int G, int d, int e, int bs, void* out, int splits,
                          float* part_ml, float* part_o, int is_fp32, int use_mma, void* stream);
int llmctl_diff_attention_mma_ok(int H, int G, int d, int e, int tile_tokens);
/* portions: int32 [n, 4] = (first token row, tokens, position of the first token, state slot). */
int llmctl_gla_scan(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv, const void* z,
                    long long ldz, const float* z_bias, const int* portions, int nportions, int tokens, float* state, float* out,
                    float* work /* fp32 [tokens, 3 H d] scratch */, int H, int d, int e, float q_scale, float tau, int is_fp32,
                    void* stream);
int llmctl_gla_output(const float* o, const float* w, const void* gate, long long ldg, void* out, int tokens, int H, int e,
                      float eps, int is_fp32, void* stream);
int llmctl_causal_conv_silu(const void* x, long long ldx, const float* w, const float* wb, const int* portions,
                            const int* seq_rows, const float* conv_state, void* out, int tokens, int C, int taps, int is_fp32,
                            void* stream);
int llmctl_selective_scan(const void* u, const void* bc, long long ldbc, int off_b, int off_c, const void* dtp, long long lddt,
                          const float* dt_bias, const float* A, const float* D, const void* z, long long ldz, const void* x,
                          long long ldx, const int* portions, int nportions, float* state, float* conv_state, void* out, int C,
                          int N, int taps, int is_fp32, void* stream);

/* ---- pre-norm with an input convolution, soft-capped window attention (csrc/norm/canon_norm.cu,
 *      csrc/attention/softcap_window_attention.cu, csrc/activation/xielu.cu) ---- */
/* x += a + f in place (each optional, bf16 or fp32); r[row] = 1 / sqrt(mean(x[row]^2) + eps). */
int llmctl_residual_rms(const void* a, int a_is_fp32, long long lda, const void* f, int f_is_fp32, long long ldf, float* x,
                        float* r, int tokens, int W, float eps, void* stream);
/* out_s = h_s + causal depthwise conv(h_s) over time, h_s = norm_w_s * x * r, for S = 1 or 2 sublayers; state: fp32
 * [slots, taps - 1, W], the last unweighted normed rows of every sequence (read, then rewritten by a second launch). */
int llmctl_norm_canon(const float* x, const float* r, int S, const float* norm_w0, const float* conv_w0, void* out0,
                      const float* norm_w1, const float* conv_w1, void* out1, const int* portions, int nportions,
                      const int* seq_rows, float* state, int tokens, int W, int taps, int out_is_fp32, void* stream);
/* llmctl_residual_rms + llmctl_norm_canon in one launch for portions of at most 8 tokens each (one block per portion). */
int llmctl_residual_norm_canon_small(const void* a, int a_is_fp32, long long lda, const void* f, int f_is_fp32, long long ldf, float* x,
                                     float eps, int S, const float* norm_w0, const float* conv_w0, void* out0, const float* norm_w1,
                                     const float* conv_w1, void* out1, const int* portions, int nportions, float* state, int W, int taps,
                                     int out_is_fp32, void* stream);
int llmctl_gated_gelu_tanh(const void* gate_up, long long ld, void* out, int is_fp32, int rows, int F, void* stream);
int llmctl_sigmoid_gate(void* y, const void* z, long long ldz, int is_fp32, int rows, int F, void* stream);
/* fp32 biases (or null), optional unit-RMS norm of every value head; q -> fp32, [k | v] -> cache row. */
int llmctl_window_kv_append(const void* proj, long long ld, const float* bias, int H, int G, int d, int e, int value_norm,
                            float eps, const long long* slots, float* q_out, void* cache, int tokens, int is_fp32, void* stream);
int llmctl_softcap_attention_heads_per_cta(int H, int G, int tile_tokens, int use_mma);
int llmctl_softcap_attention_mma_ok(int H, int G, int d, int e, int tile_tokens);
/* Sliding window (0: none) with kept first tokens, tanh soft cap (0: none), per-head distance slopes and sinks (null:
 * none), sigmoid output gate (null: none). */
int llmctl_softcap_window_attention(const float* q, const void* cache, const int* block_tables, int max_blocks, const int* tiles,
                                    int ntiles, int tile_tokens, const int* positions, const void* gate, long long gate_ld,
                                    const float* slopes, const float* sinks, float scale, float cap, int window, int keep_first,
                                    int H, int G, int d, int e, int bs, void* out, int splits, float* part_ml, float* part_o,
                                    int is_fp32, int use_mma, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LLMCTL_B200_H_ */
