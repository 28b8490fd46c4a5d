/* C ABI of libjllama_b200.so — hand-written sm_100a kernels for LLaMA inference on NVIDIA B200.
 *
 * Conventions
 *  - every entry point returns 0 on success, non-zero on failure; jl_last_error() describes the failure;
 *  - `stream` is a cudaStream_t passed as void*; launches are asynchronous on it and are legal inside
 *    CUDA-graph stream capture unless stated otherwise;
 *  - activations / weights are bf16, row-major; linear weights are [N, K] (out, in) i.e. K-major;
 *  - kernels are launched with Programmatic Dependent Launch enabled and are safe in PDL chains.
 *
 * Each declaration cites the reference op it replaces (paths under /root/reference/jax_llama/).
 */
#ifndef JLLAMA_B200_H
#define JLLAMA_B200_H
#include <stddef.h>
#ifndef JL_API
#define JL_API __attribute__((visibility("default")))
#endif
#ifdef __cplusplus
extern "C" {
#endif

const char* jl_last_error(void);
int jl_version(void);
/* number of kernel launches issued through this library since load (bench.py reports it) */
unsigned long long jl_launch_count(void);

/* model.py:611-617,638 — embedding lookup. ids int32 [M]; table [V,H]; out [M,H]. */
int jl_embed(const int* ids, const void* table, void* out, int M, int H, int V, void* stream);

/* model.py:42-48 — RMSNorm over rows of x [M,H]; optional fused residual add: if `delta` is given the
 * row normalised is x+delta and (if x_out != NULL) the sum is stored to x_out (may alias x). */
int jl_rmsnorm(const void* x, const void* delta, const void* w, void* out, void* x_out, int M, int H,
               float eps, void* stream);

/* model.py:58-92 + 177-199 — interleaved-pair RoPE on the q|k column blocks of the fused qkv activation
 * [B*S, (nh+2nkv)*hd] and append of k,v to this layer's cache [B][nkv][T][hd].  Token (b,s) goes to slot
 * *cache_len_ptr + s at rotary position slot - pad_left[b] (or positions[b*S+s] if given).  q is rotated
 * in place, or written to q_out [B*S, nh*hd] when q_out != NULL. */
int jl_rope_kv_write(void* qkv, void* q_out, void* k_cache, void* v_cache, const float* cos_t,
                     const float* sin_t, const int* cache_len_ptr, const int* pad_left, const int* positions,
                     int B, int S, int nh, int nkv, int hd, int T, int max_pos, void* stream);

/* model.py:338 — silu(gate)*up.  in [M,2F] (interleaved pairs if `interleaved`, else two halves). */
int jl_swiglu(const void* in, void* out, int M, int F, int interleaved, void* stream);

/* model.py:119-150,311-338,699-706 at decode — y = f(x) W^T for M <= 8 rows, weight-streaming bound.
 * norm_w != NULL fuses RMSNorm(x)*norm_w; mode 0 plain, 1 out = residual + y, 2 SwiGLU over interleaved
 * (w1,w3) rows (out is [M,N/2]); out_f32 selects fp32 output (plain mode). */
int jl_gemv(const void* x, const void* w, const void* norm_w, const void* residual, void* out, int M, int N,
            int K, float eps, int mode, int out_f32, int num_sms, void* stream);

/* jl_gemv for M <= 4 with the weights streamed by TMA bulk copies (cp.async.bulk + mbarrier) through a
 * shared-memory ring that starts filling before the programmatic-dependent-launch wait.  Returns 3
 * (unsupported, nothing launched) when the activations leave no room for the ring: call jl_gemv then. */
int jl_gemv_tma(const void* x, const void* w, const void* norm_w, const void* residual, void* out, int M, int N,
                int K, float eps, int mode, int out_f32, int num_sms, void* stream);

/* Same linear layers for any M on the tcgen05 tensor cores (TMA-fed, TMEM accumulators).  M > 128 runs
 * token-major tiles (prefill); M <= 128 runs swap-AB so the weight rows fill the 128-wide MMA and the
 * batch is the MMA N (decode at batch 9..128).  Modes / out_f32 as in jl_gemv.  N % 8 == 0, K % 8 == 0;
 * SwiGLU needs N % 16 == 0. */
int jl_gemm(const void* x, const void* w, const void* residual, void* out, int M, int N, int K, int mode,
            int out_f32, int num_sms, void* stream);
/* Optional scratch for jl_gemm on the CURRENT device: with it, small-batch (M <= 128) launches that have fewer
 * 128-row weight tiles than half the SMs (N = 4096: 32 tiles) split K over the idle SMs; partial sums meet in `ws`
 * (fp32, ws_bytes); once all splits of a tile have arrived (`tickets`: n_tickets ints, zero on entry and between
 * calls, half of them arrival and half completion counters) each split adds the partials of its share of the tokens
 * in split order and runs the epilogue — results do not depend on arrival order.  The splits of a tile wait for each
 * other, so such a launch needs its CTAs resident together (at most one per SM is launched).  The caller owns both
 * buffers and keeps them alive; ws == NULL unregisters.  Calls that share the scratch must be ordered on one stream. */
int jl_gemm_set_workspace(void* ws, size_t ws_bytes, int* tickets, int n_tickets);
/* Timeline hook of the single-CTA GEMM kernel for scripts/gemm_trace.py: [grid][16] u64 device buffer of
 * %globaltimer stamps, NULL = off (default). */
void jl_gemm_set_trace(void* buf);

/* model.py:194-198,263-288 at S=1 — split-KV GQA decode attention over [pad_left[b], *cache_len+n_new).
 * q [B,nh,hd] with batch pitch q_bstride elements (0 = dense; lets q live inside the fused qkv
 * activation); caches [B][nkv][T][hd]; out [B,nh*hd].  `scratch` must hold
 * jl_decode_attn_scratch_bytes(B,nh,hd,splits) bytes when splits > 1. */
size_t jl_decode_attn_scratch_bytes(int B, int nh, int hd, int splits);
int jl_decode_attn_splits(int B, int nkv, int max_len, int num_sms);
int jl_decode_attn(const void* q, const void* k_cache, const void* v_cache, const int* cache_len_ptr,
                   const int* pad_left, void* scratch, void* out, int B, int nh, int nkv, int hd, int T,
                   int n_new, float scale, int splits, int q_bstride, void* stream);

/* model.py:201-300 at S=1 in ONE launch — RoPE of q and of the new token's k, append of (k,v) at slot
 * *cache_len, split-KV GQA attention over [pad_left[b], *cache_len] and the split merge (last-arriving CTA,
 * atomic ticket).  qkv [B,(nh+2nkv)*hd] is the un-rotated fused projection; out [B,nh*hd].  `scratch` must
 * hold jl_decode_attn_fused_scratch_bytes(...) bytes and be ZERO when first used (ticket counters; the kernel
 * leaves them zero).  *cache_len is not advanced here. */
size_t jl_decode_attn_fused_scratch_bytes(int B, int nh, int nkv, int hd, int splits);
int jl_decode_attn_fused_splits(int B, int nkv, int max_len, int num_sms);
int jl_decode_attn_fused(const void* qkv, void* k_cache, void* v_cache, const float* cos_t, const float* sin_t,
                         const int* cache_len_ptr, const int* pad_left, void* scratch, void* out, int B, int nh,
                         int nkv, int hd, int T, int max_pos, float scale, int splits, void* stream);
/* Two kernels stand behind jl_decode_attn_fused: a SIMT one with many short splits (lowest latency at batch 1) and,
 * for head_dim 128 with batch * nkv >= 16, a tensor-core one (mma.sync, K/V from global memory straight into MMA
 * fragments) that streams the cache ~3x faster at batch 16-64.  variant: 0 = choose by shape, 1 = SIMT, 2 = tensor
 * core (where it applies).  Process-wide; meant for tests and A/B measurements. */
int jl_decode_attn_fused_set_variant(int variant);

/* No counterpart in the reference: an allocation-free form of jl_decode_attn for callers that cannot get
 * device memory themselves (HBM fully owned by another runtime's arena, hosts that ban cudaMalloc/cudaFree
 * inside the token loop, bare C callers without an allocator).  Same arguments minus `scratch`: the split-KV
 * workspace is a fixed 4 MiB array inside the library image, resident on every GPU that loads the library
 * until process exit.  B*nh*splits*(hd+2) floats must not exceed jl_decode_attn_noalloc_max_floats();
 * otherwise the call fails with a message naming the limit.  It calls no allocating routine.  The first call
 * on each device looks the array's address up — do it before any stream capture.  All calls share the array
 * (it keeps the previous call's contents; nothing needs zeroing), so calls that may overlap on the GPU race:
 * keep them on one stream.  Output equals jl_decode_attn's for the same `splits`. */
size_t jl_decode_attn_noalloc_max_floats(void);
int jl_decode_attn_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* cache_len_ptr,
                           const int* pad_left, void* out, int B, int nh, int nkv, int hd, int T, int n_new,
                           float scale, int splits, int q_bstride, void* stream);

/* model.py:236-288 at S>1 — causal flash attention of S new tokens per row (cache slots start..start+S,
 * already appended) on tcgen05: q [B*S, nh*hd] rotated, caches [B][nkv][T][hd], out [B*S, nh*hd].
 * Keys [pad_left[b], slot of the query] are visible.  head_dim 128 only.  cache_len_ptr is reserved. */
int jl_flash_prefill_occupancy(int smem_override /* -1 */); /* resident CTAs per SM (diagnostic; 2 expected) */
int jl_flash_prefill(const void* q, const void* k_cache, const void* v_cache, const int* cache_len_ptr,
                     const int* pad_left, void* out, int B, int S, int nh, int nkv, int hd, int T, int start,
                     float scale, void* stream);
/* Same contract on warp-level tensor cores (mma.sync, K / V from global memory straight into fragments, one warp per
 * 16 query rows): head_dim 64 and 128.  jl_flash_prefill routes head_dim 64 here (model.py:115 allows any
 * hidden / heads; the 1B-class LLaMA-architecture models have 64-wide heads). */
int jl_prefill_attn_mma(const void* q, const void* k_cache, const void* v_cache, const int* pad_left, void* out, int B,
                        int S, int nh, int nkv, int hd, int T, int start, float scale, void* stream);

/* generation.py:28-41 (HF warpers + categorical/argmax) — logits fp32 [B, ld] (V valid columns). */
int jl_argmax(const float* logits, int B, int V, int ld, int idx_offset, float* out_val, int* out_idx,
              void* stream);
int jl_topk(const float* logits, int B, int V, int ld, int idx_offset, int k, float* cand_val, int* cand_idx,
            void* stream);
int jl_sample(const float* cand_val, const int* cand_idx, int B, int n_lists, size_t list_stride, int k,
              int top_k, float top_p, float temperature, unsigned long long seed, const int* step_ptr,
              int* out_tok, void* stream);
/* HF _sample/_greedy_search body: pad finished rows, mark EOS, append to sequences,
 * advance cur_len / cache_len / step on device. */
int jl_decode_advance(const int* tok, int* next_ids, int* finished, int* sequences, int B, int max_len,
                      int eos, int pad, int* cur_len, int* cache_len, int* step, int* n_unfinished,
                      void* stream);

/* ---------------------------------------------------------------------------------------------------------
 * Whole-model decode step (model.py:743-790 at S=1, i.e. everything FlaxLLaMAForCausalLMModule.__call__ does
 * for one new token) in ONE persistent cooperative kernel for M <= 8 rows: embedding, L x (RMSNorm+wqkv, RoPE,
 * cache append, GQA attention, wo+residual, RMSNorm+w13+SwiGLU, w2+residual), final norm and LM head with a
 * running arg-max.  Weights are the per-op stacks [L*N, K].  There is no grid barrier: activations cross CTAs as
 * tagged 8-byte packets that consumers poll (csrc/decode_mega.cu).  `scratch` holds the packet buffers
 * (jl_decode_mega_scratch_bytes() bytes, ZERO when first used, never cleared afterwards); `gen` is a device
 * counter of the steps this engine has run (zero at start; the kernel advances it; it is the tag base, so every
 * scratch / peer buffer ever used with it must only be used with it).  `logits` fp32 [M, V] (V = this rank's
 * vocab shard, vocab_full the whole vocabulary) may be NULL: then only the per-CTA arg-max candidates are
 * produced (read by jl_mega_select).  Row pitch `logits_ld` (0 = V), this rank's columns start at `logits_col0`;
 * with `logits_multicast` the pointer is the NVLS multicast address of a symmetric [M, vocab_full] buffer and every
 * rank receives every shard (input of jl_sample_full under tensor parallelism).  Needs a cooperative launch of one CTA per SM (num_sms CTAs co-resident).
 * With tp > 1 the wo / w2 outputs are all-reduced inside the kernel (partition.py:67,70 is what GSPMD
 * all-reduced there): fp32 partial packets go to every rank with one multimem.st on `mc_partials` (the NVLS
 * multicast address of the symmetric buffer whose per-rank mappings are `peer_partials`; NULL = one unicast
 * store per peer), candidates likewise through `peer_cand` / `mc_cand`; sizes from jl_decode_mega_peer_bytes. */
size_t jl_decode_mega_scratch_bytes(int M, int H, int F, int nh, int nkv, int num_sms);
size_t jl_decode_mega_cand_offset(int M, int H, int F, int nh, int nkv, int num_sms);   /* tp == 1: candidates inside scratch */
size_t jl_decode_mega_peer_bytes(int M, int H, int tp, int num_sms, size_t* cand_offset);
int jl_decode_mega_stages(int M, int H, int F, int nh, int nkv, int hd); /* weight-ring depth; 0 = shape does not fit */
void jl_decode_mega_set_trace(void* buf /* device u64 [num_sms][L][32] %globaltimer stamps, NULL = off */);
int jl_decode_mega(const void* wqkv_all, const void* wo_all, const void* w13_all, const void* w2_all,
                   const void* lm_head, const void* attn_norm, const void* ffn_norm, const void* final_norm,
                   const void* embedding, const int* ids, float* logits, int logits_ld, int logits_col0,
                   int logits_multicast, void* k_cache, void* v_cache,
                   const float* cos_t, const float* sin_t, const int* cache_len, const int* pad_left, void* scratch,
                   unsigned int* gen, int M, int L, int H, int F, int V, int vocab_full, int nh, int nkv, int hd,
                   int T, int max_pos, float eps, float scale, int num_sms, int tp, int rank,
                   void* const* peer_partials, void* mc_partials, void* const* peer_cand, void* mc_cand,
                   void* stream);
/* HF _greedy_search body (generation.py:28-41 with temperature 0) for the step jl_decode_mega just ran on this
 * stream: merges the num_sms x tp arg-max candidates per row (ties: lower vocabulary index; waits for ranks whose
 * kernel is still finishing), then the bookkeeping of jl_decode_advance.  `cand` = this rank's candidate packets. */
int jl_mega_select(const void* cand, const unsigned int* gen, int tp, int rank, int num_sms, int M, int L, int* tok,
                   int* next_ids, int* finished, int* sequences, int max_len, int eos, int pad, int* cur_len,
                   int* cache_len, int* step, int* n_unfinished, void* stream);

/* ---------------------------------------------------------------------------------------------------------
 * Tensor parallelism over NVLink peer memory (partition.py:62-78 names the sharding; XLA/GSPMD inserted NCCL
 * collectives, here they run inside the compute kernels).  Peer buffers are cudaMalloc'd + exported with
 * CUDA IPC; `peer_*` arguments are host arrays of tp device pointers (index = rank, own entry local). */
int jl_ipc_alloc(size_t bytes, void** ptr, void* handle64 /* out: 64-byte IPC handle */);
int jl_ipc_open(const void* handle64, void** ptr);
int jl_ipc_close(void* ptr);
int jl_ipc_free(void* ptr);

/* Row-parallel linear at decode (wo, w2; M <= 8): local GEMV over this rank's K shard, partial sums pushed to
 * every peer's inbox, one-shot all-reduce in rank order (bitwise identical on all ranks) + residual, in one
 * launch.  The epoch that tags the flags is *seq_ptr + call_index (device counter advanced with jl_comm_bump,
 * so the same CUDA graph replays with fresh epochs).  peer_flags must hold jl_gemv_allreduce_flags(N) ints at
 * flag_offset. */
int jl_gemv_allreduce_flags(int N);
int jl_gemv_allreduce(const void* x, const void* w, const void* residual, void* out, int M, int N, int K, int tp,
                      int rank, void* const* peer_inbox, void* const* peer_flags,
                      size_t inbox_parity_stride_floats, int flag_offset, const int* seq_ptr, int call_index,
                      int num_sms, void* stream);
/* All-gather of a small record (<= slot_bytes, multiples of 16) from every rank: push to every inbox + flag.
 * Used for the cross-rank sampler (per-rank top-k candidates of the vocab-sharded logits). */
int jl_allgather_small(const void* src, void* out, int n_bytes, int slot_bytes, int tp, int rank,
                       void* const* peer_inbox, void* const* peer_flags, size_t parity_stride_bytes,
                       int flag_offset, const int* seq_ptr, int call_index, void* stream);
int jl_comm_bump(int* seq_ptr, int n, void* stream);
/* one warp: flags[r][flag_off + rank] = epoch on every rank r, then wait until this rank's flags[flag_off + 0..tp) >= epoch
 * ("every rank has finished the kernel before this one on its stream") */
int jl_flag_exchange(void* const* peer_flags, int flag_off, int epoch, const int* base /* device int added to epoch, or NULL */,
                     int tp, int rank, void* stream);
/* one warp waits (on the stream) until flags[0..tp) >= epoch (+ *seq_ptr if given: device epoch counter, graph safe):
 * later kernels may read what the peers published first */
int jl_wait_flags(const int* flags, int epoch, const int* seq_ptr, int tp, int rank, void* stream);
int jl_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);

/* HF Flax warpers + categorical sampling + `_sample` bookkeeping (generation.py:28-41) over the WHOLE vocabulary, exact
 * for any top_k / top_p (no candidate budget), deterministic ties (lower index), identical on every rank: see
 * csrc/sample_full.cu.  logits fp32 [B, ld] with V valid columns; temperature 0 = arg-max; top_k <= 0 or >= V and
 * top_p >= 1 disable the filters.  `cand`/`gen` (may be NULL) = candidate packets / step counter of jl_decode_mega: wait
 * for every rank's logits shard first.  `next_ids` == NULL: selection only (tok[B]).  `ticket` = one zero int. */
int jl_sample_full(const float* logits, int B, int V, int ld, float temperature, int top_k, float top_p,
                   unsigned long long seed, const int* step, int* tok, const void* cand, const unsigned int* gen, int tp,
                   int rank, int num_sms, int L, int* ticket, int* next_ids, int* finished, int* sequences, int max_len,
                   int eos, int pad, int* cur_len, int* cache_len, int* step_rw, int* n_unfinished, void* stream);

/* All-gather of a column-sharded fp32 block over NVLS: this rank's [rows, cols] goes to columns [col0, col0+cols) of
 * every rank's [rows, dst_ld] buffer (`dst_mc` = its multicast address) with multimem.st; flags[r][flag_off + rank] =
 * epoch (+ *seq_ptr if given) on every rank afterwards (pair with jl_wait_flags).  The reference gathers the vocab-sharded logits with the
 * all-gather GSPMD derives from partition.py:77. */
int jl_nvls_bcast_f32(const float* src, float* dst_mc, int rows, int cols, int src_ld, int dst_ld, int col0, int tp,
                      int rank, void* const* peer_flags, int flag_off, int epoch, const int* seq_ptr, int* ticket,
                      void* stream);

/* The same linear layers on CTA PAIRS (2-CTA clusters, tcgen05.mma.cta_group::2, 256 x 256 tiles, TMA-store epilogue):
 * token-major GEMMs with M >= 256, N % 256 == 0, K % 64 == 0 (every prefill GEMM of model.py:119-150, 311-338).
 * Returns 3 (nothing launched) for other shapes; jl_gemm tries this first and falls back to its single-CTA kernel. */
int jl_gemm_2cta(const void* x, const void* w, const void* residual, void* out, int M, int N, int K, int mode,
                 int num_sms, void* stream);
int jl_gemm_2cta_pairs(void);   /* 2-CTA clusters resident at once on this GPU (the persistent grid uses exactly these) */

/* NVLS form of the owner-side step of the sequence-parallel prefill, and the all-reduce of a row-parallel GEMM for any
 * token count (partition.py:67,70 is what GSPMD all-reduced there).  The GEMM before it stored this rank's bf16 partial
 * product into its own copy of a symmetric buffer; `part_mc` is the multicast address of that buffer at the first of
 * the `rows` rows this call owns: x[rows, H] += sum over ranks (multimem.ld_reduce, fp32 in the switch).  With `xn_mc`
 * (multicast address of the gathered-activation buffer at the same first row) the updated rows are RMS-normalised and
 * stored into every rank's copy with multimem.st, then the "rows ready" flag is published; without it the call is a
 * plain all-reduce into a replicated residual stream (rows = all tokens).  With `xn_local` instead (an ordinary
 * [rows, H] buffer) the normalised rows stay on this rank: all-reduce + residual add + the next RMSNorm of a batched
 * decode step in one launch.  has_partials: 0 = no reduction (chain start), 2 = the caller already exchanged the "GEMM
 * done" flags (jl_flag_exchange), 1 = exchange them inside this kernel (rows <= 128 only: a small resident grid). */
int jl_rs_reduce_mm(void* x, const void* part_mc, const void* norm_w, void* xn_mc, void* xn_local, int rows, int H,
                    int has_partials, int tp, int rank, void* const* peer_flags, int gemm_flag_off, int ready_flag_off,
                    int gemm_epoch, int ready_epoch, const int* epoch_base /* device int added to both epochs, or NULL */,
                    int* ticket, float eps, void* stream);

/* NVLS self-test over a multicast mapping of a symmetric buffer (parallel/symm.py): `mc` is the multicast
 * address.  op 0: out[i] = sum over ranks of fp32 buf[i] (multimem.ld_reduce); 1: 8-byte packets {src[i], tag}
 * stored into every rank's copy (multimem.st); 2: every copy += src[i] (multimem.red); 3 / 4: the bf16 forms of
 * 0 / (plain store); 5: u32 arrival counter at buf[0] += 1 with release semantics.  The reference's collectives
 * are NCCL calls emitted by XLA for partition.py:62-78; these instructions are what the fused kernels use instead. */
int jl_nvls_selftest(void* mc, const void* src, void* out, int n, int op, unsigned int tag, void* stream);

/* ---- Kernels of the hybrid decoder family (softmax attention and linear-recurrence mixers over an fp32 residual
 * stream).  `dtype` 0 = bfloat16, 1 = true float32 (operands, cache and outputs; statistics and sums are fp32 in both).
 * These designs have no counterpart in the reference; the mechanisms are described at the kernels. */

/* ids int32 [M]; table [V, W] of dtype; out fp32 [M, W]. */
int jl_embed_f32(const int* ids, const void* table, float* out, int M, int W, int V, int dtype, void* stream);
/* out[m] = x[m] / sqrt(mean(x[m]^2) + eps) * (offset + w); x fp32 [M, W]; w, out of dtype. */
int jl_norm_f32(const float* x, const void* w, void* out, int M, int W, float eps, float offset, int dtype, void* stream);
/* x[m] += norm(y[m]) * (offset + w_post) with y fp32 [M, W] (row pitch ldy); if w_next: h[m] = norm(x[m]) * (offset + w_next). */
int jl_postnorm_add(const float* y, int ldy, const void* w_post, float* x, const void* w_next, void* h, int M, int W, float eps,
                    float offset, int dtype, void* stream);
/* out[m, h, :] = o[m, h, :] / rms * w[:] * act(gate[m, h*V + :]); o fp32 [M, H, V]; gate fp32 with row pitch ldg. */
int jl_headnorm_gate(const float* o, const void* w, const float* gate, int ldg, void* out, int M, int H, int V, float eps,
                     int gate_act, int dtype, void* stream);
/* out = act(in) for an fp32 [M, N] block (pitch ldi) into out_dtype (pitch ldo).  act: 0 none, 1 relu^2, 2 gelu (tanh form),
 * 3 silu, 4 scale by p0 then soft cap p1 * tanh(. / p1) (p1 <= 0: no cap). */
int jl_act_cast(const float* in, int ldi, void* out, int ldo, int M, int N, int act, float p0, float p1, int out_dtype,
                void* stream);
/* data = act(data) in place for an [M, N] block (pitch ld) of dtype. */
int jl_act_inplace(void* data, int ld, int M, int N, int act, float p0, float p1, int dtype, void* stream);
/* out[:, 0:N] (pitch ldo; fp32 if out_f32 else dtype) = act(x W^T): x [M, K] (pitch ldx), W [N, K]; any M, N, K. */
int jl_linear_any(const void* x, int ldx, const void* w, void* out, int ldo, int M, int N, int K, int act, float p0, float p1,
                  int dtype, int out_f32, void* stream);
/* Rotary embedding (first `rot` channels, interleaved pairs), optional unit-RMS per head, cache append.  y fp32 [B*S, ldy] holds
 * q at q_off ([H*D]), k at k_off ([G*D]; < 0: queries only), v at v_off ([G*Dv]); caches [B][G][T_cap][D|Dv] of dtype. */
int jl_attn_prep(const float* y, int ldy, int q_off, int k_off, int v_off, void* q_out, void* k_cache, void* v_cache,
                 const float* cos_t, const float* sin_t, int max_pos, int rot, int unit_norm, float eps, const int* cache_len,
                 const int* pad_left, int B, int S, int H, int G, int D, int Dv, int T_cap, const float* bias, int v_norm,
                 int v_token_major, int dtype, void* stream);
/* (jl_attn_prep) bias: fp32 indexed like the columns of y, added first (NULL: none); v_norm: values scaled to unit RMS per head
 * before they are cached; v_token_major: value cache [B][T_cap][G*Dv] instead of [B][G][T_cap][Dv]. */
/* Causal softmax attention of S new tokens per row (slots *cache_len .. *cache_len+S-1) over slots [pad_left[b], own slot];
 * q [B*S, H, D], out [B*S, H, Dv]; gate (optional) fp32 [B*S, ldg], column h: out *= sigmoid(gate).
 * One new token (S == 1) with `scratch` (B*H*splits*(Dv+2) floats, splits from jl_attn_generic_splits, at most 64): the keys
 * are split over `splits` CTAs per key/value head and block of 16 query heads, and merged by a second launch. */
int jl_attn_generic_splits(int B, int H, int G, int T_cap);
int jl_attn_generic(const void* q, const void* k_cache, const void* v_cache, void* out, const float* gate, int ldg,
                    const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv, int T_cap, float scale,
                    float* scratch, int splits, int dtype, void* stream);
/* out[m, h, :] *= sigmoid(gate[m, h]) in place. */
int jl_head_gate(void* out, const float* gate, int ldg, int M, int H, int Dv, int dtype, void* stream);
/* Gated linear attention scan: state [B][H][D][Dv] fp32 (in/out), o fp32 [B*S, H, Dv]; a2 [H*D, R], a2_bias [H*D] of dtype.
 * ws == NULL: one fused launch (decoding).  ws = jl_gla_scan_ws_floats(...) floats: token-parallel preparation into ws, then
 * a scan that streams it through a two-stage cp.async pipeline (prompts). */
size_t jl_gla_scan_ws_floats(int B, int S, int H, int D, int Dv);
int jl_gla_scan(const float* y, int ldy, int q_off, int k_off, int v_off, int a_off, const void* a2, const void* a2_bias,
                float* state, float* o, const int* cache_len, const int* pad_left, int B, int S, int H, int D, int Dv, int R,
                float q_scale, float tau, float* ws, int dtype, void* stream);

/* Retention scan: the scan above with one fixed decay per head (head_decay fp32 [H]) instead of the projected one, the rotary
 * embedding of q and k at the token's position on the first `rot` channels of a head (layout 0: channel 2i with 2i+1; 1: channel
 * i with i + rot/2; tables fp32 [max_pos][rot/2], any factor on cos / sin already in them) and k scaled by k_scale after it. */
int jl_retention_scan(const float* y, int ldy, int q_off, int k_off, int v_off, const float* head_decay, const float* cos_t,
                      const float* sin_t, int max_pos, int rot, int layout, float q_scale, float k_scale, float* state, float* o,
                      const int* cache_len, const int* pad_left, int B, int S, int H, int D, int Dv, float* ws, void* stream);
/* Residual step of a block whose branches read the same input: x[m] += mult * (y1[m] + y2[m]) (either may be NULL), then up to
 * two norms of the new row with plain weights: h1 = norm(x) * w1, h2 = norm(x) * w2 (a weight and its output come together). */
int jl_branch_add_norm(const float* y1, int ld1, const float* y2, int ld2, float mult, float* x, const void* w1, void* h1,
                       const void* w2, void* h2, int M, int W, float eps, int dtype, void* stream);
/* Many products act(x W^T) in one launch.  Plain batches (tile_group == NULL): batch z < nbatch reads x + (z / x_div) * x_bs,
 * the weights w + (w_index ? w_index[z] : z) * w_bs and writes out + z * o_bs, M rows each.  Sorted rows (tile_group != NULL):
 * M rows in tiles of jl_linear_tile_rows(), tile t uses the weights w + tile_group[t] * w_bs (< 0: skipped), row p reads
 * input row row_src[p] (< 0: zero; NULL: p) and writes output row p. */
int jl_linear_tile_rows(void);
int jl_linear_grouped(const void* x, int ldx, long long x_bs, const void* w, long long w_bs, void* out, int ldo, long long o_bs,
                      int nbatch, int x_div, int M, int N, int K, int act, float p0, float p1, const int* w_index,
                      const int* tile_group, const int* row_src, int dtype, int out_f32, void* stream);
/* jl_attn_generic with cache row pitches ldk / ldv (keys and values may be columns of one cached row), batch-row and head
 * strides in elements (all four 0: the [B][G][T_cap][ld] cache layout; token-major projections [B*T][G][d] have bs = T*G*d,
 * hs = d, ld = G*d) and a sliding window: window > 0: a query at slot i sees slots i - window + 1 .. i only. */
int jl_attn_windowed(const void* q, const void* k_cache, const void* v_cache, void* out, const int* cache_len,
                     const int* pad_left, int B, int S, int H, int G, int D, int Dv, int T_cap, int ldk, int ldv,
                     long long k_bs, long long k_hs, long long v_bs, long long v_hs, int window, float scale, float* scratch,
                     int splits, int sink, float* out32, int dtype, void* stream);
/* (jl_attn_windowed) sink: the softmax denominator has one more term exp(0) — a key with score 0 that carries no value;
 * out32: fp32 output [B*S, H, Dv] written instead of `out`. */
/* Latent attention, preparation.  y fp32 [B*S, ldy] holds the query latent (q_rank columns at q_off; 0: none) and the key /
 * value latent followed by the rotated key part shared by the heads (kv_rank + rot_dim columns at kv_off).  The latents are
 * RMS-normed with plain weights; the key part is rotated on its first `rot` channels.  cq [B*S, q_rank]; cache
 * [B][T_cap][kv_rank + rot_dim], the token's row at slot *cache_len + s; c_out [B*S, kv_rank] / kr_out [B*S, rot_dim]
 * (optional): token-major copies of the two parts of the appended row. */
int jl_latent_prep(const float* y, int ldy, int q_off, int q_rank, int kv_off, int kv_rank, int rot_dim, int rot, int layout,
                   const void* wq_norm, const void* wkv_norm, void* cq, void* cache, const float* cos_t, const float* sin_t,
                   int max_pos, float eps, const int* cache_len, const int* pad_left, int B, int S, int T_cap, void* c_out,
                   void* kr_out, int dtype, void* stream);
/* out[m, h, out_off + d] = rotary(in[m, h, in_off + d]), d < n, at the token's position: a slice of every head rotated and
 * copied into another head layout (head pitches in_hs / out_hs, row pitches ldi / ldo). */
int jl_rotary_slice(const void* in, int ldi, int in_hs, int in_off, void* out, int ldo, int out_hs, int out_off, int H, int n,
                    int rot, int layout, const float* cos_t, const float* sin_t, int max_pos, const int* cache_len,
                    const int* pad_left, int B, int S, int dtype, void* stream);
/* Mixture-of-experts routing.  z fp32 [M, ldz]: router logits in columns 0 .. E-1.  score 0: sigmoid, 1: softmax.  groups > 1:
 * experts form `groups` equal groups of neighbours, a group scores the sum of its group_top largest scores, and only experts
 * of the `keep` best groups can be chosen.  idx int32 / wt fp32 [M, top]: the top largest, weights = scores (over their sum
 * + 1e-20 when normalise) * scale. */
int jl_moe_route(const float* z, int ldz, int M, int E, int top, int groups, int keep, int group_top, int score, int normalise,
                 float scale, const float* bias, int* idx, float* wt, void* stream);
/* (jl_moe_route) bias: fp32 [E] added to the logits (NULL: none). */
/* Order the M * top (token, choice) pairs by expert into segments rounded up to `tile` rows (cap >= jl_moe_sorted_rows rows):
 * pos [M * top]: row of each pair; row_src [cap]: token of each row (-1: padding); tile_group [cap / tile]: expert (-1: none);
 * tiles_used (optional): the number of leading tiles that belong to an expert. */
int jl_moe_sorted_rows(int n, int E, int tile);
int jl_moe_sort(const int* idx, int M, int top, int E, int tile, int cap, int* pos, int* row_src, int* tile_group,
                int* tiles_used, void* stream);
/* out[m] = sum_k wt[m, k] * z[pos ? pos[m*top+k] : m*top+k] (+ (gate ? sigmoid(gate[m*ldg]) : 1) * shared[m] when shared). */
int jl_moe_combine(const float* z, int ldz, const int* pos, const float* wt, int top, const float* shared, int lds,
                   const float* gate, int ldg, float* out, int M, int W, void* stream);
/* xs[p] = x[row_src[p]] (zeros where row_src[p] < 0): the rows of a step in sorted order; rows x W of dtype. */
int jl_moe_gather(const void* x, int ldx, const int* row_src, void* xs, int rows, int W, int dtype, void* stream);
/* Grouped token-major tcgen05 GEMM: x bf16 [M, K], M a multiple of 128, every 128-row tile t using the weight matrix
 * w[tile_group[t]] of w bf16 [groups][N, K] (< 0: a padding tile); out [M, N] bf16 or fp32.  N % 8 == 0, K % 8 == 0.
 * tiles_used (optional, device int): only that many leading tiles are computed. */
int jl_gemm_grouped(const void* x, const void* w, void* out, int M, int N, int K, int groups, const int* tile_group,
                    const int* tiles_used, int out_f32, int num_sms, void* stream);

/* ---- token embedding with a hashed pair table, short convolutions with state, delta-rule and state-space scans,
 *      gated activations and the norms around mixers that run side by side (csrc/seq_mix.cu, delta_scan.cu, gla_scan.cu) */

/* out[m] = norm(table[id] + pair[r]) * norm_w (fp32 [B*S, W]; norm_w NULL: no norm), r = (prev * mul_prev + id * mul_cur) mod
 * buckets with prev the token before it in its sequence, r = buckets for a sequence's first token (position
 * *cache_len + s - pad_left[b] == 0); rows at negative positions are zero.  prev_tok int32 [B]: the last token of the
 * previous call, replaced by this call's last. */
int jl_embed_pair_norm(const int* ids, const void* table, const void* pair, const void* norm_w, float* out, int* prev_tok,
                       const int* cache_len, const int* pad_left, int B, int S, int W, int V, int buckets, long long mul_prev,
                       long long mul_cur, float eps, int dtype, void* stream);
/* Causal convolution over time per channel: out[m, c] = act(bias[c] + sum_j w[c][taps-1-j] * in[token - j][c]), inputs fp32
 * columns col0 .. col0+C-1 of y, zeros before a sequence's start; state fp32 [B][taps-1][C] holds the last taps-1 inputs of
 * every row (read for the first tokens of the call, replaced by the call's last inputs).  w [C][taps], bias [C] or NULL. */
int jl_causal_conv(const float* y, int ldy, int col0, int C, const void* w, const void* bias, float* state, float* out, int ldo,
                   const int* cache_len, const int* pad_left, int B, int S, int taps, int act, int dtype, void* stream);
/* out[m] = c * (norm(a[m]) * wa + norm(b[m]) * wb), fp32 [M, W] (b NULL: one branch). */
int jl_norm_mean2(const float* a, int lda, const void* wa, const float* b, int ldb, const void* wb, float c, float* out, int M,
                  int W, float eps, int dtype, void* stream);
/* out[m, i] = norm_group((o[m, i] + skip[i / P] * x[m, i]) * act(z[m, i])) * w[i]: the gate first, then an RMS norm over each
 * of `groups` equal parts of the N = H * P columns.  skip [H] and x may be NULL. */
int jl_gated_groupnorm(const float* o, const float* x, int ldx, const void* skip, int P, const float* z, int ldz, const void* w,
                       void* out, int M, int N, int groups, float eps, int gate_act, int dtype, void* stream);
/* Gated activation of a fused gate | up product: out[m, j] = f(in[m, g_off + j], in[m, u_off + j]).  kind 0: act(g) * u;
 * kind 1: g' = min(g, limit), u' = clamp(u, -limit, limit), g' * sigmoid(alpha * g') * (u' + 1).  With the device counter
 * rows_used only the first *rows_used * rows_mult rows are computed. */
int jl_glu_act(const float* in, int ldi, int g_off, int u_off, void* out, int ldo, int M, int F, int kind, int act, float limit,
               float alpha, const int* rows_used, int rows_mult, int dtype, void* stream);
/* Mixing of attention weights across heads, applied after the weighted sums: o fp32 [M][H][Gc][Dv] holds, for query head g
 * and key/value head c0 + c, sum_j weight_g(j) v_c(j); out[m, h, :] = sum_g mix[h][g] * o[m, g, kv(h) - c0, :] for the heads
 * whose key/value head kv(h) = h / (H / G) lies in [c0, c0 + Gc). */
int jl_talk_mix(const float* o, const void* mix, void* out, int M, int H, int G, int Gc, int c0, int Dv, int dtype, void* stream);
/* Per token and head of a selective state space layer: dt = softplus(y[m, dt_off + h] + dt_bias[h]),
 * aux[m, h] = exp(-exp(A_log[h]) * dt), aux[m, H + h] = dt  (fp32 [M, 2H]). */
int jl_ssd_gates(const float* y, int ldy, int dt_off, const void* dt_bias, const void* a_log, float* aux, int M, int H, int dtype,
                 void* stream);
/* State space scan on the gated-linear-attention kernels: S_t = aux[t, h] S_(t-1) + (aux[t, H + h] v_t) k_t^T, o_t = S_t^T q_t,
 * q / k shared by the H / G heads of a group (columns q_off + g * D ...), v [H * Dv]; state fp32 [B, H, D, Dv]. */
int jl_ssd_scan(const float* u, int ldu, int q_off, int k_off, int v_off, int G, const float* aux, float* state, float* o,
                const int* cache_len, const int* pad_left, int B, int S, int H, int D, int Dv, float* ws, void* stream);
/* Gated delta rule with one decay per key channel, per head: S <- diag(a_t) S; e = beta_t (v_t - S^T k_t); S <- S + k_t e^T;
 * o_t = S^T q_t.  u fp32 [M, ldu]: q, k (G heads of D, after their convolutions) and v (H heads of Dv); q and k are scaled to
 * unit length per head (1e-6 inside the root), q also by D^(-1/2).  y fp32 [M, ldy]: beta logits (H columns at b_off) and
 * the rank-R decay input (a_off); a_t = exp(-exp(a_log[h]) * softplus(a2 (.) + a_bias)), a2 [H*D, R], a_bias [H*D].
 * state fp32 [B, H, D, Dv]; o fp32 [M, H*Dv]; ws: jl_delta_scan_ws_floats floats. */
size_t jl_delta_scan_ws_floats(int B, int S, int H, int D, int Dv);
int jl_delta_scan(const float* u, int ldu, int q_off, int k_off, int v_off, int G, const float* y, int ldy, int b_off, int a_off,
                  const void* a2, const void* a_bias, const void* a_log, float* state, float* o, const int* cache_len,
                  const int* pad_left, int B, int S, int H, int D, int Dv, int R, float* ws, int dtype, void* stream);

/* ---- Pieces added with the looped chunked-attention design (Datozen): learned positions, a per-layer token input, attention
 * with a weighted q / k norm before the rotation, rotated values, blocks of positions and a learned sink, a router with a
 * choice bias and identity experts. */

/* out[m] = table[ids[m]] + pos_table[position of m] (fp32 [B*S, W]); token (b, s) is at position *cache_len + s - pad_left[b]
 * (clamped to P - 1; a negative position is padding and gives a zero row). */
int jl_embed_pos(const int* ids, const void* table, const void* pos_table, float* out, const int* cache_len, const int* pad_left,
                 int B, int S, int W, int V, int P, int dtype, void* stream);
/* out[m, c] = gelu_tanh(t[m, c]) * side[ids[m], col0 + c], c < n; t fp32 (row pitch ldt), side and out of dtype (pitches lds, ldo). */
int jl_side_gate(const float* t, int ldt, const int* ids, const void* side, int lds, int col0, void* out, int ldo, int M, int n,
                 int V, int dtype, void* stream);
/* The same gate for M <= 8 rows with the small projection inside: out[m, c] = gelu_tanh(w_gate[c, :] . x[m, :]) * side[ids[m], col0 + c];
 * x fp32 [M, W] (row pitch ldx) is read as it is; w_gate [n, W], side and out of dtype. */
int jl_side_gate_rows(const float* x, int ldx, const int* ids, const void* side, int lds, int col0, const void* w_gate, void* out,
                      int ldo, int M, int W, int n, int V, int dtype, void* stream);
/* x[m] += mult * (y1[m] + y2[m]) in place (fp32 [M, W]; either branch may be NULL) and xc[m] = the updated row in dtype. */
int jl_branch_add_cast(const float* y1, int ld1, const float* y2, int ld2, float mult, float* x, void* xc, int M, int W, int dtype,
                       void* stream);
/* jl_attn_prep with: `layout` of the rotated q / k pairs (0: (2i, 2i+1), 1: (i, i + rot/2)); q_norm_w / k_norm_w [D] of dtype, an RMS
 * norm of every head before the rotation (NULL: none); v_cos / v_sin fp32 [v_max_pos][Dv/2]: values rotated at their own position
 * over all Dv channels before they are cached, pairs as v_layout (NULL: cached as they are). */
int jl_attn_prep_ex(const float* y, int ldy, int q_off, int k_off, int v_off, void* q_out, void* k_cache, void* v_cache,
                    const float* cos_t, const float* sin_t, int max_pos, int rot, int layout, int unit_norm, const void* q_norm_w,
                    const void* k_norm_w, float eps, const float* v_cos, const float* v_sin, int v_max_pos, int v_layout,
                    const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv, int T_cap,
                    const float* bias, int v_norm, int v_token_major, int dtype, void* stream);
/* jl_attn_windowed with: gate (fp32 pre-activation of a sigmoid per head, column h of row m, pitch ldg; NULL: none); chunk > 0:
 * positions form blocks of `chunk` and a query sees the keys of its own block only; sink_logit fp32 [H]: the extra term of the
 * denominator is exp(sink_logit[h]) (needs sink = 1; NULL: exp(0)); v_cos / v_sin: the cached values were rotated at their own
 * positions and every head's sum is rotated back by the query's position before the gate. */
int jl_attn_masked(const void* q, const void* k_cache, const void* v_cache, void* out, const float* gate, int ldg,
                   const int* cache_len, const int* pad_left, int B, int S, int H, int G, int D, int Dv, int T_cap, int ldk, int ldv,
                   long long k_bs, long long k_hs, long long v_bs, long long v_hs, int window, int chunk, float scale, float* scratch,
                   int splits, int sink, const float* sink_logit, const float* v_cos, const float* v_sin, int v_max_pos,
                   int v_layout, float* out32, int dtype, void* stream);
/* The tcgen05 prompt attention kernel (bfloat16, 128-wide heads; caches [B, nkv, T, 128]) with blocks of `chunk` positions, a sink in
 * the denominator (sink_logit fp32 [nh] or NULL for exp(0)), a sigmoid gate per (token, head) (fp32 pre-activation, pitch ldg) and the
 * turn back of values cached rotated at their own positions (v_cos / v_sin fp32 [v_max_pos][64], pairs m, m + 64).  `start`: slots
 * filled before this call's S tokens per row. */
int jl_flash_prefill_masked(const void* q, const void* k_cache, const void* v_cache, const int* pad_left, void* out, int B, int S,
                            int nh, int nkv, int hd, int T, int start, float scale, int chunk, int sink, const float* sink_logit,
                            const float* gate, int ldg, const float* v_cos, const float* v_sin, int v_max_pos, void* stream);
/* jl_moe_route with: choice_bias fp32 [E] added to the scores for the choice (group scores and top) only; experts n_real .. E-1
 * are identity experts: a chosen one is reported as expert -1 (jl_moe_sort and the grouped linears skip it) and its weight is
 * added to ident_w[m]. */
int jl_moe_route_ex(const float* z, int ldz, int M, int E, int top, int groups, int keep, int group_top, int score, int normalise,
                    float scale, const float* bias, const float* choice_bias, int n_real, float* ident_w, int* idx, float* wt,
                    void* stream);
/* jl_moe_combine that skips the pairs with idx < 0 and adds ident_w[m] * x[m] (x of dtype, row pitch ldx). */
int jl_moe_combine_ex(const float* z, int ldz, const int* pos, const float* wt, int top, const float* shared, int lds,
                      const float* gate, int ldg, float* out, int M, int W, const int* idx, const float* ident_w, const void* x,
                      int ldx, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif
