/*
 * b200tp — C ABI of the B200 (sm_100a) tensor-parallel layer path for nano-vllm.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*; NULL = the legacy default stream) and
 * returns an int status (B2_OK = 0).  Nothing here allocates, synchronises or
 * creates streams inside a compute call, so calls may be captured in CUDA
 * graphs.  All activations and weights are bf16 (16-bit words, row-major, the
 * innermost dimension contiguous) unless stated otherwise.  PyTorch (or any
 * caller) owns every tensor passed in; the library owns only what
 * b2_ctx_create allocates.
 *
 * Citations name the reference lines (nano-vllm, path within the project)
 * whose behaviour the entry point reproduces.
 */
#ifndef B200TP_H
#define B200TP_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B2_OK = 0,
  B2_ERR_ARG = 1,         /* null pointer, bad alignment, negative size            */
  B2_ERR_SHAPE = 2,       /* a size outside what the context was created for       */
  B2_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed (see b2_last_error) */
  B2_ERR_STATE = 4,       /* peers not imported, context destroyed, ...            */
  B2_ERR_TIMEOUT = 5,     /* a bounded device-side wait ran out (from b2_status)   */
  B2_ERR_UNSUPPORTED = 6
};

#define B2_HANDLE_BYTES 64 /* one exported symmetric-memory handle */

typedef struct b2_ctx b2_ctx;

typedef struct b2_config {
  int rank;            /* tensor-parallel rank of this process                         */
  int world;           /* tensor-parallel size (1, 2, 4 or 8)                          */
  int device;          /* CUDA device ordinal of this process                          */
  int max_tokens;      /* largest token count M of any call (prefill budget)           */
  int hidden;          /* largest row length N of an all-reduced activation            */
  int oneshot_tokens;  /* largest M one fused row-parallel launch handles; larger M is
                          processed in chunks of this many tokens                      */
  int vocab;           /* full vocabulary size for the LM-head gather (0 = unused)     */
  int max_seqs;        /* rows of the gathered logits buffer (0 = unused)              */
  int timeout_ms;      /* limit of every cross-GPU wait; 0 = default (5000)            */
} b2_config;

/* ---- context: replaces the NCCL process-group state the reference keeps in
 *      nanovllm/engine/model_runner.py:26 (init) and :50-59 (exit) ------------ */

/* Allocates the rank's symmetric buffers, split-K workspace, arrival counters
 * and the host-visible status word.  Call once per process after selecting
 * `device`. */
int b2_ctx_create(const b2_config* cfg, b2_ctx** out);

/* Writes this rank's B2_HANDLE_BYTES-byte handle; ranks exchange them with any
 * host collective (e.g. torch.distributed.all_gather over the group that
 * nanovllm/engine/model_runner.py:26 creates). */
int b2_symm_export(b2_ctx* ctx, void* handle_out);

/* `handles` = world * B2_HANDLE_BYTES bytes ordered by rank.  Maps every
 * peer's buffer.  Not needed when world == 1.  A host barrier must follow
 * before the first collective call. */
int b2_symm_import(b2_ctx* ctx, const void* handles);

/* Frees everything; call before torch.distributed.destroy_process_group
 * (nanovllm/engine/model_runner.py:50-59), after the stream has drained. */
int b2_ctx_destroy(b2_ctx* ctx);

/* Reads the status word that bounded device-side waits write (no CUDA call, no
 * synchronisation): *code is B2_OK or B2_ERR_TIMEOUT, *detail says which wait.
 * Check it after the step's own synchronisation point
 * (nanovllm/engine/model_runner.py:218, the .tolist()). */
int b2_status(b2_ctx* ctx, int* code, int* detail);
int b2_status_clear(b2_ctx* ctx);

/* After B2_ERR_TIMEOUT the context is poisoned on EVERY rank: an abandoned
 * launch leaves partial sums in the split-K workspace, counters that are not
 * back at zero, partial rows in the peers' inboxes, and launch-sequence
 * numbers that may differ between ranks.  b2_status_clear clears only the
 * word; later collective calls on the same context may return wrong sums.
 * Either destroy and re-create the context on all ranks, or call
 * b2_ctx_reset on all ranks: it synchronises the device, puts every buffer,
 * counter and sequence number of this rank back to its initial state and
 * clears the status word.  No rank may have a b2_* kernel in flight: the
 * caller brackets the call with host barriers (all ranks idle -> barrier ->
 * b2_ctx_reset -> barrier -> resume).  The reference has no counterpart: a
 * hung NCCL collective there ends the process
 * (nanovllm/engine/model_runner.py:50-59 is reached only on a clean exit).
 * Not for use during graph capture; captured graphs stay valid (addresses do
 * not change). */
int b2_ctx_reset(b2_ctx* ctx);

/* Phase tracing of the GEMM / fused row-parallel kernel (the reference has
 * only per-step wall-clock in nanovllm/engine/llm_engine.py:72-83).  While
 * enabled, every CTA of those kernels records 8 (SM clock, global ns) stamps:
 * 0 set-up done, 1 first operand tile landed, 2 last MMA issued, 3 earlier
 * kernels complete (dependency wait passed), 4 epilogue done, 5 GEMM part
 * left, 6 reduce phase done, 7 kernel entry.  If
 * host_out is non-NULL the call synchronises the device, copies
 * min(max_ctas, SM count) * 16 uint64 stamps of the most recent launch and
 * clears them.  Not for use during graph capture. */
int b2_trace(b2_ctx* ctx, int enable, unsigned long long* host_out, int max_ctas);

/* Message of the last failed CUDA call made by this library on this thread. */
const char* b2_last_error(void);

/* Number of kernels this library has launched in this process. */
int64_t b2_launch_count(void);

/* ---- GEMM: replaces F.linear in ReplicatedLinear / ColumnParallelLinear /
 *      MergedColumnParallelLinear / QKVParallelLinear.forward
 *      (nanovllm/layers/linear.py:51,73) and in ParallelLMHead.forward
 *      (nanovllm/layers/embed_head.py:61) -----------------------------------
 * C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]), bf16 in, fp32 accumulate, bf16 out.
 * lda/ldw/ldc are row strides in elements (multiples of 8); K a multiple of 8.
 * tcgen05 tensor-core kernel fed by TMA; the work is split along K over the
 * SMs (stream-K) when there are fewer output tiles than SMs.  W is treated as
 * a constant: the kernel may start fetching it while the previous b2_* kernel
 * on the stream is still running, so W must not be the output of a b2_* call
 * that immediately precedes this one (A, bias and C have no such rule). */
int b2_gemm(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias,
            void* C, int64_t ldc, int M, int N, int K, void* stream);

/* ---- qkv projection with the per-head work that follows it: replaces
 *      QKVParallelLinear.forward (nanovllm/layers/linear.py:73), q_norm / k_norm
 *      (nanovllm/models/qwen3.py:82-84), the rotary embedding (:85) and
 *      store_kvcache (nanovllm/layers/attention.py:59-63) -----------------------
 * qkv[M, (nq + 2 nkv) head_dim] = A W^T (+ bias); then, per token and head:
 * q and k heads are RMS-normalised (weights may both be NULL) and rotated,
 * k and v heads are also written to the paged cache (k_cache may be NULL).
 * Arguments as b2_gemm and b2_qk_norm_rope_store.  For up to 64 tokens and
 * head_dim 128 everything happens in the GEMM's epilogue (one launch);
 * otherwise the projection and the head kernel run as two launches. */
int b2_qkv_fused(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias, void* qkv,
                 int64_t ld_qkv, int M, int nq, int nkv, int head_dim, int K, const void* q_norm_w,
                 const void* k_norm_w, float eps, const int64_t* positions, const float* cos_sin, void* k_cache,
                 void* v_cache, const int32_t* slot_mapping, void* stream);

/* ---- gate_up projection fused with SiLU(gate) * up: replaces the pair
 *      MergedColumnParallelLinear.forward + SiluAndMul.forward in Qwen3MLP
 *      (nanovllm/models/qwen3.py:113-116; nanovllm/layers/activation.py:8-11) --
 * W_pairs [2 I, K] holds the rank's gate and up rows interleaved: row 2 j is
 * gate row j, row 2 j + 1 is up row j.  out[M, I] = silu(A gate_j^T) * (A up_j^T)
 * with the reference's roundings (both products to bf16, the activation to
 * bf16, then the product).  The [M, 2 I] intermediate never reaches HBM. */
int b2_gemm_silu_mul(b2_ctx* ctx, const void* A, int64_t lda, const void* W_pairs, int64_t ldw, void* out, int64_t ldo,
                     int M, int I, int K, void* stream);

/* ---- the same GEMM for callers that cannot allocate device memory.  It has
 *      no counterpart in the reference. ----------------------------------------
 * b2_gemm needs a context, and creating one calls cudaMalloc.  Some users of
 * this library never get that chance: a plug-in loaded after the serving
 * engine has already handed every free byte of HBM to its KV cache (the
 * reference sizes the cache from whatever is left, so a later cudaMalloc
 * fails), or code that is only ever given a stream and tensors.  This variant
 * takes no context: the kernel's scratch (the fp32 partials of output tiles
 * whose K range is shared by several CTAs, and the tiles' arrival counters)
 * is a fixed array compiled into the library, 9.3 MiB that every GPU using
 * the library holds until the process ends.  Same arithmetic and result as
 * b2_gemm, for decode-sized inputs only:
 *   M <= 64 token rows and N <= 524288, otherwise B2_ERR_SHAPE (b2_last_error
 *   says which limit was hit).
 * The call allocates nothing, on the device or through any library.  The
 * first call on each device looks up the array's address on that device
 * (the device must be current); make that first call before any stream
 * capture begins.  All calls share the one array: the counters are cleared on
 * the stream at the start of every call, but two calls that overlap on the
 * GPU (different streams, or different threads) race on it and corrupt each
 * other's result - keep calls stream-ordered.  Without a context there is no
 * status word: b2_status does not cover this entry point. */
int b2_gemm_static_scratch(const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias,
                           void* C, int64_t ldc, int M, int N, int K, void* stream);

/* ---- row-parallel linear fused with its all-reduce, the residual add and
 *      the next RMSNorm: replaces RowParallelLinear.forward
 *      (nanovllm/layers/linear.py:152-156: F.linear then dist.all_reduce) AND
 *      the RMSNorm.add_rms_forward that consumes it
 *      (nanovllm/layers/layernorm.py:28-40; wired at
 *      nanovllm/models/qwen3.py:155,157,182) ---------------------------------
 * Per rank: partial = A[M,Kr] * W[N,Kr]^T (+ bias on rank 0), pushed as bf16
 * into peers' symmetric buffers from the GEMM epilogue; then
 *   s = sum_over_ranks(partial) + residual_in        (fp32)
 *   residual_out = bf16(s)
 *   normed_out   = bf16(bf16(s * rsqrt(mean(s^2) + eps)) * norm_w)
 * in the same launch.  residual_out may alias residual_in.  If norm_w is NULL
 * the call is the plain RowParallelLinear.forward: normed_out receives
 * bf16(sum) and residual_in/residual_out are ignored.  One launch per
 * `oneshot_tokens` rows.  Every rank must issue the same sequence of
 * collective calls (b2_rowpar_fused, b2_embed with world > 1, b2_lm_head).
 * The library picks one of two forms per launch, with the same inputs, outputs
 * and arithmetic (every rank ends up with all rows of both outputs):
 *   one-shot   every rank receives every rank's partial and reduces all rows
 *              itself: one NVLink store latency, (world-1) M N 2 bytes sent
 *              per rank.  Used for up to 64 tokens (decode) everywhere, at
 *              world 2 up to oneshot_tokens, and at world 4 / 8 wherever the
 *              row-owner form is not.
 *   row-owner  token row t is reduced by rank t mod world only: partial rows
 *              go to their owner, which sums, adds the residual, normalises
 *              and sends the finished row and the new residual row to every
 *              rank: two NVLink store latencies and two system-scope fences,
 *              about 3 (world-1)/world M N 2 bytes sent per rank.  Used where
 *              it was measured to win: Kr <= 6144 and 65 .. 1023 tokens at
 *              world 8, 192 .. 511 tokens at world 4 (bounded by
 *              oneshot_tokens), unless set otherwise with b2_ctx_set_option.
 *              -0.0 in an output of this form is stored as +0.0.
 * On one rank with more than 64 tokens nothing crosses a link and the call
 * runs as the plain GEMM followed by the add + RMSNorm kernel in place (two
 * launches), unless a form is forced. */
int b2_rowpar_fused(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias,
                    int M, int N, int Kr, const void* residual_in, const void* norm_w, float eps,
                    void* normed_out, void* residual_out, void* stream);

/* Forms of the fused row-parallel block, and the knobs that choose between
 * them (no counterpart in the reference, whose only form is F.linear + NCCL).
 * Every rank must set the same values. */
enum {
  B2_FORM_AUTO = 0,
  B2_FORM_ONESHOT = 1,  /* b2_rowpar_fused, every rank reduces every row          */
  B2_FORM_OWNER = 2,    /* b2_rowpar_fused, row t reduced by rank t mod world      */
  B2_FORM_TWOSHOT = 3   /* b2_rowpar_fused_twoshot (different output contract)     */
};
enum {
  B2_OPT_ROWPAR_FORM = 1,        /* B2_FORM_AUTO (default), _ONESHOT or _OWNER: what b2_rowpar_fused launches */
  B2_OPT_OWNER_MAX_TOKENS = 2,   /* AUTO: largest M the row-owner form takes (default 1023 at world 8,
                                    511 at world 4, at most oneshot_tokens)                                */
  B2_OPT_TWOSHOT_MIN_TOKENS = 3, /* b2_rowpar_form answers B2_FORM_TWOSHOT from this M on (default: the
                                    row-owner form's largest M + 1 at world >= 4, 1025 at world 2)         */
  B2_OPT_OWNER_MIN_TOKENS = 5,   /* AUTO: smallest M the row-owner form takes (default 65: decode-sized calls
                                    stay on the one-shot form; at world 4 never below 192)                  */
  B2_OPT_WHOLE_TILES = 4         /* 1 (default): fused row-parallel calls with more than 64 tokens whose output
                                    tiles fit the SMs in one wave, and whose K is at most 6144, give every CTA
                                    one whole tile (no K split, no fp32 combine in L2); 0: always a stream-K
                                    split over all SMs                                                      */
};
int b2_ctx_set_option(b2_ctx* ctx, int option, int64_t value);
/* Which entry point and form serve M rows of N features on this context:
 * B2_FORM_TWOSHOT = call b2_rowpar_fused_twoshot (its output contract
 * differs), otherwise call b2_rowpar_fused (which will run the form named).
 * Negative on bad input.  Host arithmetic only. */
int b2_rowpar_form(b2_ctx* ctx, int M, int N);

/* The same block in its two-shot form, for many tokens (M above a few hundred)
 * at tensor-parallel size >= 2.  Token rows are dealt to the ranks in blocks
 * of 16 rows, round-robin (rank r owns rows [16 b, 16 b + 16) for
 * b = r, r + world, ...).  Each rank's GEMM epilogue sends
 * a partial row only to the rank that owns it; the owner reduces, adds the
 * residual, normalises and stores the finished row into every rank's output
 * buffer.  NVLink carries 2 (world-1)/world M N 2 bytes per rank (the one-shot
 * form carries (world-1) M N 2).  Differences from b2_rowpar_fused:
 *  - *normed_out receives the address of a context-owned [M, N] bf16 buffer
 *    (N must equal the context's hidden size).  It is valid until the next
 *    two-shot call on this context; consume it before that.
 *  - residual_out is written only for the rows this rank owns, and only those
 *    rows of residual_in are read:
 *    the residual stream stays sharded by rows between two-shot calls of the
 *    same M, which is all the decoder layer needs (reference wiring:
 *    nanovllm/models/qwen3.py:146-159). */
int b2_rowpar_fused_twoshot(b2_ctx* ctx, const void* A, int64_t lda, const void* W, int64_t ldw, const void* bias,
                            int M, int N, int Kr, const void* residual_in, const void* norm_w, float eps,
                            void** normed_out, void* residual_out, void* stream);

/* ---- RMSNorm: replaces RMSNorm.rms_forward / add_rms_forward
 *      (nanovllm/layers/layernorm.py:16-26, 28-40) ---------------------------
 * x, out: [rows, dim] with row strides ldx / ldo (elements); dim % 8 == 0. */
int b2_rmsnorm(const void* x, int64_t ldx, const void* w, float eps, int rows, int dim,
               void* out, int64_t ldo, void* stream);
/* out, res_out contiguous [rows, dim]; res_out may alias res; out may alias x. */
int b2_add_rmsnorm(const void* x, const void* res, const void* w, float eps, int rows, int dim,
                   void* out, void* res_out, void* stream);

/* ---- paged-KV scatter: replaces store_kvcache / store_kvcache_kernel
 *      (nanovllm/layers/attention.py:10-30, 33-40) ---------------------------
 * For token i < n_tokens with slot = slot_mapping[i] (int32): if slot != -1,
 * copy D 16-bit elements from key + i*key_stride and value + i*value_stride to
 * k_cache + slot*D and v_cache + slot*D.  Strides in elements; D % 8 == 0 and
 * all pointers 16-byte aligned.  Bit-exact copy. */
int b2_store_kvcache(const void* key, int64_t key_stride, const void* value, int64_t value_stride,
                     void* k_cache, void* v_cache, const int32_t* slot_mapping, int n_tokens, int D,
                     void* stream);

/* ---- vocab-parallel embedding: replaces VocabParallelEmbedding.forward
 *      (nanovllm/layers/embed_head.py:34-42: mask, lookup, zero, all_reduce) --
 * ids: int64 [M].  W: this rank's shard [vocab_end - vocab_start, H].  The
 * rank that owns a token writes its row into every rank's buffer (the
 * reference's sum has exactly one non-zero term per element); out[M,H] is
 * complete on every rank when the call's kernel ends.  ctx may be NULL when
 * the whole vocabulary is local (vocab_start = 0, world = 1). */
int b2_embed(b2_ctx* ctx, const int64_t* ids, const void* W, int64_t vocab_start, int64_t vocab_end,
             int M, int H, void* out, void* stream);

/* ---- LM head: replaces ParallelLMHead.forward
 *      (nanovllm/layers/embed_head.py:56-66: F.linear, dist.gather, cat) ------
 * logits_shard[B, Vr] = h[B,H] * W[Vr,H]^T on every rank, stored straight into
 * rank 0's [B, vocab] buffer at column rank*Vr (no separate gather or cat).
 * On rank 0, *logits_out receives the device address of the gathered
 * [B, vocab] bf16 buffer (owned by the context, valid until the next
 * b2_lm_head call); other ranks get NULL, like the reference's None.
 * row_index (int32 [B], may be NULL) selects the rows of h to use, which is
 * the reference's h[cu_seqlens_q[1:] - 1] for prefill. */
int b2_lm_head(b2_ctx* ctx, const void* h, int64_t ldh, const int32_t* row_index, const void* W, int64_t ldw,
               int B, int Vr, int H, void** logits_out, void* stream);

/* ---- LM head fused with the sampler: replaces ParallelLMHead.forward
 *      (nanovllm/layers/embed_head.py:56-66) followed by Sampler.forward
 *      (nanovllm/layers/sampler.py:7-12), as run on rank 0 by
 *      ModelRunner.run (nanovllm/engine/model_runner.py:212-218) -------------
 * No [B, vocab] logits are stored or gathered.  The reference draws
 *   token = argmax_i softmax(logits / T)_i / E_i,   E_i ~ Exp(1);
 * since the softmax denominator is common to a row, that is
 *   token = argmax_i (bf16(logit_i) / T - log E_i),
 * which every rank evaluates over its own vocabulary slice inside the GEMM
 * epilogue; only the best (score, vocab id) per row travels to rank 0.
 * temperatures: fp32 [B] on the device, or NULL for greedy decoding
 * (token = argmax_i logit_i, lowest id on ties: the reference at T -> 0).
 * E_i = -log(u), u from Philox4x32-10 keyed by `seed` with counter (vocab id,
 * row / 4, number of b2_lm_head_sample calls so far on this context, tag):
 * independent of the tensor-parallel split, different on every call (also on
 * every replay of a captured CUDA graph), reproducible from the seed.  It is
 * the reference's distribution, not its random stream (torch's generator).
 * tokens_out: int64 [B], written on rank 0 only (the reference samples on
 * rank 0).  B <= 256 (B2_ERR_SHAPE otherwise: use b2_lm_head).  row_index as
 * in b2_lm_head.  Counts as one collective call in every rank's sequence;
 * two calls must be separated by an exchange that rank 0 completes after
 * reading the first one's result (b2_broadcast_tokens does). */
int b2_lm_head_sample(b2_ctx* ctx, const void* h, int64_t ldh, const int32_t* row_index, const void* W, int64_t ldw,
                      int B, int Vr, int H, const float* temperatures, uint64_t seed, int64_t* tokens_out, void* stream);

/* Host copies of the fused sampler's generator, for tests (no CUDA call): the
 * 32 random bits behind E for (vocab_id, row `token`) in call number `call`
 * (u = ((bits >> 9) + 0.5) * 2^-23), and Philox4x32-10 itself. */
int b2_sampler_noise_bits(uint64_t seed, uint32_t vocab_id, uint32_t token, uint32_t call, uint32_t* bits);
int b2_philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]);

/* ---- sampled-token broadcast: replaces the data the reference ships from
 *      rank 0 to the other ranks inside its pickled "run" message
 *      (nanovllm/engine/model_runner.py:76-89: the next step's last_token of
 *      every sequence) ---------------------------------------------------------
 * buf: int64 [n] on every rank, n <= max_seqs, values >= 0.  Rank 0's values
 * are written into every other rank's buf by the end of the call's kernel.
 * No-op when world == 1. */
int b2_broadcast_tokens(b2_ctx* ctx, int64_t* buf, int n, void* stream);

/* ---- next decode step's inputs, computed on the device: what
 *      ModelRunner.prepare_decode builds on the host every step
 *      (nanovllm/engine/model_runner.py:172-188) -------------------------------
 * For i < n: input_ids[i] = tokens[i]; positions[i] += 1; context_lens[i] += 1;
 * slot_mapping[i] = block_tables[i, positions[i] / block_size] * block_size
 *                   + positions[i] % block_size.  block_tables int32 with
 * bt_width columns and row stride bt_stride.  Lets consecutive decode steps
 * run without a host round trip.  A row that has run out of room - its next
 * position lies past the table's width, its table entry is -1, the slot would
 * be >= num_slots (slots in the KV cache), or its slot already is -1 (a padded
 * or frozen row) - is frozen: slot_mapping[i] = -1 (it stores no K/V), its
 * position and context length stay as they are. */
int b2_advance_decode(const int64_t* tokens, int64_t* input_ids, int64_t* positions, int32_t* context_lens,
                      int32_t* slot_mapping, const int32_t* block_tables, int64_t bt_stride, int bt_width,
                      int block_size, int64_t num_slots, int n, void* stream);

/* ---- elementwise neighbours of the path (the reference generates these with
 *      torch.compile -> Triton) ----------------------------------------------
 * SiluAndMul.forward (nanovllm/layers/activation.py:8-11):
 * out[M,I] = silu(x[:, :I]) * x[:, I:], x row stride ldx. */
int b2_silu_and_mul(const void* x, int64_t ldx, int M, int I, void* out, void* stream);

/* q/k head RMSNorm (nanovllm/models/qwen3.py:82-84) + neox RoPE
 * (nanovllm/layers/rotary_embedding.py:37-48) + paged-KV scatter of the
 * resulting K and of V (nanovllm/layers/attention.py:59-63), in place on the
 * qkv GEMM output [M, (nq + 2*nkv)*head_dim] (row stride ld_qkv).  positions
 * int64 [M]; cos_sin fp32 [max_pos, head_dim] (cos || sin).  q_norm_w /
 * k_norm_w may both be NULL (no head norm).  k_cache may be NULL (no scatter,
 * as during the reference's warm-up, nanovllm/layers/attention.py:57,62).
 * head_dim must be 128 or 64. */
int b2_qk_norm_rope_store(void* qkv, int64_t ld_qkv, int M, int nq, int nkv, int head_dim,
                          const void* q_norm_w, const void* k_norm_w, float eps,
                          const int64_t* positions, const float* cos_sin,
                          void* k_cache, void* v_cache, const int32_t* slot_mapping, void* stream);

/* Greedy pick: out[i] = argmax_j logits[i, j] (first index on ties), int64.
 * The reference's Sampler (nanovllm/layers/sampler.py:7-12) at temperature -> 0. */
int b2_argmax(const void* logits, int64_t ld, int B, int V, int64_t* out, void* stream);

/* ---- the launch planner as data (no counterpart in the reference; no CUDA
 *      call, usable without a GPU) -------------------------------------------
 * How the GEMM entry points would split a problem over the device: which
 * operand layout and tile width, how many CTAs share the K blocks, and which
 * kernel runs.  The host tests use it to check that every K block of every
 * output tile is computed exactly once for any shape. */
typedef struct b2_gemm_plan {
  int swap;          /* 1: weights on the 128-row side of the MMA (M <= 256)     */
  int bn;            /* rows of the other operand's tile                         */
  int tiles_p, tiles_q, kblocks; /* tile grid and 64-wide K blocks per tile      */
  int gemm_ctas;     /* CTAs that share the GEMM work                            */
  int round_robin;   /* 1: whole tiles dealt round-robin (no split tiles)        */
  int grid;          /* CTAs launched                                            */
  int cluster_split; /* > 0: cluster kernel, K split this many ways; 0: stream-K */
} b2_gemm_plan;

/* epilogue: 0 = b2_gemm / b2_lm_head / b2_gemm_silu_mul / b2_qkv_fused,
 * 1 = b2_rowpar_fused (one-shot form), 2 = b2_rowpar_fused_twoshot, 3 = b2_lm_head_sample,
 * 4 = b2_rowpar_fused (row-owner form).  resident_clusters: NULL
 * (cluster kernel not considered) or int[18]: entry [S] for 32-token tiles and
 * [9 + S] for 64-token tiles = clusters of S CTAs the device holds at once
 * (on a GPU the library asks the occupancy calculator). */
int b2_plan_gemm(int epilogue, int M, int N, int K, int num_sms, const int* resident_clusters, b2_gemm_plan* plan);
/* The same with planner options: bit 0 = one whole tile per CTA when a many-token problem fits one wave (what
 * B2_OPT_WHOLE_TILES switches on for the fused row-parallel launches). */
int b2_plan_gemm_opts(int epilogue, int M, int N, int K, int num_sms, const int* resident_clusters, int options,
                      b2_gemm_plan* plan);

/* The K blocks CTA `cta` computes under `plan`, in order, as triples
 * (tile, k_block, starts_segment) written to units[3 * cap].  Returns their
 * number (which may exceed cap), or a negative error code if the producer's
 * and the consumers' walks over the plan disagree. */
int b2_plan_cta_units(const b2_gemm_plan* plan, int cta, int* units, int cap);

/* The CTAs that hold K blocks of output tile `tile`: first_cta .. last_cta.
 * The stream-K kernel's "last arriver stores" counter expects exactly
 * last - first + 1 arrivals. */
int b2_plan_tile_contributors(const b2_gemm_plan* plan, int tile, int* first_cta, int* last_cta);

/* Which kernel the calling thread's most recent GEMM-shaped call launched: 0 = persistent stream-K kernel,
 * 1 = cluster split-K kernel, 2 = CTA-pair kernel (problems of at least 512 tokens). */
int b2_last_gemm_kernel(void);

/* Two-shot row ownership: the rank that reduces token row `token` (blocks of
 * 16 rows dealt round-robin) and the row's index in that rank's inbox; the
 * number of rows of an M-row call that `rank` owns.  Negative on bad input. */
int b2_row_owner(int token, int world, int* local_row);
int b2_owned_rows(int M, int world, int rank);
/* The same for the row-owner form of b2_rowpar_fused: row t belongs to rank
 * t mod world, at row t / world of that rank's inbox. */
int b2_owner_form_row(int token, int world, int* local_row);
int b2_owner_form_rows(int M, int world, int rank);

#ifdef __cplusplus
}
#endif
#endif /* B200TP_H */
