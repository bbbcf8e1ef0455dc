/*
 * vn_b200.h -- C ABI of the B200 (sm_100a) speculative-decoding library.
 *
 * The reference (CUI-hyg/VerseNext) has no C FFI for this path: its only
 * native binding is the PyO3 module `verse_rs` (packages/verse_torch/src/lib.rs:51-65),
 * which is not on the decode path.  These entry points are what a ctypes /
 * cffi stub inside the reference's Python packages binds instead of the
 * NumPy / torch calls cited beside each group.
 *
 * Conventions
 *  - every function returns an int32 status (VN_OK == 0); nothing throws or
 *    aborts across this boundary; vn_last_error() gives the message.
 *  - pointers named *_dev are device pointers obtained from vn_alloc();
 *    all other pointers are host memory owned by the caller.
 *  - one vn_ctx per GPU; all work of a context is issued on its one stream.
 *  - matrices are row-major; weights are (out_features, in_features) as in
 *    the reference's Linear (verse_torch/vnnn.py:394-430).
 */
#ifndef VN_B200_H
#define VN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum vn_status {
  VN_OK = 0,
  VN_ERR_INVALID = 1,     /* bad argument            -> ValueError   */
  VN_ERR_OOM = 2,         /* device allocation failed -> MemoryError */
  VN_ERR_OVERFLOW = 3,    /* KV cache capacity        -> RuntimeError (kv_cache_parallel.py:152-159) */
  VN_ERR_TIMEOUT = 4,     /* a bounded device wait ran out */
  VN_ERR_CUDA = 5,        /* CUDA runtime error       -> RuntimeError */
  VN_ERR_NCCL = 6,
  VN_ERR_INDEX = 7,       /* layer / sequence index   -> IndexError (kv_cache_parallel.py:136-139) */
  VN_ERR_UNSUPPORTED = 8
};

enum vn_dtype { VN_F32 = 0, VN_BF16 = 1, VN_I8 = 2, VN_I4 = 3, VN_I64 = 4, VN_I32 = 5, VN_U8 = 6 };

typedef struct vn_ctx vn_ctx;
typedef struct vn_model vn_model;
typedef struct vn_kv vn_kv;
typedef struct vn_comm vn_comm;

/* ---- lifecycle ------------------------------------------------------- */
int32_t vn_version(void);
int32_t vn_ctx_create(int32_t device, vn_ctx** out);
int32_t vn_ctx_destroy(vn_ctx* ctx);
const char* vn_last_error(vn_ctx* ctx);       /* ctx may be NULL: last error of the calling thread */
int32_t vn_sync(vn_ctx* ctx);
/* number of kernels this context has launched since creation */
int32_t vn_launch_count(vn_ctx* ctx, uint64_t* out);
/* opaque handle of the context's CUDA stream (cudaStream_t) */
int32_t vn_stream(vn_ctx* ctx, void** out);

/* ---- memory (replaces Tensor.to(device): verse_torch/tensor.py:394) --- */
int32_t vn_alloc(vn_ctx* ctx, size_t bytes, void** out_dev);
int32_t vn_free(vn_ctx* ctx, void* dev);
int32_t vn_memset(vn_ctx* ctx, void* dev, int32_t byte, size_t bytes);
int32_t vn_h2d(vn_ctx* ctx, void* dst_dev, const void* src, size_t bytes);   /* synchronous */
int32_t vn_d2h(vn_ctx* ctx, void* dst, const void* src_dev, size_t bytes);   /* synchronous */
int32_t vn_d2d(vn_ctx* ctx, void* dst_dev, const void* src_dev, size_t bytes);
/* `rows` rows of width_bytes each between two pitched device buffers (asynchronous, on the context's stream) */
int32_t vn_copy_2d(vn_ctx* ctx, void* dst_dev, size_t dst_pitch, const void* src_dev, size_t src_pitch, size_t width_bytes,
                   size_t rows);
int32_t vn_host_alloc(vn_ctx* ctx, size_t bytes, void** out);                /* pinned */
int32_t vn_host_free(vn_ctx* ctx, void* p);
int32_t vn_h2d_async(vn_ctx* ctx, void* dst_dev, const void* src_pinned, size_t bytes);
int32_t vn_d2h_async(vn_ctx* ctx, void* dst_pinned, const void* src_dev, size_t bytes);
int32_t vn_mem_info(vn_ctx* ctx, size_t* free_bytes, size_t* total_bytes);

/* ---- device timing on the context's stream --------------------------- */
int32_t vn_event_create(vn_ctx* ctx, void** out_event);
int32_t vn_event_destroy(vn_ctx* ctx, void* event);
int32_t vn_event_record(vn_ctx* ctx, void* event);
int32_t vn_event_elapsed_ms(vn_ctx* ctx, void* start, void* stop, float* out_ms); /* synchronises on stop */
/* Per-kernel timing: while enabled, every launch of this context is bracketed by CUDA events on
 * its stream.  vn_profile(ctx, 1) clears and starts, vn_profile(ctx, 0) clears and stops;
 * vn_profile_report writes {"kernel": {"launches": n, "ms": total}, ...} as JSON text. */
int32_t vn_profile(vn_ctx* ctx, int32_t enable);
int32_t vn_profile_report(vn_ctx* ctx, char* buf, size_t buf_bytes);
/* overwrite a scratch buffer twice the size of L2 (bench hygiene) */
int32_t vn_flush_l2(vn_ctx* ctx);

/* ---- DeviceBackend ops, fp32 (verse_torch/device.py:219-270, :285-335) - */
/* c[b] = a[b] @ b[b]; a: batch x M x K, b: (batch | 1) x K x N */
int32_t vn_matmul(vn_ctx* ctx, const float* a_dev, const float* b_dev, float* c_dev,
                  int64_t batch, int64_t M, int64_t N, int64_t K, int32_t b_broadcast);
/* y = x @ w.T + bias; x: M x K, w: N x K */
int32_t vn_linear(vn_ctx* ctx, const float* x_dev, const float* w_dev, const float* bias_dev,
                  float* y_dev, int64_t M, int64_t N, int64_t K);
/* softmax over the middle axis of an (outer, n, inner) view; inner == 1 for the last axis */
int32_t vn_softmax(vn_ctx* ctx, const float* x_dev, float* y_dev, int64_t outer, int64_t n, int64_t inner);
int32_t vn_layernorm(vn_ctx* ctx, const float* x_dev, const float* w_dev, const float* b_dev,
                     float* y_dev, int64_t rows, int64_t cols, float eps);
int32_t vn_rmsnorm(vn_ctx* ctx, const float* x_dev, const float* w_dev, float* y_dev,
                   int64_t rows, int64_t cols, float eps);
/* NeoX half-split rotation; x: outer x T x D, cos/sin: T x half (D/2) */
int32_t vn_rope(vn_ctx* ctx, const float* x_dev, const float* cos_dev, const float* sin_dev,
                float* y_dev, int64_t outer, int64_t T, int64_t D);
/* softmax(q k^T / sqrt(D) + mask) v; q: BH x Tq x D, k,v: BH x Tk x D, mask: Tq x Tk additive or NULL */
int32_t vn_attention(vn_ctx* ctx, const float* q_dev, const float* k_dev, const float* v_dev,
                     const float* mask_dev, float* out_dev, int64_t BH, int64_t Tq, int64_t Tk, int64_t D);

/* Row-level pieces of the acceptance rule for a vocabulary split across GPUs (no counterpart in the reference, which
 * has no sharded head; they are the kernels of vn_accept driven with softmax statistics supplied by the caller).
 * A rank holds V consecutive columns of R logit rows (row pitch in elements).  All pointers are device pointers.
 *   vn_row_stats:    per row max and sum exp(x - max) of logits / temperature over these columns (float32 exp,
 *                    float64 sum), and the scaled logit at column tokens[r] (-inf when the token is not one of these
 *                    columns, i.e. outside [0, V); pass ids relative to the first column).
 *   vn_row_residual: out_mass[r] = { sum max(0, p - q), sum p } over these columns, with p = exp(x - m_p) / s_p from
 *                    the GLOBAL statistics m_p, s_p (and m_q, s_q).  mode[r]: 0 skip, 1 residual of (p, q), 2 plain p,
 *                    3 p with column removed[r] zeroed (deterministic proposals).
 *   vn_row_pick:     inverse CDF over ascending columns of the same weights: the smallest column whose running
 *                    weight exceeds u[r] times this block's weight total; out_token[r] is relative to the first
 *                    column; rows with mode 0 are left untouched. */
int32_t vn_row_stats(vn_ctx* ctx, const float* logits_dev, int64_t row_stride, int32_t R, int32_t V, float temperature,
                     const int64_t* tokens_dev, float* out_max_dev, double* out_sum_dev, float* out_logit_dev);
int32_t vn_row_residual(vn_ctx* ctx, const float* p_dev, int64_t p_stride, const float* q_dev, int64_t q_stride, int32_t R,
                        int32_t V, float temperature, const int32_t* mode_dev, const float* m_p_dev, const double* s_p_dev,
                        const float* m_q_dev, const double* s_q_dev, const int64_t* removed_dev, double* out_mass_dev);
int32_t vn_row_pick(vn_ctx* ctx, const float* p_dev, int64_t p_stride, const float* q_dev, int64_t q_stride, int32_t R,
                    int32_t V, float temperature, const int32_t* mode_dev, const float* m_p_dev, const double* s_p_dev,
                    const float* m_q_dev, const double* s_q_dev, const int64_t* removed_dev, const float* u_dev,
                    int64_t* out_token_dev);

/* ---- collectives: the vocabulary-sharded LM head + acceptance is the one step of this path with an exchange.
 * The reference's only collective is torch.distributed.all_reduce in its training loop
 * (packages/verse_torch/verse_torch/training.py:2260-2266); nothing on its decode path communicates.
 * NCCL is bound at run time (libnccl.so.2); without it these calls return VN_ERR_NCCL.  One communicator per context,
 * all traffic on the context's stream, peers' data lands in this GPU's own memory before any kernel reads it. */
int32_t vn_comm_unique_id(uint8_t* out128);      /* rank 0 makes it, every rank passes the same 128 bytes below */
int32_t vn_comm_create(vn_ctx* ctx, const uint8_t* unique_id128, int32_t world, int32_t rank, vn_comm** out);
int32_t vn_comm_destroy(vn_comm* comm);
int32_t vn_comm_info(vn_comm* comm, int32_t* world, int32_t* rank);
/* recv_dev [world][bytes_per_rank] <- every rank's send_dev [bytes_per_rank]; asynchronous on the stream */
int32_t vn_all_gather(vn_comm* comm, const void* send_dev, void* recv_dev, size_t bytes_per_rank);
/* Acceptance with the vocabulary split over the ranks of `comm` (NULL: one rank), decisions taken on the device:
 * every rank passes its columns [v_lo, v_lo + Vs) of the target logits p_dev [Bt, k+1, Vs] and draft logits q_dev
 * [Bt, k, Vs] (or NULL) of ALL Bt = world x B_local sequences, and the draft tokens draft_dev [Bt, k]; three
 * all-gathers of a few numbers per row (softmax statistics, residual masses, the picked token) give every rank
 * the same out_len_dev [Bt] / out_tokens_dev [Bt, k+1] as vn_accept on the unsplit logits (full-vocabulary rule,
 * temperature > 0, bonus token).  Philox: sequence g draws as request g % B_local with seed + (g / B_local) *
 * seed_stride, i.e. what rank g / B_local draws in its own vn_accept calls when it folds its rank into the seed
 * the same way.  No host synchronisation. */
int32_t vn_shard_accept(vn_ctx* ctx, vn_comm* comm, const float* p_dev, const float* q_dev, const int64_t* draft_dev,
                        int32_t v_lo, int32_t Vs, float temperature, uint64_t seed, uint64_t seed_stride, uint32_t offset,
                        int32_t B_local, int32_t Bt, int32_t k, int32_t bonus, int32_t* out_len_dev,
                        int64_t* out_tokens_dev);

/* ---- acceptance / rejection sampling ---------------------------------- */
/* Replaces the argmax compare + accept loop of SpeculativeDecoder
 * (verse_nex/speculative.py:218-223, :280-287) and the softmax / top-k /
 * rng.choice sampling of cometspark.py:892-911.
 *   p_logits_dev  [B, k+1, V] fp32 target logits (row k is used only when bonus != 0;
 *                  with bonus == 0 it may hold k rows)
 *   q_logits_dev  [B, k, V] fp32 draft logits, or NULL: proposals were deterministic
 *   draft_dev     [B, k] int64
 *   u_accept_dev  [B, k] fp32 / u_sample_dev [B, k+1] fp32 injected uniforms, or both NULL:
 *                  Philox4x32-10, key = seed, counter = (position, row, purpose, offset)
 *   temperature <= 0 selects the greedy rule; top_k <= 0 disables top-k
 *   out_len_dev   [B] int32 number of accepted draft tokens
 *   out_tokens_dev[B, k+1] int64 committed tokens, padded with -1
 * k may be 0 (plain sampling of one token per row from p). */
int32_t vn_accept(vn_ctx* ctx, const float* p_logits_dev, const float* q_logits_dev,
                  const int64_t* draft_dev, const float* u_accept_dev, const float* u_sample_dev,
                  uint64_t seed, uint32_t offset, float temperature, int32_t top_k, int32_t bonus,
                  int32_t B, int32_t k, int32_t V, int32_t* out_len_dev, int64_t* out_tokens_dev);
/* Same rule on rows that are not contiguous: row (b, i) of p starts at
 * p_logits_dev + b * p_stride_b + i * p_stride_i (strides in elements), likewise q.
 * Lets the logits of [context, draft] (speculative.py:202-213) be used in place. */
int32_t vn_accept_strided(vn_ctx* ctx, const float* p_logits_dev, int64_t p_stride_b, int64_t p_stride_i,
                          const float* q_logits_dev, int64_t q_stride_b, int64_t q_stride_i,
                          const int64_t* draft_dev, const float* u_accept_dev, const float* u_sample_dev,
                          uint64_t seed, uint32_t offset, float temperature, int32_t top_k, int32_t bonus,
                          int32_t B, int32_t k, int32_t V, int32_t* out_len_dev, int64_t* out_tokens_dev);
/* vn_accept for callers that must not allocate.  It has no counterpart in the reference.
 * Some hosts drive this library from places where device allocation is forbidden or fails: inside a
 * serving loop whose memory pool already owns the whole GPU, under a framework that traps cudaMalloc
 * after start-up, or in a latency-critical thread where an allocation's implicit device
 * synchronisation is not acceptable.  vn_accept grows a scratch buffer on demand; this variant keeps
 * its scratch (chunk statistics, decisions, residual masses) in a fixed 2 MiB array that is part of
 * the library image on every GPU that loads it, and calls no cudaMalloc / cudaFree or any other
 * allocating routine.
 *   - full-vocabulary rule and greedy rule only (no top-k argument); contiguous [B, k+1, V] /
 *     [B, k, V] inputs as for vn_accept; the caller still owns inputs and outputs;
 *   - sizes whose scratch exceeds the array (B * (2k+1) * ceil(V/4096) * 16 bytes plus about
 *     1 KB per sequence must stay below 2 MiB: e.g. B=128, k=4, V=248320 fits, B=256 does not)
 *     are rejected with VN_ERR_INVALID and a message that names both numbers;
 *   - the first call on a device looks up the array's device address (the CUDA runtime may load the
 *     library's device code at that moment, which is when the 2 MiB become resident): make that first
 *     call at start-up, before any stream capture is begun;
 *   - a round counter installed with vn_set_offset_source shifts the Philox offset as it does for vn_accept;
 *   - all calls share the one array: two calls that overlap on the GPU (different contexts /
 *     streams of the same device) race; calls on one context are ordered by its stream. */
int32_t vn_accept_noalloc(vn_ctx* ctx, const float* p_logits_dev, const float* q_logits_dev,
                          const int64_t* draft_dev, const float* u_accept_dev, const float* u_sample_dev,
                          uint64_t seed, uint32_t offset, float temperature, int32_t bonus,
                          int32_t B, int32_t k, int32_t V, int32_t* out_len_dev, int64_t* out_tokens_dev);
/* One token per row of logits (row r at logits_dev + r * row_stride): argmax when temperature <= 0,
 * else inverse-CDF draw from softmax(logits / T) restricted to the top-k (cometspark.py:892-911).
 * uniforms_dev [R] or NULL: Philox counter (position, row, purpose, offset). */
int32_t vn_sample(vn_ctx* ctx, const float* logits_dev, int64_t row_stride, int32_t R, int32_t V, float temperature,
                  int32_t top_k, const float* uniforms_dev, uint64_t seed, uint32_t offset, uint32_t position,
                  uint32_t purpose, int64_t* out_tokens_dev);
/* vn_sample that also leaves every row's kept list -- the (token, scaled logit) pairs at or above the k-th largest
 * value, ascending token id -- in lists_out_dev ([R] records of vn_topk_row_bytes() bytes each, or NULL): a draft
 * model samples its proposal from that list, and vn_verify_accept later needs the very same list as q. */
int32_t vn_sample_lists(vn_ctx* ctx, const float* logits_dev, int64_t row_stride, int32_t R, int32_t V, float temperature,
                        int32_t top_k, const float* uniforms_dev, uint64_t seed, uint32_t offset, uint32_t position,
                        uint32_t purpose, int64_t* out_tokens_dev, void* lists_out_dev);
size_t vn_topk_row_bytes(void);
/* Philox uniforms exactly as vn_accept draws them (for tests) */
int32_t vn_philox_uniform(vn_ctx* ctx, uint64_t seed, uint32_t offset, int32_t B, int32_t n,
                          int32_t purpose, float* out_dev);

/* ---- target / draft model (verse_nex/cometspark.py:294-698) ------------ */
/* config_json: the keyword arguments of CometSparkNexLM.__init__ (cometspark.py:334-364)
 * plus "embedding_scale" (spark/src/base_model.py:161) and "dtype": "f32" | "bf16".
 * "layer_pattern" takes every kind of VerseNexBlock.VALID_KINDS (cometspark.py:110): "trisparse", "mod", and the
 * delta attention kinds "vda", "dsa", "kda", "gmla" (verse_nex/delta_attention.py; "anchor_interval", "latent_dim").
 * A delta layer computes the whole-sequence forward of its class on the cache (masks from absolute positions). */
int32_t vn_model_create(vn_ctx* ctx, const char* config_json, vn_model** out);
int32_t vn_model_destroy(vn_model* m);
/* name: dotted state_dict name (verse_torch/vnnn.py:235-252); data: host fp32, C order */
int32_t vn_model_load_tensor(vn_model* m, const char* name, const float* data,
                             int32_t ndim, const int64_t* shape);
/* checks that every tensor arrived, precomputes sink K/V and the RoPE table */
int32_t vn_model_finalize(vn_model* m);
/* weight-only quantisation of every Linear: "int8" (per output channel,
 * quantize.py:187-214), "int4" (per output channel, :231-258), "int4g128" */
int32_t vn_model_quantize(vn_model* m, const char* scheme);
int32_t vn_model_param_bytes(vn_model* m, uint64_t* out);
/* The quantiser on its own: w_dev float32 [rows, K] (device) -> q_dev and scale_dev (device), byte for byte what
 * quantize_int8 / quantize_int4 + _pack_int4 return (verse_torch/quantize.py:187-258, :36-66):
 *   "int8"      q int8 [rows, K],                scale float32 [rows]
 *   "int4"      packed uint8 [rows, ceil(K/2)],  scale float32 [rows]   (even index in the low nibble)
 *   "int4g128"  packed uint8 [rows, K/2],        scale float32 [rows, ceil(K/128)] holding bf16-representable values */
int32_t vn_quantize(vn_ctx* ctx, const float* w_dev, int64_t rows, int32_t K, const char* scheme, void* q_dev,
                    float* scale_dev);
/* One linear that is already quantised -- the `packed` and `scale` arrays of a reference QuantizedLinear
 * (verse_torch/quantize.py:382-440; scale (rows, 1) float32) -- goes to the device as it is, no re-quantisation.
 * name: the linear's state_dict name ("blocks.3.attn.wq.weight", "head.weight", ...); host pointers.  A model takes
 * all its linears this way or none (the other tensors still arrive through vn_model_load_tensor); the head needs
 * its own quantised copy, as the reference's compressed models have (compress.py:817-822).  bf16 models only. */
int32_t vn_model_load_quant_tensor(vn_model* m, const char* name, const char* scheme, const void* packed,
                                   const float* scale, int64_t rows, int64_t K);
/* Read the quantised bytes and the scales of one linear back (host buffers of exactly the tensor's size):
 * what vn_model_quantize produced on the device, or what vn_model_load_quant_tensor was given. */
int32_t vn_model_read_quant(vn_model* m, const char* name, void* q_host, size_t q_bytes, float* scale_host,
                            size_t n_scales);
/* LM head restricted to vocabulary columns [v_lo, v_lo + n_cols): out[r, j] = hidden[r] . head.weight[v_lo + j]
 * for `rows` rows of final-norm hidden states (float32 [rows, dim], as vn_model_forward returns them in
 * out_hidden); out row pitch out_ld floats.  The building block of a head split by columns over several GPUs
 * (no counterpart in the reference, whose head is one Linear, cometspark.py:690-696). */
int32_t vn_model_head(vn_model* m, const float* hidden_dev, int32_t rows, int32_t v_lo, int32_t n_cols,
                      float* out_logits_dev, int64_t out_ld);
/* Which ALiBi rule the following forwards of this model use.  0 (default): the whole-sequence forward's -- every
 * earlier key, path switched off once more than 1024 keys are visible (tri_sparse_attn.py:489-530, :600).
 * Non-zero: the one-token recurrent step's -- its state keeps the last window_size keys only, so the path sees
 * those and stays on while that count is at most 1024 (tri_sparse_attn.py:676-731).  No effect without ALiBi. */
int32_t vn_model_set_recurrent(vn_model* m, int32_t on);
/* A small bf16 model whose layers are all TriSparse (the draft of a speculative round; at most 4 layers, dim <= 256,
 * head_dim 64, no RoPE, at most 64 new rows per forward) can run its whole layer stack and the final norm as ONE
 * cooperative kernel whose CTAs meet at bounded grid barriers, instead of a chain of launches.  Off by default (the
 * chain is as fast on B200); non-zero switches it on for this model.  The two agree to rounding: the order of
 * summation inside a dot product differs.  A barrier wait that runs out raises the same time-out condition as the
 * GEMM kernels' waits (vn_model_status returns VN_ERR_TIMEOUT), and the kernel still terminates. */
int32_t vn_model_set_fused_stack(vn_model* m, int32_t on);
/* Every wait inside the tensor-core GEMM kernels (for a pipeline stage, for the accumulator) gives up after a limit
 * and raises the time-out condition that vn_model_status reports; the kernel then drains and returns, the context
 * stays usable.  vn_model_set_wait_limit sets that limit in SM cycles for this GPU (0: the default, about a second).
 * vn_model_probe_wait runs one such wait that nothing ever ends -- a barrier no one arrives at -- so that the whole
 * path (limit, error word, status, exception) can be exercised without a fault: it returns VN_OK, the wait's length
 * goes to *waited_cycles, and the next vn_model_status returns VN_ERR_TIMEOUT. */
int32_t vn_model_set_wait_limit(vn_model* m, uint64_t cycles);
int32_t vn_model_probe_wait(vn_model* m, int64_t* waited_cycles);
/* Device-side conditions raised by forwards since the last call, read after a stream synchronisation and
 * cleared: *bad_token != 0 when a token id outside [0, vocab) was met (the kernels clamp it instead of reading
 * outside the embedding table; the reference raises IndexError from NumPy fancy indexing, vnnn.py:453-460);
 * *wait_timeout != 0 when a bounded wait inside a kernel ran out (the affected logits are undefined).
 * Returns VN_OK when both are clear, VN_ERR_INDEX for a bad token, VN_ERR_TIMEOUT for a timeout. */
int32_t vn_model_status(vn_model* m, int32_t* bad_token, int32_t* wait_timeout);

/* KV cache: per attention module K and V of shape [max_batch, max_seq, n_kv_head, head_dim]
 * with per-sequence lengths (verse_nex/kv_cache_parallel.py:42-283).  One K / V pair per layer, three (DSA, KDA,
 * GMLA) for a "vda" layer; vn_kv_read's `layer` counts these pairs.  A GMLA module caches the K / V rebuilt from
 * its latents. */
int32_t vn_kv_create(vn_model* m, int32_t max_batch, int32_t max_seq, vn_kv** out);
int32_t vn_kv_destroy(vn_kv* kv);
/* A second handle on sequences [first, first + count) of a cache: forwards, commits, resets and length calls on it
 * act on those sequences only (a serving loop prefills one free slot while the others keep their state).  The view
 * shares the parent's memory; destroy it before the parent. */
int32_t vn_kv_view(vn_kv* kv, int32_t first, int32_t count, vn_kv** out);
int32_t vn_kv_reset_seq(vn_kv* kv, int32_t seq);          /* seq < 0: all */
int32_t vn_kv_lengths(vn_kv* kv, int32_t* out_host);      /* [max_batch] */
int32_t vn_kv_set_lengths(vn_kv* kv, const int32_t* lens_host);
/* Commit / roll back the entries appended by the last forward of `n_new`
 * positions: sequence b keeps slots keep_idx[b*stride .. +n_keep[b]) (slot
 * numbers 0..n_new-1, ascending), compacted in place behind its committed
 * prefix; everything else appended is dropped.  keep_idx_dev == NULL keeps
 * the first n_keep[b] slots (chain proposals). */
int32_t vn_kv_commit(vn_kv* kv, int32_t n_new, const int32_t* keep_idx_dev, int32_t stride,
                     const int32_t* n_keep_dev, int32_t keep_add /* kept = n_keep[b] + keep_add */);
int32_t vn_kv_read(vn_kv* kv, int32_t layer, int32_t seq, int32_t which /*0=k 1=v*/, float* out_host,
                   int32_t n_positions);

/* One forward over T new positions per sequence on top of the cache.
 *   tokens_dev [B, T] int64; parents_host [T] int32 tree parents (-1 = child of the last
 *   committed token) or NULL for a chain.  Appends K/V at slots len[b] .. len[b]+T-1
 *   and advances nothing: call vn_kv_commit to make them permanent.
 *   out_hidden_dev [B, T, dim] fp32 or NULL; out_logits_dev [B, T, V] fp32 or NULL;
 *   last_only != 0: logits / hidden of the last position only ([B, 1, ...]).
 *   slot_offset: the new positions start behind `slot_offset` entries that earlier forwards
 *   appended and that are not committed yet (a draft model proposing token by token). */
int32_t vn_model_forward(vn_model* m, vn_kv* kv, const int64_t* tokens_dev, int32_t B, int32_t T,
                         const int32_t* parents_host, float* out_hidden_dev, float* out_logits_dev,
                         int32_t last_only, int32_t slot_offset);

/* The draft side of one speculative round with a draft MODEL (the north star's replacement for the k linear heads of
 * SpeculativeDecoder.draft, speculative.py:110-162): k proposals per request, token by token, all on the device.
 *   pair_dev [B, 2] int64: the last two committed tokens of every request; the draft's cache holds everything
 *   before them.  Step 0 forwards both (slots len, len + 1), step i > 0 forwards proposal i - 1 (slot len + i + 1);
 *   nothing is committed: after the round keep the first n entries with vn_kv_commit(kv, k + 1, ...).
 *   Step i writes its last-position logits to q_logits_dev [k, B, V] (the acceptance test needs q), samples with
 *   the Philox counter (position i, row b, purpose 2, offset) -- argmax when temperature <= 0 -- into
 *   step_tokens_dev [k, B], and, when q_lists_dev is given ([k, B] records of vn_topk_row_bytes() bytes), leaves the
 *   kept top-k list there for vn_verify_accept.  No synchronisation, no allocation once the model's buffers have the
 *   size: the whole call can sit inside a captured graph. */
int32_t vn_draft_propose(vn_model* draft, vn_kv* kv, const int64_t* pair_dev, int32_t B, int32_t k, float temperature,
                         int32_t top_k, uint64_t seed, uint32_t offset, float* q_logits_dev, int64_t* step_tokens_dev,
                         void* q_lists_dev);

/* Verify + accept in one call: the target forward over the T = k (+1 with bonus) new positions of every sequence
 * (tokens_dev [B, T]: last committed token, then the proposals), the LM head, and the acceptance rule of vn_accept
 * -- replaces head(x) (cometspark.py:690-697), the softmax / top-k (cometspark.py:892-911) and the compare
 * (speculative.py:216-223) of one verification round.  With temperature > 0 and 0 < top_k < vocab on a bf16 model
 * the head is FUSED with the selection: a GEMM over the first 8,192 vocabulary columns bounds every row's k-th
 * largest logit from below, the full head GEMM's epilogue keeps only the logits at or above that bound (a few
 * hundred per row), and the decisions are taken on those lists -- the [B, T, V] logits are never written.  Results
 * are those of vn_model_forward + vn_accept_strided bit for bit.  p_logits_scratch_dev [B, T, V] must be supplied:
 * it is written only when a row has so many ties at its bound that its candidate list (4,096 entries) overflows
 * -- a device flag then switches the stored-logits path on inside the same launch sequence -- and whenever the
 * fused head does not apply (greedy or full-vocabulary rule, fp32 or quantised model), where this call is the
 * forward followed by vn_accept_strided.
 *   q of the draft rows: q_lists_dev (records left by vn_sample_lists; row (b, i) at record b * ql_stride_b +
 *   i * ql_stride_i) and / or q_logits_dev with element strides as in vn_accept_strided (the fused head prefers
 *   the lists, the stored-logits route needs the logits), or both NULL (point-mass proposals).  Uniforms, seed, offset, outputs: as vn_accept.  Appends K/V like vn_model_forward: commit with
 *   vn_kv_commit. */
int32_t vn_verify_accept(vn_model* m, vn_kv* kv, const int64_t* tokens_dev, int32_t B, int32_t T, int32_t k,
                         const void* q_lists_dev, int64_t ql_stride_b, int64_t ql_stride_i, const float* q_logits_dev,
                         int64_t q_stride_b, int64_t q_stride_i, const int64_t* draft_dev, const float* u_accept_dev,
                         const float* u_sample_dev, uint64_t seed, uint32_t offset, float temperature, int32_t top_k,
                         int32_t bonus, float* p_logits_scratch_dev, int32_t* out_len_dev, int64_t* out_tokens_dev);

/* ---- round bookkeeping on the device (no counterpart in the reference: its loop is host code,
 *      speculative.py:280-293) -------------------------------------------------------------------- */
/* step_tokens_dev [k, B] proposals per draft step, pair_dev [B, 2] last two committed tokens ->
 * draft_dev [B, k] and verify_dev [B, n_verify] = (last committed, d_0, .., d_{n_verify-2}) */
int32_t vn_spec_gather(vn_ctx* ctx, const int64_t* step_tokens_dev, const int64_t* pair_dev, int32_t B, int32_t k,
                       int32_t n_verify, int64_t* draft_dev, int64_t* verify_dev);
/* fold one round's committed tokens (out_tokens_dev [B, k+1], -1 padded) into pair_dev, the per-request
 * history_dev [B, cap] / count_dev [B], and n_commit_dev [B] = tokens committed this round */
int32_t vn_spec_advance(vn_ctx* ctx, const int64_t* out_tokens_dev, int32_t B, int32_t k, int64_t* pair_dev,
                        int64_t* history_dev, int32_t cap, int32_t* count_dev, int32_t* n_commit_dev);

/* Tree proposals (the north star's "batched or tree verification", greedy rule).
 * vn_top_m: the m (<= 8) largest logits of each of R rows, best first, ties to the lower token id: the children a
 *   draft proposes under one tree node.  Row r at logits_dev + r * row_stride; tokens to out_dev[r * out_stride + j].
 * vn_tree_accept_greedy: after the target scored a tree (vn_model_forward with parents over T rows per sequence:
 *   row 0 = the last committed token, rows 1 .. T-1 the nodes; parent_dev [T] = row of each row's parent, -1 for
 *   row 0) and its arg-max per row is in target_arg_dev [B, T]: walk from row 0 along the children that carry the
 *   target's token.  out_len_dev [B] = nodes accepted (<= depth), out_tokens_dev [B, depth + 1] = their tokens plus
 *   the target's token at the stop, -1 padded -- exactly what greedy decoding of the target alone emits
 *   (speculative.py:280-287 generalised from a chain to a tree).  keep_target_dev / keep_draft_dev [B, depth + 1]:
 *   slot lists for vn_kv_commit of the two caches (count = accepted + 1 for both; the draft is taken to have
 *   appended the last two committed tokens at slots 0, 1 and node row r at slot r + 1). */
int32_t vn_top_m(vn_ctx* ctx, const float* logits_dev, int64_t row_stride, int32_t R, int32_t V, int32_t m,
                 int64_t* out_dev, int64_t out_stride);
int32_t vn_tree_accept_greedy(vn_ctx* ctx, const int64_t* tokens_dev, const int64_t* target_arg_dev, const int32_t* parent_dev,
                              int32_t B, int32_t T, int32_t depth, int32_t* out_len_dev, int64_t* out_tokens_dev,
                              int32_t* keep_target_dev, int32_t* keep_draft_dev);

/* Stochastic acceptance on a verified tree (temperature > 0; no counterpart in the reference).  The children of a
 * node are fixed proposals (vn_top_m), so the test is rejection sampling with point-mass proposals applied child after
 * child: child c with token x is accepted iff u * R < p(x), R = the mass not yet rejected at that row; a rejected x
 * leaves the support.  Every committed token then has exactly its target probability p(x) -- p = softmax(logits / T)
 * over the top-k set, read from the rows' kept lists.  Where no child is accepted, or the path is `depth` long, the
 * row's own token is drawn from p without the rejected children.
 *   lists_dev: [B * T] records left by vn_sample_lists on the target's logits of all T rows (row 0 = after the last
 *   committed token, row r = after node row r); tokens_dev [B, T], parent_dev [T] as for vn_tree_accept_greedy; a
 *   row has at most 8 children.  u_child_dev / u_sample_dev [B, T]: injected uniforms (tests), or both NULL: Philox
 *   (seed, offset + the device round counter; row b, position = row index, purpose 0 for a child's test, 1 for the
 *   final draw).  Outputs as vn_tree_accept_greedy. */
int32_t vn_tree_accept_sample(vn_ctx* ctx, const void* lists_dev, const int64_t* tokens_dev, const int32_t* parent_dev,
                              int32_t B, int32_t T, int32_t depth, const float* u_child_dev, const float* u_sample_dev,
                              uint64_t seed, uint32_t offset, int32_t* out_len_dev, int64_t* out_tokens_dev,
                              int32_t* keep_target_dev, int32_t* keep_draft_dev);

/* Device-side round counter: while set, every Philox offset passed to vn_accept* / vn_sample is
 * incremented by *counter_dev, and vn_spec_advance adds one to it at the end of a round. */
int32_t vn_set_offset_source(vn_ctx* ctx, const uint32_t* counter_dev);
/* CUDA-graph capture of everything issued on the context's stream between begin and end (one decode
 * round has a fixed launch sequence: lengths, tokens and the round counter all live on the device).
 * Nothing inside may allocate or synchronise: run the sequence once un-captured first. */
int32_t vn_graph_begin(vn_ctx* ctx);
int32_t vn_graph_end(vn_ctx* ctx, void** out_exec);
int32_t vn_graph_launch(vn_ctx* ctx, void* exec);
int32_t vn_graph_destroy(vn_ctx* ctx, void* exec);

#ifdef __cplusplus
}
#endif
#endif /* VN_B200_H */
