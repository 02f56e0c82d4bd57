/*
 * tarafer_b200 — C ABI of the B200-native batch-1 decode engine.
 *
 * The reference has no C ABI: its seam is the Rust-internal API of crates/core/src/cuda
 * (CudaModel / CudaKv).  Each entry point below names the reference item it stands in for
 * (paths relative to the reference project root), so that a Rust `extern "C"` module with
 * the reference's own method signatures can be a thin wrapper over this library.
 *
 * Conventions: every call returns 0 on success or a negative TFR_E_* code and never
 * throws or aborts; tfr_last_error() gives the message of the last failure on that
 * engine.  An engine is not thread-safe — the caller serialises access exactly as the
 * reference does (crates/cli/src/serve/mod.rs:28-32).  All device work runs on one CUDA
 * stream per engine.  After tfr_alloc_kv no call on the decode path allocates device
 * memory (crates/core/src/cuda/load.rs:547-607, "zero-allocation forward loop").
 * The library has no CPU fallback: without a usable CUDA device tfr_create fails.
 */
#ifndef TARAFER_B200_H
#define TARAFER_B200_H

#include <stddef.h>
#include <stdint.h>

/* Two builds come from the same sources.  libtarafer_b200.so is the product: the decode path, the loader, the stand-alone
 * operators and the read-only taps (tfr_debug_read).  libtarafer_b200_aids.so (-DTFR_TEST_AIDS) adds what only tests,
 * the timeline tool and the benchmark's model builder need: in-kernel timeline probes, the integer-contract taps, the
 * KV-store rounding as an operator and the synthetic K-quant quantiser.  Declarations of the second kind sit inside
 * #ifdef TFR_TEST_AIDS below.
 *
 * Environment variables the library reads (test and measurement aids; unset in normal use):
 *   TFR_ATTN_REGISTER_ROUTE=1   decode attention on short caches and the attention of prompt chunks stay on the CUDA-core
 *                               kernels for every head size (default: tensor cores for head sizes up to 128);
 *   TFR_GEMM_DP4A=1             the projections of prompt chunks and verification batches stay on the dp4a kernel
 *                               (default: int8 tensor-core MMAs for Q4_K / Q6_K matrices from five tokens on);
 *   TFR_LOOP_SLOTS, TFR_LOOP_LPB, TFR_LOOP_PBUF, TFR_LOOP_ATTN_KEYS, TFR_LOOP_ATTN_INLINE
 *                               sizes of the opt-in persistent decode loop (tfr_set_decode_path). */
#ifdef __cplusplus
extern "C" {
#endif

#define TFR_OK 0
#define TFR_E_INVALID (-1)  /* bad argument / shape / state */
#define TFR_E_CUDA (-2)     /* a CUDA call failed */
#define TFR_E_FULL (-3)     /* "context full", crates/core/src/cuda/forward.rs:46-48 */
#define TFR_E_EMPTY (-4)    /* "empty tokens", crates/core/src/cuda/forward.rs:43-45 */
#define TFR_E_UNSUPPORTED (-5)

/* ggml tensor type ids, crates/gguf/src/types.rs:7-60 */
#define TFR_TYPE_F32 0
#define TFR_TYPE_Q4_K 12
#define TFR_TYPE_Q6_K 14

typedef struct tfr_engine tfr_engine;
typedef struct tfr_kv tfr_kv;
typedef struct tfr_mat tfr_mat;

/* Fields of ModelConfig, crates/core/src/config.rs:67-104 (GGUF keys: config.rs:107-264). */
typedef struct {
    int32_t n_layer;        /* block_count */
    int32_t n_embd;         /* embedding_length */
    int32_t n_head;         /* attention.head_count */
    int32_t n_kv_head;      /* attention.head_count_kv */
    int32_t head_dim;       /* attention.key_length */
    int32_t n_ff;           /* feed_forward_length */
    int32_t n_vocab;        /* vocab_size */
    int32_t context_length; /* context_length */
    float rope_theta;       /* rope.freq_base */
    float rms_eps;          /* attention.layer_norm_rms_epsilon */
    int32_t hybrid;         /* 0 dense (qwen2), 1 Gated-DeltaNet hybrid (qwen35), backend.rs:19-31 */
    int32_t rope_dim;       /* rope.dimension_count (hybrid), 0 = head_dim */
    int32_t ssm_conv_kernel;
    int32_t ssm_state_size;
    int32_t ssm_group_count;     /* K/Q heads of the linear layers */
    int32_t ssm_time_step_rank;  /* V heads of the linear layers */
    int32_t ssm_inner_size;
    int32_t full_attention_interval; /* layer i is full attention iff (i+1) % interval == 0 */
    int32_t tp_rank;        /* tensor-parallel rank of this engine (0 when tp_size == 1) */
    int32_t tp_size;        /* 1 = single GPU */
} tfr_model_config;

/* ---- engine lifetime: CudaModel::load_with, crates/core/src/cuda/load.rs:166-609 ---- */

/* init_device (crates/core/src/cuda/device.rs:84-142) without NVRTC: kernels are ahead-of-time sm_100a code. */
int tfr_create(int device_ordinal, tfr_engine** out);
void tfr_destroy(tfr_engine* e);
const char* tfr_last_error(const tfr_engine* e);
/* gpu_name / compute_major / compute_minor fields of CudaModel, model.rs:19-29 */
int tfr_device_info(const tfr_engine* e, char* name, size_t name_cap, int* cc_major, int* cc_minor, int* sm_count);

int tfr_set_config(tfr_engine* e, const tfr_model_config* cfg);
/* upload_mat / upload_vec, load.rs:135-143 and 203-260.  Called once per GGUF tensor with
 * the tensor's name (load.rs:280-417), ggml type, dims[0] = n_rows (K, contiguous) and
 * dims[1] = n_cols (N; 1 for vectors) and the raw bytes.  `bytes` may be host or device
 * memory; the library copies (and re-orders Q6_K rows for aligned loads) — the caller keeps
 * ownership and may unmap the file after tfr_finalize_load. */
int tfr_upload_tensor(tfr_engine* e, const char* name, int ggml_type, int64_t n_rows, int64_t n_cols, const void* bytes,
                      size_t nbytes);
/* End of load_with: checks every tensor the configuration needs is present, allocates workspaces. */
int tfr_finalize_load(tfr_engine* e);

/* ---- GGUF files: crates/gguf/src/reader.rs:29-215 (GgufFile), value.rs, types.rs; host code only ----
 * tfr_gguf_open maps the file read-only and parses header, metadata and tensor table with the
 * reference reader's rules (magic, version 2 or 3, count and n_dims limits, known tensor types,
 * data section at the header's end rounded up to general.alignment (default 32), every tensor's
 * bytes inside the file).  On failure *out is NULL and err receives the reason.  Pointers returned
 * by the accessors live until tfr_gguf_close. */
typedef struct tfr_gguf tfr_gguf;
int tfr_gguf_open(const char* path, tfr_gguf** out, char* err, size_t err_cap);
void tfr_gguf_close(tfr_gguf* g);
int tfr_gguf_version(const tfr_gguf* g);
uint64_t tfr_gguf_data_offset(const tfr_gguf* g);
int64_t tfr_gguf_tensor_count(const tfr_gguf* g);
int64_t tfr_gguf_find_tensor(const tfr_gguf* g, const char* name); /* index or -1 (GgufFile::tensor) */
int tfr_gguf_tensor_info(const tfr_gguf* g, int64_t i, const char** name, int* ggml_type, int* n_dims, int64_t dims[4],
                         uint64_t* offset, uint64_t* nbytes);
const void* tfr_gguf_tensor_data(const tfr_gguf* g, int64_t i); /* GgufFile::tensor_data: the mapped bytes */
/* Metadata with the reference's lenient coercions (Value::as_u64 / as_f32 / as_str, value.rs:55-100);
 * a missing key or another kind of value returns TFR_E_INVALID.  Strings above 64 MiB and arrays above 10 M
 * items are refused (value.rs:163-183, 246-262), as is invalid UTF-8. */
int tfr_gguf_meta_u64(const tfr_gguf* g, const char* key, uint64_t* out);
int tfr_gguf_meta_f32(const tfr_gguf* g, const char* key, float* out);
int tfr_gguf_meta_str(const tfr_gguf* g, const char* key, const char** out);
int64_t tfr_gguf_meta_array_len(const tfr_gguf* g, const char* key);
/* Items of a metadata array (Value::Array, value.rs:246-262): what Tokenizer::from_gguf reads
 * (crates/core/src/tokenizer/mod.rs:27-106) - tokenizer.ggml.tokens / .merges (strings, not NUL-terminated: *len
 * bytes), .scores (floats), .token_type (integers).  TFR_E_INVALID for a missing key, another item kind or an
 * index past the end. */
int tfr_gguf_meta_array_str(const tfr_gguf* g, const char* key, int64_t i, const char** out, uint64_t* len);
int tfr_gguf_meta_array_f32(const tfr_gguf* g, const char* key, int64_t i, float* out);
int tfr_gguf_meta_array_i64(const tfr_gguf* g, const char* key, int64_t i, int64_t* out);
/* ModelConfig::from_gguf, crates/core/src/config.rs:107-264: `<arch>.*` keys, defaults and the qwen35 extras.
 * Architectures whose schedule this library does not build (smollm3's no-RoPE layers, mixture-of-experts
 * models) return TFR_E_UNSUPPORTED instead of being decoded as a plain dense model. */
int tfr_gguf_model_config(const tfr_gguf* g, tfr_model_config* out, char* err, size_t err_cap);
/* CudaModel::load_with(gguf), load.rs:166-417: tfr_set_config from the metadata, tfr_upload_tensor for every
 * tensor of the decode path straight from the mapping, tfr_finalize_load.  The file may be closed afterwards. */
int tfr_load_gguf(tfr_engine* e, const tfr_gguf* g, int tp_rank, int tp_size);

/* ---- KV cache: CudaKv, crates/core/src/cuda/kv.rs:6-42; alloc_kv model.rs:114-162 ---- */
int tfr_alloc_kv(tfr_engine* e, int max_seq, tfr_kv** out);
void tfr_free_kv(tfr_kv* kv);
int tfr_kv_len(const tfr_kv* kv);                 /* CudaKv::len */
int tfr_kv_max_seq(const tfr_kv* kv);             /* CudaKv::max_seq */
int tfr_kv_set_len(tfr_kv* kv, int len);          /* callers assign cache.len, session.rs:345 */
int tfr_kv_clear(tfr_kv* kv);                     /* CudaKv::clear */
int64_t tfr_kv_bytes_per_token(const tfr_kv* kv); /* CudaKv::bytes_per_token */
int tfr_zero_recurrent(tfr_engine* e, tfr_kv* kv); /* CudaModel::zero_recurrent, model.rs:165-194 */

/* ---- token loop ---- */
/* CudaModel::forward_greedy, forward.rs:42-71: feeds n tokens at positions kv.len.., returns the
 * greedy next token, advances kv.len by n.  n == 0 -> TFR_E_EMPTY, overflow -> TFR_E_FULL.
 * Prompts (n > 1) are fed through the decode kernels one position at a time. */
int tfr_forward_greedy(tfr_engine* e, tfr_kv* kv, const uint32_t* tokens, int n, uint32_t* next_token);
/* CudaModel::forward_greedy_all, forward.rs:268-290 (the verification primitive of speculative decoding,
 * session.rs:321-367): feeds tokens[0..n) at positions kv.len .. and returns in out[i] the greedy prediction
 * AFTER tokens[i]; kv.len advances by n.  The caller accepts a prefix and moves kv.len back with
 * tfr_kv_set_len (models with recurrent state cannot be moved back: their state has absorbed all n tokens). */
int tfr_forward_greedy_all(tfr_engine* e, tfr_kv* kv, const uint32_t* tokens, int n, uint32_t* out);
/* The on-device loop that replaces the per-token host round-trip of session.rs:288-368 /
 * forward.rs:73-105: starting from first_token at position kv.len, runs up to max_n decode
 * steps, each feeding the previous step's argmax, without returning to the host.  Stops
 * after emitting one of stop_ids (n_stop <= 8) or when the cache is full.  out receives the
 * emitted tokens, *n_out their count; kv.len advances by *n_out. */
int tfr_decode_burst(tfr_engine* e, tfr_kv* kv, uint32_t first_token, int max_n, const uint32_t* stop_ids, int n_stop,
                     uint32_t* out, int* n_out);
/* CudaModel::current_logits, forward.rs:20-39: logits of the last decoded position.  With
 * tp_size > 1 every rank holds the logits of its vocabulary rows only: the call fills
 * out[first, end) of tfr_tp_vocab_range and leaves the rest of out untouched. */
int tfr_current_logits(tfr_engine* e, float* out, int n);
/* The reference's vocabulary shortlist, load.rs:285-352 (an approximation it reports on stderr): the head runs
 * over ids [0, limit) and, when special_id lies in [limit, n_vocab), over that one extra row (the end-of-sequence
 * token), whose logit is stored at index `limit` and whose argmax index is mapped back to special_id
 * (forward.rs:107-118).  Call between tfr_set_config and tfr_finalize_load; limit must be even, >= 1024 and
 * < n_vocab; limit = 0 removes the shortlist.  tfr_load_gguf applies the reference's rule by itself
 * (TARAFER_VOCAB_LIMIT, else 49 152 for a hybrid with more than 100 000 tokens unless TARAFER_FULL_VOCAB is set).
 * tfr_current_logits then fills n_active entries; tfr_active_vocab reports n_active and the extra row's id (-1: none). */
int tfr_set_vocab_shortlist(tfr_engine* e, int limit, int special_id);
int tfr_active_vocab(const tfr_engine* e, int* n_active, int* special_id);

/* ---- tensor parallelism (new: the reference drives one GPU, device.rs:85-95) ----
 * One engine per GPU, created with tfr_model_config.tp_size = N and its tp_rank.  Every rank is
 * handed the SAME full tensors through tfr_upload_tensor and keeps its Megatron shard: rows of
 * attn_q/k/v (+bias), ffn_gate/up and the vocabulary head; K blocks of attn_output and ffn_down.
 * The row-parallel GEMVs all-reduce inside the kernel through an exchange buffer that each rank
 * owns and all peers map.  After tfr_finalize_load and before the first forward call the host
 * connects the ranks in one of two ways:
 *   - one process per GPU: tfr_tp_ipc_handle on every rank, gather the 64-byte handles in rank
 *     order over any channel, tfr_tp_attach_ipc on every rank;
 *   - one process driving all GPUs: tfr_tp_local_pointer on every engine, tfr_tp_attach_pointers
 *     with the N pointers in rank order (peer access is enabled by the call).
 * All ranks must then issue the same forward / burst calls with the same arguments; a rank
 * that does not show up makes the others return TFR_E_CUDA after a bounded wait (about 2 s). */
int tfr_tp_exchange_bytes(const tfr_engine* e, size_t* bytes);
int tfr_tp_ipc_handle(tfr_engine* e, void* handle_out_64_bytes);
int tfr_tp_attach_ipc(tfr_engine* e, const void* handles_rank_order);
int tfr_tp_local_pointer(tfr_engine* e, void** ptr);
int tfr_tp_attach_pointers(tfr_engine* e, void* const* bases_rank_order);
/* Comparison baseline only: route the row-parallel partial sums and the argmax through ncclAllReduce
 * between kernels (three graph nodes per all-reduce) instead of the in-kernel exchange.  libnccl.so.2
 * is loaded at run time; TFR_E_UNSUPPORTED if it is absent.  Rank 0 obtains an id with
 * tfr_tp_nccl_unique_id and hands it to all ranks; every rank then calls tfr_tp_use_nccl(e, id)
 * (collective: ncclCommInitRank).  tfr_tp_use_nccl(e, NULL) returns to the in-kernel exchange. */
int tfr_tp_nccl_unique_id(void* id_out_128_bytes);
int tfr_tp_use_nccl(tfr_engine* e, const void* id_128_bytes);
/* Vocabulary rows [first, end) whose logits this rank computes (all of them when tp_size == 1). */
int tfr_tp_vocab_range(const tfr_engine* e, int* first, int* end);
/* set_cuda_graph / graph_active / invalidate_decode_graph, model.rs:101-112,197 */
int tfr_set_cuda_graph(tfr_engine* e, int enabled);
int tfr_graph_active(const tfr_engine* e);
/* DecodeBackend / REGISTRY, crates/core/src/cuda/decode.rs:87-240 (the reference picks its decode backend by name,
 * `--decode flash|fastv2`).  Two schedules compute the same token loop here:
 *   1 = chained kernels: five launches per layer, one CUDA graph per token replayed back to back;
 *   2 = persistent loop: one cooperative kernel per call that runs every decode step of the call, streams the
 *       weights through shared memory without stopping at phase boundaries and hands activations over through
 *       grid-wide barriers (dense models on one GPU; Q4_K / Q6_K matrices; no vocabulary shortlist).
 * path 0 (default) takes the persistent loop when the model qualifies and the chained kernels otherwise;
 * path 2 fails with TFR_E_UNSUPPORTED when it does not.  tfr_decode_path reports which one the next call takes. */
int tfr_set_decode_path(tfr_engine* e, int path);
int tfr_decode_path(const tfr_engine* e);

/* Prompts and verification batches go through the engine in chunks of up to `tokens` tokens, each chunk reading
 * the weights once (CudaModel::forward_chunk, crates/core/src/cuda/forward.rs:54-65, 360-407; MAX_BATCH,
 * MAX_VERIFY_TOKENS, crates/core/src/cuda/types.rs:7-9).  tokens = 0 feeds every token of a prompt as a decode step;
 * values above the engine's chunk capacity are clamped.  tfr_prefill_chunk returns the size in effect, 0 for models
 * the chunk kernels do not cover (hybrid layers, tensor parallelism), which keep the step-by-step route. */
int tfr_set_prefill_chunk(tfr_engine* e, int tokens);
int tfr_prefill_chunk(const tfr_engine* e);
/* Kernel launches issued by this engine so far (graph replays count their kernel nodes). */
int64_t tfr_launch_count(const tfr_engine* e);
/* Device time of the last tfr_decode_burst / tfr_forward_greedy in milliseconds (CUDA events
 * on the engine's stream, around the kernels only). */
float tfr_last_device_ms(const tfr_engine* e);
/* Test tap: copy a named workspace of the last step to the host ("x", "q", "attn", "h", "logits",
 * "k"/"v" = cache of `layer`, "layer_x" = residual stream after every layer; the first "layer_x"
 * request switches that tap on for later steps and returns zeros).  "layer_attn", "layer_mid", "layer_h" (dense
 * single-GPU models, chained kernels): per layer the attention output, the residual stream after the output
 * projection and SiLU*mul, i.e. the vectors a layer rounds to int8 besides its input; switched on the same way. */
int tfr_debug_read(tfr_engine* e, tfr_kv* kv, const char* what, int layer, void* out, size_t nbytes);

/* Test aid: when device_buffer != NULL, thread 0 of every CTA of the matrix-vector and attention kernels stores the
 * GPU nanosecond timer at up to eight points into device_buffer[(launch * 160 + cta) * 8 + point], launch =
 * index of the kernel within the decode step (0 for the stand-alone operators). */
#ifdef TFR_TEST_AIDS
int tfr_debug_set_timeline(unsigned long long* device_buffer);
#endif

/* Test aid: dst[i] = the f16 bits the KV store writes for src[i] (crates/core/src/cuda/kernels/common.cu:9-38), over n
 * device floats; lets a test walk all 2^32 inputs against the reference's copy_kv_f16. */
#ifdef TFR_TEST_AIDS
int tfr_debug_f32_to_f16(const float* src, uint16_t* dst, int64_t n, void* stream);
#endif
/* Test aid for the persistent loop: during decode step `step` of the next calls, thread 0 of every CTA stores the
 * GPU nanosecond timer at successive points of the step into device_buffer[point * n_sm + cta] (point < points).
 * device_buffer == NULL switches it off. */
#ifdef TFR_TEST_AIDS
int tfr_debug_set_loop_timeline(tfr_engine* e, unsigned long long* device_buffer, int step, int points);
#endif

/* ---- operator level (device pointers unless stated; stream = cudaStream_t or NULL) ---- */

/* GpuMat, crates/core/src/cuda/types.rs:26-39: a weight matrix resident on the device in
 * decode layout.  rope_pair_head_dim > 0 re-orders rows so RoPE partners are adjacent. */
int tfr_mat_create(int ggml_type, int64_t n_rows, int64_t n_cols, const void* bytes, size_t nbytes,
                   int rope_pair_head_dim, tfr_mat** out);
void tfr_mat_free(tfr_mat* m);
int64_t tfr_mat_device_bytes(const tfr_mat* m);

/* quantize_q8_global, kernels/gemv.cu:43-65 */
int tfr_op_quantize_q8(const float* x, int n, int8_t* q8, float* d8, void* stream);
/* gemv / try_gemv_global_q8, crates/core/src/cuda/matmul.rs:118-302.  act_mode 0: Q8
 * activation; 1: fp32 activation (Q6_K only; the reference's attn_v route).  use_res 2:
 * out += W x.  norm_w != NULL applies RMSNorm (kernels/ops.cu:4-34) to x first. */
int tfr_op_gemv(const tfr_mat* w, const float* x, float* out, const float* bias, int use_res, int act_mode,
                const float* norm_w, float eps, void* stream);
/* gemv_q4_k_ffn_mcol, kernels/gemv.cu:2546-2575 (+ optional RMSNorm in front) */
int tfr_op_ffn_gate_up(const tfr_mat* gate, const tfr_mat* up, const float* x, const float* norm_w, float eps, float* h,
                       void* stream);
/* The FFN block of ffn_block_dense (layer.rs:1210-1456) at n_tok = 1 without the norm:
 * y (+)= down . Q8(silu(gate . Q8(x)) * (up . Q8(x))).  h_scratch: n_ff floats. */
int tfr_op_ffn_block(const tfr_mat* gate, const tfr_mat* up, const tfr_mat* down, const float* x, float* h_scratch,
                     float* y, int use_res, void* stream);
/* Same with HOST buffers: copies x in, runs the two kernels, copies y out, synchronises. */
int tfr_ffn_block_host(const tfr_mat* gate, const tfr_mat* up, const tfr_mat* down, const float* x_host, float* y_host);
/* Integer contract taps (test aid, no reference kernel exposes these): for Q4_K, a = I[N][K/32]
 * and b = S[N][K/32] of kernels/gemv.cu:71-130; for Q6_K, a = J[N][K/16] of gemv.cu:302-337; for Q8_0,
 * a = the per-32-block sums [N][K/32] of gemv.cu:1558-1582. */
#ifdef TFR_TEST_AIDS
int tfr_op_int_dots(const tfr_mat* w, const int8_t* q8, const float* d8, int32_t* a, int32_t* b, void* stream);
#endif
/* The same taps with the activation given as fp32 x[K]: it is quantised by the quantiser the matrix-vector kernels run
 * (kernels/gemv.cu:16-65 semantics), q8_out (optional, K bytes) receives the int8 values the block dots then read, and
 * b (Q4_K) the 32-group sums exactly as the dots' activation record holds them. */
#ifdef TFR_TEST_AIDS
int tfr_op_int_dots_x(const tfr_mat* w, const float* x, int32_t* a, int32_t* b, int8_t* q8_out, void* stream);
#endif
/* attn_flash_partial + attn_flash_reduce, kernels/attn/flash.cu:16-255, for one query token
 * at position pos over cache rows [0, pos].  kc / vc: [max_seq][n_kv*head_dim] f16 bits.  The split-KV scratch
 * of this stand-alone call is one buffer per device, grown on demand: calls that overlap on the same GPU
 * (different streams, or threads) race on it - serialise them. */
int tfr_op_attention(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                     int head_dim, int pos, void* stream);
/* Same computation as tfr_op_attention for callers that cannot allocate device memory when they
 * call (a graph capture in progress elsewhere in the context, a fixed memory budget, a real-time
 * loop).  It has no counterpart in the reference.  The split-KV scratch is a fixed 2 MiB array
 * inside the library image (held by every GPU that loads the library, until exit); the call
 * performs no cudaMalloc / cudaFree and uses no allocating library routine.  Shapes whose scratch
 * n_head * S * (2 + head_dim) * 4 bytes exceeds 2 MiB - 2048 B, where S is the number of key splits the
 * attention kernel uses on this GPU (a multiple of 8, at least 8, about n_sm / n_kv), or with more than 64 KV
 * heads, are refused with TFR_E_UNSUPPORTED and a message on stderr.  The first call on a device
 * looks up the array's device address (that device must be current); make that first call before
 * any stream capture begins.  All calls share the one array: calls that overlap on the GPU
 * (different streams, or threads) race on it — serialise them. */
int tfr_op_attention_noalloc(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                             int head_dim, int pos, void* stream);
/* Fused attention front end: RMSNorm + Q8 + Q/K/V projections + bias + RoPE + f16 KV store
 * (rms_norm_f32, gemv_q4_k_pair, gemv_q6_k, rope_neox_f32, copy_kv_f16; layer.rs:196-600).
 * wq / wk must have been created with rope_pair_head_dim = head_dim; biases natural order. */
int tfr_op_qkv_rope_store(const tfr_mat* wq, const tfr_mat* wk, const tfr_mat* wv, const float* bq, const float* bk,
                          const float* bv, const float* x, const float* norm_w, float eps, float theta, int head_dim,
                          int pos, float* q_out, uint16_t* kc, uint16_t* vc, void* stream);

/* Gated-DeltaNet decode step of one linear-attention layer, after the four input projections:
 * gdn_conv_qkvl2_one_f32 + gdn_delta_gated_one_d128_f32 (kernels/deltanet.cu:561-728; layer.rs:838-885)
 * in one launch.  proj = [qkv (2*n_k+n_v)*128 | z n_v*128 | beta n_v | alpha n_v] raw projections;
 * conv_w [channels][kernel] as the GGUF stores it; state [n_v][128][128] is updated in place.
 * conv_ring differs from the reference's shifted window [kernel-1][channels]: it is a ring of
 * `kernel` slots of [channels]; the call reads the kernel-1 slots before `slot` (modulo kernel,
 * oldest first) and stores the current input into `slot`.  Callers advance slot by one per token.
 * state_size must be 128 and 2 <= kernel <= 4. */
int tfr_op_gdn_step(const float* proj, const float* conv_w, float* conv_ring, float* state, const float* ssm_a,
                    const float* ssm_dt, const float* norm_w, float* out, int n_k, int n_v, int state_size, int kernel,
                    int slot, float eps, void* stream);
/* Front end of a gated full-attention layer after the raw projections: split_q_gate_interleaved_f32,
 * qk_rms_norm_partial_rope_neox_f32 on Q and K, copy_kv_f16 of K and V (kernels/deltanet.cu:144-235,
 * kernels/ops.cu:471-486; layer.rs:386-600) in one launch.  raw = [n_head x (Q_h | G_h) | K | V];
 * n_rot = rotated leading dims of every head (rope.dimension_count, or head_dim). */
int tfr_op_qk_norm_rope_store(const float* raw, const float* q_norm, const float* k_norm, float* q_out, float* gate_out,
                              uint16_t* kc, uint16_t* vc, int n_head, int n_kv, int head_dim, int n_rot, int pos,
                              float theta, float eps, void* stream);
/* tfr_op_attention with the sigmoid output gate of the hybrid's full-attention layers folded in:
 * out = attention(q) * sigmoid(gate) (mul_sigmoid_f32, kernels/deltanet.cu:176-186). */
int tfr_op_attention_gated(const float* q, const uint16_t* kc, const uint16_t* vc, const float* gate, float* out,
                           int n_head, int n_kv, int head_dim, int pos, void* stream);

/* transcode_q5_k_to_q8_0 / transcode_q5_1_to_q8_0, load.rs:33-133 (host code): src_type 13 (Q5_K, 176-byte
 * blocks) or 7 (Q5_1, 24-byte blocks) -> Q8_0 bytes (34 per 32 weights) in out.  tfr_upload_tensor and
 * tfr_mat_create apply it themselves to tensors of those types; Q8_0 (type 8) matrices run on their own
 * dot routine (kernels/gemv.cu:1558-1749). */
int tfr_transcode_to_q8_0(int src_type, const void* raw, size_t nbytes, void* out);

/* Synthetic-model aid (no counterpart in the reference, which has no quantiser): quantise
 * fp32 rows [N][K] on the device into GGUF Q4_K / Q6_K bytes. */
#ifdef TFR_TEST_AIDS
int tfr_synth_quantize(int ggml_type, const float* w, int64_t n_rows_k, int64_t n_cols_n, void* out_bytes, void* stream);
#endif

#ifdef __cplusplus
}
#endif
#endif
