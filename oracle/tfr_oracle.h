/* Shared declarations of the CPU restatement (test infrastructure only; see tfr_oracle.c). */
#ifndef TFR_ORACLE_H
#define TFR_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#define TFO_Q4_K 12 /* ggml type ids, crates/gguf/src/types.rs:7-60 */
#define TFO_Q6_K 14
#define TFO_Q8_0 8
#define TFO_Q5_K 13
#define TFO_Q5_1 7
#define TFO_Q4_K_BYTES 144
#define TFO_Q6_K_BYTES 210
#define TFO_Q8_0_BYTES 34 /* per 32 elements */

typedef struct {
    int32_t type; /* TFO_Q4_K or TFO_Q6_K */
    int32_t K;    /* input features, contiguous (GGUF dims[0]) */
    int32_t N;    /* output rows (GGUF dims[1]) */
    int32_t pad_;
    const uint8_t* data; /* raw GGUF bytes, N rows of K/256 blocks */
} tfo_mat;

/* Layer kinds: crates/core/src/config.rs (LayerKind) and backend.rs:19-31. */
#define TFO_LAYER_DENSE 0       /* qwen2 attention block */
#define TFO_LAYER_LINEAR 1      /* Gated-DeltaNet mixer (qwen35) */
#define TFO_LAYER_FULL_GATED 2  /* qwen35 full attention: fused Q|gate, q/k RMS-norm, partial RoPE, output gate */

typedef struct {
    tfo_mat wq, wk, wv, wo, gate, up, down;
    const float *bq, *bk, *bv;   /* may be NULL */
    const float *attn_norm, *ffn_norm;
    /* hybrid */
    int32_t kind, pad_;
    tfo_mat wqkv, wgate, wbeta, walpha, ssm_out;                      /* linear layers */
    const float *conv1d, *ssm_a, *ssm_dt, *ssm_norm;                  /* linear layers */
    const float *q_norm, *k_norm;                                     /* gated full-attention layers */
} tfo_layer;

typedef struct {
    int32_t n_layer, n_embd, n_head, n_kv, head_dim, n_ff, n_vocab, max_seq;
    float rope_theta, eps;
    tfo_mat token_embd;
    tfo_mat output; /* data == NULL: tied to token_embd */
    const float* output_norm;
    const tfo_layer* layers;
    /* hybrid: rope.dimension_count, ssm.group_count (K/Q heads), ssm.time_step_rank (V heads), ssm.state_size, ssm.conv_kernel */
    int32_t rope_dim, ssm_n_k, ssm_n_v, ssm_state, conv_kernel, pad_;
} tfo_model;

/* Optional taps of the residual stream, for stage-by-stage parity tests.  Any pointer may be NULL. */
typedef struct {
    float* x_final;  /* [n_embd] residual stream after the last layer */
    float* xn_final; /* [n_embd] after output_norm */
} tfo_taps;

extern int g_threads;
size_t tfo_row_bytes(const tfo_mat* m);
float tfo_half_to_float(uint16_t h);
uint16_t tfo_float_to_half_bits(float f);
int tfo_gemv(const tfo_mat* w, const float* x, float* out, const float* bias, int use_res, int act_mode);
int tfo_ffn_gate_up(const tfo_mat* gate, const tfo_mat* up, const float* x, float* out);
void tfo_rms_norm(const float* x, const float* w, float* out, int n, float eps);
void tfo_float_to_half_bits_range(uint32_t first, uint64_t count, uint16_t* out);
void tfo_set_layer_taps(float* attn, float* mid, float* h);
void tfo_copy_kv_f16(const float* src, uint16_t* cache, int pos, int stride);
void tfo_attention(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv, int hd, int pos,
                   float scale);
float tfo_dot_q8_0_q8(const uint8_t* row, int K, const int8_t* q8, const float* d8);
void tfo_q8_0_blockdots(const uint8_t* row, int K, const int8_t* q8, int32_t* sums);
int tfo_transcode_q5_k_to_q8_0(const uint8_t* raw, size_t nbytes, uint8_t* out);
int tfo_transcode_q5_1_to_q8_0(const uint8_t* raw, size_t nbytes, uint8_t* out);
/* tfr_oracle_gdn.c */
int tfo_gdn_step(const float* qkv, const float* z, const float* beta, const float* alpha, const float* conv_w,
                 float* conv_state, float* ssm, const float* ssm_a, const float* ssm_dt, const float* norm_w, float* y, int nk,
                 int nv, int d, int kernel, float eps);
void tfo_qk_norm_partial_rope(float* x, const float* w, int n_heads, int hd, int n_rot, int pos, float theta, float eps);
int tfo_linear_attn_block(const tfo_model* M, const tfo_layer* L, const float* xb, float* y, float* ssm, float* conv);
int tfo_gated_attn_block(const tfo_model* M, const tfo_layer* L, const float* xb, float* out, uint16_t* kc, uint16_t* vc, int pos);
#endif
