/*
 * CPU restatement of the hybrid (Qwen3.5-style) layer parts: the Gated-DeltaNet mixer and the
 * gated full-attention block.  TEST INFRASTRUCTURE ONLY, like tfr_oracle.c.  Citations are paths
 * inside the reference project.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "tfr_oracle.h"

/* kernels/deltanet.cu:530-559 — depthwise causal conv (kernel taps k + c*kernel, ring state
 * [kernel-1][channels] oldest first) followed by SiLU; the ring is shifted and takes x_c. */
static float conv_channel(const float* x, const float* w, float* state, int c, int channels, int kernel) {
    int km1 = kernel - 1;
    float acc = 0.f;
    for (int k = 0; k < km1; k++) acc += w[(size_t)k + (size_t)c * kernel] * state[(size_t)k * channels + c];
    float xt = x[c];
    acc += w[(size_t)(kernel - 1) + (size_t)c * kernel] * xt;
    float y = acc / (1.f + expf(-acc));
    for (int k = 0; k < km1 - 1; k++) state[(size_t)k * channels + c] = state[(size_t)(k + 1) * channels + c];
    if (km1 > 0) state[(size_t)(km1 - 1) * channels + c] = xt;
    return y;
}

/* Gated-DeltaNet decode step after the four projections (layer.rs:838-911 at n_tok = 1):
 *   conv + SiLU + split [Q|K|V] + L2-normalise Q and K per head (deltanet.cu:561-622),
 *   per V head: beta = sigmoid(b), g = exp(softplus(a + dt) * A), S *= g, delta rule column by
 *   column, read-out with q / sqrt(d), gated RMSNorm with silu(z) (deltanet.cu:628-728).
 * qkv [channels], z [n_v*d], beta/alpha [n_v] raw; y: [n_v * d]; ssm: [n_v][d][d];
 * conv_state: [kernel-1][channels], oldest first. */
int tfo_gdn_step(const float* qkv, const float* z, const float* beta, const float* alpha, const float* conv_w,
                 float* conv_state, float* ssm, const float* ssm_a, const float* ssm_dt, const float* norm_w, float* y, int nk,
                 int nv, int d, int kernel, float eps) {
    int key_dim = nk * d, val_dim = nv * d, channels = 2 * key_dim + val_dim;
    if (nk <= 0 || nv <= 0 || d <= 0 || kernel < 1) return -1;
    float* cv = (float*)malloc(sizeof(float) * (size_t)channels);
    for (int c = 0; c < channels; c++) cv[c] = conv_channel(qkv, conv_w, conv_state, c, channels, kernel);
    float* Q = cv;
    float* Kk = cv + key_dim;
    float* V = cv + 2 * key_dim;
    for (int h = 0; h < nk; h++) { /* sum of squares, not mean (deltanet.cu:598-620) */
        float sq = 0.f, sk = 0.f;
        for (int i = 0; i < d; i++) {
            sq += Q[h * d + i] * Q[h * d + i];
            sk += Kk[h * d + i] * Kk[h * d + i];
        }
        float iq = 1.0f / sqrtf(sq + eps), ik = 1.0f / sqrtf(sk + eps);
        for (int i = 0; i < d; i++) {
            Q[h * d + i] *= iq;
            Kk[h * d + i] *= ik;
        }
    }
    float qscale = 1.0f / sqrtf((float)d);
    float* o = (float*)malloc(sizeof(float) * (size_t)d);
    for (int h = 0; h < nv; h++) {
        int hk = h % nk;
        float b = 1.f / (1.f + expf(-beta[h]));
        float zz = alpha[h] + ssm_dt[h];
        float sp = zz > 20.f ? zz : log1pf(expf(zz));
        float g = expf(sp * ssm_a[h]);
        float* S = ssm + (size_t)h * d * d;
        const float* kt = Kk + (size_t)hk * d;
        const float* qt = Q + (size_t)hk * d;
        for (int i = 0; i < d * d; i++) S[i] *= g;
        for (int j = 0; j < d; j++) {
            float kv_mem = 0.f;
            for (int i = 0; i < d; i++) kv_mem += S[(size_t)i * d + j] * kt[i];
            float delta = (V[h * d + j] - kv_mem) * b;
            float acc = 0.f;
            for (int i = 0; i < d; i++) {
                float s = S[(size_t)i * d + j] + kt[i] * delta;
                S[(size_t)i * d + j] = s;
                acc += s * (qt[i] * qscale);
            }
            o[j] = acc;
        }
        float ss = 0.f;
        for (int j = 0; j < d; j++) ss += o[j] * o[j];
        float scale = 1.0f / sqrtf(ss * (1.f / (float)d) + eps);
        for (int j = 0; j < d; j++) {
            float gate = z[h * d + j];
            float silu = gate / (1.f + expf(-gate));
            y[h * d + j] = o[j] * scale * norm_w[j] * silu;
        }
    }
    free(cv); free(o);
    return 0;
}

/* The mixer of a linear layer: four projections of the normed hidden state (Q4_K x Q8,
 * layer.rs:736-798) and the step above.  xb: normed hidden [n_embd]. */
int tfo_linear_attn_block(const tfo_model* M, const tfo_layer* L, const float* xb, float* y, float* ssm, float* conv) {
    int nk = M->ssm_n_k, nv = M->ssm_n_v, d = M->ssm_state;
    int val_dim = nv * d, channels = 2 * nk * d + val_dim;
    if (L->wqkv.N != channels || L->wgate.N != val_dim || L->wbeta.N != nv || L->walpha.N != nv) return -1;
    float* qkv = (float*)malloc(sizeof(float) * (size_t)channels);
    float* z = (float*)malloc(sizeof(float) * (size_t)val_dim);
    float* beta = (float*)malloc(sizeof(float) * (size_t)nv);
    float* alpha = (float*)malloc(sizeof(float) * (size_t)nv);
    int rc = 0;
    rc |= tfo_gemv(&L->wqkv, xb, qkv, NULL, 0, 0);
    rc |= tfo_gemv(&L->wgate, xb, z, NULL, 0, 0);
    rc |= tfo_gemv(&L->wbeta, xb, beta, NULL, 0, 0);
    rc |= tfo_gemv(&L->walpha, xb, alpha, NULL, 0, 0);
    if (!rc)
        rc = tfo_gdn_step(qkv, z, beta, alpha, L->conv1d, conv, ssm, L->ssm_a, L->ssm_dt, L->ssm_norm, y, nk, nv, d,
                          M->conv_kernel, M->eps);
    free(qkv); free(z); free(beta); free(alpha);
    return rc;
}

/* Per-head RMSNorm with weight, then neox RoPE on the first n_rot dims only, pairs (i, i + n_rot/2),
 * freq = theta^(-2i/n_rot) (deltanet.cu:189-235).  w == NULL: no norm. */
void tfo_qk_norm_partial_rope(float* x, const float* w, int n_heads, int hd, int n_rot, int pos, float theta, float eps) {
    for (int h = 0; h < n_heads; h++) {
        float* base = x + (size_t)h * hd;
        if (w) {
            float ss = 0.f;
            for (int i = 0; i < hd; i++) ss += base[i] * base[i];
            float scale = 1.0f / sqrtf(ss / (float)hd + eps);
            for (int i = 0; i < hd; i++) base[i] = base[i] * scale * w[i];
        }
        int half = n_rot / 2;
        for (int i = 0; i < half; i++) {
            float freq = powf(theta, -2.f * (float)i / (float)n_rot);
            float ang = (float)pos * freq;
            float c = cosf(ang), s = sinf(ang);
            float x0 = base[i], x1 = base[i + half];
            base[i] = x0 * c - x1 * s;
            base[i + half] = x0 * s + x1 * c;
        }
    }
}

/* Gated full attention of the hybrid (layer.rs:196-659 with fused_q_gate): wq emits per head
 * [Q_h | G_h] (deltanet.cu:144-173), Q and K get a per-head RMSNorm with weight and RoPE on the
 * first rope_dim dims only (deltanet.cu:189-235), attention as usual, output *= sigmoid(G)
 * (deltanet.cu:176-186).  out: [n_head * hd]. */
int tfo_gated_attn_block(const tfo_model* M, const tfo_layer* L, const float* xb, float* out, uint16_t* kc, uint16_t* vc, int pos) {
    int H = M->n_head, Hkv = M->n_kv, hd = M->head_dim, qn = H * hd, kvn = Hkv * hd;
    int n_rot = (M->rope_dim > 0 && M->rope_dim < hd) ? M->rope_dim : hd;
    if (L->wq.N != 2 * qn) return -1;
    float* qg = (float*)malloc(sizeof(float) * (size_t)(2 * qn));
    float* q = (float*)malloc(sizeof(float) * (size_t)qn);
    float* g = (float*)malloc(sizeof(float) * (size_t)qn);
    float* kb = (float*)malloc(sizeof(float) * (size_t)kvn);
    float* vb = (float*)malloc(sizeof(float) * (size_t)kvn);
    int rc = 0;
    rc |= tfo_gemv(&L->wq, xb, qg, L->bq, 0, 0);
    rc |= tfo_gemv(&L->wk, xb, kb, L->bk, 0, 0);
    rc |= tfo_gemv(&L->wv, xb, vb, L->bv, 0, L->wv.type == TFO_Q6_K ? 1 : 0);
    for (int h = 0; h < H; h++)
        for (int i = 0; i < hd; i++) {
            q[h * hd + i] = qg[h * 2 * hd + i];
            g[h * hd + i] = qg[h * 2 * hd + hd + i];
        }
    tfo_qk_norm_partial_rope(q, L->q_norm, H, hd, n_rot, pos, M->rope_theta, M->eps);
    tfo_qk_norm_partial_rope(kb, L->k_norm, Hkv, hd, n_rot, pos, M->rope_theta, M->eps);
    tfo_copy_kv_f16(kb, kc, pos, kvn);
    tfo_copy_kv_f16(vb, vc, pos, kvn);
    tfo_attention(q, kc, vc, out, H, Hkv, hd, pos, 1.0f / sqrtf((float)hd));
    for (int i = 0; i < qn; i++) out[i] *= 1.f / (1.f + expf(-g[i]));
    free(qg); free(q); free(g); free(kb); free(vb);
    return rc;
}
