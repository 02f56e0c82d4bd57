/*
 * CPU restatement of taraference's batch-1 decode math.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: it is
 * linked or called from tests/, from the smoke check and from the CPU-baseline legs of
 * bench.py, never from the product path.  It restates, in plain C with IEEE fp32
 * arithmetic, what the reference's device code computes; every function cites the
 * reference lines it follows (paths are relative to the reference project root).
 *
 * Pinning: the reference's own tests hold no golden vectors for this path (they never
 * launch a kernel).  The pins are (1) gguf-py's `quants.dequantize` for block decoding,
 * and (2) outputs of the reference's own .cu kernels, compiled unmodified and run on a
 * B200, stored under tests/golden/ together with the script that produced them.
 *
 * Known, intended difference from the reference build: the reference is compiled with
 * fast-math (approximate division, ex2/sin/cos approximations).  This file uses exact
 * IEEE operations, so the int8 activation quantiser can differ by one unit on a few
 * elements in 1e5 and transcendental results differ in the last bits.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "tfr_oracle.h"

int g_threads = 1;

void tfo_set_threads(int n) {
    g_threads = n < 1 ? 1 : n;
#ifdef _OPENMP
    omp_set_num_threads(g_threads);
#endif
}

int tfo_get_threads(void) { return g_threads; }

int tfo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------- fp16 ---------- */

/* kernels/common.cu:2-6 — cvt.f32.f16 is an exact widening, subnormals included. */
float tfo_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* kernels/common.cu:9-38 — the KV-store rounding: add one when the highest dropped bit
 * is set (round half up in magnitude), flush below 2^-25, saturate to inf at 65536. */
uint16_t tfo_float_to_half_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx == 0u) return (uint16_t)sign;
    if (absx >= 0x7f800000u) return (uint16_t)(sign | (absx == 0x7f800000u ? 0x7c00u : 0x7e00u));
    if (absx < 0x33000000u) return (uint16_t)sign;
    if (absx >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);
    int e = (int)((absx >> 23) & 0xff) - 127 + 15;
    uint32_t mant = absx & 0x7fffffu;
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        mant |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t hm = mant >> shift;
        if ((mant >> (shift - 1)) & 1u) hm += 1u;
        return (uint16_t)(sign | hm);
    }
    uint32_t half = ((uint32_t)e << 10) | (mant >> 13);
    if (mant & 0x1000u) half += 1u;
    return (uint16_t)(sign | half);
}

/* The same conversion over a run of consecutive fp32 bit patterns [first, first + count): the exhaustive check of the
 * rounding against the reference's copy_kv_f16 walks all 2^32 patterns through this. */
void tfo_float_to_half_bits_range(uint32_t first, uint64_t count, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)count; i++) {
        uint32_t bits = first + (uint32_t)i;
        float f;
        memcpy(&f, &bits, 4);
        out[i] = tfo_float_to_half_bits(f);
    }
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ---------------------------------------------------------------- blocks -------- */

/* kernels/common.cu:40-50 — 6-bit scale / min of sub-block j from the 12 packed bytes. */
void tfo_scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* kernels/common.cu:64-84 — one 144-byte Q4_K super-block to 256 floats. */
void tfo_dequant_q4_k(const uint8_t* b, float* out) {
    float d = tfo_half_to_float(rd16(b));
    float dmin = tfo_half_to_float(rd16(b + 2));
    const uint8_t* scales = b + 4;
    const uint8_t* qs = b + 16;
    for (int t = 0; t < 4; t++) {
        uint8_t sc, m;
        tfo_scale_min_k4(2 * t, scales, &sc, &m);
        float d1 = d * (float)sc, m1 = dmin * (float)m;
        tfo_scale_min_k4(2 * t + 1, scales, &sc, &m);
        float d2 = d * (float)sc, m2 = dmin * (float)m;
        for (int l = 0; l < 32; l++) {
            out[64 * t + l] = d1 * (float)(qs[32 * t + l] & 0xF) - m1;
            out[64 * t + 32 + l] = d2 * (float)(qs[32 * t + l] >> 4) - m2;
        }
    }
}

/* Signed 6-bit value (already minus 32) of element e (0..255) of a Q6_K block;
 * kernels/common.cu:164-186. */
static inline int q6_value(const uint8_t* b, int e) {
    int n = e >> 7, r = e & 127, j = r >> 5, l = r & 31;
    const uint8_t* ql = b + 64 * n;
    const uint8_t* qh = b + 128 + 32 * n;
    int lo = (j & 1) ? ql[32 + l] : ql[l];
    lo = (j & 2) ? (lo >> 4) : (lo & 0xF);
    int hi = (qh[l] >> (2 * j)) & 3;
    return (lo | (hi << 4)) - 32;
}

/* Scale index of element e; kernels/common.cu:176-184 (sc_i + is + {0,2,4,6}). */
static inline int q6_scale_index(int e) {
    int n = e >> 7, r = e & 127, j = r >> 5, l = r & 31;
    return 8 * n + (l >> 4) + 2 * j;
}

/* kernels/common.cu:164-186 — one 210-byte Q6_K block to 256 floats. */
void tfo_dequant_q6_k(const uint8_t* b, float* out) {
    const int8_t* sc = (const int8_t*)(b + 192);
    float d = tfo_half_to_float(rd16(b + 208));
    for (int e = 0; e < 256; e++)
        out[e] = d * (float)sc[q6_scale_index(e)] * (float)q6_value(b, e);
}

/* bytes per 256 elements */
static int blk_bytes(int type) {
    return type == TFO_Q4_K ? TFO_Q4_K_BYTES : type == TFO_Q6_K ? TFO_Q6_K_BYTES : type == TFO_Q8_0 ? 8 * TFO_Q8_0_BYTES : 0;
}

/* One weight row (K elements, GGUF bytes) to floats.  kernels/embed.cu:71-131 is this
 * applied to the row of a token id. */
int tfo_dequant_row(int type, const uint8_t* row, int K, float* out) {
    int bb = blk_bytes(type);
    if (!bb || K % 256) return -1;
    for (int b = 0; b < K / 256; b++) {
        if (type == TFO_Q4_K) tfo_dequant_q4_k(row + (size_t)b * bb, out + 256 * b);
        else tfo_dequant_q6_k(row + (size_t)b * bb, out + 256 * b);
    }
    return 0;
}

/* ---------------------------------------------------------------- quantiser ----- */

/* kernels/gemv.cu:43-65 (same body at gemv.cu:16-40 and ops.cu:66-83): per 32 values
 * d = amax * (1/127) in fp32, q = round-to-nearest-even(x / d), all-zero group -> 0.
 * Groups beyond n/32 whole groups are not written (n_rows >> 5). */
void tfo_quantize_q8(const float* x, int n, int8_t* q, float* d8) {
    int nb = n >> 5;
    for (int b = 0; b < nb; b++) {
        float amax = 0.f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[32 * b + i]));
        float d = amax * (1.0f / 127.0f);
        for (int i = 0; i < 32; i++)
            q[32 * b + i] = amax == 0.f ? 0 : (int8_t)(int)nearbyintf(x[32 * b + i] / d);
        d8[b] = d;
    }
}

/* ---------------------------------------------------------------- dots ---------- */

/* Integer contract of kernels/gemv.cu:71-130: for sub-block j of one super-block,
 * I[j] = sum over its 32 elements of nibble * q8, S[j] = sum of q8.  The reference
 * builds these from four 8-element dp4a partials per lane; integer addition is exact,
 * so the totals are what matters. */
void tfo_q4k_subdots(const uint8_t* b, const int8_t* q8, int32_t* I, int32_t* S) {
    const uint8_t* qs = b + 16;
    for (int t = 0; t < 4; t++) {
        int32_t i0 = 0, i1 = 0, s0 = 0, s1 = 0;
        for (int l = 0; l < 32; l++) {
            int a0 = q8[64 * t + l], a1 = q8[64 * t + 32 + l];
            i0 += (qs[32 * t + l] & 0xF) * a0;
            i1 += (qs[32 * t + l] >> 4) * a1;
            s0 += a0;
            s1 += a1;
        }
        I[2 * t] = i0;
        I[2 * t + 1] = i1;
        S[2 * t] = s0;
        S[2 * t + 1] = s1;
    }
}

/* kernels/gemv.cu:71-130 — Q4_K row times Q8 activation.  Per super-block
 * d * sum_j d8*(float)(I_j*sc_j) - dmin * sum_j d8*(float)(S_j*m_j). */
float tfo_dot_q4k_q8(const uint8_t* row, int nb, const int8_t* q8, const float* d8) {
    float acc = 0.f;
    for (int b = 0; b < nb; b++) {
        const uint8_t* blk = row + (size_t)b * TFO_Q4_K_BYTES;
        float d = tfo_half_to_float(rd16(blk));
        float dmin = tfo_half_to_float(rd16(blk + 2));
        int32_t I[8], S[8];
        tfo_q4k_subdots(blk, q8 + 256 * b, I, S);
        float pos = 0.f, neg = 0.f;
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            tfo_scale_min_k4(j, blk + 4, &sc, &m);
            pos += d8[8 * b + j] * (float)(I[j] * (int)sc);
            neg += d8[8 * b + j] * (float)(S[j] * (int)m);
        }
        acc += d * pos;
        acc -= dmin * neg;
    }
    return acc;
}

/* Integer contract of kernels/gemv.cu:302-337: for each of the 16 scale groups g of a
 * block (16 consecutive elements 16g..16g+15) J[g] = sum (q6 - 32) * q8. */
void tfo_q6k_groupdots(const uint8_t* b, const int8_t* q8, int32_t* J) {
    for (int g = 0; g < 16; g++) J[g] = 0;
    for (int e = 0; e < 256; e++) J[e >> 4] += q6_value(b, e) * (int)q8[e];
}

/* kernels/gemv.cu:302-337 — Q6_K row times Q8 activation: d * scale_g * d8 * J. */
float tfo_dot_q6k_q8(const uint8_t* row, int nb, const int8_t* q8, const float* d8) {
    float acc = 0.f;
    for (int b = 0; b < nb; b++) {
        const uint8_t* blk = row + (size_t)b * TFO_Q6_K_BYTES;
        const int8_t* sc = (const int8_t*)(blk + 192);
        float d = tfo_half_to_float(rd16(blk + 208));
        int32_t J[16];
        tfo_q6k_groupdots(blk, q8 + 256 * b, J);
        /* element group 16g sits in 32-group (16g)/32 of this block */
        for (int g = 0; g < 16; g++) {
            /* scale index of elements 16g.. is q6_scale_index(16g) */
            acc += d * (float)sc[q6_scale_index(16 * g)] * d8[8 * b + (g >> 1)] * (float)J[g];
        }
    }
    return acc;
}

/* kernels/gemv.cu:233-264 — Q6_K row times UNQUANTISED fp32 activation (the route the
 * reference takes for a Q6_K attn_v: layer.rs:265-275 -> matmul.rs:346-412). */
float tfo_dot_q6k_f32(const uint8_t* row, int nb, const float* x) {
    float acc = 0.f;
    for (int b = 0; b < nb; b++) {
        const uint8_t* blk = row + (size_t)b * TFO_Q6_K_BYTES;
        const int8_t* sc = (const int8_t*)(blk + 192);
        float d = tfo_half_to_float(rd16(blk + 208));
        for (int e = 0; e < 256; e++)
            acc += d * (float)sc[q6_scale_index(e)] * (float)q6_value(blk, e) * x[256 * b + e];
    }
    return acc;
}

/* kernels/gemv.cu:193-231 shape — Q4_K row times fp32 activation (prefill GEMM math,
 * kernels/gemm.cu:6-67: dequantise then fp32 multiply-add). */
float tfo_dot_q4k_f32(const uint8_t* row, int nb, const float* x) {
    float acc = 0.f, w[256];
    for (int b = 0; b < nb; b++) {
        tfo_dequant_q4_k(row + (size_t)b * TFO_Q4_K_BYTES, w);
        for (int e = 0; e < 256; e++) acc += w[e] * x[256 * b + e];
    }
    return acc;
}

/* ---------------------------------------------------------------- GEMV ---------- */

/* Q8_0 x Q8, kernels/gemv.cu:1558-1582: per 32-block sum = dot(int8 weights, int8 activation);
 * acc += d_w * d_x * (float)sum. */
void tfo_q8_0_blockdots(const uint8_t* row, int K, const int8_t* q8, int32_t* sums) {
    for (int bi = 0; bi < K / 32; bi++) {
        const int8_t* qs = (const int8_t*)(row + (size_t)bi * TFO_Q8_0_BYTES + 2);
        int32_t s = 0;
        for (int t = 0; t < 32; t++) s += (int32_t)qs[t] * (int32_t)q8[32 * bi + t];
        sums[bi] = s;
    }
}
float tfo_dot_q8_0_q8(const uint8_t* row, int K, const int8_t* q8, const float* d8) {
    float acc = 0.f;
    for (int bi = 0; bi < K / 32; bi++) {
        const uint8_t* base = row + (size_t)bi * TFO_Q8_0_BYTES;
        const float dw = tfo_half_to_float((uint16_t)(base[0] | (base[1] << 8)));
        const int8_t* qs = (const int8_t*)(base + 2);
        int32_t s = 0;
        for (int t = 0; t < 32; t++) s += (int32_t)qs[t] * (int32_t)q8[32 * bi + t];
        acc += dw * d8[bi] * (float)s;
    }
    return acc;
}

/* IEEE f32 -> f16, round to nearest even (crates/core/src/quant.rs:26-62). */
static uint16_t f32_to_f16_rne(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000);
    int exponent = (int)((bits >> 23) & 0xff);
    uint32_t fraction = bits & 0x007fffffu;
    if (exponent == 255) return (uint16_t)(sign | (fraction == 0 ? 0x7c00 : 0x7e00));
    int half_exp = exponent - 127 + 15;
    if (half_exp >= 31) return (uint16_t)(sign | 0x7c00);
    if (half_exp <= 0) {
        if (half_exp < -10) return sign;
        uint32_t mantissa = fraction | 0x00800000u;
        uint32_t shift = (uint32_t)(14 - half_exp);
        uint32_t rounded = mantissa >> shift;
        uint32_t remainder = mantissa & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (remainder > halfway || (remainder == halfway && (rounded & 1u))) rounded += 1;
        return (uint16_t)(sign | rounded);
    }
    uint32_t rounded = fraction + 0x00000fffu + ((fraction >> 13) & 1u);
    uint16_t out_exp = (uint16_t)half_exp;
    if (rounded & 0x00800000u) {
        rounded = 0;
        out_exp += 1;
        if (out_exp >= 31) return (uint16_t)(sign | 0x7c00);
    }
    return (uint16_t)(sign | (out_exp << 10) | (rounded >> 13));
}

/* 32 fp32 values -> one Q8_0 block (load.rs:88-101): d = amax / 127, q = clamp(round-half-away(v / d)). */
static void q8_0_from_f32(const float* v, uint8_t* out) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) {
        float a = fabsf(v[i]);
        if (a > amax) amax = a;
    }
    volatile float d = amax == 0.f ? 0.f : amax / 127.0f;
    uint16_t h = f32_to_f16_rne(d);
    out[0] = (uint8_t)(h & 0xff);
    out[1] = (uint8_t)(h >> 8);
    for (int i = 0; i < 32; i++) {
        int q = 0;
        if (d != 0.f) {
            float r = roundf(v[i] / d);
            r = r < -127.f ? -127.f : (r > 127.f ? 127.f : r);
            q = (int)r;
        }
        out[2 + i] = (uint8_t)(int8_t)q;
    }
}

/* load.rs:33-104: Q5_K block (176 B: d, dmin, 12 scale bytes, 32 qh, 128 qs) -> 8 Q8_0 blocks. */
int tfo_transcode_q5_k_to_q8_0(const uint8_t* raw, size_t nbytes, uint8_t* out) {
    if (nbytes % 176) return -1;
    for (size_t b = 0; b < nbytes / 176; b++) {
        const uint8_t* blk = raw + b * 176;
        const float d = tfo_half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
        const float dmin = tfo_half_to_float((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t *sc = blk + 4, *qh = blk + 16, *qs = blk + 48;
        float vals[256];
        uint8_t hl = 1, hh = 2;
        for (int g = 0; g < 4; g++) {
            uint8_t s0, m0, s1, m1;
            int j = 2 * g;
            for (int w = 0; w < 2; w++, j++) {
                uint8_t s, m;
                if (j < 4) {
                    s = sc[j] & 0x3f;
                    m = sc[j + 4] & 0x3f;
                } else {
                    s = (uint8_t)((sc[j + 4] & 0x0f) | ((sc[j - 4] >> 6) << 4));
                    m = (uint8_t)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
                }
                if (w == 0) s0 = s, m0 = m;
                else s1 = s, m1 = m;
            }
            volatile float scale0 = d * (float)s0, scale1 = d * (float)s1;
            volatile float off0 = dmin * (float)m0, off1 = dmin * (float)m1;
            for (int l = 0; l < 32; l++) {
                int low = (qs[32 * g + l] & 0x0f) + ((qh[l] & hl) ? 16 : 0);
                int high = (qs[32 * g + l] >> 4) + ((qh[l] & hh) ? 16 : 0);
                volatile float p0 = scale0 * (float)low, p1 = scale1 * (float)high; /* no fused multiply-add */
                vals[64 * g + l] = p0 - off0;
                vals[64 * g + 32 + l] = p1 - off1;
            }
            hl = (uint8_t)(hl << 2);
            hh = (uint8_t)(hh << 2);
        }
        for (int k = 0; k < 8; k++) q8_0_from_f32(vals + 32 * k, out + (b * 8 + k) * 34);
    }
    return 0;
}

/* load.rs:106-133: Q5_1 block (24 B: d, min, 4 qh, 16 qs) -> one Q8_0 block. */
int tfo_transcode_q5_1_to_q8_0(const uint8_t* raw, size_t nbytes, uint8_t* out) {
    if (nbytes % 24) return -1;
    for (size_t b = 0; b < nbytes / 24; b++) {
        const uint8_t* blk = raw + b * 24;
        const float d = tfo_half_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
        const float mn = tfo_half_to_float((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint32_t qh = (uint32_t)blk[4] | ((uint32_t)blk[5] << 8) | ((uint32_t)blk[6] << 16) | ((uint32_t)blk[7] << 24);
        const uint8_t* qs = blk + 8;
        float vals[32];
        for (int j = 0; j < 16; j++) {
            uint8_t h0 = (uint8_t)(((qh >> j) << 4) & 0x10), h1 = (uint8_t)((qh >> (j + 12)) & 0x10);
            volatile float p0 = (float)((qs[j] & 0x0f) | h0) * d, p1 = (float)((qs[j] >> 4) | h1) * d;
            vals[j] = p0 + mn;
            vals[j + 16] = p1 + mn;
        }
        q8_0_from_f32(vals, out + b * 34);
    }
    return 0;
}

size_t tfo_row_bytes(const tfo_mat* m) { return (size_t)(m->K / 256) * blk_bytes(m->type); }

/* y = W x (+bias) (+y).  act_mode 0: x is quantised to Q8 first (gemv.cu:377-403,
 * 469-490, 515-536, 2081-2115); act_mode 1: fp32 activation (gemv.cu:405-438, only
 * defined by the reference for Q6_K; Q4_K accepted here for the prefill restatement).
 * use_res 0/2 as gemv.cu:367-373 (2 = accumulate into out). */
int tfo_gemv(const tfo_mat* w, const float* x, float* out, const float* bias, int use_res, int act_mode) {
    int K = w->K, N = w->N, nb = K / 256;
    if (K % 256 || !blk_bytes(w->type)) return -1;
    if (w->type == TFO_Q8_0) act_mode = 0; /* Q8_0 weights always take the Q8 activation (gemv.cu:1585-1749) */
    int8_t* q8 = NULL;
    float* d8 = NULL;
    if (act_mode == 0) {
        q8 = (int8_t*)malloc((size_t)K);
        d8 = (float*)malloc(sizeof(float) * (size_t)(K / 32));
        tfo_quantize_q8(x, K, q8, d8);
    }
    size_t rb = tfo_row_bytes(w);
#pragma omp parallel for schedule(static) if (g_threads > 1)
    for (int j = 0; j < N; j++) {
        const uint8_t* row = w->data + (size_t)j * rb;
        float acc;
        if (w->type == TFO_Q8_0)
            acc = tfo_dot_q8_0_q8(row, K, q8, d8);
        else if (act_mode == 0)
            acc = w->type == TFO_Q4_K ? tfo_dot_q4k_q8(row, nb, q8, d8) : tfo_dot_q6k_q8(row, nb, q8, d8);
        else
            acc = w->type == TFO_Q4_K ? tfo_dot_q4k_f32(row, nb, x) : tfo_dot_q6k_f32(row, nb, x);
        if (use_res == 2) acc += out[j];
        if (bias) acc += bias[j];
        out[j] = acc;
    }
    free(q8);
    free(d8);
    return 0;
}

/* kernels/gemv.cu:2546-2575 — h[j] = silu(gate_j . x) * (up_j . x), x quantised to Q8
 * once, silu(g) = g / (1 + exp(-g)). */
int tfo_ffn_gate_up(const tfo_mat* gate, const tfo_mat* up, const float* x, float* out) {
    int K = gate->K, N = gate->N, nb = K / 256;
    if (gate->type != TFO_Q4_K || up->type != TFO_Q4_K || up->K != K || up->N != N || K % 256) return -1;
    int8_t* q8 = (int8_t*)malloc((size_t)K);
    float* d8 = (float*)malloc(sizeof(float) * (size_t)(K / 32));
    tfo_quantize_q8(x, K, q8, d8);
    size_t rb = tfo_row_bytes(gate);
#pragma omp parallel for schedule(static) if (g_threads > 1)
    for (int j = 0; j < N; j++) {
        float g = tfo_dot_q4k_q8(gate->data + (size_t)j * rb, nb, q8, d8);
        float u = tfo_dot_q4k_q8(up->data + (size_t)j * rb, nb, q8, d8);
        out[j] = (g / (1.f + expf(-g))) * u;
    }
    free(q8);
    free(d8);
    return 0;
}

/* ---------------------------------------------------------------- elementwise --- */

/* kernels/ops.cu:4-34 — y = x * rsqrt(mean(x^2) + eps) * w. */
void tfo_rms_norm(const float* x, const float* w, float* out, int n, float eps) {
    float s = 0.f;
    for (int i = 0; i < n; i++) s += x[i] * x[i];
    float scale = 1.0f / sqrtf(s / (float)n + eps);
    for (int i = 0; i < n; i++) out[i] = x[i] * scale * w[i];
}

/* kernels/ops.cu:348-371 — neox rotation of pairs (i, i + hd/2), fp32 angle. */
void tfo_rope_neox(float* x, int n_heads, int head_dim, int pos, float theta) {
    int half = head_dim / 2;
    for (int h = 0; h < n_heads; h++) {
        float* base = x + (size_t)h * head_dim;
        for (int i = 0; i < half; i++) {
            float freq = powf(theta, -2.f * (float)i / (float)head_dim);
            float ang = (float)pos * freq;
            float c = cosf(ang), s = sinf(ang);
            float x0 = base[i], x1 = base[i + half];
            base[i] = x0 * c - x1 * s;
            base[i + half] = x0 * s + x1 * c;
        }
    }
}

/* kernels/ops.cu:471-486 — fp32 -> f16 bits into cache row `pos` of [pos][n_kv*hd]. */
void tfo_copy_kv_f16(const float* src, uint16_t* cache, int pos, int stride) {
    for (int d = 0; d < stride; d++) cache[(size_t)pos * stride + d] = tfo_float_to_half_bits(src[d]);
}

/* kernels/attn/flash.cu:16-116 and 222-255 — softmax(q.K^T * scale) V over positions
 * 0..pos for every query head; KV head of query head h is h / (n_head / n_kv).  The
 * reference splits the range in 8 and merges (m, l, O); the merge is exact algebra, so
 * the restatement is the unsplit softmax in fp32. */
void tfo_attention(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                   int hd, int pos, float scale) {
    int rep = n_head / n_kv, stride = n_kv * hd, T = pos + 1;
#pragma omp parallel for schedule(static) if (g_threads > 1)
    for (int h = 0; h < n_head; h++) {
        int kvh = h / rep;
        float* sc = (float*)malloc(sizeof(float) * (size_t)T);
        float m = -1e30f;
        for (int t = 0; t < T; t++) {
            const uint16_t* kr = kc + (size_t)t * stride + (size_t)kvh * hd;
            float dot = 0.f;
            for (int d = 0; d < hd; d++) dot += q[(size_t)h * hd + d] * tfo_half_to_float(kr[d]);
            sc[t] = dot * scale;
            m = fmaxf(m, sc[t]);
        }
        float l = 0.f;
        for (int t = 0; t < T; t++) {
            sc[t] = expf(sc[t] - m);
            l += sc[t];
        }
        for (int d = 0; d < hd; d++) {
            float acc = 0.f;
            for (int t = 0; t < T; t++) acc += sc[t] * tfo_half_to_float(vc[(size_t)t * stride + (size_t)kvh * hd + d]);
            out[(size_t)h * hd + d] = acc / fmaxf(l, 1e-20f);
        }
        free(sc);
    }
}

/* kernels/ops.cu:573-599 — index of the maximum; on exact ties the reference's tree can
 * return any of the tied indices, this returns the lowest. */
int tfo_argmax(const float* x, int n) {
    int bi = 0;
    float bv = -1e30f;
    for (int i = 0; i < n; i++)
        if (x[i] > bv) {
            bv = x[i];
            bi = i;
        }
    return bi;
}

/* ---------------------------------------------------------------- dense model --- */

/* One decoder layer at n_tok = 1, applied in place to the residual stream x: layer
 * schedule of layer.rs:142-709 (attention block) and layer.rs:1210-1456 (dense FFN) with
 * the BASELINE dispatch: Q4_K matrices take Q8 activations, a Q6_K attn_v takes fp32
 * activations, o-proj and down take Q8 activations.  kc / vc: this layer's cache,
 * [max_seq][n_kv*hd] f16 bits; row `pos` is written.
 * act_f32 != 0 restates the reference's PREFILL arithmetic instead (gemm.cu: every
 * projection is dequantise-then-fp32; ops.cu silu_mul), as forward.rs:54-65 fills a cache. */
/* Optional taps of a dense layer (test aid, single-threaded callers): the vectors that are quantised to int8 inside the
 * layer besides its input — the attention output (o-proj's activation, n_head*hd), the residual stream after o-proj
 * (ffn_norm's input, n_embd) and SiLU*mul (down's activation, n_ff).  NULL switches a tap off. */
static float *g_tap_attn = NULL, *g_tap_mid = NULL, *g_tap_h = NULL;
void tfo_set_layer_taps(float* attn, float* mid, float* h) {
    g_tap_attn = attn;
    g_tap_mid = mid;
    g_tap_h = h;
}

int tfo_layer_forward(const tfo_model* M, int li, float* x, uint16_t* kc, uint16_t* vc, int pos, int act_f32, float* ssm,
                      float* conv) {
    int K = M->n_embd, H = M->n_head, Hkv = M->n_kv, hd = M->head_dim, FF = M->n_ff;
    if (li < 0 || li >= M->n_layer || pos < 0 || pos >= M->max_seq) return -1;
    int qn = H * hd, kvn = Hkv * hd;
    const tfo_layer* L = &M->layers[li];
    int mix = M->ssm_n_v * M->ssm_state; /* width of the linear mixer's output */
    int wide = K > qn ? K : qn;
    if (mix > wide) wide = mix;
    float* xb = (float*)malloc(sizeof(float) * (size_t)wide);
    float* y = (float*)malloc(sizeof(float) * (size_t)wide);
    float* q = (float*)malloc(sizeof(float) * (size_t)qn);
    float* kb = (float*)malloc(sizeof(float) * (size_t)kvn);
    float* vb = (float*)malloc(sizeof(float) * (size_t)kvn);
    float* h = (float*)malloc(sizeof(float) * (size_t)FF);
    float* u = (float*)malloc(sizeof(float) * (size_t)FF);
    int rc = 0;
    tfo_rms_norm(x, L->attn_norm, xb, K, M->eps);
    if (L->kind == TFO_LAYER_LINEAR) {
        /* layer.rs:711-1208 at n_tok = 1: mixer output projected onto the residual stream */
        if (!ssm || !conv) rc = -1;
        else rc |= tfo_linear_attn_block(M, L, xb, y, ssm, conv);
        if (!rc) rc |= tfo_gemv(&L->ssm_out, y, x, NULL, 2, 0);
    } else if (L->kind == TFO_LAYER_FULL_GATED) {
        rc |= tfo_gated_attn_block(M, L, xb, y, kc, vc, pos);
        rc |= tfo_gemv(&L->wo, y, x, NULL, 2, 0);
    } else {
        rc |= tfo_gemv(&L->wq, xb, q, L->bq, 0, act_f32);
        rc |= tfo_gemv(&L->wk, xb, kb, L->bk, 0, act_f32);
        rc |= tfo_gemv(&L->wv, xb, vb, L->bv, 0, (act_f32 || L->wv.type == TFO_Q6_K) ? 1 : 0);
        tfo_rope_neox(q, H, hd, pos, M->rope_theta);
        tfo_rope_neox(kb, Hkv, hd, pos, M->rope_theta);
        tfo_copy_kv_f16(kb, kc, pos, kvn);
        tfo_copy_kv_f16(vb, vc, pos, kvn);
        tfo_attention(q, kc, vc, xb, H, Hkv, hd, pos, 1.0f / sqrtf((float)hd));
        if (g_tap_attn) memcpy(g_tap_attn, xb, sizeof(float) * (size_t)qn);
        rc |= tfo_gemv(&L->wo, xb, x, NULL, 2, act_f32);
    }
    if (g_tap_mid) memcpy(g_tap_mid, x, sizeof(float) * (size_t)K);
    tfo_rms_norm(x, L->ffn_norm, xb, K, M->eps);
    if (!act_f32) {
        rc |= tfo_ffn_gate_up(&L->gate, &L->up, xb, h);
    } else {
        rc |= tfo_gemv(&L->gate, xb, h, NULL, 0, 1);
        rc |= tfo_gemv(&L->up, xb, u, NULL, 0, 1);
        for (int j = 0; j < FF; j++) h[j] = (h[j] / (1.f + expf(-h[j]))) * u[j];
    }
    if (g_tap_h) memcpy(g_tap_h, h, sizeof(float) * (size_t)FF);
    rc |= tfo_gemv(&L->down, h, x, NULL, 2, act_f32);
    free(xb); free(y); free(q); free(kb); free(vb); free(h); free(u);
    return rc;
}

/* Sizes of the per-layer recurrent state (kv.rs:12-15, config.rs:305-316): fp32 S[n_v][d][d] and the
 * conv ring [kernel-1][channels]. */
size_t tfo_ssm_floats(const tfo_model* M) { return (size_t)M->ssm_n_v * M->ssm_state * M->ssm_state; }
size_t tfo_conv_floats(const tfo_model* M) {
    size_t ch = (size_t)(2 * M->ssm_n_k + M->ssm_n_v) * M->ssm_state;
    return M->conv_kernel > 1 ? (size_t)(M->conv_kernel - 1) * ch : 0;
}

/* Vocabulary head, layer.rs:2125-2259: logits = E . Q8(RMSNorm(x, output_norm)). */
int tfo_head_forward(const tfo_model* M, const float* x, float* logits, float* xn_out) {
    int K = M->n_embd;
    float* xb = (float*)malloc(sizeof(float) * (size_t)K);
    tfo_rms_norm(x, M->output_norm, xb, K, M->eps);
    if (xn_out) memcpy(xn_out, xb, sizeof(float) * (size_t)K);
    const tfo_mat* head = M->output.data ? &M->output : &M->token_embd;
    int rc = tfo_gemv(head, xb, logits, NULL, 0, 0);
    free(xb);
    return rc;
}

/* Embedding row of a token, kernels/embed.cu:71-131. */
int tfo_embed(const tfo_model* M, int token, float* x) {
    if (token < 0 || token >= M->token_embd.N) return -1;
    return tfo_dequant_row(M->token_embd.type, M->token_embd.data + (size_t)token * tfo_row_bytes(&M->token_embd),
                           M->n_embd, x);
}

/* One batch-1 decode step (forward.rs:360-407 at n_tok = 1): embed, every layer, head.
 * kcache/vcache: [n_layer][max_seq][n_kv*hd] f16 bits. */
int tfo_decode_token(const tfo_model* M, uint16_t* kcache, uint16_t* vcache, int pos, int token, float* logits,
                     const tfo_taps* taps, int act_f32, float* ssm_all, float* conv_all) {
    int K = M->n_embd;
    if (pos < 0 || pos >= M->max_seq) return -1;
    float* x = (float*)malloc(sizeof(float) * (size_t)K);
    size_t lstride = (size_t)M->max_seq * M->n_kv * M->head_dim;
    int rc = tfo_embed(M, token, x);
    for (int li = 0; li < M->n_layer && rc == 0; li++)
        rc = tfo_layer_forward(M, li, x, kcache + (size_t)li * lstride, vcache + (size_t)li * lstride, pos, act_f32,
                               ssm_all ? ssm_all + (size_t)li * tfo_ssm_floats(M) : NULL,
                               conv_all ? conv_all + (size_t)li * tfo_conv_floats(M) : NULL);
    if (rc == 0) {
        if (taps && taps->x_final) memcpy(taps->x_final, x, sizeof(float) * (size_t)K);
        if (logits) rc = tfo_head_forward(M, x, logits, taps ? taps->xn_final : NULL);
    }
    free(x);
    return rc;
}

/* Greedy loop over tfo_decode_token (session.rs:288-368 without EOS handling): feeds
 * `first` at position pos0, then each argmax; writes n tokens and, if margins != NULL,
 * the top-1 minus top-2 logit gap of every step (for margin-gated token comparison). */
int tfo_decode_greedy(const tfo_model* M, uint16_t* kcache, uint16_t* vcache, int pos0, int first, int n,
                      int32_t* out_tokens, float* margins, float* last_logits, float* ssm_all, float* conv_all) {
    int V = M->output.data ? M->output.N : M->token_embd.N;
    float* logits = (float*)malloc(sizeof(float) * (size_t)V);
    int tok = first, rc = 0;
    for (int s = 0; s < n && rc == 0; s++) {
        rc = tfo_decode_token(M, kcache, vcache, pos0 + s, tok, logits, NULL, 0, ssm_all, conv_all);
        if (rc) break;
        tok = tfo_argmax(logits, V);
        out_tokens[s] = tok;
        if (margins) {
            float second = -1e30f;
            for (int i = 0; i < V; i++)
                if (i != tok && logits[i] > second) second = logits[i];
            margins[s] = logits[tok] - second;
        }
    }
    if (last_logits && rc == 0) memcpy(last_logits, logits, sizeof(float) * (size_t)V);
    free(logits);
    return rc;
}
