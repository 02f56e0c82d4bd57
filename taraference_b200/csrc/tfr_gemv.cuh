// Packed-weight x Q8-activation matrix-vector machinery for batch-1 decode.
//
// Data layout in HBM
//   Q4_K  rows keep the GGUF bytes: K/256 super-blocks of 144 B (16-byte header, 128 B of
//         nibbles), so every 16-byte piece is naturally aligned.
//   Q6_K  rows are re-ordered at upload into four planes per row — ql[nb*128], qh[nb*64],
//         scales[nb*16], d[nb*2 rounded up to 16] — because the 210-byte GGUF block is not
//         16-byte aligned.  Contents are unchanged (the reference pads each block to 212 B
//         for the same reason, crates/core/src/cuda/load.rs:145-159).
//
// Work decomposition
//   The unit of work is 64 consecutive K-elements of one row ("unit"): 32 B of nibbles + the
//   block header for Q4_K, 48 B of ql/qh + scales for Q6_K.  A CTA owns a contiguous range
//   of rows; its threads walk the units of a tile of rows in flat order, so a warp always
//   reads a contiguous span of weight bytes with 16-byte loads.  Per-unit partial sums go to
//   shared memory and are added per row in a fixed order, which makes results independent
//   of grid size and run-to-run deterministic.
//
// Integer contract (what must match the reference bit for bit)
//   Q4_K: I_j = sum nibble*q8 and S_j = sum q8 over each 32-element sub-block
//         (kernels/gemv.cu:71-130).  Q6_K: sum (q6-32)*q8 over each 16-element scale group
//         (kernels/gemv.cu:302-337).  Float combination order is not part of the contract.
#pragma once
#include <cuda_fp16.h>

#include "tfr_common.cuh"

namespace tfr {

constexpr int GEMV_THREADS = 1024;  // one CTA per SM; every thread keeps GEMV_UNROLL units in flight
constexpr int GEMV_UNROLL = 2;      // units (16-byte weight loads x3) in flight per thread per tile
constexpr int GEMV_PT_MIN = GEMV_THREADS * GEMV_UNROLL;

enum { WT_Q4K = 0, WT_Q6K = 1, WT_Q6K_F32 = 2 };
enum { SWZ_Q4 = 0, SWZ_Q6 = 1 };

struct Mat {
    const uint8_t* data;
    long long row_stride;  // bytes between rows (16-byte multiple)
    int type;              // TFR_Q4_K / TFR_Q6_K
    int K, N, nb;          // nb = K / 256
};

__host__ __device__ inline long long mat_row_stride(int type, int K) {
    int nb = K / 256;
    if (type == TFR_Q4_K) return (long long)nb * 144;
    return (long long)nb * 208 + (((long long)nb * 2 + 15) / 16) * 16;
}

// Quantised activation held in shared memory for the lifetime of a CTA.
struct Act {
    int4* q8;    // K/16 chunks of 16 int8, swizzled so that consecutive units hit consecutive banks
    float* d8;   // K/32 scales
    int* ss;     // K/32 packed sums: low 16 bits = sum of the first 16 q8 of the group, high = last 16
    float* xf;   // the staged fp32 vector (normalised in place), padded layout, see xs_idx()
    float* wf;   // staged RMSNorm weights, same layout (only when a norm is fused)
};

// The fp32 vector is staged with 4 floats of padding after every 32, so that the thread that
// quantises group g can read its 32 values as float4 without shared-memory bank conflicts.
__host__ __device__ __forceinline__ int xs_idx(int i) { return i + ((i >> 5) << 2); }
__host__ __device__ inline size_t xs_floats(int K) { return (size_t)K + (size_t)(K / 32) * 4; }

// Shared-memory bytes of an Act.
__host__ __device__ inline size_t act_smem_bytes(int K, bool with_xf, bool with_wf) {
    return (size_t)K + (size_t)(K / 32) * 8 + (with_xf ? xs_floats(K) * 4 : 0) + (with_wf ? xs_floats(K) * 4 : 0);
}

__device__ __forceinline__ Act act_carve(unsigned char* smem, int K, bool with_xf, bool with_wf) {
    Act a;
    a.q8 = reinterpret_cast<int4*>(smem);
    a.d8 = reinterpret_cast<float*>(smem + K);
    a.ss = reinterpret_cast<int*>(smem + K + (K / 32) * 4);
    unsigned char* p = smem + K + (K / 32) * 8;
    a.xf = with_xf ? reinterpret_cast<float*>(p) : nullptr;
    a.wf = with_wf ? reinterpret_cast<float*>(p + xs_floats(K) * 4) : nullptr;
    return a;
}

// Position of 16-byte chunk c (elements 16c..16c+15) inside Act::q8.  G = K/64.
__device__ __forceinline__ int swz_pos(int c, int G, int mode) {
    if (mode == SWZ_Q4) return (c & 3) * G + (c >> 2);
    return ((c & 7) >> 1) * G + ((c >> 3) << 1) + (c & 1);
}

// ------------------------------------------------------------------ activation sources

// Row `token` of the embedding table, decoded element by element
// (kernels/embed.cu:71-131: x = dequant(row), no scaling).
struct SrcEmbed {
    Mat E;
    int token;
    __device__ __forceinline__ float get(int i) const {
        const uint8_t* row = E.data + (long long)token * E.row_stride;
        int b = i >> 8, e = i & 255;
        if (E.type == TFR_Q4_K) {
            const uint8_t* blk = row + b * 144;
            float d = f16_to_f32(*reinterpret_cast<const unsigned short*>(blk));
            float dmin = f16_to_f32(*reinterpret_cast<const unsigned short*>(blk + 2));
            const uint8_t* sc = blk + 4;
            int j = e >> 5, t = e >> 6, l = e & 31;
            int s, m;
            if (j < 4) {
                s = sc[j] & 63;
                m = sc[j + 4] & 63;
            } else {
                s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4);
                m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
            }
            int qb = blk[16 + 32 * t + l];
            int nib = (j & 1) ? (qb >> 4) : (qb & 0xF);
            return d * (float)s * (float)nib - dmin * (float)m;
        }
        int n = e >> 7, r = e & 127, jj = r >> 5, l = r & 31;
        const uint8_t* ql = row + b * 128 + 64 * n;
        const uint8_t* qh = row + E.nb * 128 + b * 64 + 32 * n;
        const signed char* sc = reinterpret_cast<const signed char*>(row + E.nb * 192 + b * 16);
        float d = f16_to_f32(*reinterpret_cast<const unsigned short*>(row + E.nb * 208 + 2 * b));
        int lo = (jj & 1) ? ql[32 + l] : ql[l];
        lo = (jj & 2) ? (lo >> 4) : (lo & 0xF);
        int q = (lo | (((qh[l] >> (2 * jj)) & 3) << 4)) - 32;
        return d * (float)sc[8 * n + (l >> 4) + 2 * jj] * (float)q;
    }
};

// RMSNorm scale over the vector staged in shared memory, with the reduction shape of
// kernels/ops.cu:4-34: 256 strided partial sums, then the binary tree red[t] += red[t + s]
// for s = 128 .. 1.  One warp replays that tree in registers (lane l holds red[l + 32k]),
// pairing exactly the operands the reference pairs, so the normalised vector — and with it
// the int8 activation — is bit-identical to the reference build's for the same input.
// Called by all threads of the CTA; red: 257 floats of shared memory.
__device__ float rms_scale_staged(const float* xs, int n, float eps, float* red) {
    const int tid = threadIdx.x, lane = tid & 31;
    if (tid < 256) {
        float local = 0.f;
        for (int i = tid; i < n; i += 256) {
            const float v = xs[xs_idx(i)];
            local += v * v;
        }
        red[tid] = local;
    }
    __syncthreads();
    if (tid < 32) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = red[lane + 32 * k];
#pragma unroll
        for (int k = 0; k < 4; k++) v[k] += v[k + 4];  // s = 128
        v[0] += v[2];                                  // s = 64
        v[1] += v[3];
        v[0] += v[1];                                  // s = 32
        float t = v[0];
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) t += __shfl_down_sync(TFR_FULL_MASK, t, sft);
        if (lane == 0) red[256] = rsqrtf(t / (float)n + eps);
    }
    __syncthreads();
    return red[256];
}

// Q8 activation quantiser over the staged vector, kernels/gemv.cu:16-65: per 32 values
// d = amax * (1/127), q = rn(x / d) with the build's approximate division, zero group ->
// zeros.  One THREAD per 32-value group (the reference uses a warp per group; max and the
// per-element rounding do not depend on that).  With a fused RMSNorm the normalised value
// x * scale * w is formed in the reference's order and written back for fp32-route rows.
// Also records per-half-group sums of q (pure integer, derived from q).
__device__ void act_quantize_staged(Act& act, bool has_norm, float scale, int K, int swz) {
    const int g = threadIdx.x;
    if (g >= (K >> 5)) return;
    const int G = K >> 6;
    float4* xg = reinterpret_cast<float4*>(act.xf + 36 * g);
    const float4* wg = reinterpret_cast<const float4*>(act.wf + 36 * g);
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        float4 x = xg[k];
        if (has_norm) {
            const float4 w = wg[k];
            x.x = x.x * scale * w.x;
            x.y = x.y * scale * w.y;
            x.z = x.z * scale * w.z;
            x.w = x.w * scale * w.w;
            xg[k] = x;
        }
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
    }
    const float d = amax * (1.0f / 127.0f);
    int wd[8];
    int s_lo = 0, s_hi = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const float4 x = xg[k];
        int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
        if (amax != 0.f) {
            q0 = (int)(signed char)__float2int_rn(x.x / d);
            q1 = (int)(signed char)__float2int_rn(x.y / d);
            q2 = (int)(signed char)__float2int_rn(x.z / d);
            q3 = (int)(signed char)__float2int_rn(x.w / d);
        }
        wd[k] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | ((q3 & 0xff) << 24);
        if (k < 4) s_lo += q0 + q1 + q2 + q3;
        else s_hi += q0 + q1 + q2 + q3;
    }
    act.q8[swz_pos(2 * g, G, swz)] = make_int4(wd[0], wd[1], wd[2], wd[3]);
    act.q8[swz_pos(2 * g + 1, G, swz)] = make_int4(wd[4], wd[5], wd[6], wd[7]);
    act.d8[g] = d;
    act.ss[g] = (s_lo & 0xffff) | (s_hi << 16);
}

// ------------------------------------------------------------------ unit loads / dots

// Weight bytes of one unit.  Q4_K: a, b = 32 B of nibbles, c = block header.  Q6_K: a, b = ql
// pieces, c = qh piece, s = 8 scale bytes of the half block, dbits = fp16 d.
struct UnitW {
    int4 a, b, c;
    int2 s;
    unsigned int dbits;
};

// Byte offsets of a thread's unit inside a row; a thread keeps the same unit column for the
// whole kernel, so these are computed once.
struct UnitOff {
    int q4_hdr, q4_qs;              // Q4_K
    int q6_ql, q6_qh, q6_sc, q6_d;  // Q6_K
};

__device__ __forceinline__ UnitOff unit_offsets(int u, int nb) {
    UnitOff o;
    o.q4_hdr = (u >> 2) * 144;
    o.q4_qs = o.q4_hdr + 16 + 32 * (u & 3);
    const int b = u >> 2, n = (u >> 1) & 1, is = u & 1;
    o.q6_ql = b * 128 + 64 * n + 16 * is;
    o.q6_qh = nb * 128 + b * 64 + 32 * n + 16 * is;
    o.q6_sc = nb * 192 + b * 16 + 8 * n;
    o.q6_d = nb * 208 + 2 * b;
    return o;
}

__device__ __forceinline__ void load_unit(UnitW& w, int wt, const uint8_t* row, const UnitOff& o) {
    if (wt == WT_Q4K) {
        w.c = ldg_stream(row + o.q4_hdr);
        w.a = ldg_stream(row + o.q4_qs);
        w.b = ldg_stream(row + o.q4_qs + 16);
    } else {
        w.a = ldg_stream(row + o.q6_ql);
        w.b = ldg_stream(row + o.q6_ql + 32);
        w.c = ldg_stream(row + o.q6_qh);
        w.s = ldg_stream8(row + o.q6_sc);
        w.dbits = __ldg(reinterpret_cast<const unsigned short*>(row + o.q6_d));
    }
}

// u8 x s8 dot product with 32-bit accumulate (bytes of a are unsigned, bytes of b signed).
__device__ __forceinline__ int dp4a_us(unsigned int a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dot16_us(const int4& w, unsigned int mask, const int4& a) {
    int acc = dp4a_us((unsigned)w.x & mask, a.x, 0);
    acc = dp4a_us((unsigned)w.y & mask, a.y, acc);
    acc = dp4a_us((unsigned)w.z & mask, a.z, acc);
    acc = dp4a_us((unsigned)w.w & mask, a.w, acc);
    return acc;
}
__device__ __forceinline__ int dot16(const int4& w, const int4& a, int acc) {
    acc = __dp4a(w.x, a.x, acc);
    acc = __dp4a(w.y, a.y, acc);
    acc = __dp4a(w.z, a.z, acc);
    acc = __dp4a(w.w, a.w, acc);
    return acc;
}

// Exact int -> float for |i| < 2^22 on the FP32 pipe (the conversion instruction runs at a
// quarter of the rate).  All integers converted here are below 2^22 in magnitude:
// |I * sc| <= 15*127*32*63 < 2^22, |J| <= 32*127*16 < 2^17.
__device__ __forceinline__ float i2f_small(int i) { return __int_as_float(0x4B400000 + i) - 12582912.0f; }

// The activation pieces one unit needs, read from shared memory once per pass.
struct Frag {
    int4 a0, a1, a2, a3;  // the unit's 64 int8 activations, in the order its weight pieces use them
    float4 d8;            // Q4_K: (d8 of sub-block 2t, 2t+1, -, -).  Q6_K: d8 of the four runs' groups
    int4 aux;             // Q4_K: float bits of d8*S of the two sub-blocks.  Q6_K: -32*S16 of the four runs,
                          // used as the dp4a accumulator start so that sum (q6-32)*q8 stays an exact integer
};

__device__ __forceinline__ void frag_load(Frag& f, int wt, const Act& act, int u, int G) {
    f.a0 = act.q8[u];
    f.a1 = act.q8[G + u];
    f.a2 = act.q8[2 * G + u];
    f.a3 = act.q8[3 * G + u];
    if (wt == WT_Q4K) {
        const float2 d = reinterpret_cast<const float2*>(act.d8)[u];
        const int2 ss = reinterpret_cast<const int2*>(act.ss)[u];
        const int S0 = (int)(short)(ss.x & 0xffff) + (ss.x >> 16);
        const int S1 = (int)(short)(ss.y & 0xffff) + (ss.y >> 16);
        f.d8 = make_float4(d.x, d.y, 0.f, 0.f);
        f.aux = make_int4(__float_as_int(d.x * i2f_small(S0)), __float_as_int(d.y * i2f_small(S1)), 0, 0);
    } else {
        f.d8 = reinterpret_cast<const float4*>(act.d8)[u >> 1];
        const int4 ss = reinterpret_cast<const int4*>(act.ss)[u >> 1];
        const int is = u & 1;
#define TFR_S16(v) (is ? ((v) >> 16) : (int)(short)((v) & 0xffff))
        f.aux = make_int4(-32 * TFR_S16(ss.x), -32 * TFR_S16(ss.y), -32 * TFR_S16(ss.z), -32 * TFR_S16(ss.w));
#undef TFR_S16
    }
}

// Q4_K unit (sub-blocks 2t and 2t+1 of its super-block, t = u & 3) against the fragment.
// ints (optional): I0, I1 = sum nibble*q8 of the two sub-blocks — the bit-exact contract of
// kernels/gemv.cu:71-130; the sums S are the fragment's.  High nibbles are multiplied as
// (nibble << 4) and the exact factor 16 is shifted out afterwards.
__device__ __forceinline__ float q4k_dot(const UnitW& w, const Frag& f, int t, int* ints) {
    int I0 = dot16_us(w.a, 0x0f0f0f0fu, f.a0);
    I0 += dot16_us(w.b, 0x0f0f0f0fu, f.a1);
    int I1 = dot16_us(w.a, 0xf0f0f0f0u, f.a2);
    I1 += dot16_us(w.b, 0xf0f0f0f0u, f.a3);
    I1 >>= 4;
    if (ints) {
        ints[0] = I0;
        ints[1] = I1;
    }
    // 6-bit scales / mins, kernels/common.cu:40-50 in the 16-bit form of gemv.cu:94-106.
    const int sh = 16 * (t & 1);
    const unsigned y16 = ((unsigned)w.c.y >> sh) & 0xffffu, z16 = ((unsigned)w.c.z >> sh) & 0xffffu,
                   w16 = ((unsigned)w.c.w >> sh) & 0xffffu;
    unsigned aux_sc, aux_m;
    if (t < 2) {
        aux_sc = y16 & 0x3f3fu;
        aux_m = z16 & 0x3f3fu;
    } else {
        aux_sc = (w16 & 0x0f0fu) | ((y16 & 0xc0c0u) >> 2);
        aux_m = ((w16 >> 4) & 0x0f0fu) | ((z16 & 0xc0c0u) >> 2);
    }
    const int sc0 = aux_sc & 0xff, sc1 = aux_sc >> 8, m0 = aux_m & 0xff, m1 = aux_m >> 8;
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&w.c.x));  // (d, dmin)
    return dd.x * (f.d8.x * i2f_small(I0 * sc0) + f.d8.y * i2f_small(I1 * sc1)) -
           dd.y * (__int_as_float(f.aux.x) * i2f_small(m0) + __int_as_float(f.aux.y) * i2f_small(m1));
}

// Q6_K unit: runs j = 0..3 are elements 128n + 32j + 16is + [0,16) of block b (u = 4b+2n+is).
// ints (optional): the four scale-group dots sum (q6-32)*q8 of kernels/gemv.cu:302-337.
__device__ __forceinline__ float q6k_dot(const UnitW& w, const Frag& f, int is, int* ints) {
    const int4 h = w.c;
    int4 r0, r1, r2, r3;
#define TFR_Q6W(c)                                                          \
    r0.c = (w.a.c & 0x0f0f0f0f) | ((h.c << 4) & 0x30303030);                \
    r1.c = (w.b.c & 0x0f0f0f0f) | ((h.c << 2) & 0x30303030);                \
    r2.c = (((unsigned)w.a.c >> 4) & 0x0f0f0f0f) | (h.c & 0x30303030);      \
    r3.c = (((unsigned)w.b.c >> 4) & 0x0f0f0f0f) | (((unsigned)h.c >> 2) & 0x30303030);
    TFR_Q6W(x) TFR_Q6W(y) TFR_Q6W(z) TFR_Q6W(w)
#undef TFR_Q6W
    const int J0 = dot16(r0, f.a0, f.aux.x), J1 = dot16(r1, f.a1, f.aux.y), J2 = dot16(r2, f.a2, f.aux.z),
              J3 = dot16(r3, f.a3, f.aux.w);
    const unsigned lo = (unsigned)w.s.x >> (8 * is), hi = (unsigned)w.s.y >> (8 * is);
    const float s0 = i2f_small((int)(signed char)(lo & 0xff)), s1 = i2f_small((int)(signed char)((lo >> 16) & 0xff));
    const float s2 = i2f_small((int)(signed char)(hi & 0xff)), s3 = i2f_small((int)(signed char)((hi >> 16) & 0xff));
    if (ints) {
        ints[0] = J0;
        ints[1] = J1;
        ints[2] = J2;
        ints[3] = J3;
    }
    const float d = f16_to_f32((unsigned short)w.dbits);
    return d * (s0 * f.d8.x * i2f_small(J0) + s1 * f.d8.y * i2f_small(J1) + s2 * f.d8.z * i2f_small(J2) +
                s3 * f.d8.w * i2f_small(J3));
}

// One run of 16 elements of a Q6_K row against the fp32 activation staged in shared memory
// (the reference's route for a Q6_K attn_v, kernels/gemv.cu:233-264: acc += d * scale * q * x
// with x unquantised).  u = 4b + 2n + is names the unit, j the run: elements
// 256b + 128n + 32j + 16is + [0, 16).  Reads the SoA row layout directly.
__device__ __forceinline__ float q6k_run_dot_f32(const uint8_t* row, int nb, int u, int j, const float* xf) {
    const int b = u >> 2, n = (u >> 1) & 1, is = u & 1;
    const int4 ql = __ldg(reinterpret_cast<const int4*>(row + b * 128 + 64 * n + 32 * (j & 1) + 16 * is));
    const int4 qh = __ldg(reinterpret_cast<const int4*>(row + nb * 128 + b * 64 + 32 * n + 16 * is));
    const float sc = (float)(int)*reinterpret_cast<const signed char*>(row + nb * 192 + b * 16 + 8 * n + is + 2 * j);
    const float d = f16_to_f32(__ldg(reinterpret_cast<const unsigned short*>(row + nb * 208 + 2 * b)));
    const float dsc = d * sc;
    const float4* x4 = reinterpret_cast<const float4*>(xf + xs_idx(256 * b + 128 * n + 32 * j + 16 * is));
    const int qlw[4] = {ql.x, ql.y, ql.z, ql.w};
    const int qhw[4] = {qh.x, qh.y, qh.z, qh.w};
    const int nsh = 4 * (j >> 1), hsh = 2 * j;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float4 x = x4[k];
        const float xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int by = 0; by < 4; by++) {
            const int nib = (qlw[k] >> (8 * by + nsh)) & 0xF;
            const int hb = (qhw[k] >> (8 * by + hsh)) & 3;
            acc += dsc * (float)((nib | (hb << 4)) - 32) * xv[by];
        }
    }
    return acc;
}

// ------------------------------------------------------------------ row-pair maps

// All kernels walk "row pairs": two rows whose results go to the epilogue together.
// pair p of a plain matrix = rows (2p, 2p+1); of the gate/up map = (gate row p, up row p).
struct PairRows {
    const uint8_t* r0;
    const uint8_t* r1;
    int id;  // pair id handed to the epilogue
};

// Contiguous share of n items for CTA c of C, with n = C*quot + rem split on the host so that
// the kernel needs no division: the first `rem` CTAs take quot+1 items.
struct Share {
    int quot, rem;
    __device__ __forceinline__ int begin(int c) const { return c * quot + min(c, rem); }
    __device__ __forceinline__ int count(int c) const { return quot + (c < rem ? 1 : 0); }
};
inline Share make_share(int n, int C) {
    Share s;
    s.quot = n / C;
    s.rem = n % C;
    return s;
}

struct MapSingle {
    Mat m;
    Share sh;
    __device__ __forceinline__ int n_local(int c) const { return sh.count(c); }
    __device__ __forceinline__ PairRows pair(int c, int i) const {
        const int p = sh.begin(c) + i;
        PairRows r;
        r.r0 = m.data + (long long)(2 * p) * m.row_stride;
        r.r1 = (2 * p + 1 < m.N) ? r.r0 + m.row_stride : r.r0;  // odd N: the last pair repeats its row
        r.id = p;
        return r;
    }
    __device__ __forceinline__ int nb() const { return m.nb; }
};
struct MapPair {
    Mat a, b;
    Share sh;
    __device__ __forceinline__ int n_local(int c) const { return sh.count(c); }
    __device__ __forceinline__ PairRows pair(int c, int i) const {
        const int p = sh.begin(c) + i;
        PairRows r;
        r.r0 = a.data + (long long)p * a.row_stride;
        r.r1 = b.data + (long long)p * b.row_stride;
        r.id = p;
        return r;
    }
    __device__ __forceinline__ int nb() const { return a.nb; }
};
// Q and K stacked, each spread over all CTAs: a CTA's local list is its Q pairs, then its K
// pairs.  Pair ids continue across the matrices (Q pairs first, then K, then V).
struct MapQK {
    Mat q, k;
    Share shq, shk;
    __device__ __forceinline__ int n_local(int c) const { return shq.count(c) + shk.count(c); }
    __device__ __forceinline__ PairRows pair(int c, int i) const {
        const int nq = shq.count(c);
        const bool isk = i >= nq;
        const Mat& m = isk ? k : q;
        const int p = isk ? shk.begin(c) + (i - nq) : shq.begin(c) + i;
        PairRows r;
        r.r0 = m.data + (long long)(2 * p) * m.row_stride;
        r.r1 = r.r0 + m.row_stride;
        r.id = isk ? (q.N >> 1) + p : p;
        return r;
    }
    __device__ __forceinline__ int nb() const { return q.nb; }
};

// Sum of v0 over the warp in lane 0 and of v1 in lane 16, with five shuffles.
__device__ __forceinline__ float warp_sum_pair(float v0, float v1, int lane) {
    const bool up = (lane & 16) != 0;
    float x = (up ? v1 : v0) + __shfl_xor_sync(TFR_FULL_MASK, up ? v0 : v1, 16);
    x += __shfl_xor_sync(TFR_FULL_MASK, x, 8);
    x += __shfl_xor_sync(TFR_FULL_MASK, x, 4);
    x += __shfl_xor_sync(TFR_FULL_MASK, x, 2);
    x += __shfl_xor_sync(TFR_FULL_MASK, x, 1);
    return x;
}

}  // namespace tfr
