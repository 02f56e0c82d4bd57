// Packed-weight x Q8-activation matrix-vector machinery for batch-1 decode.
//
// Data layout in HBM ("warp tiles")
//   A matrix is a flat sequence of K-quant blocks, f = row * (K/256) + block.  At upload the
//   blocks are regrouped into tiles of 32 consecutive blocks, stored piece-major: the j-th
//   16-byte piece of all 32 blocks is one contiguous 512-byte slab.  A warp that gives lane l
//   the block 32*t + l therefore reads every slab with one fully coalesced 512-byte request,
//   and each lane ends up holding one whole block (Q4_K: 9 pieces = 144 B; Q6_K: 13 pieces +
//   the fp16 d = 210 B).  Block CONTENTS are the GGUF bytes, untouched; density is exactly
//   144 B / 210 B per 256 weights.  (The reference keeps GGUF order and pads Q6_K blocks to
//   212 B for 4-byte alignment, crates/core/src/cuda/load.rs:145-159.)
//
// Work decomposition
//   One lane owns one 256-element block: it decodes the block's scales once, runs 64 dp4a
//   against the block's int8 activations held in shared memory and produces one fp32 partial.
//   Owning a whole block keeps the instruction count per weight byte low enough for an SM to
//   keep up with its share of HBM bandwidth — with smaller units the kernel is issue-bound.
//   K = 2048 puts a row in 8 adjacent lanes: three shuffles finish it.  Other K write the
//   partials to shared memory and rows are summed in a fixed order after one barrier.
//   Results never depend on grid size and are run-to-run deterministic.
//
// Integer contract (what must match the reference bit for bit)
//   Q4_K: I_j = sum nibble*q8 and S_j = sum q8 over each 32-element sub-block
//         (kernels/gemv.cu:71-130).  Q6_K: sum (q6-32)*q8 over each 16-element scale group
//         (kernels/gemv.cu:302-337).  Float combination order is not part of the contract.
#pragma once
#include <cuda_fp16.h>

#include "tfr_common.cuh"

namespace tfr {

constexpr int GEMV_THREADS = 1024;  // one CTA per SM
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int Q4_PIECES = 9, Q6_PIECES = 13, Q8_PIECES = 17;
constexpr int Q4_TILE_BYTES = 32 * 144, Q6_TILE_BYTES = 32 * 210;
// Q8_0 (34 B per 32 weights): eight consecutive blocks = 272 contiguous bytes are handled as one 256-weight block
constexpr int Q8_SUPER_BYTES = 8 * 34, Q8_TILE_BYTES = 32 * Q8_SUPER_BYTES;

enum { WT_Q4K = 0, WT_Q6K = 1 };

struct Mat {
    const uint8_t* data;  // tiled
    int type;             // TFR_Q4_K / TFR_Q6_K / TFR_Q8_0
    int K, N, nb;         // nb = K / 256
};

__host__ __device__ inline int tile_bytes(int type) {
    return type == TFR_Q4_K ? Q4_TILE_BYTES : type == TFR_Q8_0 ? Q8_TILE_BYTES : Q6_TILE_BYTES;
}
__host__ __device__ inline int block_bytes_256(int type) { return type == TFR_Q4_K ? 144 : type == TFR_Q8_0 ? Q8_SUPER_BYTES : 210; }
__host__ __device__ inline long long mat_tiles(int K, long long N) { return (N * (K / 256) + 31) / 32; }
__host__ __device__ inline long long mat_device_bytes(int type, int K, long long N) {
    return mat_tiles(K, N) * tile_bytes(type);
}

// Byte j (0..143 / 0..209) of flat block f.
__device__ __forceinline__ const uint8_t* block_byte(const Mat& m, long long f, int j) {
    const uint8_t* t = m.data + (f >> 5) * tile_bytes(m.type);
    const int lane = (int)(f & 31);
    if (m.type == TFR_Q6_K && j >= 208) return t + Q6_PIECES * 512 + lane * 2 + (j - 208);
    return t + (j >> 4) * 512 + lane * 16 + (j & 15);
}

// ------------------------------------------------------------------ activation in shared memory

// Quantised activation for the lifetime of a CTA.
struct Act {
    int4* q8;    // chunk i (16 int8) of block b at [i * nb + b]: lanes on adjacent blocks hit adjacent banks
    float* d8;   // [K/32] scale of every 32-group (block b, sub-block j at 8b + j)
    float* ds;   // [K/32] d8 * (sum of the group's q8): the Q4_K "min" term needs only this product
    int* s16n;   // [K/16] -32 * (sum of the 16-chunk's q8): start value of the Q6_K dp4a accumulators
    float* xf;   // the staged fp32 vector (normalised in place), padded layout, see xs_idx()
    float* wf;   // staged RMSNorm weights, same layout (only when a norm is fused)
};

// The fp32 vector is staged with 4 floats of padding after every 32, so that eight lanes can read
// one 32-value group as float4 while other groups' lanes hit other banks.
__host__ __device__ __forceinline__ int xs_idx(int i) { return i + ((i >> 5) << 2); }
__host__ __device__ inline size_t xs_floats(int K) { return (size_t)K + (size_t)(K / 32) * 4; }

__host__ __device__ inline size_t act_smem_bytes(int K, bool with_xf, bool with_wf) {
    return (size_t)K + (size_t)(K / 32) * 8 + (size_t)(K / 16) * 4 + (with_xf ? xs_floats(K) * 4 : 0) +
           (with_wf ? xs_floats(K) * 4 : 0);
}

__device__ __forceinline__ Act act_carve(unsigned char* smem, int K, bool with_xf, bool with_wf) {
    Act a;
    unsigned char* p = smem;
    a.q8 = reinterpret_cast<int4*>(p);
    p += K;
    a.d8 = reinterpret_cast<float*>(p);
    p += (K / 32) * 4;
    a.ds = reinterpret_cast<float*>(p);
    p += (K / 32) * 4;
    a.s16n = reinterpret_cast<int*>(p);
    p += (K / 16) * 4;
    a.xf = with_xf ? reinterpret_cast<float*>(p) : nullptr;
    if (with_xf) p += xs_floats(K) * 4;
    a.wf = with_wf ? reinterpret_cast<float*>(p) : nullptr;
    return a;
}

// Stores one quantised 32-group's derived values; the int8 themselves are written by the caller.
__device__ __forceinline__ void act_store_group(const Act& act, int g, float d, int s_lo, int s_hi) {
    act.d8[g] = d;
    act.ds[g] = d * (float)(s_lo + s_hi);
    act.s16n[2 * g] = -32 * s_lo;
    act.s16n[2 * g + 1] = -32 * s_hi;
}

// Word (4 int8) holding elements e..e+3 (e a multiple of 4) -> its slot in Act::q8.
__device__ __forceinline__ int* act_word_ptr(const Act& act, int e, int nb) {
    const int b = e >> 8, i = (e & 255) >> 4, w = (e & 15) >> 2;
    return reinterpret_cast<int*>(act.q8) + ((i * nb + b) << 2) + w;
}

// ------------------------------------------------------------------ activation sources

// Row `token` of the embedding table, decoded element by element
// (kernels/embed.cu:71-131: x = dequant(row), no scaling).
struct SrcEmbed {
    Mat E;
    int token;
    __device__ __forceinline__ float get(int i) const {
        const long long f = (long long)token * E.nb + (i >> 8);
        const int e = i & 255;
        if (E.type == TFR_Q4_K) {
            const float d = f16_to_f32(*reinterpret_cast<const unsigned short*>(block_byte(E, f, 0)));
            const float dmin = f16_to_f32(*reinterpret_cast<const unsigned short*>(block_byte(E, f, 2)));
            const uint8_t* sc = block_byte(E, f, 4);  // bytes 4..15 share piece 0
            const int j = e >> 5, t = e >> 6, l = e & 31;
            int s, m;
            if (j < 4) {
                s = sc[j] & 63;
                m = sc[j + 4] & 63;
            } else {
                s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4);
                m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
            }
            const int qb = *block_byte(E, f, 16 + 32 * t + l);
            const int nib = (j & 1) ? (qb >> 4) : (qb & 0xF);
            return d * (float)s * (float)nib - dmin * (float)m;
        }
        const int n = e >> 7, r = e & 127, jj = r >> 5, l = r & 31;
        int lo = *block_byte(E, f, 64 * n + ((jj & 1) ? 32 : 0) + l);
        lo = (jj & 2) ? (lo >> 4) : (lo & 0xF);
        const int hb = (*block_byte(E, f, 128 + 32 * n + l) >> (2 * jj)) & 3;
        const float sc = (float)(int)*reinterpret_cast<const signed char*>(block_byte(E, f, 192 + 8 * n + (l >> 4) + 2 * jj));
        const float d = f16_to_f32(*reinterpret_cast<const unsigned short*>(block_byte(E, f, 208)));
        return d * sc * (float)((lo | (hb << 4)) - 32);
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

// Q8 activation quantiser, kernels/gemv.cu:16-65: per 32 values d = amax * (1/127),
// q = rn(x / d) with the build's approximate division, zero group -> zeros.  Eight adjacent
// lanes share a group, four values each (x holds elements 4*i4 .. 4*i4+3 of the vector); max
// and the per-element rounding do not depend on how the reference spreads a group over a warp.
// Must be called by whole warps (the shuffles are warp-wide); `on` masks lanes past the end.
__device__ __forceinline__ void act_quantize4(const Act& act, float4 x, int i4, bool on, int nb) {
    float amax = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
    amax = fmaxf(amax, __shfl_xor_sync(TFR_FULL_MASK, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(TFR_FULL_MASK, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(TFR_FULL_MASK, amax, 4));
    const float d = amax * (1.0f / 127.0f);
    int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
    if (amax != 0.f) {
        q0 = (int)(signed char)__float2int_rn(x.x / d);
        q1 = (int)(signed char)__float2int_rn(x.y / d);
        q2 = (int)(signed char)__float2int_rn(x.z / d);
        q3 = (int)(signed char)__float2int_rn(x.w / d);
    }
    int s = q0 + q1 + q2 + q3;
    s += __shfl_xor_sync(TFR_FULL_MASK, s, 1);
    s += __shfl_xor_sync(TFR_FULL_MASK, s, 2);  // lanes 0-3 of the group: first 16 values, lanes 4-7: last 16
    const int other = __shfl_xor_sync(TFR_FULL_MASK, s, 4);
    if (on) {
        *act_word_ptr(act, 4 * i4, nb) = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | ((q3 & 0xff) << 24);
        if ((i4 & 7) == 0) act_store_group(act, i4 >> 3, d, s, other);
    }
}

// ------------------------------------------------------------------ block dots

// u8 x s8 dot product with 32-bit accumulate (bytes of a are unsigned, bytes of b signed).
__device__ __forceinline__ int dp4a_us(unsigned int a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dot16_us(const int4& w, unsigned int mask, const int4& a, int acc) {
    acc = dp4a_us((unsigned)w.x & mask, a.x, acc);
    acc = dp4a_us((unsigned)w.y & mask, a.y, acc);
    acc = dp4a_us((unsigned)w.z & mask, a.z, acc);
    acc = dp4a_us((unsigned)w.w & mask, a.w, acc);
    return acc;
}

// Exact int -> float for |i| < 2^22 on the FP32 pipe (the conversion instruction runs at a
// quarter of the rate).  All integers converted here are below 2^22 in magnitude:
// |I * sc| <= 15*127*32*63 < 2^22, |J| <= 32*127*16 < 2^17.
__device__ __forceinline__ float i2f_small(int i) { return __int_as_float(0x4B400000 + i) - 12582912.0f; }

// Tag types: which K-quant a kernel instance walks.
struct BlockQ4 {
    static constexpr int TILE_BYTES = Q4_TILE_BYTES;
};
struct BlockQ6 {
    static constexpr int TILE_BYTES = Q6_TILE_BYTES;
};
struct BlockQ8 {
    static constexpr int TILE_BYTES = Q8_TILE_BYTES;
};

// 16-byte piece `i` of this lane's block inside a tile.  SMEM: the tile is the shared-memory copy.
template <bool SMEM>
__device__ __forceinline__ int4 tile_piece(const uint8_t* tile, int lane, int i) {
    const uint8_t* p = tile + i * 512 + lane * 16;
    if (SMEM) {
        int4 v;
        asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
        return v;
    }
    return *reinterpret_cast<const int4*>(p);
}

// One Q4_K block (kernels/gemv.cu:71-130 over all eight sub-blocks) against block b of the
// activation.  ints (optional): I[0..7] = sum nibble*q8 per sub-block.  High nibbles are
// multiplied as (nibble << 4); the exact factor 16 is shifted out afterwards.
template <bool SMEM>
__device__ __forceinline__ float block_dot(BlockQ4, const uint8_t* tile, int lane, const Act& act, int b, int nb, int* ints) {
    const int4 wh = tile_piece<SMEM>(tile, lane, 0);  // d, dmin, 12 scale bytes
    // 6-bit scales and mins of the eight sub-blocks, kernels/common.cu:40-50, unpacked four at a time:
    // sc[0..3] = s0 & 63, sc[4..7] = (s2 & 15) | ((s0 >> 6) << 4), m[0..3] = s1 & 63, m[4..7] = (s2 >> 4) | ((s1 >> 6) << 4)
    const unsigned s0 = (unsigned)wh.y, s1 = (unsigned)wh.z, s2 = (unsigned)wh.w;
    const unsigned sc_lo = s0 & 0x3f3f3f3fu, sc_hi = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
    const unsigned m_lo = s1 & 0x3f3f3f3fu, m_hi = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
    const float4 d8a = reinterpret_cast<const float4*>(act.d8)[2 * b], d8b = reinterpret_cast<const float4*>(act.d8)[2 * b + 1];
    const float4 dsa = reinterpret_cast<const float4*>(act.ds)[2 * b], dsb = reinterpret_cast<const float4*>(act.ds)[2 * b + 1];
    const float d8[8] = {d8a.x, d8a.y, d8a.z, d8a.w, d8b.x, d8b.y, d8b.z, d8b.w};
    const float ds[8] = {dsa.x, dsa.y, dsa.z, dsa.w, dsb.x, dsb.y, dsb.z, dsb.w};
    const int4* aq = act.q8 + b;
    float acc = 0.f, accm = 0.f;
#pragma unroll
    for (int t = 0; t < 4; t++) {
        const int4 a0 = aq[(4 * t) * nb], a1 = aq[(4 * t + 1) * nb], a2 = aq[(4 * t + 2) * nb], a3 = aq[(4 * t + 3) * nb];
        const int4 qa = tile_piece<SMEM>(tile, lane, 1 + 2 * t), qb = tile_piece<SMEM>(tile, lane, 2 + 2 * t);
        int I0 = dot16_us(qa, 0x0f0f0f0fu, a0, 0);
        I0 = dot16_us(qb, 0x0f0f0f0fu, a1, I0);
        int I1 = dot16_us(qa, 0xf0f0f0f0u, a2, 0);
        I1 = dot16_us(qb, 0xf0f0f0f0u, a3, I1);
        I1 >>= 4;
        if (ints) {
            ints[2 * t] = I0;
            ints[2 * t + 1] = I1;
        }
        const int j0 = 2 * t, j1 = 2 * t + 1;
        const int sc0 = ((j0 < 4 ? sc_lo : sc_hi) >> (8 * (j0 & 3))) & 0xff, sc1 = ((j1 < 4 ? sc_lo : sc_hi) >> (8 * (j1 & 3))) & 0xff;
        const int m0 = ((j0 < 4 ? m_lo : m_hi) >> (8 * (j0 & 3))) & 0xff, m1 = ((j1 < 4 ? m_lo : m_hi) >> (8 * (j1 & 3))) & 0xff;
        acc += d8[j0] * i2f_small(I0 * sc0) + d8[j1] * i2f_small(I1 * sc1);
        accm += ds[j0] * i2f_small(m0) + ds[j1] * i2f_small(m1);
    }
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&wh.x));  // (d, dmin)
    return dd.x * acc - dd.y * accm;
}

// One Q6_K block (kernels/gemv.cu:302-337 over all sixteen scale groups).  Group c of the
// block (elements 16c..16c+15, c = 8n + 2j + is) takes its low nibbles from ql piece
// 4n + 2(j&1) + is (low half for j < 2, high half otherwise), its two high bits from bits
// 2j..2j+1 of qh piece 2n + is, and scale byte 8n + is + 2j.  ints (optional): J[c] =
// sum (q6 - 32) * q8; the accumulators start at -32 * sum(q8) so the integer is exact.
template <bool SMEM>
__device__ __forceinline__ float block_dot(BlockQ6, const uint8_t* tile, int lane, const Act& act, int b, int nb, int* ints) {
    const int4 wsc = tile_piece<SMEM>(tile, lane, 12);  // 16 int8 scales
    const unsigned int dbits = reinterpret_cast<const unsigned short*>(tile + Q6_PIECES * 512)[lane];
    const float4 d8a = reinterpret_cast<const float4*>(act.d8)[2 * b], d8b = reinterpret_cast<const float4*>(act.d8)[2 * b + 1];
    const float d8[8] = {d8a.x, d8a.y, d8a.z, d8a.w, d8b.x, d8b.y, d8b.z, d8b.w};
    const int4* aq = act.q8 + b;
    const int4* sn = reinterpret_cast<const int4*>(act.s16n) + 4 * b;
    const int scw[4] = {wsc.x, wsc.y, wsc.z, wsc.w};
    float acc = 0.f;
#pragma unroll
    for (int n = 0; n < 2; n++) {
        const int4 sA = sn[2 * n], sB = sn[2 * n + 1];  // -32*S16 of chunks 8n..8n+7
        const int s16[8] = {sA.x, sA.y, sA.z, sA.w, sB.x, sB.y, sB.z, sB.w};
#pragma unroll
        for (int is = 0; is < 2; is++) {
            const int4 la = tile_piece<SMEM>(tile, lane, 4 * n + is), lb = tile_piece<SMEM>(tile, lane, 4 * n + 2 + is),
                       h = tile_piece<SMEM>(tile, lane, 8 + 2 * n + is);
            const int4 a0 = aq[(8 * n + is) * nb], a1 = aq[(8 * n + 2 + is) * nb], a2 = aq[(8 * n + 4 + is) * nb],
                       a3 = aq[(8 * n + 6 + is) * nb];
            int J0 = s16[is], J1 = s16[2 + is], J2 = s16[4 + is], J3 = s16[6 + is];
#define TFR_Q6W(c)                                                                                         \
    J0 = __dp4a((int)((la.c & 0x0f0f0f0f) | ((h.c << 4) & 0x30303030)), a0.c, J0);                        \
    J1 = __dp4a((int)((lb.c & 0x0f0f0f0f) | ((h.c << 2) & 0x30303030)), a1.c, J1);                        \
    J2 = __dp4a((int)((((unsigned)la.c >> 4) & 0x0f0f0f0f) | (h.c & 0x30303030)), a2.c, J2);              \
    J3 = __dp4a((int)((((unsigned)lb.c >> 4) & 0x0f0f0f0f) | (((unsigned)h.c >> 2) & 0x30303030)), a3.c, J3);
            TFR_Q6W(x) TFR_Q6W(y) TFR_Q6W(z) TFR_Q6W(w)
#undef TFR_Q6W
            if (ints) {
                ints[8 * n + is] = J0;
                ints[8 * n + 2 + is] = J1;
                ints[8 * n + 4 + is] = J2;
                ints[8 * n + 6 + is] = J3;
            }
            // scale byte k = 8n + is + 2j sits in word k >> 2 at byte k & 3
            const int k0 = 8 * n + is;
            const float c0 = i2f_small((int)(signed char)((scw[k0 >> 2] >> (8 * (k0 & 3))) & 0xff));
            const float c1 = i2f_small((int)(signed char)((scw[(k0 + 2) >> 2] >> (8 * ((k0 + 2) & 3))) & 0xff));
            const float c2 = i2f_small((int)(signed char)((scw[(k0 + 4) >> 2] >> (8 * ((k0 + 4) & 3))) & 0xff));
            const float c3 = i2f_small((int)(signed char)((scw[(k0 + 6) >> 2] >> (8 * ((k0 + 6) & 3))) & 0xff));
            acc += c0 * d8[4 * n] * i2f_small(J0) + c1 * d8[4 * n + 1] * i2f_small(J1) + c2 * d8[4 * n + 2] * i2f_small(J2) +
                   c3 * d8[4 * n + 3] * i2f_small(J3);
        }
    }
    return f16_to_f32((unsigned short)dbits) * acc;
}

// Eight Q8_0 blocks (kernels/gemv.cu:1558-1582 over a 256-weight stretch): per 32-block
// sum = dot(int8 weights, int8 activation), acc += d_w * d_x * sum.  The 272 bytes are [d0 q0[32] d1 q1[32] ...]:
// the quants of even blocks start 2 bytes into a word and are realigned with a funnel shift, those of
// odd blocks are word-aligned.  ints (optional): the eight integer sums.
template <bool SMEM>
__device__ __forceinline__ float block_dot(BlockQ8, const uint8_t* tile, int lane, const Act& act, int b, int nb, int* ints) {
    const float4 d8a = reinterpret_cast<const float4*>(act.d8)[2 * b], d8b = reinterpret_cast<const float4*>(act.d8)[2 * b + 1];
    const float d8[8] = {d8a.x, d8a.y, d8a.z, d8a.w, d8b.x, d8b.y, d8b.z, d8b.w};
    const int4* aq = act.q8 + b;
    float acc = 0.f;
    // words 17m .. 17m+16 hold blocks 2m (d in the low half of word 0) and 2m+1 (d in the high half of word 8)
    auto word = [&](int w) -> unsigned int {
        const uint8_t* p = tile + (w >> 2) * 512 + lane * 16 + (w & 3) * 4;
        if (SMEM) {
            unsigned int v;
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)));
            return v;
        }
        return *reinterpret_cast<const unsigned int*>(p);
    };
#pragma unroll
    for (int m = 0; m < 4; m++) {
        unsigned int w[17];
#pragma unroll
        for (int i = 0; i < 17; i++) w[i] = word(17 * m + i);
        const int4 a0 = aq[(4 * m) * nb], a1 = aq[(4 * m + 1) * nb], a2 = aq[(4 * m + 2) * nb], a3 = aq[(4 * m + 3) * nb];
        const int ae[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const int ao[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
        int se = 0, so = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            se = __dp4a((int)__funnelshift_r(w[i], w[i + 1], 16), ae[i], se);
            so = __dp4a((int)w[9 + i], ao[i], so);
        }
        if (ints) {
            ints[2 * m] = se;
            ints[2 * m + 1] = so;
        }
        const float de = f16_to_f32((unsigned short)(w[0] & 0xffff)), dq = f16_to_f32((unsigned short)(w[8] >> 16));
        acc += de * d8[2 * m] * (float)se;
        acc += dq * d8[2 * m + 1] * (float)so;
    }
    return acc;
}

// One run of 16 elements (scale group c = 8n + 2j + is) of Q6_K block f against the fp32
// activation staged in shared memory — the reference's route for a Q6_K attn_v,
// kernels/gemv.cu:233-264: acc += d * scale * q * x with x unquantised.  b = block index in the row.
__device__ __forceinline__ float q6k_run_dot_f32(const Mat& m, long long f, int b, int c, const float* xf) {
    const int n = c >> 3, j = (c >> 1) & 3, is = c & 1;
    const int4 ql = __ldg(reinterpret_cast<const int4*>(block_byte(m, f, 64 * n + 32 * (j & 1) + 16 * is)));
    const int4 qh = __ldg(reinterpret_cast<const int4*>(block_byte(m, f, 128 + 32 * n + 16 * is)));
    const float sc = (float)(int)*reinterpret_cast<const signed char*>(block_byte(m, f, 192 + 8 * n + is + 2 * j));
    const float d = f16_to_f32(__ldg(reinterpret_cast<const unsigned short*>(block_byte(m, f, 208))));
    const float dsc = d * sc;
    const float4* x4 = reinterpret_cast<const float4*>(xf + xs_idx(256 * b + 16 * c));
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

// The same run against a plain fp32 vector in global memory (x = the row's start): the chunk kernels keep no staged
// copy per token.  Same operations in the same order as q6k_run_dot_f32.
__device__ __forceinline__ float q6k_run_dot_f32_g(const Mat& m, long long f, int b, int c, const float* x) {
    const int n = c >> 3, j = (c >> 1) & 3, is = c & 1;
    const int4 ql = __ldg(reinterpret_cast<const int4*>(block_byte(m, f, 64 * n + 32 * (j & 1) + 16 * is)));
    const int4 qh = __ldg(reinterpret_cast<const int4*>(block_byte(m, f, 128 + 32 * n + 16 * is)));
    const float sc = (float)(int)*reinterpret_cast<const signed char*>(block_byte(m, f, 192 + 8 * n + is + 2 * j));
    const float d = f16_to_f32(__ldg(reinterpret_cast<const unsigned short*>(block_byte(m, f, 208))));
    const float dsc = d * sc;
    const float4* x4 = reinterpret_cast<const float4*>(x + 256 * b + 16 * c);
    const int qlw[4] = {ql.x, ql.y, ql.z, ql.w};
    const int qhw[4] = {qh.x, qh.y, qh.z, qh.w};
    const int nsh = 4 * (j >> 1), hsh = 2 * j;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float4 xq = x4[k];
        const float xv[4] = {xq.x, xq.y, xq.z, xq.w};
#pragma unroll
        for (int by = 0; by < 4; by++) {
            const int nib = (qlw[k] >> (8 * by + nsh)) & 0xF;
            const int hb = (qhw[k] >> (8 * by + hsh)) & 3;
            acc += dsc * (float)((nib | (hb << 4)) - 32) * xv[by];
        }
    }
    return acc;
}

// The sixteen weights of that run as the factors q6k_run_dot_f32_g multiplies x by, d * scale * (q - 32) in its order of
// operations, and the dot with a vector piece in its order of additions: weights kept in registers serve many tokens.
__device__ __forceinline__ void q6k_run_weights_f32(const Mat& m, long long f, int c, float (&w)[16]) {
    const int n = c >> 3, j = (c >> 1) & 3, is = c & 1;
    const int4 ql = __ldg(reinterpret_cast<const int4*>(block_byte(m, f, 64 * n + 32 * (j & 1) + 16 * is)));
    const int4 qh = __ldg(reinterpret_cast<const int4*>(block_byte(m, f, 128 + 32 * n + 16 * is)));
    const float sc = (float)(int)*reinterpret_cast<const signed char*>(block_byte(m, f, 192 + 8 * n + is + 2 * j));
    const float d = f16_to_f32(__ldg(reinterpret_cast<const unsigned short*>(block_byte(m, f, 208))));
    const float dsc = d * sc;
    const int qlw[4] = {ql.x, ql.y, ql.z, ql.w};
    const int qhw[4] = {qh.x, qh.y, qh.z, qh.w};
    const int nsh = 4 * (j >> 1), hsh = 2 * j;
#pragma unroll
    for (int k = 0; k < 4; k++)
#pragma unroll
        for (int by = 0; by < 4; by++) {
            const int nib = (qlw[k] >> (8 * by + nsh)) & 0xF;
            const int hb = (qhw[k] >> (8 * by + hsh)) & 3;
            w[4 * k + by] = dsc * (float)((nib | (hb << 4)) - 32);
        }
}
__device__ __forceinline__ float q6k_run_dot_weights(const float (&w)[16], const float* x16) {
    const float4* x4 = reinterpret_cast<const float4*>(x16);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float4 xq = x4[k];
        acc += w[4 * k] * xq.x;
        acc += w[4 * k + 1] * xq.y;
        acc += w[4 * k + 2] * xq.z;
        acc += w[4 * k + 3] * xq.w;
    }
    return acc;
}

// ------------------------------------------------------------------ shares

// Contiguous share of n items for CTA c of C, with n = C*quot + rem split on the host so that
// the kernel needs no division: the first `rem` CTAs take quot+1 items.
struct Share {
    int quot, rem;
    __host__ __device__ __forceinline__ int begin(int c) const { return c * quot + (c < rem ? c : rem); }
    __host__ __device__ __forceinline__ int count(int c) const { return quot + (c < rem ? 1 : 0); }
};
inline Share make_share(int n, int C) {
    Share s;
    s.quot = n / C;
    s.rem = n % C;
    return s;
}

// An epilogue receives two finished dot products from exactly one thread: rows (2p, 2p+1) of a
// matrix (EPI_PAIRS) or row p of two matrices walked together (EPI_ZIP).
enum { EPI_PAIRS = 0, EPI_ZIP = 1 };

}  // namespace tfr
