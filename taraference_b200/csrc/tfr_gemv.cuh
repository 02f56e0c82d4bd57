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
#include "tfr_common.cuh"

namespace tfr {

constexpr int GEMV_THREADS = 256;  // also the reduction shape of the reference RMSNorm
constexpr int GEMV_UNROLL = 2;     // units in flight per thread per pass
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
    float* xf;   // K fp32 values (normalised input) when a fp32-activation row type needs them
};

__host__ __device__ inline size_t act_smem_bytes(int K, bool want_xf) {
    return (size_t)K + (size_t)(K / 32) * 8 + (want_xf ? (size_t)K * 4 : 0);
}

__device__ __forceinline__ Act act_carve(unsigned char* smem, int K, bool want_xf) {
    Act a;
    a.q8 = reinterpret_cast<int4*>(smem);
    a.d8 = reinterpret_cast<float*>(smem + K);
    a.ss = reinterpret_cast<int*>(smem + K + (K / 32) * 4);
    a.xf = want_xf ? reinterpret_cast<float*>(smem + K + (K / 32) * 8) : nullptr;
    return a;
}

// Position of 16-byte chunk c (elements 16c..16c+15) inside Act::q8.  G = K/64.
__device__ __forceinline__ int swz_pos(int c, int G, int mode) {
    if (mode == SWZ_Q4) return (c & 3) * G + (c >> 2);
    return ((c & 7) >> 1) * G + ((c >> 3) << 1) + (c & 1);
}

// ------------------------------------------------------------------ activation sources

struct SrcVec {
    const float* v;
    __device__ __forceinline__ float get(int i) const { return v[i]; }
};

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

// RMSNorm scale with the reduction shape of kernels/ops.cu:4-34 (256 strided partial sums,
// then a binary tree), so that the normalised vector — and with it the int8 activation —
// is bit-identical to the reference's for the same input.  Must be called by all 256 threads.
template <class Src>
__device__ float rms_scale_256(const Src& src, int n, float eps, float* red /* 256 floats */) {
    const int tid = threadIdx.x;
    float local = 0.f;
    for (int i = tid; i < n; i += GEMV_THREADS) {
        float v = src.get(i);
        local += v * v;
    }
    red[tid] = local;
    __syncthreads();
    for (int s = GEMV_THREADS / 2; s > 0; s >>= 1) {
        if (tid < s) red[tid] += red[tid + s];
        __syncthreads();
    }
    float scale = rsqrtf(red[0] / (float)n + eps);
    __syncthreads();
    return scale;
}

// Q8 activation quantiser, kernels/gemv.cu:16-65: per 32 values d = amax * (1/127),
// q = rn(x / d) with the build's approximate division, zero group -> zeros.  Additionally
// records per-half-group sums of q (pure integer, derived from q).
template <class Src>
__device__ void act_prepare(Act& act, const Src& src, const float* __restrict__ normw, float eps, int K, int swz,
                            float* __restrict__ raw_out, float* red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = K >> 6;
    float scale = 1.f;
    if (normw) scale = rms_scale_256(src, K, eps, red);
    signed char* q8b = reinterpret_cast<signed char*>(act.q8);
    for (int g = warp; g < (K >> 5); g += GEMV_THREADS / 32) {
        const int i = (g << 5) + lane;
        float raw = src.get(i);
        if (raw_out) raw_out[i] = raw;
        float xi = normw ? raw * scale * normw[i] : raw;
        if (act.xf) act.xf[i] = xi;
        float amax = warp_max(fabsf(xi));
        const float d = amax * (1.0f / 127.0f);
        int q = amax == 0.f ? 0 : (int)(signed char)__float2int_rn(xi / d);
        const int c = i >> 4;
        q8b[swz_pos(c, G, swz) * 16 + (i & 15)] = (signed char)q;
        int s = q;
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 8);
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 4);
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 2);
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 1);
        int hi = __shfl_sync(TFR_FULL_MASK, s, 16);
        if (lane == 0) {
            act.d8[g] = d;
            act.ss[g] = (s & 0xffff) | (hi << 16);
        }
    }
    __syncthreads();
}

// ------------------------------------------------------------------ unit loads / dots

struct UnitW {
    int4 a, b, c;
    int2 s;
    unsigned int dbits;
};

__device__ __forceinline__ void load_unit(UnitW& w, int wt, const uint8_t* row, int nb, int u) {
    if (wt == WT_Q4K) {
        const uint8_t* blk = row + (u >> 2) * 144;
        w.c = ldg_stream(blk);
        w.a = ldg_stream(blk + 16 + 32 * (u & 3));
        w.b = ldg_stream(blk + 32 + 32 * (u & 3));
    } else {
        const int b = u >> 2, n = (u >> 1) & 1, is = u & 1;
        const uint8_t* ql = row + b * 128 + 64 * n + 16 * is;
        w.a = ldg_stream(ql);
        w.b = ldg_stream(ql + 32);
        w.c = ldg_stream(row + nb * 128 + b * 64 + 32 * n + 16 * is);
        w.s = ldg_stream8(row + nb * 192 + b * 16 + 8 * n);
        w.dbits = __ldg(reinterpret_cast<const unsigned short*>(row + nb * 208 + 2 * b));
    }
}

__device__ __forceinline__ int dot16(const int4& w, const int4& a, int acc) {
    acc = __dp4a(w.x, a.x, acc);
    acc = __dp4a(w.y, a.y, acc);
    acc = __dp4a(w.z, a.z, acc);
    acc = __dp4a(w.w, a.w, acc);
    return acc;
}
__device__ __forceinline__ int4 and4(const int4& v, int m) { return make_int4(v.x & m, v.y & m, v.z & m, v.w & m); }
__device__ __forceinline__ int4 shr4(const int4& v, int s) {
    return make_int4((int)((unsigned)v.x >> s), (int)((unsigned)v.y >> s), (int)((unsigned)v.z >> s),
                     (int)((unsigned)v.w >> s));
}

// Integer sub-block results of one Q4_K unit (sub-blocks 2t and 2t+1 of its super-block).
struct Q4Ints {
    int I0, I1, S0, S1, sc0, sc1, m0, m1;
};

__device__ __forceinline__ Q4Ints q4k_unit_ints(const UnitW& w, const Act& act, int u, int G) {
    Q4Ints r;
    const int4 a0 = act.q8[u], a1 = act.q8[G + u], a2 = act.q8[2 * G + u], a3 = act.q8[3 * G + u];
    r.I0 = dot16(and4(w.a, 0x0f0f0f0f), a0, 0);
    r.I0 = dot16(and4(w.b, 0x0f0f0f0f), a1, r.I0);
    r.I1 = dot16(and4(shr4(w.a, 4), 0x0f0f0f0f), a2, 0);
    r.I1 = dot16(and4(shr4(w.b, 4), 0x0f0f0f0f), a3, r.I1);
    const int2 ss = reinterpret_cast<const int2*>(act.ss)[u];
    r.S0 = (int)(short)(ss.x & 0xffff) + (ss.x >> 16);
    r.S1 = (int)(short)(ss.y & 0xffff) + (ss.y >> 16);
    // 6-bit scales / mins, kernels/common.cu:40-50 in the 16-bit form of gemv.cu:94-106.
    const int t = u & 3, sh = 16 * (t & 1);
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
    r.sc0 = aux_sc & 0xff;
    r.sc1 = aux_sc >> 8;
    r.m0 = aux_m & 0xff;
    r.m1 = aux_m >> 8;
    return r;
}

__device__ __forceinline__ float q4k_unit_dot(const UnitW& w, const Act& act, int u, int G) {
    const Q4Ints r = q4k_unit_ints(w, act, u, G);
    const float d = f16_to_f32((unsigned short)(w.c.x & 0xffff));
    const float dmin = f16_to_f32((unsigned short)((unsigned)w.c.x >> 16));
    const float2 d8 = reinterpret_cast<const float2*>(act.d8)[u];
    return d * (d8.x * (float)(r.I0 * r.sc0) + d8.y * (float)(r.I1 * r.sc1)) -
           dmin * (d8.x * (float)(r.S0 * r.m0) + d8.y * (float)(r.S1 * r.m1));
}

// The four 16-element scale-group dots sum (q6-32)*q8 of one Q6_K unit: runs j = 0..3 are
// elements 128n + 32j + 16is + [0,16) of block b, where u = 4b + 2n + is.
__device__ __forceinline__ void q6k_unit_ints(const UnitW& w, const Act& act, int u, int G, int J[4]) {
    const int4 a0 = act.q8[u], a1 = act.q8[G + u], a2 = act.q8[2 * G + u], a3 = act.q8[3 * G + u];
    const int4 h = w.c;
    int4 r0, r1, r2, r3;
#define TFR_Q6W(f)                                                          \
    r0.f = (w.a.f & 0x0f0f0f0f) | ((h.f << 4) & 0x30303030);                \
    r1.f = (w.b.f & 0x0f0f0f0f) | ((h.f << 2) & 0x30303030);                \
    r2.f = (((unsigned)w.a.f >> 4) & 0x0f0f0f0f) | (h.f & 0x30303030);      \
    r3.f = (((unsigned)w.b.f >> 4) & 0x0f0f0f0f) | (((unsigned)h.f >> 2) & 0x30303030);
    TFR_Q6W(x) TFR_Q6W(y) TFR_Q6W(z) TFR_Q6W(w)
#undef TFR_Q6W
    const int4 ss = reinterpret_cast<const int4*>(act.ss)[u >> 1];
    const int is = u & 1;
#define TFR_S16(v) (is ? ((v) >> 16) : (int)(short)((v) & 0xffff))
    J[0] = dot16(r0, a0, 0) - 32 * TFR_S16(ss.x);
    J[1] = dot16(r1, a1, 0) - 32 * TFR_S16(ss.y);
    J[2] = dot16(r2, a2, 0) - 32 * TFR_S16(ss.z);
    J[3] = dot16(r3, a3, 0) - 32 * TFR_S16(ss.w);
#undef TFR_S16
}

__device__ __forceinline__ void q6k_unit_scales(const UnitW& w, int u, float sc[4]) {
    const int is = u & 1;
    const unsigned lo = (unsigned)w.s.x >> (8 * is), hi = (unsigned)w.s.y >> (8 * is);
    sc[0] = (float)(int)(signed char)(lo & 0xff);
    sc[1] = (float)(int)(signed char)((lo >> 16) & 0xff);
    sc[2] = (float)(int)(signed char)(hi & 0xff);
    sc[3] = (float)(int)(signed char)((hi >> 16) & 0xff);
}

__device__ __forceinline__ float q6k_unit_dot(const UnitW& w, const Act& act, int u, int G) {
    int J[4];
    float sc[4];
    q6k_unit_ints(w, act, u, G, J);
    q6k_unit_scales(w, u, sc);
    const float d = f16_to_f32((unsigned short)w.dbits);
    const float4 d8 = reinterpret_cast<const float4*>(act.d8)[u >> 1];
    return d * (sc[0] * d8.x * (float)J[0] + sc[1] * d8.y * (float)J[1] + sc[2] * d8.z * (float)J[2] +
                sc[3] * d8.w * (float)J[3]);
}

// Q6_K unit against the fp32 activation (the reference's route for a Q6_K attn_v,
// kernels/gemv.cu:233-264: acc += d * scale * q * x with x unquantised).
__device__ __forceinline__ float q6k_unit_dot_f32(const UnitW& w, const Act& act, int u) {
    const int b = u >> 2, n = (u >> 1) & 1, is = u & 1;
    const float* x = act.xf + 256 * b + 128 * n + 16 * is;
    float sc[4];
    q6k_unit_scales(w, u, sc);
    const float d = f16_to_f32((unsigned short)w.dbits);
    float acc = 0.f;
    const int qa[4] = {w.a.x, w.a.y, w.a.z, w.a.w};
    const int qb[4] = {w.b.x, w.b.y, w.b.z, w.b.w};
    const int qh[4] = {w.c.x, w.c.y, w.c.z, w.c.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
#pragma unroll
        for (int by = 0; by < 4; by++) {
            const int a = (qa[k] >> (8 * by)) & 0xff, bb = (qb[k] >> (8 * by)) & 0xff, hh = (qh[k] >> (8 * by)) & 0xff;
            const int e = 4 * k + by;
            const int q0 = ((a & 0xF) | ((hh & 3) << 4)) - 32;
            const int q1 = ((bb & 0xF) | (((hh >> 2) & 3) << 4)) - 32;
            const int q2 = ((a >> 4) | (((hh >> 4) & 3) << 4)) - 32;
            const int q3 = ((bb >> 4) | (((hh >> 6) & 3) << 4)) - 32;
            acc += d * sc[0] * (float)q0 * x[e];
            acc += d * sc[1] * (float)q1 * x[32 + e];
            acc += d * sc[2] * (float)q2 * x[64 + e];
            acc += d * sc[3] * (float)q3 * x[96 + e];
        }
    }
    return acc;
}

__device__ __forceinline__ float unit_dot(const UnitW& w, int wt, const Act& act, int u, int G) {
    if (wt == WT_Q4K) return q4k_unit_dot(w, act, u, G);
    if (wt == WT_Q6K) return q6k_unit_dot(w, act, u, G);
    return q6k_unit_dot_f32(w, act, u);
}

// ------------------------------------------------------------------ row maps

// vrow -> (row pointer, weight type).  "Virtual rows" let one kernel walk several matrices.
struct MapSingle {
    Mat m;
    int wt;
    __device__ __forceinline__ const uint8_t* row(int v, int& t) const {
        t = wt;
        return m.data + (long long)v * m.row_stride;
    }
    __device__ __forceinline__ int nb() const { return m.nb; }
};
// Two matrices interleaved row by row: vrow 2j -> a[j], 2j+1 -> b[j] (gate / up).
struct MapPair {
    Mat a, b;
    __device__ __forceinline__ const uint8_t* row(int v, int& t) const {
        t = WT_Q4K;
        const Mat& m = (v & 1) ? b : a;
        return m.data + (long long)(v >> 1) * m.row_stride;
    }
    __device__ __forceinline__ int nb() const { return a.nb; }
};
// Up to four matrices stacked: vrows [0,n0) -> m[0], [n0, n0+n1) -> m[1], ...
struct MapStack {
    Mat m[4];
    int wt[4];
    int start[5];
    int count;
    __device__ __forceinline__ const uint8_t* row(int v, int& t) const {
        int s = 0;
#pragma unroll
        for (int i = 1; i < 4; i++)
            if (i < count && v >= start[i]) s = i;
        t = wt[s];
        return m[s].data + (long long)(v - start[s]) * m[s].row_stride;
    }
    __device__ __forceinline__ int nb() const { return m[0].nb; }
};

// ------------------------------------------------------------------ tile walker

__host__ __device__ inline int gemv_partial_floats(int K, int row_align) {
    int G = K / 64;
    int need = row_align * G;
    return need > GEMV_PT_MIN ? need : GEMV_PT_MIN;
}

// Walks row groups [grp0, grp1) (a group = Epi::ROW_ALIGN consecutive vrows reduced by one
// warp and handed to the epilogue together).  pbuf: 2 * PT floats of shared memory.
template <class Map, class Epi>
__device__ void gemv_tiles(const Map& map, Epi& epi, const Act& act, int K, int grp0, int grp1, float* pbuf, int PT) {
    constexpr int RA = Epi::ROW_ALIGN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = K >> 6, nb = map.nb();
    const unsigned magic = 0xffffffffu / (unsigned)G + 1u;  // exact f / G for f*G < 2^32
    int rows_per_tile = GEMV_PT_MIN / G;
    rows_per_tile -= rows_per_tile % RA;
    if (rows_per_tile < RA) rows_per_tile = RA;
    const int v0 = grp0 * RA, v1 = grp1 * RA;
    int buf = 0;
    for (int tv = v0; tv < v1; tv += rows_per_tile, buf ^= 1) {
        const int rows = min(rows_per_tile, v1 - tv);
        const int n = rows * G;
        float* part = pbuf + buf * PT;
        for (int base = 0; base < n; base += GEMV_THREADS * GEMV_UNROLL) {
            UnitW w[GEMV_UNROLL];
            int uu[GEMV_UNROLL], wt[GEMV_UNROLL];
#pragma unroll
            for (int k = 0; k < GEMV_UNROLL; k++) {
                const int f = base + tid + k * GEMV_THREADS;
                if (f < n) {
                    const int r = (int)__umulhi((unsigned)f, magic);
                    uu[k] = f - r * G;
                    const uint8_t* rp = map.row(tv + r, wt[k]);
                    load_unit(w[k], wt[k], rp, nb, uu[k]);
                }
            }
#pragma unroll
            for (int k = 0; k < GEMV_UNROLL; k++) {
                const int f = base + tid + k * GEMV_THREADS;
                if (f < n) part[f] = unit_dot(w[k], wt[k], act, uu[k], G);
            }
        }
        __syncthreads();
        for (int g = warp; g * RA < rows; g += GEMV_THREADS / 32) {
            float s[RA];
#pragma unroll
            for (int a = 0; a < RA; a++) {
                const float* pr = part + (g * RA + a) * G;
                float acc = 0.f;
                for (int i = lane; i < G; i += 32) acc += pr[i];
                s[a] = warp_sum(acc);
            }
            epi.apply(tv + g * RA, s, lane);
        }
    }
}

// Contiguous share of `groups` row groups for CTA c of C.
__device__ __forceinline__ void cta_share(int groups, int c, int C, int& g0, int& g1) {
    g0 = (int)(((long long)groups * c) / C);
    g1 = (int)(((long long)groups * (c + 1)) / C);
}

}  // namespace tfr
