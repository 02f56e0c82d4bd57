// Split-KV flash-decode over the f16 KV cache, one query token.
//
// Reference: kernels/attn/flash.cu:16-116 (partial) and :222-255 (merge).  The reference
// launches one CTA per (query head, split) with 8 fixed splits, so every query head
// re-reads the K/V rows of its KV head.  Here one CTA serves ALL query heads that share a
// KV head (GQA group), so each K/V row is read from HBM once per token; the number of
// splits is sized to the SM count and shrinks for short contexts.  The splits of a KV head are
// launched as thread-block clusters (eight CTAs, four in the staged instance): the splits of a cluster merge their
// (m, l, O) partials through distributed shared memory behind one cluster barrier, each CTA of the cluster
// finishing its share of the output dims (no global round trip, no second launch).  Longer
// contexts use several clusters per KV head; their merged partials meet in global memory, where for
// every share of the dims the CTA that arrives last merges the clusters' partials.
// Three routes through a split's keys: the register route (one 64-key tile in flight, fp32 on CUDA cores: head size
// 256 on short caches, and every head size when the environment asks for it), the staged route on the tensor cores
// (head sizes up to 128, every cache: f16 MMAs with fp32 operands as two f16 terms, fp32 sums) and the staged route
// on CUDA cores (head size 256, long caches).  All agree with a float64 evaluation to about 2e-7 of the largest
// output; exp is the build's ex2-based expf.
#pragma once
#include <type_traits>

#include "tfr_common.cuh"

namespace tfr {

constexpr int ATTN_THREADS = 256;         // the register-route instance
constexpr int ATTN_THREADS_STAGED = 512;  // the staged instance on CUDA cores (head size 256): sixteen warps hide the latencies of its tile loop
__host__ __device__ constexpr bool attn_staged_mma(int hd) { return hd <= 128; }  // staged route on the tensor cores
__host__ __device__ constexpr int attn_threads(bool staged, int hd) { return staged && !attn_staged_mma(hd) ? ATTN_THREADS_STAGED : ATTN_THREADS; }
constexpr int ATTN_TILE = 64;     // keys per tile
constexpr int ATTN_REP_MAX = 8;   // query heads per KV head handled by one CTA
constexpr int ATTN_CLUSTER = 8;   // CTAs per cluster (the portable maximum); AttnArgs::S is a multiple of it
// The staged instance (long caches) runs clusters of four: the device holds 14 clusters of eight of that footprint at
// once (112 of 148 SMs) but enough clusters of four to put a split on nearly every SM.
constexpr int ATTN_CLUSTER_STAGED = 4;
__host__ __device__ constexpr int attn_cluster(bool staged) { return staged ? ATTN_CLUSTER_STAGED : ATTN_CLUSTER; }
constexpr int ATTN_LONG_MIN = 128;  // a split with more keys than this walks them through shared-memory stages
// Dynamic shared memory of k_attn_decode: a few stages of one K tile and one V tile each (rows padded by 8 halfs: 16-byte
// reads of different rows hit different banks, for plain reads and for ldmatrix), then q of the group's heads in fp32.  One tile in
// flight per SM is far too little to cover the memory latency (measured: 4 us per 32 KB tile with two stages), so a
// split keeps as many tiles in flight as shared memory holds.
__host__ __device__ constexpr int attn_stages(int hd) { return hd == 256 ? 2 : 5; }
inline size_t attn_stage_bytes(int hd) { return 2 * (size_t)ATTN_TILE * (hd + 8) * 2; }
inline size_t attn_dyn_smem(int hd) { return attn_stages(hd) * attn_stage_bytes(hd) + (size_t)ATTN_REP_MAX * hd * 4; }
// With fewer stages (head sizes on the tensor-core route only): splits must not exceed 64 x stages keys, tiles past
// the end of a split are never copied, and the warps' final merge needs 33 KB of this memory.
inline size_t attn_dyn_smem(int hd, int stages) {
    if (stages <= 0 || stages >= attn_stages(hd) || !attn_staged_mma(hd)) return attn_dyn_smem(hd);
    return stages * attn_stage_bytes(hd) + (size_t)ATTN_REP_MAX * hd * 4;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Writes a float to the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ void st_dsmem_f32(float* local, unsigned rank, float v) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

struct AttnArgs {
    const float* q;             // [n_head * hd], RoPE applied
    const unsigned short* kc;   // layer base, [max_seq][n_kv * hd] f16 bits
    const unsigned short* vc;
    float* partial;             // [n_head][S][2 + hd]: per-cluster partials (contexts of more than 8 splits)
    unsigned int* counters;     // [n_kv][8] (KV head, output slice), zero between launches
    float* out;                 // [n_head * hd]
    const float* gate;          // optional [n_head * hd]: out *= sigmoid(gate) (deltanet.cu:176-186)
    int n_head, n_kv, S, min_keys;
    float scale;
    int pos;                    // used when st == nullptr
    int staged;                 // 1: the staged instance (the launch carries its dynamic shared memory, attn_dyn_smem)
    int stages;                 // host side: tile stages the launch provides (0 = all); n serve splits of up to 64 n keys
    int prof_id;                // timeline probe: which launch of the token this is (test aid)
};

// Warp-level matrix instructions of the staged route (f16 operands, fp32 accumulators).
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// Transposes an 8x8 matrix of 16-bit values held one row pair per lane (lane 4 r + c holds row r, columns 2 c, 2 c + 1).
__device__ __forceinline__ unsigned movm_trans(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// An fp32 value travels through the f16 tensor-core path as a sum of two f16 terms, x = h1 + h2 with h2 the f16 image of
// what the first rounding dropped: about 22 bits.  Measured against a float64 evaluation the route is as accurate as the
// fp32 CUDA-core routes (1.0e-7 ... 2.9e-7 of the largest output on seven shapes, against 1.3e-7 ... 2.2e-7).  Scaling
// the second term by 2^12 to keep it out of the f16 subnormals, or a third term, changed neither figure and cost 0.5 %
// and 3 % of a decode token.  x, y -> packed pairs, low half first.
__device__ __forceinline__ unsigned pack_f16x2(__half a, __half b) {
    const __half2 h = __halves2half2(a, b);
    return *reinterpret_cast<const unsigned*>(&h);
}
__device__ __forceinline__ void split2_f16x2(float x, float y, unsigned& t1, unsigned& t2) {
    const __half hx = __float2half_rn(x), hy = __float2half_rn(y);
    t1 = pack_f16x2(hx, hy);
    t2 = pack_f16x2(__float2half_rn(x - __half2float(hx)), __float2half_rn(y - __half2float(hy)));
}

// After the five butterfly steps lane L holds the sum over all lanes of v[L].
__device__ __forceinline__ float warp_transpose_reduce32(float (&v)[32], int lane) {
#pragma unroll
    for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; i++) {
            const float send = up ? v[i] : v[i + n / 2];
            const float keep = up ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(TFR_FULL_MASK, send, off);
        }
    }
    return v[0];
}

// STAGED = true compiles in the long-split route (and needs attn_dyn_smem(HD) of dynamic shared memory at launch);
// the STAGED = false instance is the register route alone, with the registers that route needs and no more.
template <int HD, bool STAGED = false>
__global__ void __launch_bounds__(attn_threads(STAGED, HD)) k_attn_decode(AttnArgs a, const TokenState* st) {
    constexpr int NT = attn_threads(STAGED, HD);
    prof_mark(0, a.prof_id);
    constexpr int DL = HD / 32;   // dims per lane in the score phase
    constexpr int DPT = HD / 64;  // dims per thread in the value phase
    constexpr int VK = ATTN_TILE / 4;  // keys per thread and tile in the value phase
    using KRaw = typename std::conditional<DL == 8, uint4, typename std::conditional<DL == 4, uint2, unsigned int>::type>::type;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int CL = attn_cluster(STAGED);
    const int g = blockIdx.y, s = blockIdx.x;  // grid (S, n_kv), clusters of CL along x
    const int rep = a.n_head / a.n_kv;
    const int kvdim = a.n_kv * HD;
    const int kg = tid >> 6, dp = tid & 63;
    // The decode state was last written by the previous token's final kernel, and every kernel of the chain
    // completes only after its predecessor: position and stop flag are final here, before the wait.
    const int done = st ? st->done : 0;
    const int T = (st ? st->pos : a.pos) + 1;
    int S_eff = (T + a.min_keys - 1) / a.min_keys;
    S_eff = S_eff < 1 ? 1 : (S_eff > a.S ? a.S : S_eff);
    // up to CL splits: the first cluster of the KV head merges on chip; its idle members
    // still attend the cluster barriers.  More splits: every CTA for itself, merge through memory.
    const int n_cl = (S_eff + CL - 1) / CL;  // clusters that have work
    const bool leave = done || (S_eff == 1 ? s >= 1 : s >= n_cl * CL);
    const bool active = s < S_eff;
    const int chunk = (T + S_eff - 1) / S_eff;
    const int t0 = min(T, s * chunk);
    const int t1 = (active && !leave) ? min(T, t0 + chunk) : t0;

    // K and V rows of one tile in registers: the value rows are used after the softmax, the key rows of both
    // score batches (batch bt of warp w covers keys 32*bt + 4*w ..) are requested before the first is used.
    // fresh = false: every row of the tile below `limit`; fresh = true: only row T-1, which the previous
    // kernel has just written (the others keep what an earlier call loaded).
    uint2 vraw[VK];
    KRaw kraw[2][4];
    auto load_v = [&](int tt, int limit, bool fresh) {
#pragma unroll
        for (int i = 0; i < VK; i++) {
            const int t = tt + kg + 4 * i;
            if (!fresh) vraw[i] = make_uint2(0u, 0u);
            if (fresh ? (t == T - 1 && t < t1) : t < limit) {
                const unsigned short* vr = a.vc + (size_t)t * kvdim + g * HD + dp * DPT;
                if constexpr (DPT == 4) vraw[i] = *reinterpret_cast<const uint2*>(vr);
                else if constexpr (DPT == 2) vraw[i].x = *reinterpret_cast<const unsigned int*>(vr);
                else vraw[i].x = *vr;
            }
        }
    };
    auto load_k = [&](int tt, int limit, bool fresh) {
#pragma unroll
        for (int bt = 0; bt < 2; bt++) {
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                const int t = tt + (bt * 8 + warp) * 4 + kk;
                if (!fresh) kraw[bt][kk] = KRaw{};
                if (fresh ? (t == T - 1 && t < t1) : t < limit) {
                    const unsigned short* kr = a.kc + (size_t)t * kvdim + g * HD + lane * DL;
                    if constexpr (DL == 1) kraw[bt][kk] = *kr;
                    else kraw[bt][kk] = *reinterpret_cast<const KRaw*>(kr);
                }
            }
        }
    };
    // Rows of earlier positions do not depend on the previous kernel: the first tile's are requested before
    // the grid-dependency wait, so their latency hides behind the kernel boundary.
    // A split with many keys stages its tiles in shared memory instead (below): no register preload then.
    const bool long_path = STAGED && t1 > t0;  // the staged instance walks every split through shared memory
    if constexpr (!STAGED) {
        load_k(t0, min(t1, T - 1), false);
        load_v(t0, min(t1, T - 1), false);
    }
    // The staged route does the same with its first NST - 1 tiles, as asynchronous copies; row T - 1 is left out of
    // them and fetched with plain loads after the wait.
    extern __shared__ __align__(16) unsigned char attn_dyn[];
    constexpr int KROW = HD + 8, CPR = HD / 8;  // halfs per staged K row; 16-byte chunks per cache row
    constexpr int NST = attn_stages(HD);
    constexpr size_t stage_b = 2 * (size_t)ATTN_TILE * KROW * 2;
    auto k_stage = [&](int st_) { return reinterpret_cast<unsigned short*>(attn_dyn + (size_t)st_ * stage_b); };
    auto v_stage = [&](int st_) { return reinterpret_cast<unsigned short*>(attn_dyn + (size_t)st_ * stage_b + (size_t)ATTN_TILE * KROW * 2); };
    auto issue_tile = [&](int tt, int st_, int skip_row) {
        unsigned short* ks = k_stage(st_);
        unsigned short* vs = v_stage(st_);
        if (tt < t1)
            for (int i = tid; i < ATTN_TILE * CPR; i += NT) {
                const int row = i / CPR, c8 = i - row * CPR;
                const bool in = tt + row < t1;
                if (tt + row == skip_row) continue;
                const size_t off = (size_t)(in ? tt + row : t1 - 1) * kvdim + (size_t)g * HD + c8 * 8;
                cp_async16(ks + row * KROW + c8 * 8, a.kc + off, in ? 16 : 0);
                cp_async16(vs + row * KROW + c8 * 8, a.vc + off, in ? 16 : 0);
            }
        cp_async_commit();  // a group per tile slot, empty past the end: the wait in the tile loop counts groups
    };
    if constexpr (STAGED) if (long_path) {
#pragma unroll
        for (int p = 0; p < NST - 1; p++) issue_tile(t0 + p * ATTN_TILE, p, T - 1);
    }
    griddep_wait();  // q and the new K/V row come from the previous kernel
    griddep_launch_dependents();
    prof_mark(1, a.prof_id);
    if (leave) return;
    if constexpr (!STAGED) {
        load_k(t0, 0, true);
        load_v(t0, 0, true);
    }

    __shared__ __align__(16) float sc[ATTN_TILE][ATTN_REP_MAX];  // [key][head]: the value phase reads a key's eight weights as two float4
    __shared__ __align__(16) float m_s[ATTN_REP_MAX];
    __shared__ __align__(16) float l_s[ATTN_REP_MAX];
    __shared__ __align__(16) float alpha_s[ATTN_REP_MAX];
    __shared__ float ored[4][ATTN_REP_MAX][HD];
    __shared__ int is_last_s;
    // on-chip merge: slice s of every member's O, and every member's (m, l), land here
    __shared__ float gath[ATTN_REP_MAX * HD];  // [member][per], per = rep * HD / CL
    __shared__ float gm[CL][ATTN_REP_MAX], gl[CL][ATTN_REP_MAX];

    // q fragment of every head of the group: dims lane*DL .. lane*DL+DL-1 (the register route's; the staged route
    // keeps q in shared memory)
    float qr[ATTN_REP_MAX][DL];
#pragma unroll
    for (int h = 0; h < ATTN_REP_MAX; h++)
#pragma unroll
        for (int d = 0; d < DL; d++) qr[h][d] = (h < rep && !STAGED) ? a.q[(g * rep + h) * HD + lane * DL + d] : 0.f;
    if (tid < ATTN_REP_MAX) {
        m_s[tid] = -1e30f;
        l_s[tid] = 0.f;
        alpha_s[tid] = 1.f;
    }
    float o[ATTN_REP_MAX][DPT];
#pragma unroll
    for (int h = 0; h < ATTN_REP_MAX; h++)
#pragma unroll
        for (int d = 0; d < DPT; d++) o[h][d] = 0.f;
    __syncthreads();
    prof_mark(4, a.prof_id);

    // The register route (short splits): one tile in flight, K and V rows in registers.  It leaves the sums of its four
    // key groups in `ored`, like the staged route.
    auto register_route = [&]() {
        for (int tt = t0; tt < t1; tt += ATTN_TILE) {
            const int tn = min(ATTN_TILE, t1 - tt);
            // ---- scores
#pragma unroll
            for (int bt = 0; bt < 2; bt++) {
                const int kbase = (bt * 8 + warp) * 4;
                if (kbase >= tn) {
                    if (kbase + (lane >> 3) < ATTN_TILE && (lane & 7) < ATTN_REP_MAX) sc[kbase + (lane >> 3)][lane & 7] = -1e30f;
                    continue;
                }
                float v[32];
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {
                    float kf[DL];
                    if constexpr (DL == 4) {
                        const uint2 raw = kraw[bt][kk];
                        kf[0] = f16_to_f32((unsigned short)(raw.x & 0xffff));
                        kf[1] = f16_to_f32((unsigned short)(raw.x >> 16));
                        kf[2] = f16_to_f32((unsigned short)(raw.y & 0xffff));
                        kf[3] = f16_to_f32((unsigned short)(raw.y >> 16));
                    } else if constexpr (DL == 8) {
                        const uint4 raw = kraw[bt][kk];
                        const unsigned int rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                        for (int d = 0; d < 4; d++) {
                            kf[2 * d] = f16_to_f32((unsigned short)(rw[d] & 0xffff));
                            kf[2 * d + 1] = f16_to_f32((unsigned short)(rw[d] >> 16));
                        }
                    } else if constexpr (DL == 2) {
                        kf[0] = f16_to_f32((unsigned short)(kraw[bt][kk] & 0xffff));
                        kf[1] = f16_to_f32((unsigned short)(kraw[bt][kk] >> 16));
                    } else {
                        kf[0] = f16_to_f32((unsigned short)kraw[bt][kk]);
                    }
#pragma unroll
                    for (int h = 0; h < ATTN_REP_MAX; h++) {
                        float acc = 0.f;
#pragma unroll
                        for (int d = 0; d < DL; d++) acc += qr[h][d] * kf[d];
                        v[kk * 8 + h] = acc;
                    }
                }
                const float tot = warp_transpose_reduce32(v, lane);
                const int kk = lane >> 3, h = lane & 7;
                const int t = tt + kbase + kk;
                sc[kbase + kk][h] = (t < t1 && h < rep) ? tot * a.scale : -1e30f;
            }
            // the key registers are free: the next tile's key rows travel during the softmax and the value phase
            if (tt + ATTN_TILE < t1) load_k(tt + ATTN_TILE, t1, false);
            __syncthreads();
            prof_mark(6, a.prof_id);
            // ---- online softmax bookkeeping: warp h owns head h
            if (warp < rep) {
                const float s0 = sc[lane][warp], s1 = sc[lane + 32][warp];
                const float tile_m = warp_max(fmaxf(s0, s1));
                const float m_old = m_s[warp];
                const float m_new = fmaxf(m_old, tile_m);
                const float p0 = (tt + lane < t1) ? expf(s0 - m_new) : 0.f;
                const float p1 = (tt + lane + 32 < t1) ? expf(s1 - m_new) : 0.f;
                const float tile_l = warp_sum(p0 + p1);
                sc[lane][warp] = p0;
                sc[lane + 32][warp] = p1;
                if (lane == 0) {
                    const float alpha = expf(m_old - m_new);
                    alpha_s[warp] = alpha;
                    l_s[warp] = l_s[warp] * alpha + tile_l;
                    m_s[warp] = m_new;
                }
            }
            __syncthreads();
            prof_mark(7, a.prof_id);
            // ---- values: thread (kg, dp) accumulates keys kg, kg+4, ... for dims dp*DPT..
#pragma unroll
            for (int h = 0; h < ATTN_REP_MAX; h++) {
                const float al = h < rep ? alpha_s[h] : 1.f;
#pragma unroll
                for (int d = 0; d < DPT; d++) o[h][d] *= al;
            }
            // Keys past the end of the tile carry weight 0 and value 0, so groups of four keys run without
            // per-key branches; a group that lies wholly past the end is skipped (uniform over the CTA).
#pragma unroll
            for (int i0 = 0; i0 < VK; i0 += 4) {
                if (4 * i0 >= tn) break;
                float4 pa[4], pb[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int k = kg + 4 * (i0 + j);
                    pa[j] = *reinterpret_cast<const float4*>(&sc[k][0]);
                    pb[j] = *reinterpret_cast<const float4*>(&sc[k][4]);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float vf[DPT];
                    vf[0] = f16_to_f32((unsigned short)(vraw[i0 + j].x & 0xffff));
                    if constexpr (DPT >= 2) vf[1] = f16_to_f32((unsigned short)(vraw[i0 + j].x >> 16));
                    if constexpr (DPT == 4) {
                        vf[2] = f16_to_f32((unsigned short)(vraw[i0 + j].y & 0xffff));
                        vf[3] = f16_to_f32((unsigned short)(vraw[i0 + j].y >> 16));
                    }
                    const float p[ATTN_REP_MAX] = {pa[j].x, pa[j].y, pa[j].z, pa[j].w, pb[j].x, pb[j].y, pb[j].z, pb[j].w};
#pragma unroll
                    for (int h = 0; h < ATTN_REP_MAX; h++) {
                        if (h < rep) {
#pragma unroll
                            for (int d = 0; d < DPT; d++) o[h][d] += p[h] * vf[d];
                        }
                    }
                }
            }
            // the next tile's value rows are requested now and used after the next tile's softmax
            if (tt + ATTN_TILE < t1) load_v(tt + ATTN_TILE, t1, false);
            __syncthreads();
        }

#pragma unroll
        for (int h = 0; h < ATTN_REP_MAX; h++)
#pragma unroll
            for (int d = 0; d < DPT; d++) ored[kg][h][dp * DPT + d] = o[h][d];
    };
    if constexpr (STAGED && attn_staged_mma(HD)) {
        // ---- the staged route on the tensor cores (head sizes up to 128).  K and V tiles travel global -> shared
        // memory as asynchronous 16-byte copies, five stages deep (the first four requested before the dependency
        // wait).  A warp owns 16 keys of a tile: scores S[16 keys x 8 heads] = K[16 x HD] Q^T as HD / 16 m16n8k16 MMAs,
        // online softmax on the accumulator fragment (a lane holds two keys x two heads; the maxima meet by three
        // shuffles), the weights transposed in registers (movmatrix) into the B operand of O^T[HD x 8 heads] +=
        // V^T[HD x 16 keys] P, whose A operand ldmatrix.trans reads straight from the V rows.  K and V are f16
        // already; q and the weights are fp32 and go through as sums of two f16 terms (split2_f16x2),
        // the products are exact and the sums fp32.  Every warp keeps its own running (m, l, O); the eight meet once, after the loop.
        // A step takes two tiles (warps 0-3 the first, 4-7 the second) and costs one barrier.
        static_assert(attn_stages(HD) == 5, "the issue schedule below is written for five stages");
        {
            // row T - 1, written by the previous kernel, if it lies in one of the tiles requested before the wait
            const int row = T - 1 - t0;
            if (T - 1 < t1 && row < (NST - 1) * ATTN_TILE && tid < 2 * CPR) {
                const int st_ = row / ATTN_TILE, r = row % ATTN_TILE, c8 = tid % CPR;
                const size_t off = (size_t)(T - 1) * kvdim + (size_t)g * HD + c8 * 8;
                if (tid < CPR) *reinterpret_cast<int4*>(k_stage(st_) + r * KROW + c8 * 8) = *reinterpret_cast<const int4*>(a.kc + off);
                else *reinterpret_cast<int4*>(v_stage(st_) + r * KROW + c8 * 8) = *reinterpret_cast<const int4*>(a.vc + off);
            }
        }
        constexpr int KS = HD / 16;  // 16-dim steps of the score product = 16-dim blocks of the value product
        const int gq = lane >> 2, tq = lane & 3;
        // B fragments of Q^T (k = dims, n = heads): lane (gq, tq) holds q[head gq][dims 16 ks + 2 tq, + 1] and [+ 8, + 9]
        unsigned q1[KS][2], q2[KS][2];
#pragma unroll
        for (int ks = 0; ks < KS; ks++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                float2 qv = make_float2(0.f, 0.f);
                if (gq < rep) qv = *reinterpret_cast<const float2*>(a.q + (size_t)(g * rep + gq) * HD + 16 * ks + 2 * tq + 8 * j);
                split2_f16x2(qv.x, qv.y, q1[ks][j], q2[ks][j]);
            }
        float oacc[KS][4];  // O^T fragments: [0], [1] = dim 16 mb + gq, heads 2 tq, 2 tq + 1; [2], [3] = dim 16 mb + gq + 8
#pragma unroll
        for (int mb = 0; mb < KS; mb++)
#pragma unroll
            for (int i = 0; i < 4; i++) oacc[mb][i] = 0.f;
        float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};  // heads 2 tq, 2 tq + 1 (l: this lane's keys only)
        const int n_tiles = (t1 - t0 + ATTN_TILE - 1) / ATTN_TILE, n_steps = (n_tiles + 1) >> 1;
        const int kb = warp & 3;
        // lane addresses of the ldmatrix reads inside a 16-key block (matrix mi = lane / 8, row lane % 8)
        const int mi = lane >> 3, mr = lane & 7;
        const int k_off = ((mi & 1) * 8 + mr) * KROW + (mi >> 1) * 8;  // K: keys 0-7 / 8-15 by mi & 1, dims + 0 / + 8 by mi >> 1
        const int v_off = ((mi >> 1) * 8 + mr) * KROW + (mi & 1) * 8;  // V: dims + 0 / + 8 by mi & 1, keys 0-7 / 8-15 by mi >> 1
        for (int j = 0; j < n_steps; j++) {
            // tiles 2 j and 2 j + 1 must have landed: four tiles were requested before the loop, one in step 0 and two
            // in every later step, one copy group per tile in order
            if (j == 0) cp_async_wait_group<2>();
            else cp_async_wait_group<1>();
            __syncthreads();  // everybody's pieces, and everybody is done with the tiles of step j - 1
            if (j == 0) {
                issue_tile(t0 + 4 * ATTN_TILE, 4, -1);
            } else {
                issue_tile(t0 + (2 * j + 3) * ATTN_TILE, (2 * j + 3) % NST, -1);
                issue_tile(t0 + (2 * j + 4) * ATTN_TILE, (2 * j + 4) % NST, -1);
            }
            if (j == 0) prof_mark(6, a.prof_id);
            const int ti = 2 * j + (warp >> 2), key0 = t0 + ti * ATTN_TILE + kb * 16;
            if (key0 < t1) {  // the same for the whole warp
                const int stg = ti % NST;
                float sacc[4] = {0.f, 0.f, 0.f, 0.f};  // S[key gq][heads 2 tq, 2 tq + 1], S[key gq + 8][the same heads]
                {
                    const unsigned kaddr = smem_u32(k_stage(stg) + kb * 16 * KROW + k_off);
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) {
                        unsigned af[4];
                        ldsm_x4(af, kaddr + ks * 32);
                        // The tensor core adds into its accumulator with truncation: every 16-term product sum starts
                        // from zero and joins the running sum by a round-to-nearest add, which keeps fp32-level accuracy.
                        float part[4] = {0.f, 0.f, 0.f, 0.f};
                        mma_16816(part, af, q2[ks][0], q2[ks][1]);
                        mma_16816(part, af, q1[ks][0], q1[ks][1]);
#pragma unroll
                        for (int i = 0; i < 4; i++) sacc[i] += part[i];
                    }
                }
                const bool on_a = key0 + gq < t1, on_b = key0 + gq + 8 < t1;
                float pw[4], al[2];
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const float sa = on_a ? sacc[c] * a.scale : -1e30f, sb = on_b ? sacc[2 + c] * a.scale : -1e30f;
                    float mx = fmaxf(sa, sb);
#pragma unroll
                    for (int off = 4; off <= 16; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(TFR_FULL_MASK, mx, off));
                    const float mn = fmaxf(m_run[c], mx);
                    al[c] = expf(m_run[c] - mn);
                    pw[c] = on_a ? expf(sa - mn) : 0.f;
                    pw[2 + c] = on_b ? expf(sb - mn) : 0.f;
                    l_run[c] = l_run[c] * al[c] + pw[c] + pw[2 + c];
                    m_run[c] = mn;
                }
                if (__any_sync(TFR_FULL_MASK, al[0] != 1.f || al[1] != 1.f)) {
#pragma unroll
                    for (int mb = 0; mb < KS; mb++) {
                        oacc[mb][0] *= al[0], oacc[mb][1] *= al[1];
                        oacc[mb][2] *= al[0], oacc[mb][3] *= al[1];
                    }
                }
                // weights as B operand (k = keys, n = heads): transpose the [key][head pair] fragments
                unsigned ph_a, pl_a, ph_b, pl_b;
                split2_f16x2(pw[0], pw[1], ph_a, pl_a);
                split2_f16x2(pw[2], pw[3], ph_b, pl_b);
                const unsigned b0h = movm_trans(ph_a), b1h = movm_trans(ph_b), b0l = movm_trans(pl_a), b1l = movm_trans(pl_b);
                const unsigned vaddr = smem_u32(v_stage(stg) + kb * 16 * KROW + v_off);
#pragma unroll
                for (int mb = 0; mb < KS; mb++) {
                    unsigned vf[4];
                    ldsm_x4_trans(vf, vaddr + mb * 32);
                    float part[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_16816(part, vf, b0l, b1l);
                    mma_16816(part, vf, b0h, b1h);
#pragma unroll
                    for (int i = 0; i < 4; i++) oacc[mb][i] += part[i];
                }
            }
            if (j == 0) prof_mark(7, a.prof_id);
        }
        // ---- the eight warps' (m, l, O) meet in shared memory (over the tile stages, which nobody reads any more).
        // A warp that had no keys leaves only its (m, l) = (-1e30, 0) and is skipped by the readers.
#pragma unroll
        for (int c = 0; c < 2; c++)
#pragma unroll
            for (int off = 4; off <= 16; off <<= 1) l_run[c] += __shfl_xor_sync(TFR_FULL_MASK, l_run[c], off);
        cp_async_wait_all();
        __syncthreads();
        constexpr int WOS = HD + 4;                                     // floats per head in wO: the four head pairs of a store hit different banks
        float* wO = reinterpret_cast<float*>(attn_dyn);                 // [warp][head][WOS]
        float* wm = wO + (NT / 32) * ATTN_REP_MAX * WOS;                // [warp][head]
        float* wl = wm + (NT / 32) * ATTN_REP_MAX;
        if (gq == 0) {
            wm[warp * ATTN_REP_MAX + 2 * tq] = m_run[0], wm[warp * ATTN_REP_MAX + 2 * tq + 1] = m_run[1];
            wl[warp * ATTN_REP_MAX + 2 * tq] = l_run[0], wl[warp * ATTN_REP_MAX + 2 * tq + 1] = l_run[1];
        }
        const bool had_keys = t0 + (warp >> 2) * ATTN_TILE + kb * 16 < t1;  // the warp's first block exists
        if (had_keys) {
#pragma unroll
            for (int mb = 0; mb < KS; mb++) {
                float* o0 = wO + ((size_t)warp * ATTN_REP_MAX + 2 * tq) * WOS + 16 * mb + gq;
                o0[0] = oacc[mb][0], o0[WOS] = oacc[mb][1], o0[8] = oacc[mb][2], o0[WOS + 8] = oacc[mb][3];
            }
        }
        __syncthreads();
        {
            // warp h folds head h: a lane takes HD / 32 adjacent dims, the weights exp(m_w - m) once per thread
            constexpr int DPL = HD / 32;
            const int h = warp;
            float mw[NT / 32], m = -1e30f;
#pragma unroll
            for (int w = 0; w < NT / 32; w++) {
                mw[w] = wm[w * ATTN_REP_MAX + h];
                m = fmaxf(m, mw[w]);
            }
            float acc[DPL], l = 0.f;
#pragma unroll
            for (int d = 0; d < DPL; d++) acc[d] = 0.f;
#pragma unroll
            for (int w = 0; w < NT / 32; w++) {
                if (mw[w] > -1e29f) {  // the same for the whole warp
                    const float wgt = expf(mw[w] - m);
                    l += wgt * wl[w * ATTN_REP_MAX + h];
                    const float* src = wO + ((size_t)w * ATTN_REP_MAX + h) * WOS + lane * DPL;
                    if constexpr (DPL == 4) {
                        const float4 v = *reinterpret_cast<const float4*>(src);
                        acc[0] += wgt * v.x, acc[1] += wgt * v.y, acc[2] += wgt * v.z, acc[3] += wgt * v.w;
                    } else {
                        const float2 v = *reinterpret_cast<const float2*>(src);
                        acc[0] += wgt * v.x, acc[1] += wgt * v.y;
                    }
                }
            }
            if (S_eff == 1) {
                // single split: the folded head is the output (the merge of one partial is the identity)
                if (h < rep) {
                    const int hg = g * rep + h;
#pragma unroll
                    for (int d = 0; d < DPL; d++) {
                        float r = acc[d] / fmaxf(l, 1e-20f);
                        if (a.gate) r *= 1.f / (1.f + expf(-a.gate[hg * HD + lane * DPL + d]));
                        a.out[hg * HD + lane * DPL + d] = r;
                    }
                }
                prof_mark(5, a.prof_id);
                return;
            }
#pragma unroll
            for (int d = 0; d < DPL; d++) {
                ored[0][h][lane * DPL + d] = acc[d];
                ored[1][h][lane * DPL + d] = 0.f, ored[2][h][lane * DPL + d] = 0.f, ored[3][h][lane * DPL + d] = 0.f;
            }
            if (lane == 0) {
                m_s[h] = m;
                l_s[h] = l;
            }
        }
    } else if constexpr (STAGED) {
        // ---- the staged route on CUDA cores (head size 256): K and V tiles travel global -> shared memory as asynchronous 16-byte copies, NST stages
        // deep (the first ones requested before the dependency wait), so the loads of the next tiles run under the
        // arithmetic of tile i and no register holds cache data.  Sixteen warps.
        float* q_s = reinterpret_cast<float*>(attn_dyn + NST * stage_b);
        {
            // row T - 1, written by the previous kernel, if it lies in one of the tiles requested before the wait
            const int row = T - 1 - t0;
            if (T - 1 < t1 && row < (NST - 1) * ATTN_TILE && tid < 2 * CPR) {
                const int st_ = row / ATTN_TILE, r = row % ATTN_TILE, c8 = tid % CPR;
                const size_t off = (size_t)(T - 1) * kvdim + (size_t)g * HD + c8 * 8;
                if (tid < CPR) *reinterpret_cast<int4*>(k_stage(st_) + r * KROW + c8 * 8) = *reinterpret_cast<const int4*>(a.kc + off);
                else *reinterpret_cast<int4*>(v_stage(st_) + r * KROW + c8 * 8) = *reinterpret_cast<const int4*>(a.vc + off);
            }
        }
        // Both phases are register-blocked so that shared-memory reads stay well below the FMA count (a 16-byte read
        // costs the load pipe four cycles per warp even when all lanes read the same address), and both split the
        // eight heads in two halves so that a thread's state fits the 128 registers of a 512-thread CTA.
        // Scores: a thread takes KPT keys x four heads x one slice of DSL dims; the DS slices of a (key group, head half)
        // are DS adjacent lanes, the two halves of a key group sit in the same warp (one shared-memory read serves
        // both); the partial sums meet in a halving butterfly that leaves every lane with ONE score.  With 8-dim
        // slices the thread's q values (four heads x eight dims) stay in registers for the whole split.  Group kgrp
        // takes keys kgrp, kgrp + NG, ...: a short last tile costs less.
        // Values: a warp takes KPI keys per round for one head half, HD / 8 lanes per key, a lane eight dims: per key
        // one read of the four weights and one 16-byte read of V for 32 FMAs.
        constexpr int HH = ATTN_REP_MAX / 2;            // heads per half
        constexpr int DS = HD >= 128 ? 16 : 8;          // dim slices (lanes) per group
        constexpr int DSL = HD / DS;                    // dims per slice: 8 or 16
        constexpr int NG = NT / DS / 2;                 // key groups
        constexpr int KPT = ATTN_TILE / NG;             // keys per thread
        constexpr int NV = KPT * HH;                    // partial sums per thread (= DS)
        static_assert(NV == DS, "the butterfly leaves one value per lane");
        constexpr int DV = 8;                           // value dims per lane: one 16-byte read of a V row
        constexpr int LPK = HD / DV, KPI = 32 / LPK;    // lanes per key and keys per warp and round in the value phase
        constexpr int KW = NT / 64;                     // warps per head half in the value phase
        constexpr bool QREG = DSL == 8;
        const int ds = lane & (DS - 1);
        const int grp = warp * (32 / DS) + lane / DS, kgrp = grp >> 1, hh = grp & 1;   // scores: key group and head half
        const int vkl = lane / LPK, vdl = lane % LPK, vkw = warp >> 1, vhh = warp & 1;  // values
        float qreg[QREG ? HH : 1][8];
        if constexpr (QREG) {
#pragma unroll
            for (int h = 0; h < HH; h++) {
                const bool on = hh * HH + h < rep;
                const float* qp = a.q + (size_t)(g * rep + (on ? hh * HH + h : 0)) * HD + ds * DSL;
                const float4 a0 = *reinterpret_cast<const float4*>(qp), a1 = *reinterpret_cast<const float4*>(qp + 4);
                qreg[h][0] = on ? a0.x : 0.f, qreg[h][1] = on ? a0.y : 0.f, qreg[h][2] = on ? a0.z : 0.f, qreg[h][3] = on ? a0.w : 0.f;
                qreg[h][4] = on ? a1.x : 0.f, qreg[h][5] = on ? a1.y : 0.f, qreg[h][6] = on ? a1.z : 0.f, qreg[h][7] = on ? a1.w : 0.f;
            }
        } else {
            for (int i = tid; i < ATTN_REP_MAX * HD; i += NT) q_s[i] = i < rep * HD ? a.q[g * rep * HD + i] : 0.f;
        }
        float o2[HH][DV];
#pragma unroll
        for (int h = 0; h < HH; h++)
#pragma unroll
            for (int d = 0; d < DV; d++) o2[h][d] = 0.f;
        // Softmax bookkeeping without a serial section.  The tile's row maxima are gathered by warp shuffles and one
        // shared-memory atomic max per warp and head (maxima do not depend on the order); after a barrier every thread
        // derives the new running maxima and its rescale factors for itself, the owning lane turns its score into a
        // weight, and the weight sums go through per-warp slots that eight threads add in a fixed order.
        __shared__ __align__(16) unsigned int tmax[2][ATTN_REP_MAX];  // ordered-integer image of the tile maxima (read as uint4)
        __shared__ __align__(16) float tl[NT / 32][ATTN_REP_MAX];     // per-warp sums of the tile's weights
        auto enc = [](float f) { const unsigned u = __float_as_uint(f); return (u & 0x80000000u) ? ~u : (u | 0x80000000u); };
        auto dec = [](unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); };
        if (tid < 2 * ATTN_REP_MAX) tmax[tid >> 3][tid & 7] = enc(-1e30f);
        int it = 0;
        for (int tt = t0; tt < t1; tt += ATTN_TILE, it++) {
            const int tn = min(ATTN_TILE, t1 - tt), cur = it % NST, par = it & 1;
            cp_async_wait_group<NST - 2>();  // this thread's pieces of tile `it`
            __syncthreads();                 // everybody's pieces, and everybody is done with tile it - 1
            issue_tile(tt + (NST - 1) * ATTN_TILE, (it + NST - 1) % NST, -1);  // into the stage tile it - 1 has just left
            if (it == 0) prof_mark(6, a.prof_id);
            float sv = 0.f;  // this lane's score of the tile
            auto scores = [&](auto kact_tag) {
                constexpr int KACT = decltype(kact_tag)::value;  // keys per thread that the tile reaches
                float v[NV];
#pragma unroll
                for (int i = 0; i < NV; i++) v[i] = 0.f;
                const unsigned short* kbase = k_stage(cur) + kgrp * KROW + ds * DSL;
#pragma unroll
                for (int c = 0; c < DSL; c += 8) {
#pragma unroll
                    for (int kk = 0; kk < KACT; kk++) {
                        const int4 kw = *reinterpret_cast<const int4*>(kbase + kk * NG * KROW + c);
                        const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kw.x)), k1 = __half22float2(*reinterpret_cast<const __half2*>(&kw.y));
                        const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kw.z)), k3 = __half22float2(*reinterpret_cast<const __half2*>(&kw.w));
#pragma unroll
                        for (int h = 0; h < HH; h++) {
                            float4 a0, a1;
                            if constexpr (QREG) {
                                a0 = make_float4(qreg[h][0], qreg[h][1], qreg[h][2], qreg[h][3]);
                                a1 = make_float4(qreg[h][4], qreg[h][5], qreg[h][6], qreg[h][7]);
                            } else {
                                const float* qp = q_s + (hh * HH + h) * HD + ds * DSL + c;
                                a0 = *reinterpret_cast<const float4*>(qp), a1 = *reinterpret_cast<const float4*>(qp + 4);
                            }
                            float t = v[kk * HH + h];
                            t = fmaf(a0.x, k0.x, t), t = fmaf(a0.y, k0.y, t), t = fmaf(a0.z, k1.x, t), t = fmaf(a0.w, k1.y, t);
                            t = fmaf(a1.x, k2.x, t), t = fmaf(a1.y, k2.y, t), t = fmaf(a1.z, k3.x, t), t = fmaf(a1.w, k3.y, t);
                            v[kk * HH + h] = t;
                        }
                    }
                }
                // halving butterfly over the DS lanes of the group
#pragma unroll
                for (int off = DS / 2, n = NV; off >= 1; off >>= 1, n >>= 1) {
                    const bool up = (lane & off) != 0;
#pragma unroll
                    for (int i = 0; i < n / 2; i++) {
                        const float send = up ? v[i] : v[i + n / 2];
                        const float keep = up ? v[i + n / 2] : v[i];
                        v[i] = keep + __shfl_xor_sync(TFR_FULL_MASK, send, off);
                    }
                }
                sv = v[0];
            };
            // rows past the end of the split arrive as zeros, so the full schedule is right for any tile; a tile that
            // reaches only the first key of every group (the short tail of a split) runs a quarter of it
            if (tn > NG) scores(std::integral_constant<int, KPT>{});
            else scores(std::integral_constant<int, 1>{});
            // the lane holds value ds of the group's KPT x 4: the group's key number ds / 4, head ds % 4 of its half
            const int sk = (ds >> 2) * NG + kgrp, sh = hh * HH + (ds & 3);
            const bool s_on = sk < tn && sh < rep;
            sv = s_on ? sv * a.scale : -1e30f;
            {
                float mx = sv;  // lanes that agree in lane & 3 and in the head-half bit hold the same head
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1)
                    if (off != DS) mx = fmaxf(mx, __shfl_xor_sync(TFR_FULL_MASK, mx, off));
                if ((lane & (28 & ~DS)) == 0) atomicMax(&tmax[par][sh], enc(mx));
            }
            __syncthreads();
            {
                const float4 mo0 = *reinterpret_cast<const float4*>(&m_s[0]), mo1 = *reinterpret_cast<const float4*>(&m_s[4]);
                const uint4 t0v = *reinterpret_cast<const uint4*>(&tmax[par][0]), t1v = *reinterpret_cast<const uint4*>(&tmax[par][4]);
                const float m_old[ATTN_REP_MAX] = {mo0.x, mo0.y, mo0.z, mo0.w, mo1.x, mo1.y, mo1.z, mo1.w};
                const unsigned tm[ATTN_REP_MAX] = {t0v.x, t0v.y, t0v.z, t0v.w, t1v.x, t1v.y, t1v.z, t1v.w};
                float m_new[ATTN_REP_MAX];
#pragma unroll
                for (int h = 0; h < ATTN_REP_MAX; h++) m_new[h] = fmaxf(m_old[h], dec(tm[h]));
                // the running maxima of a long split settle after its first tiles: rescale only when one has moved
                bool moved = false;
#pragma unroll
                for (int h = 0; h < HH; h++) moved |= (vhh ? m_new[HH + h] != m_old[HH + h] : m_new[h] != m_old[h]);
                if (moved) {
#pragma unroll
                    for (int h = 0; h < HH; h++) {
                        const float al = vhh ? expf(m_old[HH + h] - m_new[HH + h]) : expf(m_old[h] - m_new[h]);
#pragma unroll
                        for (int d = 0; d < DV; d++) o2[h][d] *= al;
                    }
                }
                const int sel = lane & 3;
                const float mlo = sel == 0 ? m_new[0] : sel == 1 ? m_new[1] : sel == 2 ? m_new[2] : m_new[3];
                const float mhi = sel == 0 ? m_new[4] : sel == 1 ? m_new[5] : sel == 2 ? m_new[6] : m_new[7];
                const float pw = s_on ? expf(sv - (hh ? mhi : mlo)) : 0.f;
                sc[sk][sh] = pw;
                float ls = pw;
#pragma unroll
                for (int off = 4; off <= 16; off <<= 1)
                    if (off != DS) ls += __shfl_xor_sync(TFR_FULL_MASK, ls, off);
                if ((lane & (28 & ~DS)) == 0) tl[warp][sh] = ls;
            }
            __syncthreads();
            if (tid < ATTN_REP_MAX) {
                const float m_old = m_s[tid], mn = fmaxf(m_old, dec(tmax[par][tid]));
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < NT / 32; w++) sum += tl[w][tid];
                l_s[tid] = l_s[tid] * expf(m_old - mn) + sum;
                m_s[tid] = mn;
                tmax[par][tid] = enc(-1e30f);  // free for tile it + 2
            }
            const unsigned short* vs = v_stage(cur);
#pragma unroll 2
            for (int k = vkw * KPI + vkl; k < tn; k += KW * KPI) {
                const float4 pa = *reinterpret_cast<const float4*>(&sc[k][vhh * HH]);
                const float p[HH] = {pa.x, pa.y, pa.z, pa.w};
                const uint4 raw = *reinterpret_cast<const uint4*>(vs + k * KROW + vdl * DV);
                const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), v1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&raw.z)), v3 = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
                const float vf[DV] = {v0.x, v0.y, v1.x, v1.y, v2.x, v2.y, v3.x, v3.y};
#pragma unroll
                for (int h = 0; h < HH; h++)
#pragma unroll
                    for (int d = 0; d < DV; d++) o2[h][d] = fmaf(p[h], vf[d], o2[h][d]);
            }
            if (it == 0) prof_mark(7, a.prof_id);
        }
        __syncthreads();  // the last tile's weights and the final (m, l) are settled
        // the key lanes of a warp fold by shuffles, then the eight key warps of a head half fold into the four slots the epilogue sums
#pragma unroll
        for (int off = 16; off >= LPK; off >>= 1)
#pragma unroll
            for (int h = 0; h < HH; h++)
#pragma unroll
                for (int d = 0; d < DV; d++) o2[h][d] += __shfl_xor_sync(TFR_FULL_MASK, o2[h][d], off);
#pragma unroll
        for (int half = 0; half < KW / 4; half++) {
            if ((vkw >> 2) == half && lane < LPK) {
#pragma unroll
                for (int h = 0; h < HH; h++)
#pragma unroll
                    for (int d = 0; d < DV; d++) {
                        float* dst = &ored[vkw & 3][vhh * HH + h][lane * DV + d];
                        *dst = half ? *dst + o2[h][d] : o2[h][d];
                    }
            }
            __syncthreads();
        }
    } else {
        register_route();
    }
    prof_mark(2, a.prof_id);
    __syncthreads();
    const int po = 2 + HD;
    if (S_eff == 1) {
        // single split: normalise and store directly (the merge of one partial is the identity)
        for (int idx = tid; idx < rep * HD; idx += NT) {
            const int h = idx / HD, d = idx % HD;
            const int hg = g * rep + h;
            const float tot = ored[0][h][d] + ored[1][h][d] + ored[2][h][d] + ored[3][h][d];
            float r = tot / fmaxf(l_s[h], 1e-20f);
            if (a.gate) r *= 1.f / (1.f + expf(-a.gate[hg * HD + d]));
            a.out[hg * HD + d] = r;
        }
        prof_mark(5, a.prof_id);
        return;
    }
    // ---- level 1, inside the cluster.  Every member sends slice j of its O (the sum of its four key
    // groups) and its (m, l) into member j's shared memory: remote stores stream out without waiting,
    // where remote loads cost a round trip each.  After one cluster barrier member j merges slice j of the
    // cluster's eight splits from local memory; nothing remote is touched afterwards, so members leave
    // independently.  Members past the last split send zeros that the merge skips, and still own a slice.
    const int cl = s / CL, rk = s % CL;
    const int total = rep * HD, per = total / CL;
    for (int idx = tid; idx < total; idx += NT) {
        const int h = idx / HD, d = idx % HD;
        const float v = ored[0][h][d] + ored[1][h][d] + ored[2][h][d] + ored[3][h][d];
        st_dsmem_f32(&gath[rk * per + idx % per], (unsigned)(idx / per), v);
    }
    if (tid < CL * ATTN_REP_MAX) {
        const int r = tid / ATTN_REP_MAX, h = tid % ATTN_REP_MAX;
        st_dsmem_f32(&gm[rk][h], (unsigned)r, m_s[h]);
        st_dsmem_f32(&gl[rk][h], (unsigned)r, l_s[h]);
    }
    cluster_sync_all();
    prof_mark(3, a.prof_id);
    const int in_cl = min(CL, S_eff - cl * CL);  // splits of this cluster that had keys
    if (n_cl == 1) {
        for (int i = tid; i < per; i += NT) {
            const int idx = rk * per + i;
            const int h = idx / HD, d = idx % HD;
            const int hg = g * rep + h;
            float m = -1e30f;
            for (int r = 0; r < in_cl; r++) m = fmaxf(m, gm[r][h]);
            float l = 0.f, acc = 0.f;
            for (int r = 0; r < in_cl; r++) {
                const float al = expf(gm[r][h] - m);
                l += al * gl[r][h];
                acc += al * gath[r * per + i];
            }
            float res = acc / fmaxf(l, 1e-20f);
            if (a.gate) res *= 1.f / (1.f + expf(-a.gate[hg * HD + d]));
            a.out[hg * HD + d] = res;
        }
        prof_mark(5, a.prof_id);
        return;
    }
    // ---- level 2, across clusters (long contexts).  Member j of every cluster writes its cluster's merged
    // slice j — (m, l) of the heads it touches and the unnormalised O — to global memory; the member j that
    // arrives last (one counter per KV head and slice) merges the n_cl cluster partials of that slice.  The
    // eight slices of a KV head finish independently on eight SMs.
    {
        float* pbase = a.partial;
        for (int i = tid; i < per; i += NT) {
            const int idx = rk * per + i;
            const int h = idx / HD, d = idx % HD;
            float m = -1e30f;
            for (int r = 0; r < in_cl; r++) m = fmaxf(m, gm[r][h]);
            float l = 0.f, acc = 0.f;
            for (int r = 0; r < in_cl; r++) {
                const float al = expf(gm[r][h] - m);
                l += al * gl[r][h];
                acc += al * gath[r * per + i];
            }
            float* base = pbase + ((size_t)(g * rep + h) * a.S + cl) * po;
            base[2 + d] = acc;
            if (d == 0 || i == 0) {  // the first element of every head inside the slice
                base[0] = m;
                base[1] = l;
            }
        }
    }
    // release: the CTA's stores are ordered before thread 0's fence by the barrier, and the fence is cumulative
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        unsigned int* ctr = a.counters + g * ATTN_CLUSTER + rk;
        const unsigned int old = atomicAdd(ctr, 1u);
        is_last_s = (old == (unsigned int)(n_cl - 1));
        if (is_last_s) {
            *ctr = 0u;
            __threadfence();  // acquire side: the other clusters' partials, read below with L2 loads
        }
    }
    __syncthreads();
    if (!is_last_s) return;
    for (int i = tid; i < per; i += NT) {
        const int idx = rk * per + i;
        const int h = idx / HD, d = idx % HD;
        const int hg = g * rep + h;
        const float* hb = a.partial + (size_t)hg * a.S * po;
        // RC cluster partials per round, all of a round's loads in flight together (one trip to L2 per round)
        constexpr int RC = STAGED ? 16 : 8;
        float m = -1e30f, l = 0.f, acc = 0.f;
        for (int c0 = 0; c0 < n_cl; c0 += RC) {
            float mm[RC], ll[RC], aa[RC];
#pragma unroll
            for (int j = 0; j < RC; j++) {
                const bool on = c0 + j < n_cl;
                const float* b = hb + (size_t)(on ? c0 + j : c0) * po;
                mm[j] = on ? __ldcg(b) : -1e30f;
                ll[j] = on ? __ldcg(b + 1) : 0.f;
                aa[j] = on ? __ldcg(b + 2 + d) : 0.f;
            }
            float m_new = m;
#pragma unroll
            for (int j = 0; j < RC; j++) m_new = fmaxf(m_new, mm[j]);
            const float keep = expf(m - m_new);
            l *= keep;
            acc *= keep;
            m = m_new;
#pragma unroll
            for (int j = 0; j < RC; j++) {
                const float al = expf(mm[j] - m);
                l += al * ll[j];
                acc += al * aa[j];
            }
        }
        float r = acc / fmaxf(l, 1e-20f);
        if (a.gate) r *= 1.f / (1.f + expf(-a.gate[hg * HD + d]));
        a.out[hg * HD + d] = r;
    }
    prof_mark(5, a.prof_id);
}

}  // namespace tfr
