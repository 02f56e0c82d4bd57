// Split-KV flash-decode over the f16 KV cache, one query token.
//
// Reference: kernels/attn/flash.cu:16-116 (partial) and :222-255 (merge).  The reference
// launches one CTA per (query head, split) with 8 fixed splits, so every query head
// re-reads the K/V rows of its KV head.  Here one CTA serves ALL query heads that share a
// KV head (GQA group), so each K/V row is read from HBM once per token; the number of
// splits is sized to the SM count and shrinks for short contexts.  The splits of a KV head are
// launched as thread-block clusters of eight: the eight splits of a cluster merge their (m, l, O)
// partials through distributed shared memory behind one cluster barrier, each CTA of the cluster
// finishing an eighth of the output dims (no global round trip, no second launch).  Longer
// contexts use several clusters per KV head; their merged partials meet in global memory, where for
// every eighth of the dims the CTA that arrives last merges the clusters' partials
// from global memory.  Arithmetic is fp32 on f16 data as in the reference; exp is the build's
// ex2-based expf.
#pragma once
#include <type_traits>

#include "tfr_common.cuh"

namespace tfr {

constexpr int ATTN_THREADS = 256;
constexpr int ATTN_TILE = 64;     // keys per tile
constexpr int ATTN_REP_MAX = 8;   // query heads per KV head handled by one CTA
constexpr int ATTN_CLUSTER = 8;   // CTAs per cluster (the portable maximum); AttnArgs::S is a multiple of it
constexpr int ATTN_LONG_MIN = 128;  // a split with more keys than this walks them through shared-memory stages
// Dynamic shared memory of k_attn_decode: a few stages of one K tile (rows padded by 8 halfs: 16-byte reads of 32
// different rows hit 32 different banks) and one V tile each, then q of the group's heads in fp32.  One tile in
// flight per SM is far too little to cover the memory latency (measured: 4 us per 32 KB tile with two stages), so a
// split keeps as many tiles in flight as shared memory holds.
__host__ __device__ constexpr int attn_stages(int hd) { return hd == 256 ? 2 : 5; }
inline size_t attn_stage_bytes(int hd) { return (size_t)ATTN_TILE * (hd + 8) * 2 + (size_t)ATTN_TILE * hd * 2; }
inline size_t attn_dyn_smem(int hd) { return attn_stages(hd) * attn_stage_bytes(hd) + (size_t)ATTN_REP_MAX * hd * 4; }

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
    int staged;                 // 1: the launch carries the dynamic shared memory of the long-split route (attn_dyn_smem)
    int prof_id;                // timeline probe: which launch of the token this is (test aid)
};

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
__global__ void __launch_bounds__(ATTN_THREADS) k_attn_decode(AttnArgs a, const TokenState* st) {
    prof_mark(0, a.prof_id);
    constexpr int DL = HD / 32;   // dims per lane in the score phase
    constexpr int DPT = HD / 64;  // dims per thread in the value phase
    constexpr int VK = ATTN_TILE / 4;  // keys per thread and tile in the value phase
    using KRaw = typename std::conditional<DL == 8, uint4, typename std::conditional<DL == 4, uint2, unsigned int>::type>::type;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.y, s = blockIdx.x;  // grid (S, n_kv), clusters of ATTN_CLUSTER along x
    const int rep = a.n_head / a.n_kv;
    const int kvdim = a.n_kv * HD;
    const int kg = tid >> 6, dp = tid & 63;
    // The decode state was last written by the previous token's final kernel, and every kernel of the chain
    // completes only after its predecessor: position and stop flag are final here, before the wait.
    const int done = st ? st->done : 0;
    const int T = (st ? st->pos : a.pos) + 1;
    int S_eff = (T + a.min_keys - 1) / a.min_keys;
    S_eff = S_eff < 1 ? 1 : (S_eff > a.S ? a.S : S_eff);
    // up to ATTN_CLUSTER splits: the first cluster of the KV head merges on chip; its idle members
    // still attend the cluster barriers.  More splits: every CTA for itself, merge through memory.
    const int n_cl = (S_eff + ATTN_CLUSTER - 1) / ATTN_CLUSTER;  // clusters that have work
    const bool leave = done || (S_eff == 1 ? s >= 1 : s >= n_cl * ATTN_CLUSTER);
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
    const bool long_path = STAGED && a.staged && t1 - t0 > ATTN_LONG_MIN;
    if (!long_path) {
        load_k(t0, min(t1, T - 1), false);
        load_v(t0, min(t1, T - 1), false);
    }
    griddep_wait();  // q and the new K/V row come from the previous kernel
    griddep_launch_dependents();
    prof_mark(1, a.prof_id);
    if (leave) return;
    if (!long_path) {
        load_k(t0, 0, true);
        load_v(t0, 0, true);
    }

    __shared__ __align__(16) float sc[ATTN_TILE][ATTN_REP_MAX];  // [key][head]: the value phase reads a key's eight weights as two float4
    __shared__ float m_s[ATTN_REP_MAX], l_s[ATTN_REP_MAX], alpha_s[ATTN_REP_MAX];
    __shared__ float ored[4][ATTN_REP_MAX][HD];
    __shared__ int is_last_s;
    // on-chip merge: slice s of every member's O, and every member's (m, l), land here
    __shared__ float gath[ATTN_CLUSTER][HD];
    __shared__ float gm[ATTN_CLUSTER][ATTN_REP_MAX], gl[ATTN_CLUSTER][ATTN_REP_MAX];

    // q fragment of every head of the group: dims lane*DL .. lane*DL+DL-1
    float qr[ATTN_REP_MAX][DL];
#pragma unroll
    for (int h = 0; h < ATTN_REP_MAX; h++)
#pragma unroll
        for (int d = 0; d < DL; d++) qr[h][d] = h < rep ? a.q[(g * rep + h) * HD + lane * DL + d] : 0.f;
    if (tid < ATTN_REP_MAX) {
        m_s[tid] = -1e30f;
        l_s[tid] = 0.f;
    }
    float o[ATTN_REP_MAX][DPT];
#pragma unroll
    for (int h = 0; h < ATTN_REP_MAX; h++)
#pragma unroll
        for (int d = 0; d < DPT; d++) o[h][d] = 0.f;
    __syncthreads();
    prof_mark(4, a.prof_id);

    if constexpr (STAGED) if (long_path) {
        // ---- long splits: K and V tiles travel global -> shared memory as asynchronous 16-byte copies, NST stages
        // deep, so the loads of the next tiles run under the arithmetic of tile i and no register holds cache data.
        extern __shared__ __align__(16) unsigned char attn_dyn[];
        constexpr int KROW = HD + 8, CPR = HD / 8;  // halfs per staged K row; 16-byte chunks per cache row
        constexpr int NST = attn_stages(HD);
        const size_t stage_b = (size_t)ATTN_TILE * KROW * 2 + (size_t)ATTN_TILE * HD * 2;
        float* q_s = reinterpret_cast<float*>(attn_dyn + NST * stage_b);
        auto k_stage = [&](int st_) { return reinterpret_cast<unsigned short*>(attn_dyn + (size_t)st_ * stage_b); };
        auto v_stage = [&](int st_) { return reinterpret_cast<unsigned short*>(attn_dyn + (size_t)st_ * stage_b + (size_t)ATTN_TILE * KROW * 2); };
        auto issue_tile = [&](int tt, int st_) {
            unsigned short* ks = k_stage(st_);
            unsigned short* vs = v_stage(st_);
            if (tt < t1)
                for (int i = tid; i < ATTN_TILE * CPR; i += ATTN_THREADS) {
                    const int row = i / CPR, c8 = i - row * CPR;
                    const bool in = tt + row < t1;
                    const size_t off = (size_t)(in ? tt + row : t1 - 1) * kvdim + (size_t)g * HD + c8 * 8;
                    cp_async16(ks + row * KROW + c8 * 8, a.kc + off, in ? 16 : 0);
                    cp_async16(vs + row * HD + c8 * 8, a.vc + off, in ? 16 : 0);
                }
            cp_async_commit();  // a group per tile slot, empty past the end: the wait below counts groups
        };
#pragma unroll
        for (int p = 0; p < NST - 1; p++) issue_tile(t0 + p * ATTN_TILE, p);
        for (int i = tid; i < rep * HD; i += ATTN_THREADS) q_s[i] = a.q[g * rep * HD + i];
        // Both phases are register-blocked so that shared-memory reads stay well below the FMA count (a 16-byte read
        // costs the load pipe four cycles per warp even when all lanes read the same address).
        // Scores: a thread takes KPT keys x all heads x one slice of DSL dims: per 8 dims it reads q once for the
        // eight heads (16 reads) and each key once (KPT reads) for KPT * 64 FMAs; the DS slices of a key group are
        // DS adjacent lanes, their partial sums meet in a halving butterfly that leaves lane ds with values 2 ds, 2 ds + 1.
        // Values: warp w takes keys w, w + 8, ... of the tile, lane l the dims l * DV ..: per key 2 reads of the eight
        // weights and one of V for 8 * DV FMAs.
        constexpr int DS = HD >= 128 ? 16 : 8;          // dim slices (lanes) per key group
        constexpr int DSL = HD / DS;                    // dims per slice: 8 or 16
        constexpr int KPT = DS / 4;                     // keys per thread: 8 warps x (32 / DS) groups x KPT = 64
        constexpr int NV = KPT * ATTN_REP_MAX;          // partial sums per thread
        constexpr int DV = HD / 32;                     // value dims per lane
        const int ds = lane & (DS - 1), kgrp = warp * (32 / DS) + lane / DS;
        const int key0 = kgrp * KPT;
        float o2[ATTN_REP_MAX][DV];
#pragma unroll
        for (int h = 0; h < ATTN_REP_MAX; h++)
#pragma unroll
            for (int d = 0; d < DV; d++) o2[h][d] = 0.f;
        int it = 0;
        for (int tt = t0; tt < t1; tt += ATTN_TILE, it++) {
            const int tn = min(ATTN_TILE, t1 - tt), cur = it % NST;
            issue_tile(tt + (NST - 1) * ATTN_TILE, (it + NST - 1) % NST);  // the stage tile it - 1 has just left
            cp_async_wait_group<NST - 1>();
            __syncthreads();
            if (it == 0) prof_mark(6, a.prof_id);
            {
                float v[NV];
#pragma unroll
                for (int i = 0; i < NV; i++) v[i] = 0.f;
                const unsigned short* kbase = k_stage(cur) + key0 * KROW + ds * DSL;
#pragma unroll
                for (int c = 0; c < DSL; c += 8) {
                    float kf[KPT][8];
#pragma unroll
                    for (int kk = 0; kk < KPT; kk++) {
                        const int4 kw = *reinterpret_cast<const int4*>(kbase + kk * KROW + c);
                        const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kw.x)), k1 = __half22float2(*reinterpret_cast<const __half2*>(&kw.y));
                        const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kw.z)), k3 = __half22float2(*reinterpret_cast<const __half2*>(&kw.w));
                        kf[kk][0] = k0.x, kf[kk][1] = k0.y, kf[kk][2] = k1.x, kf[kk][3] = k1.y;
                        kf[kk][4] = k2.x, kf[kk][5] = k2.y, kf[kk][6] = k3.x, kf[kk][7] = k3.y;
                    }
#pragma unroll
                    for (int h = 0; h < ATTN_REP_MAX; h++) {
                        if (h < rep) {
                            const float* qp = q_s + h * HD + ds * DSL + c;
                            const float4 a0 = *reinterpret_cast<const float4*>(qp), a1 = *reinterpret_cast<const float4*>(qp + 4);
#pragma unroll
                            for (int kk = 0; kk < KPT; kk++)
                                v[kk * ATTN_REP_MAX + h] += a0.x * kf[kk][0] + a0.y * kf[kk][1] + a0.z * kf[kk][2] + a0.w * kf[kk][3] +
                                                            a1.x * kf[kk][4] + a1.y * kf[kk][5] + a1.z * kf[kk][6] + a1.w * kf[kk][7];
                        }
                    }
                }
                // halving butterfly over the DS lanes of the key group
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
                // this lane now holds values 2 ds and 2 ds + 1 of the group's KPT x 8: key 2 ds / 8, heads 2 ds % 8, + 1
                const int kl = (2 * ds) >> 3, h0 = (2 * ds) & 7, k = key0 + kl;
                sc[k][h0] = (k < tn && h0 < rep) ? v[0] * a.scale : -1e30f;
                sc[k][h0 + 1] = (k < tn && h0 + 1 < rep) ? v[1] * a.scale : -1e30f;
            }
            __syncthreads();
            if (warp < rep) {  // online softmax bookkeeping: warp h owns head h
                const float s0 = sc[lane][warp], s1 = sc[lane + 32][warp];
                const float tile_m = warp_max(fmaxf(s0, s1));
                const float m_old = m_s[warp];
                const float m_new = fmaxf(m_old, tile_m);
                const float p0 = (lane < tn) ? expf(s0 - m_new) : 0.f;
                const float p1 = (lane + 32 < tn) ? expf(s1 - m_new) : 0.f;
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
#pragma unroll
            for (int h = 0; h < ATTN_REP_MAX; h++) {
                const float al = h < rep ? alpha_s[h] : 1.f;
#pragma unroll
                for (int d = 0; d < DV; d++) o2[h][d] *= al;
            }
            const unsigned short* vs = v_stage(cur);
#pragma unroll 2
            for (int k = warp; k < tn; k += 8) {
                const float4 pa = *reinterpret_cast<const float4*>(&sc[k][0]), pb = *reinterpret_cast<const float4*>(&sc[k][4]);
                const float p[ATTN_REP_MAX] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
                float vf[DV];
                const unsigned short* vr = vs + k * HD + lane * DV;
                if constexpr (DV == 8) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(vr);
                    const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), v1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&raw.z)), v3 = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
                    vf[0] = v0.x, vf[1] = v0.y, vf[2] = v1.x, vf[3] = v1.y, vf[4] = v2.x, vf[5] = v2.y, vf[6] = v3.x, vf[7] = v3.y;
                } else if constexpr (DV == 4) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(vr);
                    const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), v1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    vf[0] = v0.x, vf[1] = v0.y, vf[2] = v1.x, vf[3] = v1.y;
                } else {
                    const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(vr));
                    vf[0] = v0.x, vf[1] = v0.y;
                }
#pragma unroll
                for (int h = 0; h < ATTN_REP_MAX; h++) {
                    if (h < rep) {
#pragma unroll
                        for (int d = 0; d < DV; d++) o2[h][d] += p[h] * vf[d];
                    }
                }
            }
            __syncthreads();  // the next iteration overwrites sc and refills the stage just used
            if (it == 0) prof_mark(7, a.prof_id);
        }
        // the eight key groups (warps) fold into the four slots the epilogue sums
#pragma unroll
        for (int half = 0; half < 2; half++) {
            if ((warp >> 2) == half) {
#pragma unroll
                for (int h = 0; h < ATTN_REP_MAX; h++)
#pragma unroll
                    for (int d = 0; d < DV; d++) {
                        float* dst = &ored[warp & 3][h][lane * DV + d];
                        *dst = half ? *dst + o2[h][d] : o2[h][d];
                    }
            }
            __syncthreads();
        }
    }
    for (int tt = t0; tt < t1 && !long_path; tt += ATTN_TILE) {
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

    prof_mark(2, a.prof_id);
    // ---- combine the four key groups and write this split's (m, l, O)
    if (!long_path) {
#pragma unroll
        for (int h = 0; h < ATTN_REP_MAX; h++)
#pragma unroll
            for (int d = 0; d < DPT; d++) ored[kg][h][dp * DPT + d] = o[h][d];
    }
    __syncthreads();
    const int po = 2 + HD;
    if (S_eff == 1) {
        // single split: normalise and store directly (the merge of one partial is the identity)
        for (int idx = tid; idx < rep * HD; idx += ATTN_THREADS) {
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
    const int cl = s / ATTN_CLUSTER, rk = s % ATTN_CLUSTER;
    const int total = rep * HD, per = total / ATTN_CLUSTER;  // per <= HD
    for (int idx = tid; idx < total; idx += ATTN_THREADS) {
        const int h = idx / HD, d = idx % HD;
        const float v = ored[0][h][d] + ored[1][h][d] + ored[2][h][d] + ored[3][h][d];
        st_dsmem_f32(&gath[rk][idx % per], (unsigned)(idx / per), v);
    }
    if (tid < ATTN_CLUSTER * ATTN_REP_MAX) {
        const int r = tid / ATTN_REP_MAX, h = tid % ATTN_REP_MAX;
        st_dsmem_f32(&gm[rk][h], (unsigned)r, m_s[h]);
        st_dsmem_f32(&gl[rk][h], (unsigned)r, l_s[h]);
    }
    cluster_sync_all();
    prof_mark(3, a.prof_id);
    const int in_cl = min(ATTN_CLUSTER, S_eff - cl * ATTN_CLUSTER);  // splits of this cluster that had keys
    if (n_cl == 1) {
        for (int i = tid; i < per; i += ATTN_THREADS) {
            const int idx = rk * per + i;
            const int h = idx / HD, d = idx % HD;
            const int hg = g * rep + h;
            float m = -1e30f;
            for (int r = 0; r < in_cl; r++) m = fmaxf(m, gm[r][h]);
            float l = 0.f, acc = 0.f;
            for (int r = 0; r < in_cl; r++) {
                const float al = expf(gm[r][h] - m);
                l += al * gl[r][h];
                acc += al * gath[r][i];
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
        for (int i = tid; i < per; i += ATTN_THREADS) {
            const int idx = rk * per + i;
            const int h = idx / HD, d = idx % HD;
            float m = -1e30f;
            for (int r = 0; r < in_cl; r++) m = fmaxf(m, gm[r][h]);
            float l = 0.f, acc = 0.f;
            for (int r = 0; r < in_cl; r++) {
                const float al = expf(gm[r][h] - m);
                l += al * gl[r][h];
                acc += al * gath[r][i];
            }
            float* base = pbase + ((size_t)(g * rep + h) * a.S + cl) * po;
            base[2 + d] = acc;
            if (d == 0 || i == 0) {  // the first element of every head inside the slice
                base[0] = m;
                base[1] = l;
            }
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned int* ctr = a.counters + g * ATTN_CLUSTER + rk;
        const unsigned int old = atomicAdd(ctr, 1u);
        is_last_s = (old == (unsigned int)(n_cl - 1));
        if (is_last_s) *ctr = 0u;
    }
    __syncthreads();
    if (!is_last_s) return;
    __threadfence();
    for (int i = tid; i < per; i += ATTN_THREADS) {
        const int idx = rk * per + i;
        const int h = idx / HD, d = idx % HD;
        const int hg = g * rep + h;
        const float* hb = a.partial + (size_t)hg * a.S * po;
        float m = -1e30f;
#pragma unroll 4
        for (int c = 0; c < n_cl; c++) m = fmaxf(m, __ldcg(hb + (size_t)c * po));
        float l = 0.f, acc = 0.f;
#pragma unroll 4
        for (int c = 0; c < n_cl; c++) {
            const float* b = hb + (size_t)c * po;
            const float al = expf(__ldcg(b) - m);
            l += al * __ldcg(b + 1);
            acc += al * __ldcg(b + 2 + d);
        }
        float r = acc / fmaxf(l, 1e-20f);
        if (a.gate) r *= 1.f / (1.f + expf(-a.gate[hg * HD + d]));
        a.out[hg * HD + d] = r;
    }
    prof_mark(5, a.prof_id);
}

}  // namespace tfr
