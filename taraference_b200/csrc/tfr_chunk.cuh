// Multi-token ("chunk") forward: prompts and verification batches.
//
// The reference feeds a prompt in chunks of up to MAX_BATCH tokens (crates/core/src/cuda/forward.rs:54-65,
// 360-407) and verifies up to MAX_VERIFY_TOKENS tokens in one pass (forward.rs:268-358): its GEMM kernels
// (kernels/gemm.cu:6-190) read every weight block once per chunk, and attn_fast_v2 (kernels/attn/fast_v2.cu:12-192)
// runs causal attention over the f16 cache.  Here a chunk of M tokens goes through
//
//   k_embed_rows     x[m] = embedding row of token m                                  (kernels/embed.cu:71-131)
//   k_prep_rows      per token: RMSNorm (kernels/ops.cu:4-34) + Q8 quantiser (kernels/gemv.cu:16-65) -> global
//   k_gemm_q8        every weight tile is brought on chip once per launch and dotted with the activations of up
//                    to Mt tokens at a time; same block dots, row sums and epilogues as the batch-1 kernels
//   k_attn_chunk     causal attention of a tile of query tokens x the query heads of one KV head over the f16 cache
//   k_argmax_rows    greedy token of every row                                        (kernels/ops.cu:601-629)
//
// The projections use the arithmetic of the decode path (Q8 activations, integer block dots), not the reference's
// prefill arithmetic (fp32 activations against dequantised weights): a prompt fed in chunks then leaves the same
// K/V rows and residual stream as the same prompt fed token by token, up to the summation order inside attention.
#pragma once
#include "tfr_kernels.cuh"

namespace tfr {

constexpr int CHUNK_MAX_TOKENS = 64;   // tokens per chunk forward
constexpr int CHUNK_VERIFY_MAX = 16;   // tokens per chunk when every row's greedy token is wanted (logits [M][V])
constexpr int CHUNK_ATTN_SPLITS_MAX = 32;  // most key splits of the chunk attention

// ------------------------------------------------------------------ embedding rows

__global__ void k_embed_rows(Mat E, const int* tokens, int K, float* x, TokenState* st) {
    const int m = blockIdx.x;
    int tok = tokens[m];
    if (tok < 0 || tok >= E.N) {
        if (st && threadIdx.x == 0) st->err = 1;
        tok = 0;
    }
    const SrcEmbed src{E, tok};
    for (int i = threadIdx.x; i < K; i += blockDim.x) x[(size_t)m * K + i] = src.get(i);
}

// ------------------------------------------------------------------ RMSNorm + Q8 per token, to global memory

struct PrepRowsArgs {
    const float* x;      // [M][ldx]
    int ldx, K;
    const float* normw;  // RMSNorm weight or nullptr
    float eps;
    unsigned char* act;  // [M][act_stride]: the Act arrays of every token (act_carve layout)
    size_t act_stride;
    float* xn;           // optional [M][K]: the normalised fp32 vector (fp32-route rows read it)
};

// One CTA per token.  Dynamic shared memory: the staged vector + 272 floats when a norm is fused, else nothing.
__global__ void __launch_bounds__(GEMV_THREADS, 1) k_prep_rows(PrepRowsArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int m = blockIdx.x, tid = threadIdx.x, K = a.K, n4 = K >> 2, nb = K >> 8;
    const float* x = a.x + (size_t)m * a.ldx;
    const Act act = act_carve(a.act + (size_t)m * a.act_stride, K, false, false);
    griddep_wait();
    griddep_launch_dependents();
    if (a.normw) {
        float* xs = reinterpret_cast<float*>(smem);
        float* red = xs + xs_floats(K);
        for (int i4 = tid; i4 < n4; i4 += GEMV_THREADS)
            *reinterpret_cast<float4*>(xs + xs_idx(4 * i4)) = reinterpret_cast<const float4*>(x)[i4];
        __syncthreads();
        const float scale = rms_scale_staged(xs, K, a.eps, red);
        for (int k0 = 0; k0 < n4; k0 += GEMV_THREADS) {
            const int i4 = k0 + tid;
            const bool on = i4 < n4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on) {
                v = *reinterpret_cast<const float4*>(xs + xs_idx(4 * i4));
                const float4 w = reinterpret_cast<const float4*>(a.normw)[i4];
                v.x = v.x * scale * w.x;
                v.y = v.y * scale * w.y;
                v.z = v.z * scale * w.z;
                v.w = v.w * scale * w.w;
                if (a.xn) reinterpret_cast<float4*>(a.xn + (size_t)m * K)[i4] = v;
            }
            act_quantize4(act, v, i4, on, nb);
        }
    } else {
        for (int k0 = 0; k0 < n4; k0 += GEMV_THREADS) {
            const int i4 = k0 + tid;
            const bool on = i4 < n4;
            const float4 v = on ? reinterpret_cast<const float4*>(x)[i4] : make_float4(0.f, 0.f, 0.f, 0.f);
            act_quantize4(act, v, i4, on, nb);
        }
    }
}

// ------------------------------------------------------------------ epilogues with a token index

enum { CEPI_STORE = 0, CEPI_SILU = 1, CEPI_QKV = 2 };

struct ChunkEpi {
    int kind;
    float* out;          // [M][ldo]
    int ldo, n_rows, use_res;
    const float* bias;
    // CEPI_QKV (EpiQkv per token): q rows go to out; K and V rows of position pos0 + m to the cache
    unsigned short *kc, *vc;
    int nq, nk, hd, kvdim, pos0;
    float theta;
};

// The epilogue of token m in the shape reduce_rows expects.
struct ChunkEpiTok {
    const ChunkEpi* e;
    int m;
    __device__ __forceinline__ void store_one(int row, float acc) const {
        float* o = e->out + (size_t)m * e->ldo;
        if (e->use_res == 2) acc += o[row];
        if (e->bias) acc += e->bias[row];
        o[row] = acc;
    }
    __device__ __forceinline__ void apply(int p, float x0, float x1) const {
        if (e->kind == CEPI_SILU) {
            e->out[(size_t)m * e->ldo + p] = (x0 / (1.f + __expf(-x0))) * x1;  // kernels/gemv.cu:2570-2574
            return;
        }
        if (e->kind == CEPI_STORE) {  // kernels/gemv.cu:367-373
            store_one(2 * p, x0);
            if (2 * p + 1 < e->n_rows) store_one(2 * p + 1, x1);
            return;
        }
        // bias, neox RoPE (kernels/ops.cu:348-371), f16 KV store (kernels/ops.cu:471-486): EpiQkv at position pos0 + m
        const int v = 2 * p, nq = e->nq, nk = e->nk, hd = e->hd, pos = e->pos0 + m;
        if (e->bias) {
            x0 += e->bias[v];
            x1 += e->bias[v + 1];
        }
        if (v < nq + nk) {
            const bool isq = v < nq;
            const int vv = isq ? v : v - nq;
            const int head = vv / hd, i = (vv % hd) >> 1, half = hd >> 1;
            const float freq = powf(e->theta, -2.f * (float)i / (float)hd);
            const float ang = (float)pos * freq;
            const float c = cosf(ang), sn = sinf(ang);
            const float y0 = x0 * c - x1 * sn;
            const float y1 = x0 * sn + x1 * c;
            if (isq) {
                float* q = e->out + (size_t)m * e->ldo;
                q[head * hd + i] = y0;
                q[head * hd + i + half] = y1;
            } else {
                unsigned short* kr = e->kc + (size_t)pos * e->kvdim + head * hd;
                kr[i] = f32_to_f16_bits_ref(y0);
                kr[i + half] = f32_to_f16_bits_ref(y1);
            }
        } else {
            const int vv = v - nq - nk;
            unsigned short* vr = e->vc + (size_t)pos * e->kvdim;
            vr[vv] = f32_to_f16_bits_ref(x0);
            vr[vv + 1] = f32_to_f16_bits_ref(x1);
        }
    }
};

// reduce_rows (same lanes, same order of additions) run by a group of `gw` warps; wig = the warp's index in its group.
template <int MODE, class Epi>
__device__ __forceinline__ void reduce_rows_group(const float* pa, const float* pb, int n_rows, int nb, int id0, const Epi& epi, int wig,
                                                  int gw) {
    const int lane = threadIdx.x & 31;
    if (nb <= 16) {
        const int LPR = nb <= 8 ? 8 : 16, RPW = 32 / LPR;
        const int k = lane & (LPR - 1), rl = lane / LPR;
        for (int base = wig * RPW; base < n_rows; base += gw * RPW) {
            const int r = base + rl;
            const bool on = r < n_rows && k < nb;
            float a = on ? pa[r * nb + k] : 0.f;
            float b = (MODE == EPI_ZIP && on) ? pb[r * nb + k] : 0.f;
            for (int o = LPR >> 1; o > 0; o >>= 1) {
                a += __shfl_xor_sync(TFR_FULL_MASK, a, o);
                if (MODE == EPI_ZIP) b += __shfl_xor_sync(TFR_FULL_MASK, b, o);
            }
            if (MODE == EPI_ZIP) {
                if (k == 0 && r < n_rows) epi.apply(id0 + r, a, b);
            } else {
                const float other = __shfl_down_sync(TFR_FULL_MASK, a, LPR);
                if (k == 0 && !(rl & 1) && r < n_rows) epi.apply(id0 + (r >> 1), a, other);
            }
        }
    } else {
        const int items = MODE == EPI_ZIP ? n_rows : (n_rows + 1) >> 1;
        for (int it = wig; it < items; it += gw) {
            const float* ra = MODE == EPI_ZIP ? pa + it * nb : pa + (2 * it) * nb;
            const float* rb = MODE == EPI_ZIP ? pb + it * nb : ra + nb;
            const bool has_b = MODE == EPI_ZIP || 2 * it + 1 < n_rows;
            float a = 0.f, b = 0.f;
            for (int i = lane; i < nb; i += 32) {
                a += ra[i];
                if (has_b) b += rb[i];
            }
            a = warp_sum(a);
            b = warp_sum(b);
            if (lane == 0) epi.apply(id0 + it, a, b);
        }
    }
}

// ------------------------------------------------------------------ the chunk GEMM

// Shared memory: [ Act x Mt | partial sums x Mt | mbarriers | tile slots ].
// Warp w < wa owns the tiles w, w + wa, ... of the CTA and `nsw` ring slots; it refills a slot as soon as it has used
// the tile in it, so the stream runs `nsw` tiles ahead of the dots.  With more tokens than Mt the CTA walks its
// tiles once per group of Mt tokens (the second pass finds them in L2).
struct GemmGeom {
    int M, Mt, K, pbuf_floats, nsw;
    int wa;              // warps that run block dots (each owns nsw ring slots); a power of two <= 32
    size_t act_stride;   // bytes between tokens in the global activation buffer
    int act_b16;         // bytes of one token's Act in shared memory (a multiple of 16)
};

template <class BLK>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
k_gemm_q8(const unsigned char* act_g, const float* xn, RowJob ja, RowJob jb, F32Seg fseg, ChunkEpi epi, GemmGeom g, TokenState* st) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cta = blockIdx.x;
    const int K = g.K, nb = K >> 8, Mt = g.Mt, nsw = g.nsw, wa = g.wa;
    constexpr int TB = BLK::TILE_BYTES;
    unsigned char* act_s = smem;
    float* pbuf = reinterpret_cast<float*>(act_s + (size_t)Mt * g.act_b16);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(pbuf + (size_t)Mt * g.pbuf_floats);
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(full + wa * nsw) + 127) & ~(uintptr_t)127);

    const int rows_a0 = ja.sh.begin(cta) * ja.rows_per_item;
    const int rows_a = max(0, min(ja.sh.count(cta) * ja.rows_per_item, ja.m.N - rows_a0));
    const int rows_b0 = jb.m.data ? jb.sh.begin(cta) * jb.rows_per_item : 0;
    const int rows_b = jb.m.data ? max(0, min(jb.sh.count(cta) * jb.rows_per_item, jb.m.N - rows_b0)) : 0;
    const long long fa0 = (long long)rows_a0 * nb, fa1 = fa0 + (long long)rows_a * nb;
    const long long fb0 = (long long)rows_b0 * nb, fb1 = fb0 + (long long)rows_b * nb;
    const int ta0 = (int)(fa0 >> 5), tiles_a = rows_a > 0 ? (int)((fa1 + 31) >> 5) - ta0 : 0;
    const int tb0 = (int)(fb0 >> 5), tiles_b = rows_b > 0 ? (int)((fb1 + 31) >> 5) - tb0 : 0;
    const int n_jobs = tiles_a + tiles_b;
    const int ntw = (warp < wa && warp < n_jobs) ? (n_jobs - warp + wa - 1) / wa : 0;  // tiles of this warp
    const int n_groups = (g.M + Mt - 1) / Mt;
    const int uses = ntw * n_groups;  // tile uses of this warp over the whole launch
    unsigned long long* wfull = full + (warp < wa ? warp : 0) * nsw;
    unsigned char* wring = ring + (size_t)(warp < wa ? warp : 0) * nsw * TB;
    auto issue = [&](int k) {  // use k of this warp: tile warp + wa * (k mod ntw) into slot k mod nsw
        const int j = warp + wa * (k % ntw), s = k % nsw;
        const uint8_t* src = j < tiles_a ? ja.m.data + (long long)(ta0 + j) * TB : jb.m.data + (long long)(tb0 + j - tiles_a) * TB;
        mbar_expect_tx(wfull + s, TB);
        bulk_load(wring + (size_t)s * TB, src, TB, wfull + s);
    };
    if (lane == 0 && warp < wa) {
        for (int s = 0; s < nsw; s++) mbar_init(wfull + s, 1);
        mbar_fence_init();
        for (int k = 0; k < nsw && k < uses; k++) issue(k);  // weights do not depend on the previous kernel
    }
    __syncwarp();
    griddep_wait();
    griddep_launch_dependents();

    const int G = Mt >= 8 ? 8 : (Mt >= 4 ? 4 : (Mt >= 2 ? 2 : 1));  // token groups of the row-sum phase
    const int gw = GEMV_WARPS / G, grp = warp / gw, wig = warp % gw;
    bool ok = true, dead = false;  // dead: this warp saw a copy time out and takes no further tiles
    int late_slot = -1;
    unsigned late_parity = 0;
    for (int grp_i = 0; grp_i < n_groups; grp_i++) {
        const int m0 = grp_i * Mt, mt = min(Mt, g.M - m0);
        // the Q8 activations of tokens m0 .. m0 + mt - 1
        {
            const int per = g.act_b16 >> 4;
            for (int i = tid; i < mt * per; i += GEMV_THREADS) {
                const int m = i / per, r = i - m * per;
                reinterpret_cast<int4*>(act_s + (size_t)m * g.act_b16)[r] =
                    reinterpret_cast<const int4*>(act_g + (size_t)(m0 + m) * g.act_stride)[r];
            }
        }
        __syncthreads();
        // rows on the fp32 activation route (kernels/gemv.cu:233-264): a task = (row, block, run of 16) reads its
        // weights once and walks the tokens of the group, each token's normalised vector straight from global memory
        if (fseg.m.data) {
            const int np = fseg.sh.count(cta), pbase = fseg.sh.begin(cta);
            const int per_row = 16 * nb, ppp = max(1, g.pbuf_floats / (2 * per_row));  // row pairs per pass
            for (int p0 = 0; p0 < np; p0 += ppp) {
                const int pn = min(ppp, np - p0), tn = pn * 2 * per_row;
                for (int t = tid; t < tn; t += GEMV_THREADS) {
                    const int row_l = t / per_row, rem = t - row_l * per_row;
                    const int row_g = 2 * (pbase + p0) + row_l;
                    for (int m = 0; m < mt; m++) {
                        float v = 0.f;
                        if (row_g < fseg.m.N)
                            v = q6k_run_dot_f32_g(fseg.m, (long long)row_g * nb + (rem >> 4), rem >> 4, rem & 15, xn + (size_t)(m0 + m) * K);
                        pbuf[(size_t)m * g.pbuf_floats + t] = v;
                    }
                }
                __syncthreads();
                for (int item = warp; item < pn * mt; item += GEMV_WARPS) {
                    const int m = item / pn, rr = item - m * pn;
                    const float* a = pbuf + (size_t)m * g.pbuf_floats + (2 * rr) * per_row;
                    float s0 = 0.f, s1 = 0.f;
                    for (int i = lane; i < per_row; i += 32) {
                        s0 += a[i];
                        s1 += a[per_row + i];
                    }
                    s0 = warp_sum(s0);
                    s1 = warp_sum(s1);
                    if (lane == 0) ChunkEpiTok{&epi, m0 + m}.apply(fseg.id_base + pbase + p0 + rr, s0, s1);
                }
                __syncthreads();
            }
        }
        // phase A: per-block partials of every token out of the tiles
        for (int i = 0; i < ntw && !dead; i++) {
            const int k = grp_i * ntw + i, j = warp + wa * i, s = k % nsw;
            const bool is_b = j >= tiles_a;
            const long long f = (long long)(is_b ? tb0 + (j - tiles_a) : ta0 + j) * 32 + lane;
            const bool mine = is_b ? (f >= fb0 && f < fb1) : (f >= fa0 && f < fa1);
            // a copy that did not land within the wait limit: its tile is not read, the error word marks the call invalid
            // and the warp stops issuing; it waits for that copy once more before the CTA leaves
            const bool landed = mbar_wait(wfull + s, (unsigned)((k / nsw) & 1));
            if (!landed) {
                ok = false;
                late_slot = s;
                late_parity = (unsigned)((k / nsw) & 1);
            }
            if (mine) {
                const int off = is_b ? rows_a * nb + (int)(f - fb0) : (int)(f - fa0);
                const int b = (int)(f % nb);
                // (Sharing the nibble masks / 6-bit assembly of a block across four tokens was measured: at the 64
                // registers a 1024-thread CTA allows it spills and runs 13 % slower than one block_dot per token.)
                for (int m = 0; m < mt; m++) {
                    const Act act = act_carve(act_s + (size_t)m * g.act_b16, K, false, false);
                    pbuf[(size_t)m * g.pbuf_floats + off] = landed ? block_dot<true>(BLK{}, wring + (size_t)s * TB, lane, act, b, nb, nullptr) : 0.f;
                }
            }
            __syncwarp();
            if (!landed) {
                dead = true;
                break;
            }
            if (lane == 0 && k + nsw < uses) {
                fence_proxy_async();
                issue(k + nsw);
            }
        }
        __syncthreads();
        // phase B: row sums in the decode kernels' order + epilogue, token groups side by side
        for (int m = grp; m < mt; m += G) {
            const ChunkEpiTok et{&epi, m0 + m};
            const float* part_a = pbuf + (size_t)m * g.pbuf_floats;
            const float* part_b = part_a + rows_a * nb;
            if (epi.kind == CEPI_SILU) {
                reduce_rows_group<EPI_ZIP>(part_a, part_b, rows_a, nb, ja.id_base + rows_a0, et, wig, gw);
            } else {
                reduce_rows_group<EPI_PAIRS>(part_a, part_a, rows_a, nb, ja.id_base + (rows_a0 >> 1), et, wig, gw);
                if (rows_b > 0) reduce_rows_group<EPI_PAIRS>(part_b, part_b, rows_b, nb, jb.id_base + (rows_b0 >> 1), et, wig, gw);
            }
        }
        __syncthreads();
    }
    if (!ok && st) st->err = 2;
    if (late_slot >= 0) mbar_wait(wfull + late_slot, late_parity);  // bounded: a second limit, then the CTA leaves regardless
}

struct GemmLaunch {
    GemmGeom g;
    size_t smem;
    bool fits;
};

// Picks Mt (tokens per pass) and the ring depth for a launch.
inline GemmLaunch gemm_plan(int tile_bytes, int M, int K, const RowJob& ja, const RowJob& jb, bool with_f32) {
    GemmLaunch L{};
    const int nb = K / 256;
    const int ra = (ja.sh.quot + 1) * ja.rows_per_item, rb = jb.m.data ? (jb.sh.quot + 1) * jb.rows_per_item : 0;
    int pf = ((ra + rb) * nb + 3) & ~3;
    if (with_f32 && pf < 2 * 16 * nb) pf = 2 * 16 * nb;
    const size_t act_b16 = (act_smem_bytes(K, false, false) + 15) & ~(size_t)15;
    const size_t xf = 0;  // fp32-route rows read the normalised vectors from global memory
    L.fits = false;
    // The dot work of a launch does not depend on Mt, the per-pass overhead shrinks with it: take the widest set of
    // dot warps that still leaves room for a few tokens per pass, then as many tokens as fit.
    const int want = std::min(M, 4);
    for (int pass = 0; pass < 2 && !L.fits; pass++)
        for (int wa = GEMV_WARPS; wa >= 8 && !L.fits; wa >>= 1)
            for (int Mt = std::min(M, 16); Mt >= (pass == 0 ? want : 1); Mt--) {
                const size_t fixed = (size_t)Mt * act_b16 + xf + (size_t)Mt * pf * 4 + 256;
                if (fixed + (size_t)wa * (8 + tile_bytes) > GEMV_SMEM_MAX) continue;
                int nsw = (int)((GEMV_SMEM_MAX - fixed) / ((size_t)wa * (8 + tile_bytes)));
                if (nsw > 4) nsw = 4;
                L.g = GemmGeom{M, Mt, K, pf, nsw, wa, 0, (int)act_b16};
                L.smem = fixed + (size_t)wa * nsw * (8 + tile_bytes);
                L.fits = true;
                break;
            }
    return L;
}

template <class BLK>
inline cudaError_t launch_gemm(cudaStream_t stream, int grid, const unsigned char* act_g, size_t act_stride, const float* xn, int M,
                               const RowJob& ja, const RowJob& jb, const F32Seg& fseg, const ChunkEpi& epi, int K, TokenState* st) {
    GemmLaunch L = gemm_plan(BLK::TILE_BYTES, M, K, ja, jb, fseg.m.data != nullptr);
    if (!L.fits) return cudaErrorInvalidValue;
    L.g.act_stride = act_stride;
    return launch_pdl(k_gemm_q8<BLK>, dim3(grid), dim3(GEMV_THREADS), L.smem, stream, act_g, xn, ja, jb, fseg, epi, L.g, st);
}

// ------------------------------------------------------------------ causal attention of a chunk

// CTA = (KV head g, tile of QT query tokens, split s of the keys); its rows are the QT x rep (query token, query head
// of the group) pairs.  Keys are walked in tiles of 32 that travel global -> shared memory as asynchronous 16-byte
// copies, ATTC_STAGES tiles deep; a warp owns rows, a lane owns one key of the tile for the scores and HD / 32 output
// dims for the values (fp32 math on the f16 cache, as kernels/attn/fast_v2.cu:12-192; row (m, h) sees keys
// 0 .. pos0 + m).  With S > 1 splits (long contexts: a chunk has few query tiles, the keys supply the parallelism)
// every CTA leaves (m, l, O) partials that k_attn_chunk_merge combines (kernels/attn/flash.cu:236-254 algebra).
constexpr int ATTC_THREADS = 256, ATTC_WARPS = ATTC_THREADS / 32, ATTC_TK = 32, ATTC_STAGES = 4;
constexpr int ATTC_ROWS_MAX = 32;  // rows per CTA: 4 per warp
inline size_t attn_chunk_smem(int hd) {
    return sizeof(float) * ATTC_ROWS_MAX * hd + (size_t)ATTC_STAGES * (2 * ATTC_TK * (hd + 8) + 2 * ATTC_TK * hd);
}

struct AttnChunkArgs {
    const float* q;   // [M][n_head * hd]
    const unsigned short *kc, *vc;  // layer base [max_seq][kvdim]
    float* out;       // [M][n_head * hd]
    float* partial;   // [M * n_head][S][2 + hd] when S > 1
    int M, QT, S, n_head, n_kv, pos0, kvdim, ldq;
    float scale;
};

template <int HD>
__global__ void __launch_bounds__(ATTC_THREADS) k_attn_chunk(AttnChunkArgs a) {
    constexpr int KROW = HD + 8, DPL = HD / 32, RPW = ATTC_ROWS_MAX / ATTC_WARPS, CPR = HD / 8;
    extern __shared__ __align__(128) unsigned char attc_smem[];
    float (*q_s)[HD] = reinterpret_cast<float (*)[HD]>(attc_smem);
    constexpr size_t STAGE_B = 2 * ATTC_TK * KROW + 2 * ATTC_TK * HD;
    unsigned char* stages = attc_smem + sizeof(float) * ATTC_ROWS_MAX * HD;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.x, rep = a.n_head / a.n_kv, sp = blockIdx.z;
    const int m_first = blockIdx.y * a.QT, qt = min(a.QT, a.M - m_first);
    const int n_rows = qt * rep;
    const int T = a.pos0 + m_first + qt;  // keys the tile's last token sees
    // this split's run of whole key tiles
    const int n_tiles = (T + ATTC_TK - 1) / ATTC_TK, per = (n_tiles + a.S - 1) / a.S;
    const int k0 = min(T, sp * per * ATTC_TK), k1 = min(T, (sp + 1) * per * ATTC_TK);
    auto issue_tile = [&](int tt, int st_) {
        unsigned short* ks = reinterpret_cast<unsigned short*>(stages + (size_t)st_ * STAGE_B);
        unsigned short* vs = ks + ATTC_TK * KROW;
        if (tt < k1)
            for (int i = tid; i < ATTC_TK * CPR; i += ATTC_THREADS) {
                const int row = i / CPR, c8 = i - row * CPR;
                const bool in = tt + row < k1;
                const size_t off = (size_t)(in ? tt + row : k1 - 1) * a.kvdim + (size_t)g * HD + c8 * 8;
                cp_async16(ks + row * KROW + c8 * 8, a.kc + off, in ? 16 : 0);
                cp_async16(vs + row * HD + c8 * 8, a.vc + off, in ? 16 : 0);
            }
        cp_async_commit();
    };
    griddep_wait();
    griddep_launch_dependents();
#pragma unroll
    for (int p = 0; p < ATTC_STAGES - 1; p++) issue_tile(k0 + p * ATTC_TK, p);
    for (int i = tid; i < n_rows * (HD / 4); i += ATTC_THREADS) {
        const int r = i / (HD / 4), c4 = i - r * (HD / 4);
        const int m = m_first + r / rep, h = g * rep + r % rep;
        reinterpret_cast<float4*>(&q_s[r][0])[c4] = reinterpret_cast<const float4*>(a.q + (size_t)m * a.ldq + (size_t)h * HD)[c4];
    }
    float o[RPW][DPL], mx[RPW], ls[RPW];
#pragma unroll
    for (int rr = 0; rr < RPW; rr++) {
        mx[rr] = -1e30f;
        ls[rr] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; d++) o[rr][d] = 0.f;
    }
    int it = 0;
    for (int tt = k0; tt < k1; tt += ATTC_TK, it++) {
        issue_tile(tt + (ATTC_STAGES - 1) * ATTC_TK, (it + ATTC_STAGES - 1) % ATTC_STAGES);
        cp_async_wait_group<ATTC_STAGES - 1>();
        __syncthreads();
        const unsigned short* k_s = reinterpret_cast<const unsigned short*>(stages + (size_t)(it % ATTC_STAGES) * STAGE_B);
        const unsigned short* v_s = k_s + ATTC_TK * KROW;
#pragma unroll
        for (int rr = 0; rr < RPW; rr++) {
            const int r = warp * RPW + rr;
            if (r >= n_rows) break;  // uniform over the warp
            const int last_key = a.pos0 + m_first + r / rep;  // causal limit of this row
            if (tt > last_key) continue;
            float acc = 0.f;
            const unsigned short* kr = k_s + lane * KROW;
#pragma unroll 4
            for (int d = 0; d < HD; d += 8) {
                const int4 kw = *reinterpret_cast<const int4*>(kr + d);
                const float4 qa = *reinterpret_cast<const float4*>(&q_s[r][d]), qb = *reinterpret_cast<const float4*>(&q_s[r][d + 4]);
                const float2 k0f = __half22float2(*reinterpret_cast<const __half2*>(&kw.x)), k1f = __half22float2(*reinterpret_cast<const __half2*>(&kw.y));
                const float2 k2f = __half22float2(*reinterpret_cast<const __half2*>(&kw.z)), k3f = __half22float2(*reinterpret_cast<const __half2*>(&kw.w));
                acc += qa.x * k0f.x + qa.y * k0f.y;
                acc += qa.z * k1f.x + qa.w * k1f.y;
                acc += qb.x * k2f.x + qb.y * k2f.y;
                acc += qb.z * k3f.x + qb.w * k3f.y;
            }
            const bool seen = tt + lane <= last_key && tt + lane < k1;
            const float sc = seen ? acc * a.scale : -1e30f;
            const float m_new = fmaxf(mx[rr], warp_max(sc));
            const float p = seen ? expf(sc - m_new) : 0.f;
            const float alpha = expf(mx[rr] - m_new);
            ls[rr] = ls[rr] * alpha + warp_sum(p);
            mx[rr] = m_new;
#pragma unroll
            for (int d = 0; d < DPL; d++) o[rr][d] *= alpha;
            const int n_keys = min(min(ATTC_TK, k1 - tt), last_key - tt + 1);
            for (int key = 0; key < n_keys; key++) {
                const float pk = __shfl_sync(TFR_FULL_MASK, p, key);
                if (DPL == 4) {
                    const uint2 vv = *reinterpret_cast<const uint2*>(v_s + key * HD + lane * 4);
                    const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&vv.x)), v1 = __half22float2(*reinterpret_cast<const __half2*>(&vv.y));
                    o[rr][0] += pk * v0.x;
                    o[rr][1] += pk * v0.y;
                    o[rr][2] += pk * v1.x;
                    o[rr][3] += pk * v1.y;
                } else {
#pragma unroll
                    for (int d = 0; d < DPL; d += 2) {
                        const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(v_s + key * HD + lane * DPL + d));
                        o[rr][d] += pk * v0.x;
                        o[rr][d + 1] += pk * v0.y;
                    }
                }
            }
        }
        __syncthreads();  // the stage is refilled at the top of the next iteration
    }
    cp_async_wait_all();
#pragma unroll
    for (int rr = 0; rr < RPW; rr++) {
        const int r = warp * RPW + rr;
        if (r >= n_rows) break;
        const int m = m_first + r / rep, h = g * rep + r % rep;
        if (a.S == 1) {
            const float inv = 1.f / fmaxf(ls[rr], 1e-20f);
            float* dst = a.out + (size_t)m * a.ldq + (size_t)h * HD + lane * DPL;
#pragma unroll
            for (int d = 0; d < DPL; d++) dst[d] = o[rr][d] * inv;
        } else {
            float* dst = a.partial + (((size_t)m * a.n_head + h) * a.S + sp) * (2 + HD);
            if (lane == 0) {
                dst[0] = mx[rr];
                dst[1] = ls[rr];
            }
#pragma unroll
            for (int d = 0; d < DPL; d++) dst[2 + lane * DPL + d] = o[rr][d];
        }
    }
}

// out[row][d] = sum_s exp(m_s - m) O_s[d] / max(sum_s exp(m_s - m) l_s, 1e-20) over the S partials of a row
// (kernels/attn/flash.cu:236-254).  One CTA of hd threads per (token, head) row.
__global__ void k_attn_chunk_merge(const float* partial, float* out, int S, int hd, int n_head, int ldq) {
    const int row = blockIdx.x, d = threadIdx.x;
    griddep_wait();
    griddep_launch_dependents();
    const float* pb = partial + (size_t)row * S * (2 + hd);
    float m = -1e30f;
    for (int s = 0; s < S; s++) m = fmaxf(m, pb[(size_t)s * (2 + hd)]);
    float l = 0.f, acc = 0.f;
    for (int s = 0; s < S; s++) {
        const float* p = pb + (size_t)s * (2 + hd);
        const float al = expf(p[0] - m);
        l += al * p[1];
        acc += al * p[2 + d];
    }
    const int tok = row / n_head, h = row - tok * n_head;
    out[(size_t)tok * ldq + (size_t)h * hd + d] = acc / fmaxf(l, 1e-20f);
}

// ------------------------------------------------------------------ greedy token of every row

// kernels/ops.cu:601-629 (argmax_rows_f32); ties resolve to the lowest index.  A row of the vocabulary's size is too
// long for one CTA: ARGMAX_SLICES CTAs per row fold their slice into a packed key each, the last one to arrive (per
// row counter, zero between launches) folds the keys and writes the token.
constexpr int ARGMAX_SLICES = 32;
__global__ void k_argmax_rows(const float* logits, int V, int* out, unsigned long long* keys, unsigned int* counters) {
    __shared__ unsigned long long sb[32];
    __shared__ int is_last;
    const int m = blockIdx.x, sl = blockIdx.y, tid = threadIdx.x;
    const float* row = logits + (size_t)m * V;
    const int per = (V + ARGMAX_SLICES - 1) / ARGMAX_SLICES, i0 = sl * per, i1 = min(V, i0 + per);
    unsigned long long best = 0ull;
    for (int i = i0 + tid; i < i1; i += blockDim.x) {
        const unsigned long long k = argmax_key(row[i], i);
        best = k > best ? k : best;
    }
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(TFR_FULL_MASK, best, o);
        best = other > best ? other : best;
    }
    if ((tid & 31) == 0) sb[tid >> 5] = best;
    __syncthreads();
    if (tid == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); i++) best = sb[i] > best ? sb[i] : best;
        keys[(size_t)m * ARGMAX_SLICES + sl] = best;
        __threadfence();
        const unsigned int old = atomicAdd(counters + m, 1u);
        is_last = old == ARGMAX_SLICES - 1;
        if (is_last) {
            counters[m] = 0u;
            __threadfence();
            unsigned long long b = 0ull;
            for (int i = 0; i < ARGMAX_SLICES; i++) {
                const unsigned long long k = __ldcg(keys + (size_t)m * ARGMAX_SLICES + i);
                b = k > b ? k : b;
            }
            out[m] = argmax_key_index(b);
        }
    }
}

}  // namespace tfr
