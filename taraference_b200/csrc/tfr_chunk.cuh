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
//                    (K rows, fp32-route V rows, Q8_0 matrices, batches of fewer than five tokens)
//   k_gemm_mma_q4 / k_gemm_mma_q6   the other projections: the same integer sub-block dots as int8 tensor-core MMAs
//                    over CTA tiles of rows x tokens, scale arithmetic on the accumulator fragments
//   k_attn_chunk / k_attn_chunk_mma   causal attention of a tile of query tokens x the query heads of one KV head
//                    over the f16 cache, on CUDA cores / on the tensor cores (head sizes up to 128)
//   k_argmax_rows    greedy token of every row                                        (kernels/ops.cu:601-629)
//
// The projections use the arithmetic of the decode path (Q8 activations, integer block dots), not the reference's
// prefill arithmetic (fp32 activations against dequantised weights): a prompt fed in chunks then leaves the same
// K/V rows of layer 0, bit for bit, and below that the same cache and residual stream up to the summation order of
// attention and of the tensor-core projections' row sums (fp32 rounding, now and then an int8 flip).
#pragma once
#include "tfr_attn.cuh"
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
    // Rows on the fp32 activation route whose tasks fit one pass of the CTA (the usual case: one or two V row pairs per
    // CTA): a thread unpacks the sixteen weights of its task ONCE, keeps them in registers and walks the tokens of the
    // whole launch, every token's normalised vector straight from global memory; with fewer tasks than threads the
    // tokens of a group are shared out among the threads of a task.  Same operations in the same order as
    // q6k_run_dot_f32_g, hence the same bits.
    bool f32_done = false;
    if (fseg.m.data) {
        const int np = fseg.sh.count(cta), pbase = fseg.sh.begin(cta);
        const int per_row = 16 * nb, tn = np * 2 * per_row;
        if (tn <= GEMV_THREADS && tn <= g.pbuf_floats) {
            f32_done = true;
            if (np > 0) {
                const int TG = GEMV_THREADS / tn;  // threads per task
                const int t = tid % tn, tsel = tid / tn;
                const bool on = tid < TG * tn;
                const int row_l = t / per_row, rem = t - row_l * per_row, row_g = 2 * pbase + row_l;
                float w[16];
#pragma unroll
                for (int i = 0; i < 16; i++) w[i] = 0.f;
                if (on && row_g < fseg.m.N) q6k_run_weights_f32(fseg.m, (long long)row_g * nb + (rem >> 4), rem & 15, w);
                for (int m0 = 0; m0 < g.M; m0 += Mt) {
                    const int mt = min(Mt, g.M - m0);
                    if (on)
                        for (int m = tsel; m < mt; m += TG)
                            pbuf[(size_t)m * g.pbuf_floats + t] = q6k_run_dot_weights(w, xn + (size_t)(m0 + m) * K + 256 * (rem >> 4) + 16 * (rem & 15));
                    __syncthreads();
                    for (int item = warp; item < np * mt; item += GEMV_WARPS) {
                        const int m = item / np, rr = item - m * np;
                        const float* a = pbuf + (size_t)m * g.pbuf_floats + (2 * rr) * per_row;
                        float s0 = 0.f, s1 = 0.f;
                        for (int i = lane; i < per_row; i += 32) {
                            s0 += a[i];
                            s1 += a[per_row + i];
                        }
                        s0 = warp_sum(s0);
                        s1 = warp_sum(s1);
                        if (lane == 0) ChunkEpiTok{&epi, m0 + m}.apply(fseg.id_base + pbase + rr, s0, s1);
                    }
                    __syncthreads();
                }
            }
        }
    }
    if (n_jobs == 0 && (f32_done || !fseg.m.data)) return;  // nothing on the Q8 route in this CTA, and no copy was requested
    for (int grp_i = 0; grp_i < n_groups; grp_i++) {
        const int m0 = grp_i * Mt, mt = min(Mt, g.M - m0);
        // the Q8 activations of tokens m0 .. m0 + mt - 1 (a CTA without tiles, e.g. in a launch of fp32-route rows alone,
        // has no use for them)
        if (n_jobs > 0) {
            const int per = g.act_b16 >> 4;
            for (int i = tid; i < mt * per; i += GEMV_THREADS) {
                const int m = i / per, r = i - m * per;
                reinterpret_cast<int4*>(act_s + (size_t)m * g.act_b16)[r] =
                    reinterpret_cast<const int4*>(act_g + (size_t)(m0 + m) * g.act_stride)[r];
            }
        }
        __syncthreads();
        // rows on the fp32 activation route (kernels/gemv.cu:233-264), when their tasks do not fit one pass of the CTA
        // (otherwise they ran before this loop): a task = (row, block, run of 16) and a token per thread and turn
        if (fseg.m.data && !f32_done) {
            const int np = fseg.sh.count(cta), pbase = fseg.sh.begin(cta);
            const int per_row = 16 * nb, ppp = max(1, g.pbuf_floats / (2 * per_row));  // row pairs per pass
            for (int p0 = 0; p0 < np; p0 += ppp) {
                const int pn = min(ppp, np - p0), tn = pn * 2 * per_row;
                for (int tt = tid; tt < tn * mt; tt += GEMV_THREADS) {
                    const int m = tt / tn, t = tt - m * tn;
                    const int row_l = t / per_row, rem = t - row_l * per_row;
                    const int row_g = 2 * (pbase + p0) + row_l;
                    float v = 0.f;
                    if (row_g < fseg.m.N)
                        v = q6k_run_dot_f32_g(fseg.m, (long long)row_g * nb + (rem >> 4), rem >> 4, rem & 15, xn + (size_t)(m0 + m) * K);
                    pbuf[(size_t)m * g.pbuf_floats + t] = v;
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
        // phase A: per-block partials of every token out of the tiles.
        // A CTA with few tiles (the K rows of a prompt chunk, the projections of a verification batch on 2 048 rows)
        // would leave most warps idle while a tile's owner walks it through the tokens one block dot after the other:
        // when every tile sits in a slot of its own for the whole launch (no refills), the warps without a tile help —
        // warp w takes tile w % n_jobs and every H-th token of the group, each (tile, token) pair is still one
        // block_dot into the same partial-sum slot, so the results are the same bits.
        const int H = n_jobs > 0 ? GEMV_WARPS / n_jobs : 0;
        const bool helpers = H >= 2 && n_jobs <= wa && n_groups <= nsw;
        if (helpers) {
            if (warp < H * n_jobs) {
                const int j = warp % n_jobs, q = warp / n_jobs, s = grp_i % nsw;  // the owner (warp j) has one tile: its use grp_i sits in slot grp_i
                const bool is_b = j >= tiles_a;
                const long long f = (long long)(is_b ? tb0 + (j - tiles_a) : ta0 + j) * 32 + lane;
                const bool mine = is_b ? (f >= fb0 && f < fb1) : (f >= fa0 && f < fa1);
                const bool landed = mbar_wait(full + j * nsw + s, 0u);
                if (!landed) {
                    ok = false;
                    if (q == 0) late_slot = s, late_parity = 0u;
                }
                if (mine) {
                    const int off = is_b ? rows_a * nb + (int)(f - fb0) : (int)(f - fa0);
                    const int b = (int)(f % nb);
                    const unsigned char* tile = ring + (size_t)(j * nsw + s) * TB;
                    for (int m = q; m < mt; m += H) {
                        const Act act = act_carve(act_s + (size_t)m * g.act_b16, K, false, false);
                        pbuf[(size_t)m * g.pbuf_floats + off] = landed ? block_dot<true>(BLK{}, tile, lane, act, b, nb, nullptr) : 0.f;
                    }
                }
            }
        } else
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

// ------------------------------------------------------------------ the chunk GEMM on the tensor cores (Q4_K)

// CTA tile = 16 * RG rows x 64 tokens, k-loop over the 256-weight blocks, both operands staged in shared memory three
// or four k steps deep by 16-byte asynchronous copies: the 144-byte block of (row r, block b) is nine pieces of the tiled layout, the
// tokens' int8 groups of block b are sixteen pieces of their activation record, their group scales and scaled sums four
// more.  A warp owns 16 rows and NBW blocks of eight tokens.  The sub-block dots I_j = sum nibble * q8 (kernels/gemv.cu:
// 71-130) run as m16n8k32 u8 x s8 MMAs — the low nibbles of a 32-byte stretch are sub-block 2 t, the high nibbles, left
// in place and shifted out of the sum afterwards, sub-block 2 t + 1 — and are the exact integers of block_dot; the scale
// arithmetic runs on the accumulator fragments (a lane holds two rows x two tokens), block partials d * acc - dmin *
// accm are summed along k in registers.  That order of a row's sum differs from reduce_rows' butterfly: results agree
// with the decode kernels' to fp32 rounding, not bit for bit.
constexpr int GM_MT = 64;         // tokens per CTA tile (16 for batches of up to 16 tokens)
constexpr int GM_ASTRIDE = 160;   // bytes per staged Q4_K block (144 + 16): 8 words modulo 32, four rows' 8-byte reads of four lanes each fill the banks
constexpr int GM4_BSTRIDE = 288;  // bytes per staged token in the Q4_K kernel (256 int8 + 32): 8 words modulo 32 as well
constexpr int GM_BSTRIDE = 272;   // bytes per staged token in the Q6_K kernel (256 int8 + 16): 4 words modulo 32 for its 4-byte reads
constexpr int GM_THREADS = 256;
constexpr int GEMM_MMA_MIN_TOKENS = 5;   // smaller batches keep the dp4a kernel
inline size_t gemm_mma_stage_bytes(int rg, bool zip, int mt) { return (size_t)rg * 16 * GM_ASTRIDE * (zip ? 2 : 1) + (size_t)mt * GM4_BSTRIDE + (size_t)mt * 64; }
// Stages of the copy pipeline: the 16-row tiles do little per k step and need the copies of three steps in flight to hide
// a trip to L2; the others take three stages (one barrier per k step).
__host__ __device__ constexpr int gemm_mma_stages(int rg) { return rg == 1 ? 4 : 3; }
inline size_t gemm_mma_smem(int rg, bool zip, int mt) { return gemm_mma_stages(rg) * gemm_mma_stage_bytes(rg, zip, mt); }

__device__ __forceinline__ void mma_16832_u8s8(int (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ZIP: two matrices of the same shape (gate, up), epilogue apply(row, gate, up); otherwise one matrix and the
// pair-ordered epilogues (store / Q, K rows with RoPE), whose two rows meet by a shuffle.
template <int RG, bool ZIP, int MT>
__global__ void __launch_bounds__(GM_THREADS, 2)
k_gemm_mma_q4(const unsigned char* act_g, size_t act_stride, Mat A1, Mat B2, int id_base1, int id_base2, ChunkEpi epi, int M, int m_base) {
    constexpr int NBW = MT * RG / 64;            // 8-token blocks per warp: 8 warps = RG row groups x (8 / RG) token parts of MT * RG / 8 tokens
    static_assert(NBW >= 1, "a token part holds at least one block of eight tokens");
    constexpr int NMAT = ZIP ? 2 : 1;
    constexpr int TB = Q4_TILE_BYTES;
    extern __shared__ __align__(128) unsigned char gm_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
    // Without ZIP a second matrix of the same K may follow the first in the grid (the K rows behind the Q rows: one launch
    // instead of two): a CTA's rows lie in one of them.
    const int tiles1 = (A1.N + RG * 16 - 1) / (RG * 16);
    const bool second = !ZIP && B2.data != nullptr && (int)blockIdx.x >= tiles1;
    const Mat A = second ? B2 : A1;
    const int id_base = second ? id_base2 : id_base1;
    const int K = A.K, nb = A.nb;
    const int row0 = (second ? (int)blockIdx.x - tiles1 : (int)blockIdx.x) * RG * 16;
    const size_t a_bytes = (size_t)RG * 16 * GM_ASTRIDE, stage_b = a_bytes * NMAT + (size_t)MT * GM4_BSTRIDE + (size_t)MT * 64;
    const int mt = min(MT, M - m_base);       // tokens of this launch's token tile
    const unsigned char* act_t = act_g + (size_t)m_base * act_stride;
    auto stage_a = [&](int st_, int mat) { return gm_smem + (size_t)st_ * stage_b + (size_t)mat * a_bytes; };
    auto stage_q = [&](int st_) { return gm_smem + (size_t)st_ * stage_b + a_bytes * NMAT; };
    auto stage_s = [&](int st_) { return reinterpret_cast<float*>(gm_smem + (size_t)st_ * stage_b + a_bytes * NMAT + (size_t)MT * GM4_BSTRIDE); };
    constexpr int NST = gemm_mma_stages(RG);
    auto issue = [&](int b, int st_) {
        if (b >= nb) {
            cp_async_commit();  // an empty group keeps the count of the wait below
            return;
        }
#pragma unroll
        for (int mat = 0; mat < NMAT; mat++) {
            const uint8_t* data = mat ? B2.data : A.data;
            unsigned char* dst = stage_a(st_, mat);
            for (int i = tid; i < RG * 16 * 9; i += GM_THREADS) {
                const int r = i / 9, piece = i - r * 9;
                const long long f = (long long)min(row0 + r, A.N - 1) * nb + b;  // rows past the matrix repeat its last row
                cp_async16(dst + r * GM_ASTRIDE + piece * 16, data + (f >> 5) * TB + piece * 512 + (f & 31) * 16, 16);
            }
        }
        unsigned char* q = stage_q(st_);
        for (int i = tid; i < MT * 16; i += GM_THREADS) {
            const int t = i >> 4, c = i & 15;
            const bool in = t < mt;
            cp_async16(q + t * GM4_BSTRIDE + c * 16, act_t + (size_t)(in ? t : 0) * act_stride + ((size_t)c * nb + b) * 16, in ? 16 : 0);
        }
        float* sc = stage_s(st_);
        for (int i = tid; i < MT * 4; i += GM_THREADS) {
            const int t = i >> 2, part = i & 3;  // parts 0, 1: group scales d8[8 b ..]; 2, 3: scaled sums ds[8 b ..]
            const bool in = t < mt;
            const unsigned char* rec = act_t + (size_t)(in ? t : 0) * act_stride + K + (part >> 1) * (K / 32) * 4;
            cp_async16(sc + t * 16 + part * 4, rec + (size_t)(8 * b + 4 * (part & 1)) * 4, in ? 16 : 0);
        }
        cp_async_commit();
    };
    griddep_wait();
    griddep_launch_dependents();
    const int rg = warp % RG, tpart = warp / RG;  // row group and token part of this warp
    float total[NMAT][NBW][4];
#pragma unroll
    for (int mat = 0; mat < NMAT; mat++)
#pragma unroll
        for (int n = 0; n < NBW; n++)
#pragma unroll
            for (int i = 0; i < 4; i++) total[mat][n][i] = 0.f;
#pragma unroll
    for (int p = 0; p < NST - 1; p++) issue(p, p);
    for (int b = 0; b < nb; b++) {
        const int st_ = b % NST;
        cp_async_wait_group<NST - 2>();  // this thread's pieces of step b
        __syncthreads();                 // everybody's pieces, and everybody is done with step b - 1
        issue(b + NST - 1, (b + NST - 1) % NST);  // into the stage step b - 1 has just left
        const unsigned char* qs = stage_q(st_);
        const float* scs = stage_s(st_);
#pragma unroll
        for (int mat = 0; mat < NMAT; mat++) {
            const unsigned char* ar = stage_a(st_, mat) + (size_t)(rg * 16 + gq) * GM_ASTRIDE;  // row gq of the group; row gq + 8 is 8 strides on
            // d, dmin and the 6-bit scales and mins of the two rows (kernels/common.cu:40-50, as in block_dot)
            unsigned sc_lo[2], sc_hi[2], m_lo[2], m_hi[2];
            float2 dd[2];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int4 wh = *reinterpret_cast<const int4*>(ar + r * 8 * GM_ASTRIDE);
                const unsigned s0 = (unsigned)wh.y, s1 = (unsigned)wh.z, s2 = (unsigned)wh.w;
                sc_lo[r] = s0 & 0x3f3f3f3fu, sc_hi[r] = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
                m_lo[r] = s1 & 0x3f3f3f3fu, m_hi[r] = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
                dd[r] = __half22float2(*reinterpret_cast<const __half2*>(&wh.x));
            }
#pragma unroll
            for (int n = 0; n < NBW; n++) {
                const int tok0 = (tpart * NBW + n) * 8;
                if (tok0 >= mt) continue;  // the same for the whole warp
                // group scales (d8) and scaled sums (ds) of tokens tok0 + 2 tq, + 1 for the eight sub-blocks
                float d8[2][8], ds[2][8];
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const float4* sp = reinterpret_cast<const float4*>(scs + (tok0 + 2 * tq + c) * 16);
                    const float4 x0 = sp[0], x1 = sp[1], y0 = sp[2], y1 = sp[3];
                    d8[c][0] = x0.x, d8[c][1] = x0.y, d8[c][2] = x0.z, d8[c][3] = x0.w, d8[c][4] = x1.x, d8[c][5] = x1.y, d8[c][6] = x1.z, d8[c][7] = x1.w;
                    ds[c][0] = y0.x, ds[c][1] = y0.y, ds[c][2] = y0.z, ds[c][3] = y0.w, ds[c][4] = y1.x, ds[c][5] = y1.y, ds[c][6] = y1.z, ds[c][7] = y1.w;
                }
                // The order of a sub-block's 32 products is free: MMA k slots 4 tq .. and 16 + 4 tq .. take elements
                // 8 tq .. 8 tq + 3 and 8 tq + 4 .. 8 tq + 7, so a lane's two weight words and two activation words are
                // one 8-byte read each.
                const unsigned char* qt = qs + (size_t)(tok0 + gq) * GM4_BSTRIDE + 8 * tq;  // B operand: token tok0 + gq
                float acc[4] = {0.f, 0.f, 0.f, 0.f}, accm[4] = {0.f, 0.f, 0.f, 0.f};  // [0], [1]: row gq, tokens 2 tq, + 1; [2], [3]: row gq + 8
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    const uint2 wa = *reinterpret_cast<const uint2*>(ar + (1 + 2 * t) * 16 + tq * 8);                   // row gq
                    const uint2 wb = *reinterpret_cast<const uint2*>(ar + 8 * GM_ASTRIDE + (1 + 2 * t) * 16 + tq * 8);  // row gq + 8
                    const unsigned w[4] = {wa.x, wb.x, wa.y, wb.y};
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const int j = 2 * t + half;
                        const unsigned mask = half ? 0xf0f0f0f0u : 0x0f0f0f0fu;
                        const unsigned af[4] = {w[0] & mask, w[1] & mask, w[2] & mask, w[3] & mask};
                        const uint2 bw = *reinterpret_cast<const uint2*>(qt + j * 32);
                        const unsigned b0 = bw.x, b1 = bw.y;
                        int c[4] = {0, 0, 0, 0};
                        mma_16832_u8s8(c, af, b0, b1);
                        if (half) {
#pragma unroll
                            for (int i = 0; i < 4; i++) c[i] >>= 4;  // the high nibbles were multiplied as nibble * 16
                        }
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const int scj = ((j < 4 ? sc_lo[r] : sc_hi[r]) >> (8 * (j & 3))) & 0xff;
                            const float mj = i2f_small((int)(((j < 4 ? m_lo[r] : m_hi[r]) >> (8 * (j & 3))) & 0xff));
#pragma unroll
                            for (int cc = 0; cc < 2; cc++) {
                                acc[2 * r + cc] = fmaf(d8[cc][j], i2f_small(c[2 * r + cc] * scj), acc[2 * r + cc]);
                                accm[2 * r + cc] = fmaf(ds[cc][j], mj, accm[2 * r + cc]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < 2; r++)
#pragma unroll
                    for (int cc = 0; cc < 2; cc++) total[mat][n][2 * r + cc] += dd[r].x * acc[2 * r + cc] - dd[r].y * accm[2 * r + cc];
            }
        }
    }
    cp_async_wait_all();
    // ---- epilogue: a lane holds rows gq, gq + 8 of its group x tokens 2 tq, 2 tq + 1 of its token blocks
#pragma unroll
    for (int n = 0; n < NBW; n++) {
        const int tok0 = (tpart * NBW + n) * 8;
        if (tok0 >= mt) continue;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int row = row0 + rg * 16 + gq + 8 * r;
            if (ZIP) {
#pragma unroll
                for (int cc = 0; cc < 2; cc++) {
                    const int t = tok0 + 2 * tq + cc;
                    if (row < A.N && t < mt) ChunkEpiTok{&epi, m_base + t}.apply(id_base + row, total[0][n][2 * r + cc], total[NMAT - 1][n][2 * r + cc]);
                }
            } else {
                // rows 2 p and 2 p + 1 sit in lanes gq and gq ^ 1: the even lane takes token 2 tq, the odd one 2 tq + 1
                const float mine0 = total[0][n][2 * r], mine1 = total[0][n][2 * r + 1];
                const float other0 = __shfl_xor_sync(TFR_FULL_MASK, mine0, 4), other1 = __shfl_xor_sync(TFR_FULL_MASK, mine1, 4);
                const bool odd = gq & 1;
                const int t = tok0 + 2 * tq + (odd ? 1 : 0), row_even = row & ~1;
                const float x0 = odd ? other1 : mine0, x1 = odd ? mine1 : other0;
                if (row_even < A.N && t < mt) ChunkEpiTok{&epi, m_base + t}.apply(id_base + (row_even >> 1), x0, x1);
            }
        }
    }
}

// Launches k_gemm_mma_q4 for one matrix or two in a row (pair-ordered epilogues) or a gate / up pair (ZIP).  Row tiles of 64 when
// that still gives every SM a CTA, of 16 otherwise (the output and down projections have 2 048 rows).
inline cudaError_t launch_gemm_mma_q4(cudaStream_t stream, int sms, const unsigned char* act_g, size_t act_stride, int M, const RowJob& ja,
                                      const RowJob& jb, const ChunkEpi& epi) {
    const bool zip = epi.kind == CEPI_SILU;
    const bool two = !zip && jb.m.data != nullptr;  // a second matrix behind the first (Q rows, then K rows)
    const int rows = ja.m.N + (two ? jb.m.N : 0);
    const bool big = (rows + 63) / 64 >= sms;
    const bool few = M <= 16 && big;  // a token tile of 16: every warp of a 64-row CTA has a token block
    // 64-row tiles that do not divide evenly over the SMs leave some SMs twice the rows of the others (11 008 rows: 172
    // tiles on 148 SMs): 32-row tiles then even the load out at a little more unpacking per MMA
    const int t64 = (rows + 63) / 64, t32 = (rows + 31) / 32;
    const bool mid = big && !few && ((t32 + sms - 1) / sms) * 32 < ((t64 + sms - 1) / sms) * 64;
    const int rg = mid ? 2 : big ? 4 : 1, mt_tile = few ? 16 : GM_MT;
    const int tile_rows = 16 * rg;
    const dim3 grid((ja.m.N + tile_rows - 1) / tile_rows + (two ? (jb.m.N + tile_rows - 1) / tile_rows : 0)), block(GM_THREADS);
    const size_t smem = gemm_mma_smem(rg, zip, mt_tile);
    const Mat m2 = (zip || two) ? jb.m : Mat{};
    const int id1 = ja.id_base, id2 = two ? jb.id_base : 0;
    for (int m_base = 0; m_base < M; m_base += mt_tile) {
        cudaError_t r;
        if (zip) r = few   ? launch_pdl(k_gemm_mma_q4<4, true, 16>, grid, block, smem, stream, act_g, act_stride, ja.m, m2, id1, id2, epi, M, m_base)
                     : mid ? launch_pdl(k_gemm_mma_q4<2, true, 64>, grid, block, smem, stream, act_g, act_stride, ja.m, m2, id1, id2, epi, M, m_base)
                     : big ? launch_pdl(k_gemm_mma_q4<4, true, 64>, grid, block, smem, stream, act_g, act_stride, ja.m, m2, id1, id2, epi, M, m_base)
                           : launch_pdl(k_gemm_mma_q4<1, true, 64>, grid, block, smem, stream, act_g, act_stride, ja.m, m2, id1, id2, epi, M, m_base);
        else r = few   ? launch_pdl(k_gemm_mma_q4<4, false, 16>, grid, block, smem, stream, act_g, act_stride, ja.m, m2, id1, id2, epi, M, m_base)
                 : mid ? launch_pdl(k_gemm_mma_q4<2, false, 64>, grid, block, smem, stream, act_g, act_stride, ja.m, m2, id1, id2, epi, M, m_base)
                 : big ? launch_pdl(k_gemm_mma_q4<4, false, 64>, grid, block, smem, stream, act_g, act_stride, ja.m, m2, id1, id2, epi, M, m_base)
                       : launch_pdl(k_gemm_mma_q4<1, false, 64>, grid, block, smem, stream, act_g, act_stride, ja.m, m2, id1, id2, epi, M, m_base);
        if (r != cudaSuccess) return r;
    }
    return cudaSuccess;
}

// ------------------------------------------------------------------ the chunk GEMM on the tensor cores (Q6_K)

// The same frame for Q6_K matrices (down, the head): 64 rows x 64 tokens per CTA, eight warps = four row groups x two
// token halves, and optionally a part of the k range (grid.y parts: a matrix of 2 048 rows has only 32 row tiles).
// A block's sixteen scale groups are one m16n8k16 s8 x s8 MMA each: the 6-bit values are assembled from the ql nibbles
// and qh bit pairs as in block_dot(BlockQ6) (kernels/gemv.cu:302-337), the accumulators start at -32 * sum(q8) of the
// group, so the MMA leaves the exact J = sum (q6 - 32) * q8.  With k parts the CTA stores its partial sums and
// k_gemm_splitk_finish adds the parts in a fixed order and runs the epilogue.
constexpr int GM6_ASTRIDE = 240;  // 13 pieces + the d pair + padding: eight rows' words hit 32 different banks
inline size_t gemm_mma_q6_smem(int mt) { return 2 * ((size_t)64 * GM6_ASTRIDE + (size_t)mt * GM_BSTRIDE + (size_t)mt * 96); }

__device__ __forceinline__ void mma_16816_s8(int (&c)[4], unsigned a0, unsigned a1, unsigned b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

template <int MT>
__global__ void __launch_bounds__(GM_THREADS, 2)
k_gemm_mma_q6(const unsigned char* act_g, size_t act_stride, Mat A, int id_base, ChunkEpi epi, int M, float* partial) {
    constexpr int RG = 4, NBW = MT / 16, TB = Q6_TILE_BYTES;  // eight warps = four row groups x two token halves of MT / 2 tokens
    extern __shared__ __align__(128) unsigned char gm_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
    const int K = A.K, nb = A.nb;
    const int row0 = blockIdx.x * RG * 16;
    const int kparts = gridDim.y, kp = blockIdx.y;
    const int b_begin = (int)((long long)nb * kp / kparts), b_end = (int)((long long)nb * (kp + 1) / kparts);
    constexpr size_t a_bytes = (size_t)RG * 16 * GM6_ASTRIDE, q_bytes = (size_t)MT * GM_BSTRIDE, stage_b = a_bytes + q_bytes + (size_t)MT * 96;
    const int mt = min(MT, M);
    auto stage_a = [&](int st_) { return gm_smem + (size_t)st_ * stage_b; };
    auto stage_q = [&](int st_) { return gm_smem + (size_t)st_ * stage_b + a_bytes; };
    auto stage_x = [&](int st_) { return gm_smem + (size_t)st_ * stage_b + a_bytes + q_bytes; };  // per token: 8 floats d8, 16 ints -32 * S16
    auto issue = [&](int b, int st_) {
        unsigned char* dst = stage_a(st_);
        for (int i = tid; i < RG * 16 * 14; i += GM_THREADS) {
            const int r = i / 14, piece = i - r * 14;
            const long long f = (long long)min(row0 + r, A.N - 1) * nb + b;  // rows past the matrix repeat its last row
            const uint8_t* tile = A.data + (f >> 5) * TB;
            if (piece < 13) cp_async16(dst + r * GM6_ASTRIDE + piece * 16, tile + piece * 512 + (f & 31) * 16, 16);
            else cp_async4(dst + r * GM6_ASTRIDE + 208, tile + Q6_PIECES * 512 + ((f & 31) & ~1) * 2);  // d of this block and its neighbour
        }
        unsigned char* q = stage_q(st_);
        for (int i = tid; i < MT * 16; i += GM_THREADS) {
            const int t = i >> 4, c = i & 15;
            const bool in = t < mt;
            cp_async16(q + t * GM_BSTRIDE + c * 16, act_g + (size_t)(in ? t : 0) * act_stride + ((size_t)c * nb + b) * 16, in ? 16 : 0);
        }
        unsigned char* x = stage_x(st_);
        for (int i = tid; i < MT * 6; i += GM_THREADS) {
            const int t = i / 6, part = i - t * 6;  // parts 0, 1: d8[8 b ..]; 2 .. 5: s16n[16 b ..]
            const bool in = t < mt;
            const unsigned char* rec = act_g + (size_t)(in ? t : 0) * act_stride + K;
            const unsigned char* src = part < 2 ? rec + (size_t)(8 * b + 4 * part) * 4 : rec + (size_t)(K / 32) * 8 + (size_t)(16 * b + 4 * (part - 2)) * 4;
            cp_async16(x + t * 96 + part * 16, src, in ? 16 : 0);
        }
        cp_async_commit();
    };
    griddep_wait();
    griddep_launch_dependents();
    const int rg = warp & 3, tpart = warp >> 2;
    float total[NBW][4];
#pragma unroll
    for (int n = 0; n < NBW; n++)
#pragma unroll
        for (int i = 0; i < 4; i++) total[n][i] = 0.f;
    if (b_begin < b_end) issue(b_begin, 0);
    for (int b = b_begin; b < b_end; b++) {
        const int st_ = (b - b_begin) & 1;
        if (b + 1 < b_end) {
            issue(b + 1, st_ ^ 1);
            cp_async_wait_group<1>();
        } else {
            cp_async_wait_all();
        }
        __syncthreads();
        const unsigned char* qs = stage_q(st_);
        const unsigned char* xs = stage_x(st_);
        const unsigned char* ar = stage_a(st_) + (size_t)(rg * 16 + gq) * GM6_ASTRIDE;  // row gq of the group; row gq + 8 is 8 strides on
        int4 wsc[2];
        float dw[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            wsc[r] = *reinterpret_cast<const int4*>(ar + r * 8 * GM6_ASTRIDE + 12 * 16);
            const unsigned dpair = *reinterpret_cast<const unsigned*>(ar + r * 8 * GM6_ASTRIDE + 208);
            const long long f = (long long)min(row0 + rg * 16 + gq + 8 * r, A.N - 1) * nb + b;
            dw[r] = f16_to_f32((unsigned short)((f & 1) ? dpair >> 16 : dpair & 0xffffu));
        }
#pragma unroll
        for (int n = 0; n < NBW; n++) {
            const int tok0 = (tpart * NBW + n) * 8;
            if (tok0 >= mt) continue;  // the same for the whole warp
            float d8[2][8];
            int s16[2][16];
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const int4* xp = reinterpret_cast<const int4*>(xs + (size_t)(tok0 + 2 * tq + c) * 96);
                const int4 x0 = xp[0], x1 = xp[1];
                d8[c][0] = __int_as_float(x0.x), d8[c][1] = __int_as_float(x0.y), d8[c][2] = __int_as_float(x0.z), d8[c][3] = __int_as_float(x0.w);
                d8[c][4] = __int_as_float(x1.x), d8[c][5] = __int_as_float(x1.y), d8[c][6] = __int_as_float(x1.z), d8[c][7] = __int_as_float(x1.w);
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int4 y = xp[2 + k];
                    s16[c][4 * k] = y.x, s16[c][4 * k + 1] = y.y, s16[c][4 * k + 2] = y.z, s16[c][4 * k + 3] = y.w;
                }
            }
            const unsigned char* qt = qs + (size_t)(tok0 + gq) * GM_BSTRIDE + 4 * tq;  // B operand: token tok0 + gq
            float acc[4] = {0.f, 0.f, 0.f, 0.f};  // [0], [1]: row gq, tokens 2 tq, + 1; [2], [3]: row gq + 8
#pragma unroll
            for (int nn = 0; nn < 2; nn++)
#pragma unroll
                for (int is = 0; is < 2; is++) {
                    unsigned la[2], lb[2], hw[2];
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const unsigned char* rowp = ar + r * 8 * GM6_ASTRIDE + tq * 4;
                        la[r] = *reinterpret_cast<const unsigned*>(rowp + (4 * nn + is) * 16);
                        lb[r] = *reinterpret_cast<const unsigned*>(rowp + (4 * nn + 2 + is) * 16);
                        hw[r] = *reinterpret_cast<const unsigned*>(rowp + (8 + 2 * nn + is) * 16);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int c = 8 * nn + 2 * j + is;  // the scale group: elements 16 c .. 16 c + 15 of the block
                        unsigned af[2];
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const unsigned nibw = (j & 1) ? lb[r] : la[r];
                            af[r] = ((nibw >> (4 * (j >> 1))) & 0x0f0f0f0fu) | (((hw[r] >> (2 * j)) << 4) & 0x30303030u);
                        }
                        const unsigned b0 = *reinterpret_cast<const unsigned*>(qt + c * 16);
                        int cj[4] = {s16[0][c], s16[1][c], s16[0][c], s16[1][c]};
                        mma_16816_s8(cj, af[0], af[1], b0);
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const int w = r ? (c < 4 ? wsc[1].x : c < 8 ? wsc[1].y : c < 12 ? wsc[1].z : wsc[1].w)
                                            : (c < 4 ? wsc[0].x : c < 8 ? wsc[0].y : c < 12 ? wsc[0].z : wsc[0].w);
                            const float cf = i2f_small((int)(signed char)((w >> (8 * (c & 3))) & 0xff));
#pragma unroll
                            for (int cc = 0; cc < 2; cc++) acc[2 * r + cc] = fmaf(cf * d8[cc][c >> 1], i2f_small(cj[2 * r + cc]), acc[2 * r + cc]);
                        }
                    }
                }
#pragma unroll
            for (int r = 0; r < 2; r++)
#pragma unroll
                for (int cc = 0; cc < 2; cc++) total[n][2 * r + cc] += dw[r] * acc[2 * r + cc];
        }
        __syncthreads();
    }
#pragma unroll
    for (int n = 0; n < NBW; n++) {
        const int tok0 = (tpart * NBW + n) * 8;
        if (tok0 >= mt) continue;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int row = row0 + rg * 16 + gq + 8 * r;
            if (kparts > 1) {
#pragma unroll
                for (int cc = 0; cc < 2; cc++) {
                    const int t = tok0 + 2 * tq + cc;
                    if (row < A.N && t < mt) partial[((size_t)kp * M + t) * A.N + row] = total[n][2 * r + cc];
                }
            } else {
                const float mine0 = total[n][2 * r], mine1 = total[n][2 * r + 1];
                const float other0 = __shfl_xor_sync(TFR_FULL_MASK, mine0, 4), other1 = __shfl_xor_sync(TFR_FULL_MASK, mine1, 4);
                const bool odd = gq & 1;
                const int t = tok0 + 2 * tq + (odd ? 1 : 0), row_even = row & ~1;
                const float x0 = odd ? other1 : mine0, x1 = odd ? mine1 : other0;
                if (row_even < A.N && t < mt) ChunkEpiTok{&epi, t}.apply(id_base + (row_even >> 1), x0, x1);
            }
        }
    }
}

// Adds the k parts of k_gemm_mma_q6 in their order and runs the pair-ordered epilogue: one thread per (token, row pair).
__global__ void k_gemm_splitk_finish(const float* partial, int kparts, int M, int N, int id_base, ChunkEpi epi) {
    griddep_wait();
    griddep_launch_dependents();
    const int pairs = (N + 1) >> 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * pairs) return;
    const int t = i / pairs, p = i - t * pairs;
    float x0 = 0.f, x1 = 0.f;
    for (int k = 0; k < kparts; k++) {
        const float* src = partial + ((size_t)k * M + t) * N + 2 * p;
        x0 += src[0];
        if (2 * p + 1 < N) x1 += src[1];
    }
    ChunkEpiTok{&epi, t}.apply(id_base + p, x0, x1);
}

// ws: scratch for the k parts (ws_floats floats; nullptr: no split).
inline cudaError_t launch_gemm_mma_q6(cudaStream_t stream, int sms, const unsigned char* act_g, size_t act_stride, int M, const RowJob& ja,
                                      const ChunkEpi& epi, float* ws, size_t ws_floats) {
    const int rows = ja.m.N, tiles = (rows + 63) / 64;
    int kparts = 1;
    if (ws && tiles < sms) {
        kparts = std::min(std::min(4, ja.m.nb), std::max(1, sms / tiles));
        if ((size_t)kparts * M * rows > ws_floats) kparts = 1;
    }
    cudaError_t r = M <= 16 ? launch_pdl(k_gemm_mma_q6<16>, dim3(tiles, kparts), dim3(GM_THREADS), gemm_mma_q6_smem(16), stream, act_g, act_stride,
                                         ja.m, ja.id_base, epi, M, ws)
                            : launch_pdl(k_gemm_mma_q6<64>, dim3(tiles, kparts), dim3(GM_THREADS), gemm_mma_q6_smem(64), stream, act_g, act_stride,
                                         ja.m, ja.id_base, epi, M, ws);
    if (r != cudaSuccess || kparts == 1) return r;
    const int items = M * ((rows + 1) / 2);
    return launch_pdl(k_gemm_splitk_finish, dim3((items + 255) / 256), dim3(256), (size_t)0, stream, (const float*)ws, kparts, M, rows, ja.id_base, epi);
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

// The same CTA shape on the tensor cores (head sizes up to 128, prompt chunks): a warp owns 16 rows — (query token,
// query head) pairs of one KV head — and walks every key of the split, eight warps share the staged tiles.  Scores
// S[16 rows x 64 keys] = Q K^T and O[16 rows x HD] += P V run as m16n8k16 MMAs (f16 operands, fp32 accumulators) the
// way k_attn_decode's staged route does: K and V are f16 in the cache (exact), q and the softmax weights are fp32 and
// travel as two f16 terms (split2_f16x2), every 16-term product sum starts from zero and joins the running sum by a
// round-to-nearest add.  The softmax runs on the accumulator fragments (a lane holds two rows x two keys of every 8-key block), whose
// layout is also that of the A operand of P V, so the weights never leave registers.
constexpr int ATTM_TK = 64, ATTM_STAGES = 4, ATTM_ROWS = 128;
inline size_t attn_chunk_mma_smem(int hd) { return (size_t)ATTM_STAGES * 2 * ATTM_TK * (hd + 8) * 2; }

template <int HD>
__global__ void __launch_bounds__(ATTC_THREADS) k_attn_chunk_mma(AttnChunkArgs a) {
    constexpr int KROW = HD + 8, CPR = HD / 8, KS = HD / 16, NB = HD / 8, KB = ATTM_TK / 16;
    extern __shared__ __align__(128) unsigned char attc_smem[];
    constexpr size_t STAGE_B = 2 * (size_t)ATTM_TK * KROW * 2;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
    const int g = blockIdx.x, rep = a.n_head / a.n_kv, sp = blockIdx.z;
    const int m_first = blockIdx.y * a.QT, qt = min(a.QT, a.M - m_first);
    const int n_rows = qt * rep;
    const int T = a.pos0 + m_first + qt;  // keys the tile's last token sees
    const int n_tiles = (T + ATTM_TK - 1) / ATTM_TK, per = (n_tiles + a.S - 1) / a.S;
    const int k0 = min(T, sp * per * ATTM_TK), k1 = min(T, (sp + 1) * per * ATTM_TK);
    auto k_stage = [&](int st_) { return reinterpret_cast<unsigned short*>(attc_smem + (size_t)st_ * STAGE_B); };
    auto v_stage = [&](int st_) { return k_stage(st_) + ATTM_TK * KROW; };
    auto issue_tile = [&](int tt, int st_) {
        unsigned short* ks = k_stage(st_);
        unsigned short* vs = v_stage(st_);
        if (tt < k1)
            for (int i = tid; i < ATTM_TK * CPR; i += ATTC_THREADS) {
                const int row = i / CPR, c8 = i - row * CPR;
                const bool in = tt + row < k1;
                const size_t off = (size_t)(in ? tt + row : k1 - 1) * a.kvdim + (size_t)g * HD + c8 * 8;
                cp_async16(ks + row * KROW + c8 * 8, a.kc + off, in ? 16 : 0);  // rows past the split arrive as zeros
                cp_async16(vs + row * KROW + c8 * 8, a.vc + off, in ? 16 : 0);
            }
        cp_async_commit();
    };
    griddep_wait();
    griddep_launch_dependents();
#pragma unroll
    for (int p = 0; p < ATTM_STAGES - 1; p++) issue_tile(k0 + p * ATTM_TK, p);
    // rows gq and gq + 8 of this warp's 16; a row past the tile's last one repeats row 0 and is never written back
    const int r_a = warp * 16 + gq, r_b = r_a + 8;
    const bool row_a = r_a < n_rows, row_b = r_b < n_rows, warp_on = warp * 16 < n_rows;
    const int ra = row_a ? r_a : 0, rb = row_b ? r_b : 0;
    const int last_a = a.pos0 + m_first + ra / rep, last_b = a.pos0 + m_first + rb / rep;  // causal limits
    // the warp's rows are in token order: its last valid row sees the most keys
    const int last_w = a.pos0 + m_first + (min(n_rows, warp * 16 + 16) - 1) / rep;
    // A fragments of Q (16 rows x 16 dims per step): [0] row gq dims 2 tq, + 1; [1] row gq + 8; [2], [3] the same, dims + 8
    unsigned qh[KS][4], ql[KS][4];
    {
        const float* qa = a.q + (size_t)(m_first + ra / rep) * a.ldq + (size_t)(g * rep + ra % rep) * HD;
        const float* qb = a.q + (size_t)(m_first + rb / rep) * a.ldq + (size_t)(g * rep + rb % rep) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ks++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const float2 va = warp_on ? *reinterpret_cast<const float2*>(qa + 16 * ks + 2 * tq + 8 * j) : make_float2(0.f, 0.f);
                const float2 vb = warp_on ? *reinterpret_cast<const float2*>(qb + 16 * ks + 2 * tq + 8 * j) : make_float2(0.f, 0.f);
                split2_f16x2(va.x, va.y, qh[ks][2 * j], ql[ks][2 * j]);
                split2_f16x2(vb.x, vb.y, qh[ks][2 * j + 1], ql[ks][2 * j + 1]);
            }
    }
    float oacc[NB][4];  // [0], [1] = row gq, dims 8 nb + 2 tq, + 1; [2], [3] = row gq + 8
#pragma unroll
    for (int nb = 0; nb < NB; nb++)
#pragma unroll
        for (int i = 0; i < 4; i++) oacc[nb][i] = 0.f;
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};  // rows gq, gq + 8 (l: this lane's keys only)
    // lane addresses of the ldmatrix reads inside a 16-key block (matrix mi = lane / 8, row lane % 8)
    const int mi = lane >> 3, mr = lane & 7;
    const int k_off = ((mi >> 1) * 8 + mr) * KROW + (mi & 1) * 8;  // K as B operand: dims + 0 / + 8 by mi & 1, keys 0-7 / 8-15 by mi >> 1
    const int v_off = ((mi & 1) * 8 + mr) * KROW + (mi >> 1) * 8;  // V as B operand (transposed read): keys by mi & 1, dims + 0 / + 8 by mi >> 1
    int it = 0;
    for (int tt = k0; tt < k1; tt += ATTM_TK, it++) {
        cp_async_wait_group<ATTM_STAGES - 2>();  // this thread's pieces of tile `it`
        __syncthreads();                         // everybody's pieces, and everybody is done with tile it - 1
        issue_tile(tt + (ATTM_STAGES - 1) * ATTM_TK, (it + ATTM_STAGES - 1) % ATTM_STAGES);
        if (!warp_on || tt > last_w) continue;  // the same for the whole warp; barriers are outside
        const int stg = it % ATTM_STAGES;
        // ---- scores of the 64 keys: eight 8-key blocks, fragments [0], [1] = row gq keys 2 tq, + 1; [2], [3] = row gq + 8
        float sacc[2 * KB][4];
#pragma unroll
        for (int nb = 0; nb < 2 * KB; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) sacc[nb][i] = 0.f;
#pragma unroll
        for (int kb = 0; kb < KB; kb++) {
            const unsigned kaddr = smem_u32(k_stage(stg) + kb * 16 * KROW + k_off);
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                unsigned bf[4];  // [0], [1]: keys 0-7 of the block, dims + 0 / + 8; [2], [3]: keys 8-15
                ldsm_x4(bf, kaddr + ks * 32);
                float p0[4] = {0.f, 0.f, 0.f, 0.f}, p1[4] = {0.f, 0.f, 0.f, 0.f};
                mma_16816(p0, ql[ks], bf[0], bf[1]);
                mma_16816(p0, qh[ks], bf[0], bf[1]);
                mma_16816(p1, ql[ks], bf[2], bf[3]);
                mma_16816(p1, qh[ks], bf[2], bf[3]);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    sacc[2 * kb][i] += p0[i];
                    sacc[2 * kb + 1][i] += p1[i];
                }
            }
        }
        // ---- online softmax on the fragments
        float mx_a = -1e30f, mx_b = -1e30f;
#pragma unroll
        for (int nb = 0; nb < 2 * KB; nb++)
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const int key = tt + nb * 8 + 2 * tq + c;
                const bool in = key < k1;
                sacc[nb][c] = (in && key <= last_a) ? sacc[nb][c] * a.scale : -1e30f;
                sacc[nb][2 + c] = (in && key <= last_b) ? sacc[nb][2 + c] * a.scale : -1e30f;
                mx_a = fmaxf(mx_a, sacc[nb][c]);
                mx_b = fmaxf(mx_b, sacc[nb][2 + c]);
            }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(TFR_FULL_MASK, mx_a, 1)), mx_a = fmaxf(mx_a, __shfl_xor_sync(TFR_FULL_MASK, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(TFR_FULL_MASK, mx_b, 1)), mx_b = fmaxf(mx_b, __shfl_xor_sync(TFR_FULL_MASK, mx_b, 2));
        const float mn_a = fmaxf(m_run[0], mx_a), mn_b = fmaxf(m_run[1], mx_b);
        const float al_a = expf(m_run[0] - mn_a), al_b = expf(m_run[1] - mn_b);
        m_run[0] = mn_a, m_run[1] = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int nb = 0; nb < 2 * KB; nb++)
#pragma unroll
            for (int c = 0; c < 2; c++) {
                // a masked score is -1e30: its weight must be zero even while the row's maximum is still -1e30
                const float pa = sacc[nb][c] > -1e29f ? expf(sacc[nb][c] - mn_a) : 0.f;
                const float pb = sacc[nb][2 + c] > -1e29f ? expf(sacc[nb][2 + c] - mn_b) : 0.f;
                sacc[nb][c] = pa, sacc[nb][2 + c] = pb;
                sum_a += pa, sum_b += pb;
            }
        l_run[0] = l_run[0] * al_a + sum_a;
        l_run[1] = l_run[1] * al_b + sum_b;
        if (__any_sync(TFR_FULL_MASK, al_a != 1.f || al_b != 1.f)) {
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                oacc[nb][0] *= al_a, oacc[nb][1] *= al_a;
                oacc[nb][2] *= al_b, oacc[nb][3] *= al_b;
            }
        }
        // ---- O += P V: the score fragments of two adjacent 8-key blocks are the A fragment of a 16-key step
#pragma unroll
        for (int kb = 0; kb < KB; kb++) {
            unsigned ph[4], pl[4];
            split2_f16x2(sacc[2 * kb][0], sacc[2 * kb][1], ph[0], pl[0]);
            split2_f16x2(sacc[2 * kb][2], sacc[2 * kb][3], ph[1], pl[1]);
            split2_f16x2(sacc[2 * kb + 1][0], sacc[2 * kb + 1][1], ph[2], pl[2]);
            split2_f16x2(sacc[2 * kb + 1][2], sacc[2 * kb + 1][3], ph[3], pl[3]);
            const unsigned vaddr = smem_u32(v_stage(stg) + kb * 16 * KROW + v_off);
#pragma unroll
            for (int nb = 0; nb < NB; nb += 2) {
                unsigned bf[4];  // [0], [1]: dims 8 nb .. + 7, keys 0-7 / 8-15; [2], [3]: dims 8 (nb + 1) ..
                ldsm_x4_trans(bf, vaddr + nb * 16);
                float p0[4] = {0.f, 0.f, 0.f, 0.f}, p1[4] = {0.f, 0.f, 0.f, 0.f};
                mma_16816(p0, pl, bf[0], bf[1]);
                mma_16816(p0, ph, bf[0], bf[1]);
                mma_16816(p1, pl, bf[2], bf[3]);
                mma_16816(p1, ph, bf[2], bf[3]);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    oacc[nb][i] += p0[i];
                    oacc[nb + 1][i] += p1[i];
                }
            }
        }
    }
    cp_async_wait_all();
    if (!warp_on) return;
#pragma unroll
    for (int c = 0; c < 2; c++) {
        l_run[c] += __shfl_xor_sync(TFR_FULL_MASK, l_run[c], 1);
        l_run[c] += __shfl_xor_sync(TFR_FULL_MASK, l_run[c], 2);
    }
#pragma unroll
    for (int half = 0; half < 2; half++) {
        if (!(half ? row_b : row_a)) continue;
        const int r = half ? r_b : r_a;
        const int m = m_first + r / rep, h = g * rep + r % rep;
        if (a.S == 1) {
            const float inv = 1.f / fmaxf(l_run[half], 1e-20f);
            float* dst = a.out + (size_t)m * a.ldq + (size_t)h * HD + 2 * tq;
#pragma unroll
            for (int nb = 0; nb < NB; nb++) *reinterpret_cast<float2*>(dst + 8 * nb) = make_float2(oacc[nb][2 * half] * inv, oacc[nb][2 * half + 1] * inv);
        } else {
            float* dst = a.partial + (((size_t)m * a.n_head + h) * a.S + sp) * (2 + HD);
            if (tq == 0) {
                dst[0] = m_run[half];
                dst[1] = l_run[half];
            }
#pragma unroll
            for (int nb = 0; nb < NB; nb++) *reinterpret_cast<float2*>(dst + 2 + 8 * nb + 2 * tq) = make_float2(oacc[nb][2 * half], oacc[nb][2 * half + 1]);
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
