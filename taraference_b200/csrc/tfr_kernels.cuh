// __global__ kernels of the batch-1 decode path and their launch helpers.
#pragma once
#include "tfr_attn.cuh"
#include "tfr_gdn.cuh"
#include "tfr_gemv.cuh"
#include "tfr_tp.cuh"

namespace tfr {

// ------------------------------------------------------------------ epilogues
//
// (EPI_PAIRS / EPI_ZIP are declared in tfr_gemv.cuh.)

// y = W x (+y) (+bias): kernels/gemv.cu:367-373 residual rule (2 = accumulate in place).
struct EpiStore {
    static constexpr int MODE = EPI_PAIRS;
    float* out;
    const float* bias;
    int use_res;
    int n_rows;
    const float* res_smem = nullptr;  // the CTA's residual values, fetched right after the dependency wait
    int res_row0 = 0;
    __device__ void begin(const TokenState*) {}
    // The in-place residual is read long before the epilogue needs it: by then the successor's weight
    // requests already fill the memory system and a plain load would queue behind them.
    __device__ __forceinline__ bool wants_residual() const { return use_res == 2; }
    __device__ __forceinline__ float residual(int row) const { return row < n_rows ? out[row] : 0.f; }
    __device__ __forceinline__ void set_residual(const float* buf, int row0) {
        res_smem = buf;
        res_row0 = row0;
    }
    __device__ __forceinline__ void one(int row, float acc) {
        if (use_res == 2) acc += res_smem ? res_smem[row - res_row0] : out[row];
        if (bias) acc += bias[row];
        out[row] = acc;
    }
    __device__ __forceinline__ void apply(int p, float v0, float v1) {
        one(2 * p, v0);
        if (2 * p + 1 < n_rows) one(2 * p + 1, v1);
    }
    __device__ void end(TokenState*) {}
};

// h = silu(gate.x) * (up.x), kernels/gemv.cu:2570-2574.  Pair p = (gate row p, up row p).
struct EpiSilu {
    static constexpr int MODE = EPI_ZIP;
    float* out;
    __device__ __forceinline__ bool wants_residual() const { return false; }
    __device__ __forceinline__ float residual(int) const { return 0.f; }
    __device__ __forceinline__ void set_residual(const float*, int) {}
    __device__ void begin(const TokenState*) {}
    __device__ __forceinline__ void apply(int p, float gate, float up) {
        out[p] = (gate / (1.f + __expf(-gate))) * up;
    }
    __device__ void end(TokenState*) {}
};

// Fused Q/K/V epilogue: bias, neox RoPE (kernels/ops.cu:348-371) and the f16 KV store
// (kernels/ops.cu:471-486).  Q and K rows were re-ordered at upload so that the RoPE
// partners (i, i + hd/2) of a head are the two rows of a pair; biases likewise.
struct EpiQkv {
    static constexpr int MODE = EPI_PAIRS;
    float* q_out;            // [n_head * hd] natural order
    unsigned short* kc;      // layer base [max_seq][kvdim]
    unsigned short* vc;
    const float* bias;       // [nq + nk + nv] in stored-row order, or nullptr
    int nq, nk, hd, kvdim;
    float theta;
    int pos;
    __device__ void begin(const TokenState* st) {
        if (st) pos = st->pos;
    }
    __device__ __forceinline__ bool wants_residual() const { return false; }
    __device__ __forceinline__ float residual(int) const { return 0.f; }
    __device__ __forceinline__ void set_residual(const float*, int) {}
    __device__ __forceinline__ void apply(int p, float x0, float x1) {
        const int v = 2 * p;
        if (bias) {
            x0 += bias[v];
            x1 += bias[v + 1];
        }
        if (v < nq + nk) {
            const bool isq = v < nq;
            const int vv = isq ? v : v - nq;
            const int head = vv / hd, i = (vv % hd) >> 1, half = hd >> 1;
            const float freq = powf(theta, -2.f * (float)i / (float)hd);
            const float ang = (float)pos * freq;
            const float c = cosf(ang), sn = sinf(ang);
            const float y0 = x0 * c - x1 * sn;
            const float y1 = x0 * sn + x1 * c;
            if (isq) {
                q_out[head * hd + i] = y0;
                q_out[head * hd + i + half] = y1;
            } else {
                unsigned short* kr = kc + (size_t)pos * kvdim + head * hd;
                kr[i] = f32_to_f16_bits_ref(y0);
                kr[i + half] = f32_to_f16_bits_ref(y1);
            }
        } else {
            const int vv = v - nq - nk;
            unsigned short* vr = vc + (size_t)pos * kvdim;
            vr[vv] = f32_to_f16_bits_ref(x0);
            vr[vv + 1] = f32_to_f16_bits_ref(x1);
        }
    }
    __device__ void end(TokenState*) {}
};

// Vocabulary head with the greedy argmax folded in (kernels/ops.cu:573-599 picks the
// maximum; here ties resolve to the lowest index).  The CTA that finishes last publishes
// the token and advances the device-resident decode state, so the next token's first
// kernel can start without the host (the reference reads the argmax back every token,
// crates/core/src/cuda/forward.rs:100-104).
// End of a decode step: record the greedy token and choose the next input — the token itself, or, in a
// verification pass (forward.rs:268-290), the next token the caller supplied.
__device__ __forceinline__ void advance_state(TokenState* st, int tok, int* out_tokens, const int* prompt) {
    const int step = st->step;
    out_tokens[step] = tok;
    int next = tok;
    if (st->force_prompt) {
        st->prompt_idx += 1;
        if (step + 1 < st->max_steps) next = prompt[st->prompt_idx];
    }
    st->token = next;
    st->pos += 1;
    st->step = step + 1;
    int stop = (step + 1 >= st->max_steps) || (st->pos >= st->max_seq);
    for (int i = 0; i < st->n_stop; i++) stop |= (st->stop_ids[i] == tok);
    if (stop) st->done = 1;
}

struct EpiLogits {
    static constexpr int MODE = EPI_PAIRS;
    float* logits;
    int* out_tokens;   // ring of emitted tokens, indexed by TokenState::step
    const int* prompt; // forced inputs of a verification pass (TokenState::force_prompt)
    int n_rows;
    int row_offset;    // vocabulary id of local row 0 (vocabulary-parallel head)
    int use_tp;
    TpComm c;
    unsigned long long* defer_best;  // non-null: publish the local winner here and leave the state alone
                                     // (a library all-reduce and k_state_advance finish the step)
    int special_row, special_id;     // shortlisted head: local row special_row stands for vocabulary id special_id (-1: none)
    unsigned long long best;
    __device__ void begin(const TokenState*) { best = 0ull; }
    __device__ __forceinline__ bool wants_residual() const { return false; }
    __device__ __forceinline__ float residual(int) const { return 0.f; }
    __device__ __forceinline__ void set_residual(const float*, int) {}
    __device__ __forceinline__ void one(int row, float v) {
        logits[row] = v;
        const unsigned long long k = argmax_key(v, row + row_offset);
        best = k > best ? k : best;
    }
    __device__ __forceinline__ void apply(int p, float v0, float v1) {
        one(2 * p, v0);
        if (2 * p + 1 < n_rows) one(2 * p + 1, v1);
    }
    __device__ void end(TokenState* st) {
        __shared__ unsigned long long sbest[GEMV_WARPS];
        __shared__ int last;
        const int tid = threadIdx.x;
        // several lanes of a warp may have handled rows: fold their candidates first
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(TFR_FULL_MASK, best, o);
            best = other > best ? other : best;
        }
        if ((tid & 31) == 0) sbest[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            unsigned long long b = 0ull;
            for (int i = 0; i < GEMV_WARPS; i++) b = sbest[i] > b ? sbest[i] : b;
            atomicMax(&st->best, b);
            __threadfence();
            const unsigned int old = atomicAdd(&st->head_done, 1u);
            last = (old == gridDim.x - 1);
        }
        __syncthreads();
        if (last && tid == 0) {
            __threadfence();
            unsigned long long b = atomicMax(&st->best, 0ull);
            if (defer_best) {
                *defer_best = b;
                st->best = 0ull;
                st->head_done = 0u;
                return;
            }
            if (use_tp) {
                // every rank's local winner -> the global one, identical on all ranks
                if (!tp_allreduce_best(c, st->ar_epoch + (unsigned)c.ops_per_token, b)) {
                    st->err = 3;
                    st->done = 1;
                }
                st->ar_epoch += (unsigned)c.ops_per_token;
            }
            int tok = argmax_key_index(b);
            if (special_id >= 0 && tok == special_row) tok = special_id;  // forward.rs:107-118 (map_output_id)
            advance_state(st, tok, out_tokens, prompt);
            st->best = 0ull;
            st->head_done = 0u;
        }
    }
};

// ------------------------------------------------------------------ the GEMV kernel

struct PrepArgs {
    const float* vec;     // source vector; nullptr -> embedding row of TokenState::token
    Mat embed;
    const float* normw;   // RMSNorm weight or nullptr
    float eps;
    float* raw_out;       // embedding source only: CTA 0 stores the decoded row here (residual stream)
    int token;            // embedding source without TokenState
    int prof_id;          // timeline probe: which launch of the token this is (test aid)
    // rows [0, pos] of these two arrays (row_bytes each) are pulled into L2 for the kernel that follows
    // (the layer's K and V cache before flash-decode); nullptr: none
    const unsigned char* l2_rows_a;
    const unsigned char* l2_rows_b;
    int l2_row_bytes;
};

// A matrix whose rows are spread over the CTAs in contiguous shares of `rows_per_item` rows.
// data == nullptr: absent.
struct RowJob {
    Mat m;
    Share sh;
    int rows_per_item;  // 2: the share counts row pairs; 1: rows
    int id_base;        // epilogue id of the matrix's first item
};

// Rows that take the fp32 activation instead (Q6_K attn_v); m.data == nullptr: none.
struct F32Seg {
    Mat m;
    Share sh;     // over row pairs
    int id_base;  // pair id of the segment's first pair
};

// Shared-memory map of k_gemv:
//   [ Act | partial sums (pbuf_floats) | 272 floats | full[slots] mbarriers | tile slots ].
// One CTA owns an SM (1024 threads, nearly all shared memory): 32 warps and up to ~46 tile slots
// keep the dot phase at HBM speed.  (Half-SM CTAs, which would let the next kernel's CTA sit
// beside this one and prefetch, were measured slower: fewer warps and slots cost more than the
// overlap gained.)  Kernels are chained with programmatic stream serialisation: a CTA requests
// its weight tiles, then sleeps in griddepcontrol.wait until the previous kernel's results are
// complete, so launch latency and the first tiles' fetch hide behind the predecessor's tail.
constexpr size_t GEMV_SMEM_MAX = 225 * 1024;  // opt-in limit is 227 KB including the kernels' small static arrays
constexpr int GEMV_L2_AHEAD = 4;  // tiles per warp requested into L2 beyond the one in its ring slot
inline size_t gemv_smem_fixed(int K, bool with_xf, bool has_norm, int pbuf_floats) {
    size_t act_bytes = (act_smem_bytes(K, with_xf, has_norm) + 15) & ~(size_t)15;
    return act_bytes + (size_t)pbuf_floats * sizeof(float) + 272 * sizeof(float);
}
inline int gemv_pbuf_floats(int rows_a, int rows_b, int nb) {
    const int need = (rows_a + rows_b) * nb;
    return need > 1024 ? ((need + 3) & ~3) : 1024;
}

// Row sums from the per-block partials and the epilogue.  LPR lanes add up one row.
template <int MODE, class Epi>
__device__ __forceinline__ void reduce_rows(const float* pa, const float* pb, int n_rows, int nb, int id0, Epi& epi) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (nb <= 16) {
        const int LPR = nb <= 8 ? 8 : 16, RPW = 32 / LPR;
        const int k = lane & (LPR - 1), rl = lane / LPR;
        for (int base = warp * RPW; base < n_rows; base += GEMV_WARPS * RPW) {
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
                const float other = __shfl_down_sync(TFR_FULL_MASK, a, LPR);  // the odd row of the pair
                if (k == 0 && !(rl & 1) && r < n_rows) epi.apply(id0 + (r >> 1), a, other);
            }
        }
    } else {
        const int items = MODE == EPI_ZIP ? n_rows : (n_rows + 1) >> 1;
        for (int it = warp; it < items; it += GEMV_WARPS) {
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

// One CTA of 1024 threads per SM.  The weight tiles of the CTA's rows are pulled into
// shared memory by bulk copies (TMA, one 4.5 / 6.6 KB request per tile).  Every warp requests
// its own tiles at kernel entry (one issuing thread cannot keep HBM busy: a thread issues
// only a few copies per microsecond), so they stream from HBM while all warps stage,
// normalise and quantise the activation.  A warp then waits on its tile's mbarrier, each
// lane reads its own block from the tile, the lane's partial goes to shared memory and,
// after a single barrier, rows are summed in a fixed order and handed to the epilogue.  When
// the CTA has more tiles than slots (the vocabulary head), a warp owns one slot and refills
// it itself after each tile.
template <class BLK, class Epi>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
k_gemv(PrepArgs pa, RowJob ja, RowJob jb, F32Seg fseg, Epi epi_in, int K, int pbuf_floats, int slots, TokenState* st) {
    extern __shared__ __align__(128) unsigned char smem[];
    prof_mark(0, pa.prof_id);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cta = blockIdx.x;
    const bool has_norm = pa.normw != nullptr;
    // the fp32 copy of the vector is staged only where something reads it back: the norm's reduction,
    // the fp32-route rows, the embedding source
    const bool with_xf = has_norm || fseg.m.data != nullptr || pa.vec == nullptr;
    Epi epi = epi_in;
    Act act = act_carve(smem, K, with_xf, has_norm);
    const size_t act_bytes = (act_smem_bytes(K, with_xf, has_norm) + 15) & ~(size_t)15;
    float* pbuf = reinterpret_cast<float*>(smem + act_bytes);
    float* red = pbuf + pbuf_floats;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(red + 272);
    float* xs = act.xf;
    const int nb = K >> 8;
    constexpr int TB = BLK::TILE_BYTES;
    unsigned char* ring = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(full + slots) + 127) & ~(uintptr_t)127);

    // flat block ranges of this CTA in A and B, and the tiles that cover them
    const int rows_a0 = ja.sh.begin(cta) * ja.rows_per_item;
    const int rows_a = max(0, min(ja.sh.count(cta) * ja.rows_per_item, ja.m.N - rows_a0));
    const int rows_b0 = jb.m.data ? jb.sh.begin(cta) * jb.rows_per_item : 0;
    const int rows_b = jb.m.data ? max(0, min(jb.sh.count(cta) * jb.rows_per_item, jb.m.N - rows_b0)) : 0;
    const long long fa0 = (long long)rows_a0 * nb, fa1 = fa0 + (long long)rows_a * nb;
    const long long fb0 = (long long)rows_b0 * nb, fb1 = fb0 + (long long)rows_b * nb;
    const int ta0 = (int)(fa0 >> 5), tiles_a = rows_a > 0 ? (int)((fa1 + 31) >> 5) - ta0 : 0;
    const int tb0 = (int)(fb0 >> 5), tiles_b = rows_b > 0 ? (int)((fb1 + 31) >> 5) - tb0 : 0;
    const int n_jobs = tiles_a + tiles_b;
    float* part_a = pbuf;
    float* part_b = pbuf + rows_a * nb;
    auto job_src = [&](int j) -> const uint8_t* {
        return j < tiles_a ? ja.m.data + (long long)(ta0 + j) * TB : jb.m.data + (long long)(tb0 + j - tiles_a) * TB;
    };
    // Tile j of the CTA belongs to warp j % stride.  Without reuse every tile has its own slot; with
    // reuse (more tiles than slots) warp w owns slot w and walks its tiles through it in order.
    const bool reuse = n_jobs > slots;
    const int stride = reuse ? slots : GEMV_WARPS;
    auto issue = [&](int j) {
        const int s = reuse ? warp : j;
        mbar_expect_tx(full + s, TB);
        bulk_load(ring + (size_t)s * TB, job_src(j), TB, full + s);
    };

    // Weights do not depend on the previous kernel: every warp requests its first tiles at once.  (Requesting
    // the tiles of a large CTA only after its vector has arrived was measured: the vector then lands within
    // 0.5 us instead of 2-3, but a bulk request costs its issuing thread a third of a microsecond, and paying
    // that after the wait instead of before it loses more than the faster vector gains.)
    if (lane == 0 && warp < stride) {
        for (int j = warp; j < n_jobs; j += stride) {
            mbar_init(full + (reuse ? warp : j), 1);
            if (reuse) break;
        }
        mbar_fence_init();
        for (int j = warp; j < n_jobs; j += stride) {
            issue(j);
            if (reuse) break;
        }
    }
    if (fseg.m.data && tid == GEMV_THREADS - 1) {
        // the fp32-route rows are read with plain loads later: have their tiles in L2 by then
        const long long f0 = 2ll * fseg.sh.begin(cta) * nb, f1 = f0 + 2ll * fseg.sh.count(cta) * nb;
        if (f1 > f0) {
            const long long t0 = f0 >> 5, t1 = (f1 + 31) >> 5;
            bulk_prefetch_l2(fseg.m.data + t0 * Q6_TILE_BYTES, (unsigned)((t1 - t0) * Q6_TILE_BYTES));
        }
    }
    // RMSNorm weights are constants: fetch them before the wait (K <= 4 * threads on this path)
    constexpr int NORM_REGS = 2;
    float4 wreg[NORM_REGS];
    if (has_norm) {
#pragma unroll
        for (int k = 0; k < NORM_REGS; k++) {
            const int i4 = k * GEMV_THREADS + tid;
            wreg[k] = i4 < (K >> 2) ? reinterpret_cast<const float4*>(pa.normw)[i4] : make_float4(1.f, 1.f, 1.f, 1.f);
        }
    }
    if (pa.l2_rows_a && st && tid == GEMV_THREADS - 32) {
        // A hint only: the position may still be the previous token's if the kernel before this one is the
        // vocabulary head; a row more or less in L2 changes nothing but timing.
        const int rows = st->pos + 1, per = (rows + (int)gridDim.x - 1) / (int)gridDim.x;
        const int r0 = cta * per, r1 = min(rows, r0 + per);
        if (r1 > r0) {
            const size_t off = (size_t)r0 * pa.l2_row_bytes;
            const unsigned bytes = (unsigned)((r1 - r0) * pa.l2_row_bytes) & ~15u;
            if (bytes) {
                bulk_prefetch_l2(pa.l2_rows_a + off, bytes);
                bulk_prefetch_l2(pa.l2_rows_b + off, bytes);
            }
        }
    }
    __syncwarp();
    prof_mark(1, pa.prof_id);
    // Everything below reads what earlier kernels wrote (the vector, the decode state).
    griddep_wait();
    prof_mark(3, pa.prof_id);
    // Only now may the next kernel start its prologue: its bulk weight requests then queue behind this
    // kernel's own latency-critical loads instead of in front of them, and never run two kernels ahead.
    griddep_launch_dependents();
    const int done = st ? st->done : 0;
    // residual values of this CTA's rows (pair-ordered epilogues only), one per thread
    const int res_row0 = 2 * (ja.id_base + (rows_a0 >> 1));
    const bool res_pre = Epi::MODE == EPI_PAIRS && epi.wants_residual() && rows_a <= 256 && rows_b == 0 && !fseg.m.data;
    float resv = 0.f;
    if (res_pre && tid < rows_a) resv = epi.residual(res_row0 + tid);
    constexpr int STAGE_REGS = 6;  // float4 per thread and pass: one pass up to K = 12288
    const int n4 = K >> 2;
    float scale = 1.f;
    if (pa.vec && !with_xf) {
        // plain vector: quantise pass by pass straight from the registers that fetched it
        if (!done) {
            for (int base = 0; base < n4; base += STAGE_REGS * GEMV_THREADS) {
                float4 sx[STAGE_REGS];
#pragma unroll
                for (int k = 0; k < STAGE_REGS; k++) {
                    const int i4 = base + k * GEMV_THREADS + tid;
                    sx[k] = i4 < n4 ? reinterpret_cast<const float4*>(pa.vec)[i4] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int k = 0; k < STAGE_REGS; k++) {
                    const int i4 = base + k * GEMV_THREADS + tid;
                    if (base + k * GEMV_THREADS < n4) act_quantize4(act, sx[k], i4, i4 < n4, nb);
                }
            }
        }
        prof_mark(2, pa.prof_id);
        prof_mark(6, pa.prof_id);
    } else {
        if (pa.vec) {
            for (int i4 = tid; i4 < n4; i4 += GEMV_THREADS)
                *reinterpret_cast<float4*>(xs + xs_idx(4 * i4)) = reinterpret_cast<const float4*>(pa.vec)[i4];
        } else {
            int tok = st ? st->token : pa.token;
            if (tok < 0 || tok >= pa.embed.N) {
                if (st && tid == 0) st->err = 1;
                tok = 0;
            }
            const SrcEmbed src{pa.embed, tok};
            for (int i = tid; i < K; i += GEMV_THREADS) {
                const float v = src.get(i);
                xs[xs_idx(i)] = v;
                if (cta == 0 && pa.raw_out && !done) pa.raw_out[i] = v;
            }
        }
        __syncthreads();
        prof_mark(2, pa.prof_id);
        if (!done) {
            if (has_norm) scale = rms_scale_staged(xs, K, pa.eps, red);
            prof_mark(6, pa.prof_id);
            for (int k0 = 0; k0 < n4; k0 += GEMV_THREADS) {
                const int i4 = k0 + tid;
                const bool on = i4 < n4;
                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (on) {
                    x = *reinterpret_cast<const float4*>(xs + xs_idx(4 * i4));
                    if (has_norm) {
                        float4 w = wreg[0];
                        if (k0 == GEMV_THREADS) w = wreg[1];
                        if (k0 >= NORM_REGS * GEMV_THREADS) w = reinterpret_cast<const float4*>(pa.normw)[i4];
                        x.x = x.x * scale * w.x;
                        x.y = x.y * scale * w.y;
                        x.z = x.z * scale * w.z;
                        x.w = x.w * scale * w.w;
                        if (fseg.m.data) *reinterpret_cast<float4*>(xs + xs_idx(4 * i4)) = x;
                    }
                }
                act_quantize4(act, x, i4, on, nb);
            }
        }
    }
    if (done) {
        // the copies already in flight must land before the CTA's shared memory is released
        if (lane == 0 && warp < stride)
            for (int j = warp; j < n_jobs; j += stride) {
                mbar_wait(full + (reuse ? warp : j), 0);
                if (reuse) break;
            }
        return;
    }
    // With a ring (one tile per warp) too few bytes are in flight to keep HBM busy: the warp's next
    // tiles are pulled into L2 ahead of time and its refills then hit L2.  Requested only now, so that
    // the bulk traffic queues behind the activation loads above, not in front of them.
    if (reuse && lane == 0 && warp < stride)
        for (int k = 1; k <= GEMV_L2_AHEAD && warp + k * stride < n_jobs; k++) bulk_prefetch_l2(job_src(warp + k * stride), TB);
    prof_mark(7, pa.prof_id);
    epi.begin(st);
    if (res_pre) {
        if (tid < rows_a) red[tid] = resv;  // red is free once the norm's reduction is over
        epi.set_residual(red, res_row0);
    }
    __syncthreads();

    // rows on the fp32 activation route: one task per (row, block, run of 16).  When their partials fit behind the
    // block partials of the tiles (the usual case: a CTA holds one or two V row pairs), the tasks run side by side
    // with the tile dots — taken from the last thread downwards, so the few warps that own tiles keep to their tiles —
    // and share the tile dots' barrier; otherwise they run first, chunk by chunk, with barriers of their own.
    const int f32_tasks = fseg.m.data ? 2 * fseg.sh.count(cta) * 16 * nb : 0;
    const int f32_off = ((rows_a + rows_b) * nb + 3) & ~3;
    const bool f32_fused = f32_tasks > 0 && f32_off + f32_tasks <= pbuf_floats;
    if (fseg.m.data && !f32_fused) {
        const int np = fseg.sh.count(cta), pbase = fseg.sh.begin(cta);
        const int per_row = 16 * nb, tasks = 2 * np * per_row;
        const int chunk = (pbuf_floats / (2 * per_row)) * (2 * per_row);  // whole row pairs per chunk
        for (int t0 = 0; t0 < tasks; t0 += chunk) {
            const int tn = min(chunk, tasks - t0);
            for (int t = tid; t < tn; t += GEMV_THREADS) {
                const int task = t0 + t;
                const int row_l = task / per_row, rem = task - row_l * per_row;
                const int row_g = 2 * pbase + row_l;
                float v = 0.f;
                if (row_g < fseg.m.N) v = q6k_run_dot_f32(fseg.m, (long long)row_g * nb + (rem >> 4), rem >> 4, rem & 15, xs);
                pbuf[t] = v;
            }
            __syncthreads();
            const int pairs_here = tn / (2 * per_row), pair_first = t0 / (2 * per_row);
            for (int rr = warp; rr < pairs_here; rr += GEMV_WARPS) {
                const float* a = pbuf + (2 * rr) * per_row;
                float s0 = 0.f, s1 = 0.f;
                for (int i = lane; i < per_row; i += 32) {
                    s0 += a[i];
                    s1 += a[per_row + i];
                }
                s0 = warp_sum(s0);
                s1 = warp_sum(s1);
                if (lane == 0) epi.apply(fseg.id_base + pbase + pair_first + rr, s0, s1);
            }
            __syncthreads();
        }
    }

    // phase A: per-block partials out of the tiles
    bool ok = true;
    int late_slot = -1;
    unsigned late_parity = 0;
    if (warp < stride) {
        int it = 0;
        for (int j = warp; j < n_jobs; j += stride, it++) {
            const int s = reuse ? warp : j;
            const bool is_b = j >= tiles_a;
            const long long f = (long long)(is_b ? tb0 + (j - tiles_a) : ta0 + j) * 32 + lane;
            const bool mine = is_b ? (f >= fb0 && f < fb1) : (f >= fa0 && f < fa1);
            // A copy that did not land within the wait limit: the tile is NOT read (its partials become zero and the
            // error word marks the step invalid), the slot is not refilled, and the warp waits for that copy once
            // more before the CTA may leave (below), so shared memory is never released under a copy in flight.
            const bool landed = mbar_wait(full + s, reuse ? (it & 1) : 0);
            if (!landed) {
                ok = false;
                late_slot = s;
                late_parity = reuse ? (it & 1) : 0;
            }
            if (mine) {
                float* dst = is_b ? part_b + (f - fb0) : part_a + (f - fa0);
                *dst = landed ? block_dot<true>(BLK{}, ring + (size_t)s * TB, lane, act, (int)(f % nb), nb, nullptr) : 0.f;
            }
            __syncwarp();
            if (!landed) {
                // without slot reuse the warp's later tiles were requested at kernel entry: let them land (bounded)
                if (!reuse)
                    for (int j2 = j + stride; j2 < n_jobs; j2 += stride) mbar_wait(full + j2, 0);
                break;
            }
            if (reuse && lane == 0 && j + stride < n_jobs) {
                fence_proxy_async();
                issue(j + stride);
                if (j + (GEMV_L2_AHEAD + 1) * stride < n_jobs) bulk_prefetch_l2(job_src(j + (GEMV_L2_AHEAD + 1) * stride), TB);
            }
        }
    }
    if (f32_fused) {
        const int pbase = fseg.sh.begin(cta), per_row = 16 * nb;
        for (int t = GEMV_THREADS - 1 - tid; t < f32_tasks; t += GEMV_THREADS) {
            const int row_l = t / per_row, rem = t - row_l * per_row;
            const int row_g = 2 * pbase + row_l;
            float v = 0.f;
            if (row_g < fseg.m.N) v = q6k_run_dot_f32(fseg.m, (long long)row_g * nb + (rem >> 4), rem >> 4, rem & 15, xs);
            pbuf[f32_off + t] = v;
        }
    }
    if (!ok && st) st->err = 2;  // a bulk copy never completed: results of this step are invalid
    __syncthreads();
    prof_mark(4, pa.prof_id);
    if (f32_fused) {
        // the same sums as the stand-alone route: lanes stride over a row's runs, then the warp tree
        const int pbase = fseg.sh.begin(cta), per_row = 16 * nb, pairs = f32_tasks / (2 * per_row);
        for (int rr = GEMV_WARPS - 1 - warp; rr < pairs; rr += GEMV_WARPS) {
            const float* a = pbuf + f32_off + (2 * rr) * per_row;
            float s0 = 0.f, s1 = 0.f;
            for (int i = lane; i < per_row; i += 32) {
                s0 += a[i];
                s1 += a[per_row + i];
            }
            s0 = warp_sum(s0);
            s1 = warp_sum(s1);
            if (lane == 0) epi.apply(fseg.id_base + pbase + rr, s0, s1);
        }
    }
    // phase B: row sums in a fixed order + epilogue
    if (Epi::MODE == EPI_ZIP) {
        reduce_rows<EPI_ZIP>(part_a, part_b, rows_a, nb, ja.id_base + rows_a0, epi);
    } else {
        reduce_rows<EPI_PAIRS>(part_a, part_a, rows_a, nb, ja.id_base + (rows_a0 >> 1), epi);
        if (rows_b > 0) reduce_rows<EPI_PAIRS>(part_b, part_b, rows_b, nb, jb.id_base + (rows_b0 >> 1), epi);
    }
    epi.end(st);
    if (late_slot >= 0) mbar_wait(full + late_slot, late_parity);  // bounded: a second limit, then the CTA leaves regardless
    prof_mark(5, pa.prof_id);
}

// Set once per process: launch with programmatic stream serialisation (overlap with the previous kernel).
inline bool& gemv_pdl_enabled() {
    static bool on = true;
    return on;
}

template <class... Args>
inline cudaError_t launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gemv_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <class BLK, class Epi>
inline cudaError_t launch_gemv(cudaStream_t stream, int grid, const PrepArgs& pa, const RowJob& ja, const RowJob& jb,
                               const F32Seg& fseg, const Epi& epi, int K, TokenState* st) {
    const int nb = K / 256;
    constexpr int TB = BLK::TILE_BYTES;
    const int ra = (ja.sh.quot + 1) * ja.rows_per_item, rb = jb.m.data ? (jb.sh.quot + 1) * jb.rows_per_item : 0;
    int pf = gemv_pbuf_floats(ra, rb, nb);
    if (fseg.m.data && pf < 2 * 16 * nb) pf = 2 * 16 * nb;
    const bool has_norm = pa.normw != nullptr;
    const bool with_xf = has_norm || fseg.m.data != nullptr || pa.vec == nullptr;  // as in the kernel
    const size_t fixed = gemv_smem_fixed(K, with_xf, has_norm, pf);
    // tiles a CTA can need: each matrix's share may straddle one extra tile at either end
    const int need = (ra * nb + 31) / 32 + 1 + (rb ? (rb * nb + 31) / 32 + 1 : 0);
    if (fixed + 256 + 1024 + TB > GEMV_SMEM_MAX) return cudaErrorInvalidValue;
    int slots = (int)((GEMV_SMEM_MAX - fixed - 256 - 1024) / (TB + 8));
    if (slots >= need) slots = need;
    else if (slots > GEMV_WARPS) slots = GEMV_WARPS;  // reuse: one slot per warp
    if (slots < 1) slots = 1;
    const size_t smem = fixed + (size_t)slots * 8 + 256 + (size_t)slots * TB;
    return launch_pdl(k_gemv<BLK, Epi>, dim3(grid), dim3(GEMV_THREADS), smem, stream, pa, ja, jb, fseg, epi, K, pf, slots, st);
}

inline RowJob make_job(const Mat& m, int rows_per_item, int C, int id_base = 0) {
    RowJob j{};
    j.m = m;
    j.rows_per_item = rows_per_item;
    j.sh = make_share((m.N + rows_per_item - 1) / rows_per_item, C);
    j.id_base = id_base;
    return j;
}

// ------------------------------------------------------------------ small kernels

// Stand-alone quantiser with linear output (A1), same expression as act_quantize_staged.
__global__ void k_quantize_q8(const float* __restrict__ x, signed char* __restrict__ q8, float* __restrict__ d8, int n) {
    const int lane = threadIdx.x & 31;
    const int g = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (g >= (n >> 5)) return;
    const int i = (g << 5) + lane;
    const float xi = x[i];
    const float amax = warp_max(fabsf(xi));
    const float d = amax * (1.0f / 127.0f);
    q8[i] = amax == 0.f ? 0 : (signed char)__float2int_rn(xi / d);
    if (lane == 0) d8[g] = d;
}

#ifdef TFR_TEST_AIDS
// Builds an Act from an already quantised activation (linear int8 + scales); test-only path
// used to expose the integer sub-block dots.
__device__ void act_from_q8(const Act& act, const signed char* q8, const float* d8, int K) {
    const int tid = threadIdx.x, j = tid & 7, nb = K >> 8;
    for (int g0 = 0; g0 < (K >> 5); g0 += blockDim.x / 8) {
        const int g = g0 + (tid >> 3);
        const bool on = g < (K >> 5);
        const int e = 32 * (on ? g : 0) + 4 * j;
        const int q0 = q8[e], q1 = q8[e + 1], q2 = q8[e + 2], q3 = q8[e + 3];
        int s = q0 + q1 + q2 + q3;
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 1);
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 2);
        const int other = __shfl_xor_sync(TFR_FULL_MASK, s, 4);
        if (on) {
            *act_word_ptr(act, e, nb) = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) | ((q3 & 0xff) << 24);
            if (j == 0) act_store_group(act, g, d8[g], s, other);
        }
    }
    __syncthreads();
}

// Integer contract taps, computed by the very routines the GEMV kernel uses.
// Q4_K: I[row][K/32], S[row][K/32].  Q6_K: J[row][K/16].  Q8_0: sums[row][K/32].
// x != nullptr: the activation is quantised here by act_quantize4 (what k_gemv runs on a plain vector) instead of being
// taken from (q8, d8); q8_out (optional) then receives the int8 values the block dots read.  S is read back from the
// Act the dots use (s16n holds -32 * the sum of every 16-chunk, an exact integer), not recomputed from the int8.
template <class BLK>
__global__ void k_int_dots(Mat m, const float* x, const signed char* q8, const float* d8, int* outA, int* outB, signed char* q8_out) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int K = m.K, nb = m.nb, lane = threadIdx.x & 31, tid = threadIdx.x;
    Act act = act_carve(smem, K, false, false);
    if (x) {
        const int n4 = K >> 2;
        for (int k0 = 0; k0 < n4; k0 += blockDim.x) {
            const int i4 = k0 + tid;
            const bool on = i4 < n4;
            const float4 v = on ? reinterpret_cast<const float4*>(x)[i4] : make_float4(0.f, 0.f, 0.f, 0.f);
            act_quantize4(act, v, i4, on, nb);
        }
        __syncthreads();
        if (q8_out && blockIdx.x == 0)
            for (int e = 4 * tid; e < K; e += 4 * blockDim.x) *reinterpret_cast<int*>(q8_out + e) = *act_word_ptr(act, e, nb);
    } else {
        act_from_q8(act, q8, d8, K);
    }
    const long long total = (long long)m.N * nb;
    const long long tiles = (total + 31) >> 5;
    const int TB = tile_bytes(m.type);
    for (long long t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < tiles; t += (long long)gridDim.x * (blockDim.x >> 5)) {
        const long long f = t * 32 + lane;
        if (f >= total) continue;
        const int r = (int)(f / nb), b = (int)(f % nb);
        int ints[16];
        block_dot<false>(BLK{}, m.data + t * TB, lane, act, b, nb, ints);
        if (BLK::TILE_BYTES == Q4_TILE_BYTES) {
            for (int j = 0; j < 8; j++) {
                outA[(size_t)r * (K / 32) + 8 * b + j] = ints[j];
                const int g = 8 * b + j;
                outB[(size_t)r * (K / 32) + g] = -(act.s16n[2 * g] + act.s16n[2 * g + 1]) / 32;
            }
        } else if (BLK::TILE_BYTES == Q8_TILE_BYTES) {
            for (int j = 0; j < 8; j++) outA[(size_t)r * (K / 32) + 8 * b + j] = ints[j];
        } else {
            for (int c = 0; c < 16; c++) outA[(size_t)r * (K / 16) + 16 * b + c] = ints[c];
        }
    }
}

#endif  // TFR_TEST_AIDS

// Row-permuting repack.  perm_hd > 0: within each head of perm_hd rows, destination row
// 2i + s takes source row i + s * perm_hd / 2 (RoPE partners become adjacent).
__device__ __forceinline__ int perm_src_row(int v, int perm_hd) {
    if (perm_hd <= 0) return v;
    const int h = v / perm_hd, w = v % perm_hd;
    return h * perm_hd + (w >> 1) + (w & 1) * (perm_hd >> 1);
}

// GGUF block bytes -> warp-tiled layout (see tfr_gemv.cuh).  One thread per (flat block, 16-byte
// piece); tail tiles are zero-filled by the caller.
__global__ void k_repack_tiled(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int type, int N, int nb,
                               int perm_hd) {
    const int pieces = type == TFR_Q4_K ? Q4_PIECES : type == TFR_Q8_0 ? Q8_PIECES : Q6_PIECES + 1;  // Q6_K: 13 pieces + the 2-byte d
    const int blk = block_bytes_256(type), TB = tile_bytes(type);
    const long long total = (long long)N * nb * pieces;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long f = i / pieces;
        const int pc = (int)(i - f * pieces);
        const int row = (int)(f / nb), b = (int)(f - (long long)row * nb);
        const uint8_t* sb = src + ((long long)perm_src_row(row, perm_hd) * nb + b) * blk;
        uint8_t* tile = dst + (f >> 5) * TB;
        const int lane = (int)(f & 31);
        if (type == TFR_Q6_K && pc == Q6_PIECES) {
            tile[Q6_PIECES * 512 + lane * 2] = sb[208];
            tile[Q6_PIECES * 512 + lane * 2 + 1] = sb[209];
        } else {
            for (int k = 0; k < 16; k++) tile[pc * 512 + lane * 16 + k] = sb[pc * 16 + k];
        }
    }
}

// One row of a tiled matrix as a one-row tiled matrix (a single tile, lanes 0 .. nb-1): the extra
// vocabulary row of a shortlisted head (load.rs:308-342).  One thread per (block, piece).
__global__ void k_extract_row(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int type, int row, int nb) {
    const int pieces = type == TFR_Q4_K ? Q4_PIECES : type == TFR_Q8_0 ? Q8_PIECES : Q6_PIECES + 1;
    const int TB = tile_bytes(type);
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nb * pieces) return;
    const int b = i / pieces, pc = i - b * pieces;
    const long long f = (long long)row * nb + b;
    const uint8_t* st = src + (f >> 5) * TB;
    const int sl = (int)(f & 31);
    if (type == TFR_Q6_K && pc == Q6_PIECES) {
        dst[Q6_PIECES * 512 + b * 2] = st[Q6_PIECES * 512 + sl * 2];
        dst[Q6_PIECES * 512 + b * 2 + 1] = st[Q6_PIECES * 512 + sl * 2 + 1];
    } else {
        for (int k = 0; k < 16; k++) dst[pc * 512 + b * 16 + k] = st[pc * 512 + sl * 16 + k];
    }
}

__global__ void k_permute_f32(const float* __restrict__ src, float* __restrict__ dst, int n, int perm_hd) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v < n) dst[v] = src[perm_src_row(v, perm_hd)];
}

// Decode-state control (single thread each).  args (device memory, copied from the host per call):
// [0] token, [1] pos, [2] max_steps, [3] max_seq, [4] n_stop, [5..12] stop ids, [13] conv ring offset,
// [14] forced-input (verification) flag.
__global__ void k_state_begin(TokenState* st, const int* __restrict__ args) {
    st->token = args[0];
    st->pos = args[1];
    st->step = 0;
    st->max_steps = args[2];
    st->max_seq = args[3];
    st->done = 0;
    st->n_stop = args[4];
    for (int i = 0; i < 8; i++) st->stop_ids[i] = args[5 + i];
    st->best = 0ull;
    st->head_done = 0u;
    st->prompt_idx = 0;
    st->err = 0;
    st->ring_off = args[13];
    st->force_prompt = args[14];
}

// Second half of the vocabulary head when the (max, argmax) exchange is done by a library all-reduce:
// publishes the token and advances the decode state (the tail of EpiLogits::end).
__global__ void k_state_advance(TokenState* st, const unsigned long long* best, int* out_tokens, const int* prompt) {
    griddep_wait();
    if (st->done) return;
    advance_state(st, argmax_key_index(*best), out_tokens, prompt);
}

// x += y (the residual add after a library all-reduce of the row-parallel partial sums)
__global__ void k_add_residual(float* __restrict__ x, const float* __restrict__ y, int n, const TokenState* st) {
    griddep_wait();
    if (st && st->done) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += y[i];
}

// Prefill by decode steps: after a head-less pass, feed the next prompt token.
__global__ void k_state_next_prompt(TokenState* st, const int* prompt, int ar_ops) {
    griddep_wait();
    if (st->done) return;
    st->ar_epoch += (unsigned)ar_ops;  // tensor parallelism: keep the epoch numbering per token fixed
    st->prompt_idx += 1;
    st->pos += 1;
    st->token = prompt[st->prompt_idx];
    if (st->pos >= st->max_seq) st->done = 1;
}

}  // namespace tfr
