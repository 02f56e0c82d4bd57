// __global__ kernels of the batch-1 decode path and their launch helpers.
#pragma once
#include "tfr_attn.cuh"
#include "tfr_gemv.cuh"

namespace tfr {

// ------------------------------------------------------------------ epilogues
//
// An epilogue receives the two finished dot products of a row pair from exactly one thread.

// y = W x (+y) (+bias): kernels/gemv.cu:367-373 residual rule (2 = accumulate in place).
struct EpiStore {
    float* out;
    const float* bias;
    int use_res;
    int n_rows;
    __device__ void begin(const TokenState*) {}
    __device__ __forceinline__ void one(int row, float acc) {
        if (use_res == 2) acc += out[row];
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
    float* out;
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
struct EpiLogits {
    float* logits;
    int* out_tokens;   // ring of emitted tokens, indexed by TokenState::step
    int n_rows;
    unsigned long long best;
    __device__ void begin(const TokenState*) { best = 0ull; }
    __device__ __forceinline__ void one(int row, float v) {
        logits[row] = v;
        const unsigned long long k = argmax_key(v, row);
        best = k > best ? k : best;
    }
    __device__ __forceinline__ void apply(int p, float v0, float v1) {
        one(2 * p, v0);
        if (2 * p + 1 < n_rows) one(2 * p + 1, v1);
    }
    __device__ void end(TokenState* st) {
        __shared__ unsigned long long sbest[GEMV_THREADS / 32];
        __shared__ int last;
        const int tid = threadIdx.x;
        if ((tid & 31) == 0) sbest[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            unsigned long long b = 0ull;
            for (int i = 0; i < GEMV_THREADS / 32; i++) b = sbest[i] > b ? sbest[i] : b;
            atomicMax(&st->best, b);
            __threadfence();
            const unsigned int old = atomicAdd(&st->head_done, 1u);
            last = (old == gridDim.x - 1);
        }
        __syncthreads();
        if (last && tid == 0) {
            __threadfence();
            const unsigned long long b = atomicMax(&st->best, 0ull);
            const int tok = argmax_key_index(b);
            const int step = st->step;
            out_tokens[step] = tok;
            st->token = tok;
            st->pos += 1;
            st->step = step + 1;
            int stop = (step + 1 >= st->max_steps) || (st->pos >= st->max_seq);
            for (int i = 0; i < st->n_stop; i++) stop |= (st->stop_ids[i] == tok);
            if (stop) st->done = 1;
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
    int wt;               // WT_Q4K / WT_Q6K: type of the rows that take the Q8 activation
    float* raw_out;       // embedding source only: CTA 0 stores the decoded row here (residual stream)
    int token;            // embedding source without TokenState
};

// Rows that take the fp32 activation instead (Q6_K attn_v); data == nullptr: none.
struct F32Seg {
    Mat m;
    Share sh;     // over row pairs
    int id_base;  // pair id of the segment's first pair
};

constexpr int GEMV_PT = 2 * GEMV_THREADS;  // floats per partial-sum buffer

// Shared-memory map of k_gemv: [ Act | partial sums x2 | 272 floats | 512 pair ids ].
inline size_t gemv_smem_bytes(int K, bool has_norm) {
    size_t act_bytes = (act_smem_bytes(K, true, has_norm) + 15) & ~(size_t)15;
    return act_bytes + 2 * (size_t)GEMV_PT * sizeof(float) + 272 * sizeof(float) + 512 * sizeof(int);
}

// One CTA of GEMV_THREADS threads per SM walks its share of row pairs.  Thread
// (r, u) = (tid / G, tid % G) owns unit column u of the r-th pair of every pass, so its byte
// offsets inside a row never change.  The weight loads of the first pass are issued before
// anything else: HBM streams while the activation is staged, normalised and quantised, and
// inside the loop the next pass is requested before the current one is reduced.
// K = 2048 (G = 32) makes a warp own a whole row pair: the reduction is five shuffles and the
// CTA never synchronises in the loop.  Other K go through shared-memory partial sums.
template <class Map, class Epi>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
k_gemv(PrepArgs pa, Map map, F32Seg fseg, Epi epi_in, int K, TokenState* st) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int NW = GEMV_THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cta = blockIdx.x;
    const bool has_norm = pa.normw != nullptr;
    Epi epi = epi_in;
    Act act = act_carve(smem, K, true, has_norm);
    const size_t act_bytes = (act_smem_bytes(K, true, has_norm) + 15) & ~(size_t)15;
    float* pbuf = reinterpret_cast<float*>(smem + act_bytes);
    float* red = pbuf + 2 * GEMV_PT;
    int* ids = reinterpret_cast<int*>(red + 272);
    float* xs = act.xf;

    const int G = K >> 6;
    const int R = GEMV_THREADS / G;  // row pairs per pass
    const int r = tid / G, u = tid - r * G;
    const bool active = r < R;
    const UnitOff off = unit_offsets(u, map.nb());
    const int wt = pa.wt;
    const int n_loc = map.n_local(cta);

    // first pass of weights: requested before anything else
    UnitW w0, w1;
    PairRows pr = map.pair(cta, (active && r < n_loc) ? r : 0);
    if (n_loc > 0) {
        load_unit(w0, wt, pr.r0, off);
        load_unit(w1, wt, pr.r1, off);
    }
    const int done = st ? st->done : 0;
    if (pa.vec) {
        for (int i4 = tid; i4 < (K >> 2); i4 += GEMV_THREADS) {
            const int at = xs_idx(4 * i4);
            *reinterpret_cast<float4*>(xs + at) = reinterpret_cast<const float4*>(pa.vec)[i4];
            if (has_norm) *reinterpret_cast<float4*>(act.wf + at) = reinterpret_cast<const float4*>(pa.normw)[i4];
        }
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
            if (has_norm) act.wf[xs_idx(i)] = pa.normw[i];
            if (cta == 0 && pa.raw_out && !done) pa.raw_out[i] = v;
        }
    }
    if (done) return;
    __syncthreads();
    float scale = 1.f;
    if (has_norm) scale = rms_scale_staged(xs, K, pa.eps, red);
    act_quantize_staged(act, has_norm, scale, K, wt == WT_Q4K ? SWZ_Q4 : SWZ_Q6);
    epi.begin(st);
    __syncthreads();

    // rows on the fp32 activation route: one task per (row, unit, run of 16), all threads
    if (fseg.m.data) {
        const int np = fseg.sh.count(cta), pbase = fseg.sh.begin(cta);
        const int per_row = 4 * G, tasks = 2 * np * per_row;
        const int chunk = ((2 * GEMV_PT) / (2 * per_row)) * (2 * per_row);  // whole row pairs per chunk
        for (int t0 = 0; t0 < tasks; t0 += chunk) {
            const int tn = min(chunk, tasks - t0);
            for (int t = tid; t < tn; t += GEMV_THREADS) {
                const int task = t0 + t;
                const int row_l = task / per_row, rem = task - row_l * per_row;
                const int row_g = 2 * pbase + row_l;
                float v = 0.f;
                if (row_g < fseg.m.N)
                    v = q6k_run_dot_f32(fseg.m.data + (long long)row_g * fseg.m.row_stride, fseg.m.nb, rem >> 2, rem & 3, xs);
                pbuf[t] = v;
            }
            __syncthreads();
            const int pairs_here = tn / (2 * per_row), pair_first = t0 / (2 * per_row);
            for (int rr = warp; rr < pairs_here; rr += NW) {
                const float* a = pbuf + (2 * rr) * per_row;
                float s0 = 0.f, s1 = 0.f;
                for (int i = lane; i < per_row; i += 32) {
                    s0 += a[i];
                    s1 += a[per_row + i];
                }
                const float x = warp_sum_pair(s0, s1, lane);
                const float y = __shfl_sync(TFR_FULL_MASK, x, 16);
                if (lane == 0) epi.apply(fseg.id_base + pbase + pair_first + rr, x, y);
            }
            __syncthreads();
        }
    }

    const int t4 = u & 3, is = u & 1;
    int buf = 0;
    for (int base = 0; base < n_loc; base += R) {
        const bool valid = active && base + r < n_loc;
        const int id = pr.id;
        float v0, v1;
        {
            Frag f;
            frag_load(f, wt, act, active ? u : 0, G);
            if (wt == WT_Q4K) {
                v0 = q4k_dot(w0, f, t4, nullptr);
                v1 = q4k_dot(w1, f, t4, nullptr);
            } else {
                v0 = q6k_dot(w0, f, is, nullptr);
                v1 = q6k_dot(w1, f, is, nullptr);
            }
        }
        const int nbase = base + R;
        if (nbase < n_loc) {
            pr = map.pair(cta, (active && nbase + r < n_loc) ? nbase + r : 0);
            load_unit(w0, wt, pr.r0, off);
            load_unit(w1, wt, pr.r1, off);
        }
        if (G == 32) {
            // warp == r: the 32 lanes hold the 32 units of both rows
            const float x = warp_sum_pair(v0, v1, lane);
            const float y = __shfl_sync(TFR_FULL_MASK, x, 16);
            if (lane == 0 && valid) epi.apply(id, x, y);
        } else {
            float* part = pbuf + buf * GEMV_PT;
            if (active) {
                part[(2 * r) * G + u] = v0;
                part[(2 * r + 1) * G + u] = v1;
                if (u == 0) ids[buf * 256 + r] = id;
            }
            __syncthreads();
            const int np = min(R, n_loc - base);
            for (int pp = warp; pp < np; pp += NW) {
                const float* a = part + (2 * pp) * G;
                float s0 = 0.f, s1 = 0.f;
                for (int i = lane; i < G; i += 32) {
                    s0 += a[i];
                    s1 += a[G + i];
                }
                const float x = warp_sum_pair(s0, s1, lane);
                const float y = __shfl_sync(TFR_FULL_MASK, x, 16);
                if (lane == 0) epi.apply(ids[buf * 256 + pp], x, y);
            }
            buf ^= 1;
        }
    }
    epi.end(st);
}

template <class Map, class Epi>
inline cudaError_t launch_gemv(cudaStream_t stream, int grid, const PrepArgs& pa, const Map& map, const F32Seg& fseg,
                               const Epi& epi, int K, TokenState* st) {
    const size_t smem = gemv_smem_bytes(K, pa.normw != nullptr);
    k_gemv<Map, Epi><<<grid, GEMV_THREADS, smem, stream>>>(pa, map, fseg, epi, K, st);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ small kernels

// Stand-alone quantiser with linear output (A1), same expression as act_quantize_group.
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

// Builds an Act from an already quantised activation (linear int8 + scales); test-only path
// used to expose the integer sub-block dots.
__device__ void act_from_q8(Act& act, const signed char* q8, const float* d8, int K, int swz) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, G = K >> 6;
    signed char* q8b = reinterpret_cast<signed char*>(act.q8);
    for (int g = warp; g < (K >> 5); g += blockDim.x >> 5) {
        const int i = (g << 5) + lane;
        const int q = q8[i];
        q8b[swz_pos(i >> 4, G, swz) * 16 + (i & 15)] = (signed char)q;
        int s = q;
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 8);
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 4);
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 2);
        s += __shfl_xor_sync(TFR_FULL_MASK, s, 1);
        const int hi = __shfl_sync(TFR_FULL_MASK, s, 16);
        if (lane == 0) {
            act.d8[g] = d8[g];
            act.ss[g] = (s & 0xffff) | (hi << 16);
        }
    }
    __syncthreads();
}

// Integer contract taps, computed by the very dot routines the GEMV kernel uses.
// Q4_K: I[row][K/32], S[row][K/32].  Q6_K: J[row][K/16].
__global__ void k_int_dots(Mat m, const signed char* q8, const float* d8, int* outA, int* outB) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int K = m.K, G = K >> 6;
    Act act = act_carve(smem, K, false, false);
    const int wt = m.type == TFR_Q4_K ? WT_Q4K : WT_Q6K;
    act_from_q8(act, q8, d8, K, m.type == TFR_Q4_K ? SWZ_Q4 : SWZ_Q6);
    const int total = m.N * G;
    for (int fidx = blockIdx.x * blockDim.x + threadIdx.x; fidx < total; fidx += gridDim.x * blockDim.x) {
        const int r = fidx / G, u = fidx % G;
        UnitW w;
        Frag f;
        const UnitOff off = unit_offsets(u, m.nb);
        load_unit(w, wt, m.data + (long long)r * m.row_stride, off);
        frag_load(f, wt, act, u, G);
        if (m.type == TFR_Q4_K) {
            int ints[2];
            q4k_dot(w, f, u & 3, ints);
            const int2 ss = reinterpret_cast<const int2*>(act.ss)[u];
            int* I = outA + (size_t)r * (K / 32) + 2 * u;
            int* S = outB + (size_t)r * (K / 32) + 2 * u;
            I[0] = ints[0];
            I[1] = ints[1];
            S[0] = (int)(short)(ss.x & 0xffff) + (ss.x >> 16);
            S[1] = (int)(short)(ss.y & 0xffff) + (ss.y >> 16);
        } else {
            int J[4];
            q6k_dot(w, f, u & 1, J);
            // run j of unit (b, n, is) is scale group 16b + 8n + 2j + is
            const int b = u >> 2, n = (u >> 1) & 1, is = u & 1;
            for (int j = 0; j < 4; j++) outA[(size_t)r * (K / 16) + 16 * b + 8 * n + 2 * j + is] = J[j];
        }
    }
}

// Row-permuting repack.  perm_hd > 0: within each head of perm_hd rows, destination row
// 2i + s takes source row i + s * perm_hd / 2 (RoPE partners become adjacent).
__device__ __forceinline__ int perm_src_row(int v, int perm_hd) {
    if (perm_hd <= 0) return v;
    const int h = v / perm_hd, w = v % perm_hd;
    return h * perm_hd + (w >> 1) + (w & 1) * (perm_hd >> 1);
}

__global__ void k_repack_q4k(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N, int nb, int perm_hd) {
    const long long row_bytes = (long long)nb * 144;
    const long long total = (long long)N * row_bytes;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int v = (int)(i / row_bytes);
        const long long off = i - (long long)v * row_bytes;
        dst[i] = src[(long long)perm_src_row(v, perm_hd) * row_bytes + off];
    }
}

__global__ void k_repack_q6k(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N, int nb,
                             long long dst_stride, int perm_hd) {
    const long long src_row = (long long)nb * 210;
    const long long total = (long long)N * src_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int v = (int)(i / src_row);
        const int off = (int)(i - (long long)v * src_row);
        const int b = off / 210, e = off % 210;
        long long d;
        if (e < 128) d = (long long)b * 128 + e;
        else if (e < 192) d = (long long)nb * 128 + b * 64 + (e - 128);
        else if (e < 208) d = (long long)nb * 192 + b * 16 + (e - 192);
        else d = (long long)nb * 208 + b * 2 + (e - 208);
        dst[(long long)v * dst_stride + d] = src[(long long)perm_src_row(v, perm_hd) * src_row + off];
    }
}

__global__ void k_permute_f32(const float* __restrict__ src, float* __restrict__ dst, int n, int perm_hd) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v < n) dst[v] = src[perm_src_row(v, perm_hd)];
}

// Decode-state control (single thread each).  args (device memory, copied from the host per call):
// [0] token, [1] pos, [2] max_steps, [3] max_seq, [4] n_stop, [5..12] stop ids.
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
}

// Prefill by decode steps: after a head-less pass, feed the next prompt token.
__global__ void k_state_next_prompt(TokenState* st, const int* prompt) {
    if (st->done) return;
    st->prompt_idx += 1;
    st->pos += 1;
    st->token = prompt[st->prompt_idx];
    if (st->pos >= st->max_seq) st->done = 1;
}

}  // namespace tfr
