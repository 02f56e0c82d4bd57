// __global__ kernels of the batch-1 decode path and their launch helpers.
#pragma once
#include "tfr_attn.cuh"
#include "tfr_gemv.cuh"

namespace tfr {

// ------------------------------------------------------------------ epilogues

// y = W x (+y) (+bias): kernels/gemv.cu:367-373 residual rule (2 = accumulate in place).
struct EpiStore {
    static constexpr int ROW_ALIGN = 1;
    float* out;
    const float* bias;
    int use_res;
    __device__ void begin(const TokenState*) {}
    __device__ __forceinline__ void apply(int v, const float* s, int lane) {
        if (lane) return;
        float acc = s[0];
        if (use_res == 2) acc += out[v];
        if (bias) acc += bias[v];
        out[v] = acc;
    }
    __device__ void end(TokenState*) {}
};

// h = silu(gate.x) * (up.x), kernels/gemv.cu:2570-2574.  vrows (2j, 2j+1) = (gate_j, up_j).
struct EpiSilu {
    static constexpr int ROW_ALIGN = 2;
    float* out;
    __device__ void begin(const TokenState*) {}
    __device__ __forceinline__ void apply(int v, const float* s, int lane) {
        if (lane) return;
        const float gate = s[0], up = s[1];
        out[v >> 1] = (gate / (1.f + __expf(-gate))) * up;
    }
    __device__ void end(TokenState*) {}
};

// Fused Q/K/V epilogue: bias, neox RoPE (kernels/ops.cu:348-371) and the f16 KV store
// (kernels/ops.cu:471-486).  Q and K rows were re-ordered at upload so that the RoPE
// partners (i, i + hd/2) of a head are adjacent vrows (2i, 2i+1); biases likewise.
struct EpiQkv {
    static constexpr int ROW_ALIGN = 2;
    float* q_out;            // [n_head * hd] natural order
    unsigned short* kc;      // layer base [max_seq][kvdim]
    unsigned short* vc;
    const float* bias;       // [nq + nk + nv] in vrow order, or nullptr
    int nq, nk, hd, kvdim;
    float theta;
    int pos;
    __device__ void begin(const TokenState* st) {
        if (st) pos = st->pos;
    }
    __device__ __forceinline__ void apply(int v, const float* s, int lane) {
        if (lane) return;
        float x0 = s[0], x1 = s[1];
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
    static constexpr int ROW_ALIGN = 1;
    float* logits;
    int* out_tokens;   // ring of emitted tokens, indexed by TokenState::step
    unsigned long long best;
    __device__ void begin(const TokenState*) { best = 0ull; }
    __device__ __forceinline__ void apply(int v, const float* s, int lane) {
        if (lane) return;
        logits[v] = s[0];
        const unsigned long long k = argmax_key(s[0], v);
        best = k > best ? k : best;
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
    int swz;
    int want_xf;
    float* raw_out;       // embedding source only: CTA 0 stores the decoded row here (residual stream)
    int token;            // embedding source without TokenState
};

template <class Map, class Epi>
__global__ void __launch_bounds__(GEMV_THREADS, 4)
k_gemv(PrepArgs pa, Map map, Epi epi_in, int K, int groups, TokenState* st) {
    if (st && st->done) return;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float red[GEMV_THREADS];
    Epi epi = epi_in;
    Act act = act_carve(smem, K, pa.want_xf != 0);
    const size_t act_bytes = (act_smem_bytes(K, pa.want_xf != 0) + 15) & ~(size_t)15;
    float* pbuf = reinterpret_cast<float*>(smem + act_bytes);
    const int PT = gemv_partial_floats(K, Epi::ROW_ALIGN);
    if (pa.vec) {
        SrcVec src{pa.vec};
        act_prepare(act, src, pa.normw, pa.eps, K, pa.swz, (float*)nullptr, red);
    } else {
        int tok = st ? st->token : pa.token;
        if (tok < 0 || tok >= pa.embed.N) {
            if (st && threadIdx.x == 0) st->err = 1;
            tok = 0;
        }
        SrcEmbed src{pa.embed, tok};
        act_prepare(act, src, pa.normw, pa.eps, K, pa.swz, blockIdx.x == 0 ? pa.raw_out : (float*)nullptr, red);
    }
    epi.begin(st);
    int g0, g1;
    cta_share(groups, blockIdx.x, gridDim.x, g0, g1);
    gemv_tiles(map, epi, act, K, g0, g1, pbuf, PT);
    epi.end(st);
}

inline size_t gemv_smem_bytes(int K, bool want_xf, int row_align) {
    size_t act_bytes = (act_smem_bytes(K, want_xf) + 15) & ~(size_t)15;
    return act_bytes + 2 * (size_t)gemv_partial_floats(K, row_align) * sizeof(float);
}

template <class Map, class Epi>
inline cudaError_t launch_gemv(cudaStream_t stream, int grid, const PrepArgs& pa, const Map& map, const Epi& epi, int K,
                               int groups, TokenState* st) {
    const size_t smem = gemv_smem_bytes(K, pa.want_xf != 0, Epi::ROW_ALIGN);
    if (grid > groups) grid = groups;
    if (grid < 1) grid = 1;
    k_gemv<Map, Epi><<<grid, GEMV_THREADS, smem, stream>>>(pa, map, epi, K, groups, st);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ small kernels

// Stand-alone quantiser with linear output (A1), same expression as act_prepare.
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

// Integer contract taps.  Q4_K: I[row][K/32], S[row][K/32].  Q6_K: J[row][K/16].
__global__ void k_int_dots(Mat m, const signed char* q8, const float* d8, int* outA, int* outB) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int K = m.K, G = K >> 6;
    Act act = act_carve(smem, K, false);
    act_from_q8(act, q8, d8, K, m.type == TFR_Q4_K ? SWZ_Q4 : SWZ_Q6);
    const int total = m.N * G;
    for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < total; f += gridDim.x * blockDim.x) {
        const int r = f / G, u = f % G;
        UnitW w;
        const uint8_t* row = m.data + (long long)r * m.row_stride;
        if (m.type == TFR_Q4_K) {
            load_unit(w, WT_Q4K, row, m.nb, u);
            const Q4Ints qi = q4k_unit_ints(w, act, u, G);
            int* I = outA + (size_t)r * (K / 32) + 2 * u;
            int* S = outB + (size_t)r * (K / 32) + 2 * u;
            I[0] = qi.I0;
            I[1] = qi.I1;
            S[0] = qi.S0;
            S[1] = qi.S1;
        } else {
            load_unit(w, WT_Q6K, row, m.nb, u);
            int J[4];
            q6k_unit_ints(w, act, u, G, J);
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

// Decode-state control (single thread each).
__global__ void k_state_begin(TokenState* st, int token, int pos, int max_steps, int max_seq, int n_stop, int s0, int s1,
                              int s2, int s3, int s4, int s5, int s6, int s7) {
    st->token = token;
    st->pos = pos;
    st->step = 0;
    st->max_steps = max_steps;
    st->max_seq = max_seq;
    st->done = 0;
    st->n_stop = n_stop;
    const int s[8] = {s0, s1, s2, s3, s4, s5, s6, s7};
    for (int i = 0; i < 8; i++) st->stop_ids[i] = s[i];
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
