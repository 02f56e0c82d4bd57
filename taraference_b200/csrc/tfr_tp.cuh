// Tensor parallelism over NVLink peer memory: the all-reduce of a row-parallel GEMV happens
// inside the GEMV kernel's epilogue.
//
// The reference is single-GPU (crates/core/src/cuda/device.rs:85-95 opens device 0 only); this is
// new functionality whose parity target is the single-GPU result of the same model.  Megatron
// split: Q/K/V, gate/up and the vocabulary head are column-parallel (rows of the GGUF matrix),
// attn_output and ffn_down row-parallel (blocks along K), so every rank ends a row-parallel
// GEMV with a partial y[K] that must be summed over ranks.
//
// One-shot exchange, per CTA: all ranks launch the same grid with the same row shares, so CTA c of
// every rank owns the same rows.  It pushes its partial rows into slot [my_rank] of EVERY rank's
// exchange buffer with plain stores through NVLink, publishes a release flag per peer, waits for
// the tp flags addressed to it, then sums the tp slots in rank order (the same order on all
// ranks: the replicated residual stream stays bit-identical) and applies the residual.  No
// grid-wide barrier and no second launch; a CTA only ever waits for its namesakes on the peers.
//
// Buffers alternate with the parity of a monotonically increasing epoch.  Rank A can only reach
// all-reduce k+2 (same parity as k) after every peer has signalled k+1, i.e. after the peers'
// kernel k has completed in stream order, so a slot is never overwritten while it is being read.
// Every wait is bounded: on expiry the kernel records an error, ends the burst and returns.
#pragma once
#include "tfr_gemv.cuh"

namespace tfr {

constexpr int TP_MAX = 8;
constexpr int TP_MAX_CTAS = 160;                       // flags per source rank (>= SM count)
constexpr unsigned long long TP_WAIT_NS = 2000000000ull;  // 2 s: far above any launch skew between ranks

// Layout of one rank's exchange buffer (device memory, opened by the peers through CUDA IPC).
struct TpLayout {
    size_t flags_off, best_off, bflags_off, data_off, total;
    int k_max;
};
inline TpLayout tp_layout(int k_max) {
    TpLayout l{};
    l.k_max = (k_max + 3) & ~3;
    l.flags_off = 0;                                                  // unsigned [TP_MAX][TP_MAX_CTAS]
    l.bflags_off = l.flags_off + sizeof(unsigned) * TP_MAX * TP_MAX_CTAS;  // unsigned [TP_MAX]
    l.best_off = (l.bflags_off + sizeof(unsigned) * TP_MAX + 15) & ~(size_t)15;  // u64 [2][TP_MAX]
    l.data_off = (l.best_off + sizeof(unsigned long long) * 2 * TP_MAX + 255) & ~(size_t)255;  // float [2][TP_MAX][k_max]
    l.total = l.data_off + sizeof(float) * 2 * TP_MAX * (size_t)l.k_max;
    return l;
}

struct TpComm {
    unsigned char* base[TP_MAX];  // exchange buffer of every rank, as mapped into this process
    TpLayout lay;
    int tp, rank;
    int ops_per_token;            // all-reduces of one decode step (2 per layer + the argmax)
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float2 ld_sys_f2(const float* p) {
    float2 v;
    asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys_f2(float* p, float a, float b) {
    asm volatile("st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Waits until *flag has reached `epoch` (wrap-safe), at most TP_WAIT_NS.
__device__ __forceinline__ bool tp_wait_flag(const unsigned* flag, unsigned epoch) {
    if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
        if (global_timer_ns() - t0 > TP_WAIT_NS) return false;
    }
}

// Row-parallel epilogue: x += sum over ranks of (W_rank . act_rank), kernels/gemv.cu:367-373 residual
// rule (2 = accumulate in place) applied once to the reduced sum.
struct EpiAllReduce {
    static constexpr int MODE = EPI_PAIRS;
    float* x;          // [n_rows] replicated residual stream, updated in place
    int n_rows;
    Share sh;          // row-pair shares of the matrix over the grid (the same on every rank)
    TpComm c;
    int op_index;      // which all-reduce of the token this is
    unsigned epoch;
    __device__ void begin(const TokenState* st) { epoch = st->ar_epoch + (unsigned)op_index + 1u; }
    __device__ __forceinline__ float* slot(int dst_rank, int src_rank) const {
        return reinterpret_cast<float*>(c.base[dst_rank] + c.lay.data_off) +
               ((size_t)(epoch & 1u) * TP_MAX + src_rank) * c.lay.k_max;
    }
    __device__ __forceinline__ void apply(int p, float v0, float v1) {
        for (int r = 0; r < c.tp; r++) st_sys_f2(slot(r, c.rank) + 2 * p, v0, v1);
    }
    __device__ void end(TokenState* st) {
        __shared__ int ok_s;
        const int tid = threadIdx.x, cta = blockIdx.x;
        const int p0 = sh.begin(cta), np = sh.count(cta);
        if (tid == 0) ok_s = 1;
        __syncthreads();  // every partial of this CTA has been issued
        if (np > 0 && tid < c.tp) {
            __threadfence_system();
            unsigned* theirs = reinterpret_cast<unsigned*>(c.base[tid] + c.lay.flags_off) + c.rank * TP_MAX_CTAS + cta;
            st_release_sys(theirs, epoch);
            const unsigned* mine = reinterpret_cast<const unsigned*>(c.base[c.rank] + c.lay.flags_off) + tid * TP_MAX_CTAS + cta;
            if (!tp_wait_flag(mine, epoch)) ok_s = 0;
        }
        __syncthreads();
        if (!ok_s) {
            if (tid == 0) {
                st->err = 3;  // a peer never delivered its partial: the step's results are invalid
                st->done = 1;
            }
            return;
        }
        for (int i = tid; i < np; i += blockDim.x) {
            const int p = p0 + i;
            float a = 0.f, b = 0.f;
            for (int r = 0; r < c.tp; r++) {
                const float2 v = ld_sys_f2(slot(c.rank, r) + 2 * p);
                a += v.x;
                b += v.y;
            }
            x[2 * p] += a;
            if (2 * p + 1 < n_rows) x[2 * p + 1] += b;
        }
    }
};

// Argmax exchange of the vocabulary-parallel head: every rank contributes its packed
// (logit, ~global index) key; all ranks take the maximum.  Called by one thread.
__device__ __forceinline__ bool tp_allreduce_best(const TpComm& c, unsigned epoch, unsigned long long& best) {
    const int par = (int)(epoch & 1u);
    for (int r = 0; r < c.tp; r++)
        st_sys_u64(reinterpret_cast<unsigned long long*>(c.base[r] + c.lay.best_off) + par * TP_MAX + c.rank, best);
    __threadfence_system();
    for (int r = 0; r < c.tp; r++)
        st_release_sys(reinterpret_cast<unsigned*>(c.base[r] + c.lay.bflags_off) + c.rank, epoch);
    bool ok = true;
    for (int r = 0; r < c.tp; r++)
        ok = tp_wait_flag(reinterpret_cast<const unsigned*>(c.base[c.rank] + c.lay.bflags_off) + r, epoch) && ok;
    if (!ok) return false;
    unsigned long long b = 0ull;
    for (int r = 0; r < c.tp; r++) {
        const unsigned long long v = ld_sys_u64(reinterpret_cast<const unsigned long long*>(c.base[c.rank] + c.lay.best_off) + par * TP_MAX + r);
        b = v > b ? v : b;
    }
    best = b;
    return true;
}

}  // namespace tfr
