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
// every rank owns the same rows.  A thread that finishes a row pair pushes it into slot [my_rank]
// of EVERY rank's exchange buffer through NVLink as ONE 16-byte store {v0, epoch, v1, epoch}: the
// value travels together with its own arrival mark (8-byte halves are written atomically), so
// there is no fence, no separate flag and no second trip.  The CTA then polls its tp slots per
// row pair until both marks carry the current epoch, sums them in rank order (the same order on
// all ranks: the replicated residual stream stays bit-identical) and applies the residual.  No
// grid-wide barrier and no second launch; a CTA only ever waits for its namesakes on the peers.
//
// The data buffers alternate with the parity of the all-reduce's index inside the token (a token has an
// even number of them, 2 per layer, so consecutive all-reduces always use different buffers, across token
// boundaries too, with or without a vocabulary head in between); a mark is only valid for its own
// monotonically increasing epoch.  Rank A can only reach all-reduce k+2 (the buffer of k) after every peer
// has delivered k+1, i.e. after the peers' kernel k has completed in stream order, so a slot is never
// overwritten while it is being read.  Every wait is bounded: on expiry the kernel records an
// error, ends the burst and returns.
#pragma once
#include "tfr_gemv.cuh"

namespace tfr {

constexpr int TP_MAX = 8;
constexpr unsigned long long TP_WAIT_NS = 2000000000ull;  // 2 s: far above any launch skew between ranks

// Layout of one rank's exchange buffer (device memory, opened by the peers through CUDA IPC).
struct TpLayout {
    size_t best_off, data_off, total;
    int k_max;
};
inline TpLayout tp_layout(int k_max) {
    TpLayout l{};
    l.k_max = (k_max + 3) & ~3;
    l.best_off = 0;                                       // uint4 [2][TP_MAX]: {lo, epoch, hi, epoch} of the argmax key
    l.data_off = (sizeof(uint4) * 2 * TP_MAX + 255) & ~(size_t)255;  // uint4 [2][TP_MAX][k_max / 2]: {v0, epoch, v1, epoch}
    l.total = l.data_off + sizeof(uint4) * 2 * TP_MAX * (size_t)(l.k_max / 2);
    return l;
}

struct TpComm {
    unsigned char* base[TP_MAX];  // exchange buffer of every rank, as mapped into this process
    TpLayout lay;
    int tp, rank;
    int ops_per_token;            // all-reduces of one decode step (2 per layer + the argmax)
};

__device__ __forceinline__ void st_sys_v4(uint4* p, unsigned a, unsigned b, unsigned c, unsigned d) {
    asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_sys_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Polls a {a, epoch, b, epoch} cell until both marks carry `epoch`, at most TP_WAIT_NS.
__device__ __forceinline__ bool tp_wait_cell(const uint4* cell, unsigned epoch, uint4& v) {
    v = ld_sys_v4(cell);
    if (v.y == epoch && v.w == epoch) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 64; i++) {
            v = ld_sys_v4(cell);
            if (v.y == epoch && v.w == epoch) return true;
        }
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
    __device__ __forceinline__ bool wants_residual() const { return false; }
    __device__ __forceinline__ float residual(int) const { return 0.f; }
    __device__ __forceinline__ void set_residual(const float*, int) {}
    __device__ __forceinline__ uint4* slot(int dst_rank, int src_rank) const {
        return reinterpret_cast<uint4*>(c.base[dst_rank] + c.lay.data_off) +
               ((size_t)(op_index & 1) * TP_MAX + src_rank) * (c.lay.k_max >> 1);
    }
    __device__ __forceinline__ void apply(int p, float v0, float v1) {
        for (int r = 0; r < c.tp; r++) st_sys_v4(slot(r, c.rank) + p, __float_as_uint(v0), epoch, __float_as_uint(v1), epoch);
    }
    __device__ void end(TokenState* st) {
        const int tid = threadIdx.x, cta = blockIdx.x;
        const int p0 = sh.begin(cta), np = sh.count(cta);
        bool ok = true;
        for (int i = tid; i < np; i += blockDim.x) {
            const int p = p0 + i;
            float a = 0.f, b = 0.f;
            for (int r = 0; r < c.tp; r++) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                ok = ok && tp_wait_cell(slot(c.rank, r) + p, epoch, v);  // after one expiry, do not wait again
                a += __uint_as_float(v.x);
                b += __uint_as_float(v.z);
            }
            if (ok) {
                x[2 * p] += a;
                if (2 * p + 1 < n_rows) x[2 * p + 1] += b;
            }
        }
        if (!ok) {
            st->err = 3;  // a peer never delivered its partial: the step's results are invalid
            st->done = 1;
        }
    }
};

// Argmax exchange of the vocabulary-parallel head: every rank contributes its packed
// (logit, ~global index) key; all ranks take the maximum.  Called by one thread.
__device__ __forceinline__ bool tp_allreduce_best(const TpComm& c, unsigned epoch, unsigned long long& best) {
    const int par = (int)(epoch & 1u);
    for (int r = 0; r < c.tp; r++)
        st_sys_v4(reinterpret_cast<uint4*>(c.base[r] + c.lay.best_off) + par * TP_MAX + c.rank, (unsigned)(best & 0xffffffffull),
                  epoch, (unsigned)(best >> 32), epoch);
    bool ok = true;
    unsigned long long b = 0ull;
    for (int r = 0; r < c.tp; r++) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        ok = ok && tp_wait_cell(reinterpret_cast<const uint4*>(c.base[c.rank] + c.lay.best_off) + par * TP_MAX + r, epoch, v);
        const unsigned long long k = ((unsigned long long)v.z << 32) | v.x;
        b = k > b ? k : b;
    }
    if (!ok) return false;
    best = b;
    return true;
}

}  // namespace tfr
