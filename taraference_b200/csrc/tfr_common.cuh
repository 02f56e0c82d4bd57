// Shared device helpers for the sm_100a decode kernels.
//
// This translation unit is compiled with --use_fast_math, -ftz=true, -prec-div=false,
// -prec-sqrt=false, -fmad=true: the options the reference hands NVRTC
// (crates/core/src/cuda/device.rs:106-120).  Expressions written the same way as in the
// reference kernels therefore lower to the same approximate instructions (div.approx,
// ex2.approx, rsqrt.approx, sin/cos.approx), which is what makes the int8 activation
// quantiser bit-identical to the reference build.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define TFR_Q4_K 12
#define TFR_Q6_K 14
#define TFR_Q8_0 8
#define TFR_Q5_K 13
#define TFR_Q5_1 7
#define TFR_FULL_MASK 0xffffffffu

namespace tfr {

// kernels/common.cu:2-6
__device__ __forceinline__ float f16_to_f32(unsigned short h) {
    float o;
    asm("cvt.f32.f16 %0, %1;" : "=f"(o) : "h"(h));
    return o;
}

// kernels/common.cu:9-38: the KV-store rounding (round half up in magnitude).
__device__ __forceinline__ unsigned short f32_to_f16_bits_ref(float f) {
    unsigned int x = __float_as_uint(f);
    unsigned int sign = (x >> 16) & 0x8000u;
    unsigned int absx = x & 0x7fffffffu;
    if (absx == 0u) return (unsigned short)sign;
    if (absx >= 0x7f800000u) return (unsigned short)(sign | (absx == 0x7f800000u ? 0x7c00u : 0x7e00u));
    if (absx < 0x33000000u) return (unsigned short)sign;
    if (absx >= 0x47800000u) return (unsigned short)(sign | 0x7c00u);
    int e = (int)((absx >> 23) & 0xff) - 127 + 15;
    unsigned int mant = absx & 0x7fffffu;
    if (e <= 0) {
        if (e < -10) return (unsigned short)sign;
        mant |= 0x800000u;
        unsigned int shift = (unsigned int)(14 - e);
        unsigned int hm = mant >> shift;
        if ((mant >> (shift - 1)) & 1u) hm += 1u;
        return (unsigned short)(sign | hm);
    }
    unsigned int half = ((unsigned int)e << 10) | (mant >> 13);
    if (mant & 0x1000u) half += 1u;
    return (unsigned short)(sign | half);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(TFR_FULL_MASK, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(TFR_FULL_MASK, v, o));
    return v;
}

// Streaming 16-byte weight load: read-only path, do not keep in L1.
__device__ __forceinline__ int4 ldg_stream(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ int2 ldg_stream8(const void* p) {
    int2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.s32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// ---- mbarrier / bulk-copy (TMA) primitives, shared::cta only, no multicast -------------------
__device__ __forceinline__ unsigned int smem_u32(const void* p) { return (unsigned int)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned int parity) {
    unsigned int ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after a fixed number of polls (each poll may itself block for a
// hardware-defined short time) so that a lost copy can never hang the GPU.
constexpr int MBAR_POLL_LIMIT = 1 << 18;
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned int parity) {
    for (int i = 0; i < MBAR_POLL_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy (bulk copy) writes.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Untiled bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned int bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// 4-byte asynchronous copy global -> shared.
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// 16-byte asynchronous copy global -> shared (LDGSTS); n_src = 0 fills the destination with zeros.
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int n_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Blocks until at most N of this thread's committed copy groups are still in flight.
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Programmatic dependent launch (sm_90+): the first lets the next kernel in the stream start its
// prologue, the second blocks until the previous kernel has completed and its writes are visible.
// Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Optional timeline probe (test aid, only in builds with -DTFR_TEST_AIDS; the product library compiles it to nothing):
// when set, thread 0 of every CTA stores %globaltimer at eight points of a kernel into
// g_prof[(launch id * 160 + cta) * 8 + point].
#ifdef TFR_TEST_AIDS
__constant__ unsigned long long* g_prof = nullptr;
__device__ __forceinline__ void prof_mark(int point, int kernel_id = 0) {
    if (g_prof && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g_prof[((size_t)kernel_id * 160 + blockIdx.y * gridDim.x + blockIdx.x) * 8 + point] = t;
    }
}
#else
__device__ __forceinline__ void prof_mark(int, int = 0) {}
#endif

// Asks the memory system to bring a range into L2 (no destination, no completion to wait for).
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, unsigned int bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// Device-resident decode state shared by every kernel of the token loop.  The host never
// reads it while a burst is in flight; kernels read pos/token from here so one captured
// graph serves every position (the reference's `_d` kernel variants do the same with
// d_pos0 / d_token, crates/core/src/cuda/model.rs:71-73).
struct TokenState {
    int pos;        // position of the token being processed (= KV rows already filled)
    int token;      // id of the token being processed
    int step;       // tokens emitted so far in this burst
    int max_steps;  // burst length
    int done;       // set once a stop id was emitted or max_steps reached
    int n_stop;
    int stop_ids[8];
    int err;                       // non-zero: a kernel saw an impossible state
    unsigned int head_done;        // CTAs of the vocabulary head that have finished
    unsigned long long best;       // packed (orderable logit, ~index) running argmax
    int prompt_left;               // prompt tokens still to be fed (prefill by decode steps)
    int prompt_idx;
    int max_seq;                   // KV capacity; reaching it sets done
    int ring_off;                  // conv-history ring: slot of the current input = (pos + ring_off) % kernel
    unsigned int ar_epoch;         // tensor parallelism: all-reduces completed before this token (never reset)
    int force_prompt;              // 1: every step is fed the next prompt token, not its own argmax (verification)
};

// Orderable 64-bit key: larger logit wins; on equal logits the lower index wins.
__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
    unsigned int b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - (unsigned int)idx);
}
__device__ __forceinline__ int argmax_key_index(unsigned long long k) {
    return (int)(0xffffffffu - (unsigned int)(k & 0xffffffffull));
}

}  // namespace tfr
