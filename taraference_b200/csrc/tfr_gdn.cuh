// Kernels of the hybrid (Qwen3.5-style) layers: the Gated-DeltaNet decode step and the
// per-head Q/K RMSNorm + partial RoPE + KV store of the gated full-attention layers.
//
// Reference: kernels/deltanet.cu:530-622 (conv + SiLU + split + L2), :628-728 (decay, delta rule,
// read-out, gated RMSNorm), :144-173 (Q|gate split), :189-235 (Q/K norm + partial RoPE),
// kernels/ops.cu:471-486 (f16 KV store).  The reference runs the mixer as two launches with Q, K, V
// bounced through global memory and walks the 128x128 state twice (decay pass, then update);
// here one CTA per V head does the conv for the 3 x 128 channels it needs, keeps its 64 KB
// state in registers and touches every state element exactly once (one load, one store).
#pragma once
#include "tfr_common.cuh"

namespace tfr {

constexpr int GDN_D = 128;        // state size per head (ssm.state_size of the supported models)
constexpr int GDN_PARTS = 4;      // row slabs of the state handled by different threads of a column
constexpr int GDN_THREADS = GDN_D * GDN_PARTS;
constexpr int GDN_MAX_KERNEL = 4;

struct GdnArgs {
    const float* proj;     // [channels | val_dim | n_v | n_v]: raw qkv, z gate, beta, alpha projections
    const float* conv_w;   // [channels][kernel], tap k of channel c at k + c * kernel (GGUF dims [kernel, channels])
    float* conv_ring;      // [kernel][channels]: slot (pos + ring_off) % kernel takes the current input
    float* state;          // [n_v][128][128] fp32
    const float* ssm_a;    // [n_v], already -exp(A_log)
    const float* ssm_dt;   // [n_v]
    const float* norm_w;   // [128]
    float* out;            // [n_v * 128]: feeds the ssm_out projection
    int n_k, n_v, kernel;
    float eps;
    int slot;              // ring slot when st == nullptr
};

// The conv history is a ring indexed by position instead of the reference's shifted window
// (deltanet.cu:552-558): nothing moves, and the two V heads that share a K head can both read
// the Q/K history without racing against a shift.
__device__ __forceinline__ float gdn_conv_channel(const GdnArgs& a, int c, int channels, int slot, bool write) {
    const int km1 = a.kernel - 1;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < GDN_MAX_KERNEL - 1; k++) {
        if (k < km1) {
            int s = slot - km1 + k;
            s += s < 0 ? a.kernel : 0;
            acc += a.conv_w[(size_t)c * a.kernel + k] * a.conv_ring[(size_t)s * channels + c];
        }
    }
    const float xt = a.proj[c];
    acc += a.conv_w[(size_t)c * a.kernel + km1] * xt;
    if (write) a.conv_ring[(size_t)slot * channels + c] = xt;
    return acc / (1.f + expf(-acc));
}

__global__ void __launch_bounds__(GDN_THREADS, 1) k_gdn_step(GdnArgs a, const TokenState* st) {
    griddep_wait();  // the projections come from the previous kernel
    griddep_launch_dependents();
    if (st && st->done) return;
    constexpr int D = GDN_D, R = D / GDN_PARTS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.x, hk = h % a.n_k;
    const int key_dim = a.n_k * D, val_dim = a.n_v * D, channels = 2 * key_dim + val_dim;
    const int slot = st ? (st->pos + st->ring_off) % a.kernel : a.slot;
    const int j = tid & (D - 1), part = tid >> 7;
    float* S = a.state + (size_t)h * D * D;

    __shared__ float sq[D], sk[D], sv[D];
    __shared__ float red[GDN_PARTS][D];
    __shared__ float wred[16];
    __shared__ float sg, sb;

    // the state loads go out first; the conv and the norms run while they are in flight
    float s[R];
#pragma unroll
    for (int r = 0; r < R; r++) s[r] = __ldcs(S + (size_t)(part * R + r) * D + j);

    float cv = 0.f;
    if (part < 3) {
        // part 0: Q channel j of K head hk, part 1: K channel, part 2: V channel j of head h
        const int c = part == 0 ? hk * D + j : part == 1 ? key_dim + hk * D + j : 2 * key_dim + h * D + j;
        cv = gdn_conv_channel(a, c, channels, slot, part == 2 || h < a.n_k);
    }
    if (tid == 0) {
        const float br = a.proj[channels + val_dim + h];
        sb = 1.f / (1.f + expf(-br));
        const float z = a.proj[channels + val_dim + a.n_v + h] + a.ssm_dt[h];
        const float sp = (z > 20.f) ? z : log1pf(expf(z));
        sg = expf(sp * a.ssm_a[h]);
    }
    // L2 norms of Q and K (sum of squares, deltanet.cu:598-620)
    const float sqr = warp_sum(part < 2 ? cv * cv : 0.f);
    if (lane == 0) wred[warp] = sqr;
    __syncthreads();
    if (part == 0) {
        const float inv = rsqrtf(wred[0] + wred[1] + wred[2] + wred[3] + a.eps);
        sq[j] = (cv * inv) * 0.08838834764f;  // 1/sqrt(128), deltanet.cu:668
    } else if (part == 1) {
        const float inv = rsqrtf(wred[4] + wred[5] + wred[6] + wred[7] + a.eps);
        sk[j] = cv * inv;
    } else if (part == 2) {
        sv[j] = cv;
    }
    __syncthreads();
    const float g = sg, b = sb;

    // decay and the memory read-out of this column slab
    float kv = 0.f;
#pragma unroll
    for (int r = 0; r < R; r++) {
        s[r] *= g;
        kv += s[r] * sk[part * R + r];
    }
    red[part][j] = kv;
    __syncthreads();
    const float delta = (sv[j] - (red[0][j] + red[1][j] + red[2][j] + red[3][j])) * b;
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const float ki = sk[part * R + r];
        s[r] += ki * delta;
        __stcs(S + (size_t)(part * R + r) * D + j, s[r]);
        o += s[r] * sq[part * R + r];
    }
    red[part][j] = o;
    __syncthreads();
    // gated RMSNorm over the head's 128 outputs (deltanet.cu:703-727)
    float oj = 0.f;
    if (part == 0) oj = red[0][j] + red[1][j] + red[2][j] + red[3][j];
    const float ss = warp_sum(oj * oj);
    if (part == 0 && lane == 0) wred[8 + warp] = ss;
    __syncthreads();
    if (part == 0) {
        const float scale = rsqrtf((wred[8] + wred[9] + wred[10] + wred[11]) * (1.f / (float)D) + a.eps);
        const float gate = a.proj[channels + h * D + j];
        const float silu = gate / (1.f + expf(-gate));
        a.out[h * D + j] = oj * scale * a.norm_w[j] * silu;
    }
}

// Gated full attention, between the raw projections and the attention kernel: one CTA per
// query head or KV head.  raw = [n_head x (Q_h | G_h) | K | V].
struct QkNormArgs {
    const float* raw;
    const float* q_norm;      // [hd] or nullptr (no norm)
    const float* k_norm;
    float* q_out;             // [n_head * hd]
    float* gate_out;          // [n_head * hd]
    unsigned short* kc;       // layer base [max_seq][n_kv * hd]
    unsigned short* vc;
    int n_head, n_kv, hd, n_rot;
    float theta, eps;
    int pos;                  // used when st == nullptr
};

__global__ void __launch_bounds__(256) k_qk_norm_rope_store(QkNormArgs a, const TokenState* st) {
    griddep_wait();
    griddep_launch_dependents();
    if (st && st->done) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.x, hd = a.hd;
    const bool isq = head < a.n_head;
    const int hk = head - a.n_head;
    const int pos = st ? st->pos : a.pos;
    const int qn2 = 2 * a.n_head * hd, kvdim = a.n_kv * hd;
    const float* src = isq ? a.raw + (size_t)head * 2 * hd : a.raw + qn2 + (size_t)hk * hd;
    const float* w = isq ? a.q_norm : a.k_norm;
    __shared__ float xs[256];
    __shared__ float wred[8];
    const float x = tid < hd ? src[tid] : 0.f;
    const float ss = warp_sum(x * x);
    if (lane == 0) wred[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < 8; i++) tot += wred[i];
    float y = x;
    if (w && tid < hd) y = x * rsqrtf(tot / (float)hd + a.eps) * w[tid];
    xs[tid] = y;
    __syncthreads();
    const int half = a.n_rot >> 1;
    if (tid < a.n_rot) {
        const int i = tid < half ? tid : tid - half;
        const float freq = powf(a.theta, -2.f * (float)i / (float)a.n_rot);
        const float ang = (float)pos * freq;
        const float c = cosf(ang), sn = sinf(ang);
        const float x0 = xs[i], x1 = xs[i + half];
        y = tid < half ? x0 * c - x1 * sn : x0 * sn + x1 * c;
    }
    if (tid >= hd) return;
    if (isq) {
        a.q_out[head * hd + tid] = y;
        a.gate_out[head * hd + tid] = src[hd + tid];
    } else {
        a.kc[(size_t)pos * kvdim + hk * hd + tid] = f32_to_f16_bits_ref(y);
        a.vc[(size_t)pos * kvdim + hk * hd + tid] = f32_to_f16_bits_ref(a.raw[qn2 + kvdim + hk * hd + tid]);
    }
}

}  // namespace tfr
