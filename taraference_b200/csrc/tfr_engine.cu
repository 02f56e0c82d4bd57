// Engine and C ABI of the B200 batch-1 decode library (see include/tarafer_b200.h).
//
// The layer schedule follows crates/core/src/cuda/layer.rs:142-709 (attention block),
// :1210-1456 (dense FFN) and :2125-2259 (vocabulary head) at n_tok = 1, folded from the
// reference's 16 launches per layer into five:
//   1. RMSNorm + Q8 + Q/K/V (+bias) + RoPE + f16 KV store
//   2. split-KV flash-decode with in-kernel merge
//   3. Q8 + o-proj + residual
//   4. RMSNorm + Q8 + gate/up + SiLU*mul
//   5. Q8 + down + residual
// plus one head kernel per token (RMSNorm + Q8 + lm_head + argmax + state advance); the
// embedding lookup is folded into layer 0's first kernel.  Position and token live in
// device memory (TokenState), so one captured CUDA graph per token is replayed back to
// back for a whole burst without any host round-trip.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <dlfcn.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/tarafer_b200.h"
#include "tfr_kernels.cuh"
#include "tfr_chunk.cuh"
#include "tfr_loop.cuh"

using namespace tfr;

// ------------------------------------------------------------------ objects

struct tfr_mat {
    Mat m{};
    void* dev = nullptr;
    size_t bytes = 0;
    int perm_hd = 0;
};

// Layer kinds of crates/core/src/config.rs (LayerKind) with the hybrid's gated variant of full attention.
enum { LAYER_DENSE = 0, LAYER_LINEAR = 1, LAYER_FULL_GATED = 2 };

struct LayerW {
    int kind = LAYER_DENSE;
    tfr_mat *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
    float* bias_qkv = nullptr;  // vrow order, or nullptr
    float *attn_norm = nullptr, *ffn_norm = nullptr;
    // linear (Gated-DeltaNet) layers: the four input projections stacked into one matrix
    tfr_mat *gdn_proj = nullptr, *ssm_out = nullptr;
    tfr_mat* proj4[4] = {nullptr, nullptr, nullptr, nullptr};  // the four projections kept apart when their types differ
    float *conv_w = nullptr, *ssm_a = nullptr, *ssm_dt = nullptr, *ssm_norm = nullptr;
    // gated full-attention layers
    float *q_norm = nullptr, *k_norm = nullptr;
};

// Raw GGUF bytes of a matrix kept on the host until tfr_finalize_load stacks it with its siblings.
struct HostRaw {
    int type = 0;
    int64_t K = 0, N = 0;
    std::vector<uint8_t> bytes;
};

struct VecT {
    float* dev = nullptr;
    int64_t n = 0;
};

// NCCL, loaded at run time and only for the comparison mode of the tensor-parallel engine (the product
// path all-reduces inside its own kernels).  Minimal declarations of the stable NCCL 2.x C API.
struct NcclId {  // ncclUniqueId: 128 opaque bytes, passed by value
    char b[128];
};
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
constexpr int NCCL_UINT64 = 5, NCCL_FLOAT32 = 7, NCCL_SUM = 0, NCCL_MAX = 2;
static NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h) {
            api.lib = h;
            api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
            api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
            api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
            api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
            if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy) api.lib = nullptr;
        }
    }
    return api.lib ? &api : nullptr;
}

// This rank's share of the model (Megatron split).  With tp == 1 it covers everything.
struct TpPlan {
    int tp = 1, rank = 0;
    int n_head = 0, n_kv = 0, nq = 0, nkv = 0;  // local heads and their widths
    int q_lo = 0;                               // first element of the local heads in the full attention output
    int wo_b0 = 0, wo_b1 = 0;                   // K blocks of attn_output that cover the local heads
    int attn_off = 0, attn_width = 0;           // local heads sit at attn[attn_off ..) of a zero-padded vector
    int ff_b0 = 0, ff_b1 = 0, ff = 0;           // block-aligned slice of the FFN width
    int v0 = 0, v1 = 0;                         // vocabulary rows of the head
};

constexpr int TFR_MAX_BURST = 8192;
constexpr int TFR_MAX_PROMPT = 65536;

struct tfr_engine {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    std::string err;
    tfr_model_config cfg{};
    TpPlan plan{};
    TpComm comm{};
    unsigned char* comm_local = nullptr;
    bool peers_wired = false, comm_ipc = false;  // peers_wired: every rank's exchange buffer is mapped (tfr_tp_attach_*)
    bool nccl_ready = false;                     // the comparison mode's communicator exists
    // comparison mode: partial sums through ncclAllReduce between kernels instead of the in-kernel exchange
    void* nccl_comm = nullptr;
    bool use_nccl = false;
    float* ypart = nullptr;
    unsigned long long* best_buf = nullptr;
    bool has_cfg = false, finalized = false;
    std::map<std::string, tfr_mat*> mats;
    std::map<std::string, VecT> vecs;
    std::map<std::string, HostRaw> held;
    std::vector<LayerW> layers;
    tfr_mat *token_embd = nullptr, *head = nullptr, *head_special = nullptr;
    int vocab_limit = 0, special_id = -1;  // shortlisted head (load.rs:285-352); 0: the whole vocabulary
    float* output_norm = nullptr;
    // workspaces
    float *x = nullptr, *q = nullptr, *attn = nullptr, *h = nullptr, *logits = nullptr, *partial = nullptr;
    float *proj = nullptr, *qgate = nullptr;  // hybrid: raw projections; sigmoid gate of the attention output
    unsigned int* counters = nullptr;
    TokenState* st = nullptr;
    TokenState* st_host = nullptr;  // pinned
    int *out_tokens = nullptr, *out_host = nullptr, *prompt = nullptr;
    int *args_dev = nullptr, *args_host = nullptr;  // per-call scalars: pinned host -> device
    int attn_S = 1, attn_S_staged = 1, attn_min_keys = 64;  // splits per KV head of the two attention instances
    float* layer_taps = nullptr;  // [n_layer][n_embd] residual stream after each layer (test aid)
    // [n_layer][...] the other vectors a dense layer quantises: attention output, residual after o-proj, SiLU*mul (test aid)
    float *tap_attn = nullptr, *tap_mid = nullptr, *tap_h = nullptr;
    // graphs
    bool use_graph = true;
    cudaGraphExec_t g_decode = nullptr, g_body = nullptr;
    const tfr_kv* graph_kv = nullptr;
    int nodes_decode = 0, nodes_body = 0;
    int64_t launches = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.f;
    // persistent decode loop (tfr_loop.cuh): one cooperative kernel per call instead of a graph per token
    bool loop_ok = false;
    int decode_path = 0;  // 0: the loop when the model qualifies, 1: chained kernels, 2: the loop or an error
    std::string loop_why;
    LoopArgs loop{};
    LoopLayer* loop_layers = nullptr;
    unsigned int* loop_bar = nullptr;
    unsigned long long* loop_best = nullptr;
    float* loop_vec = nullptr;  // the vectors the loop's phases hand to one another, one allocation
    size_t loop_vec_n = 0;
    size_t loop_smem = 0;
    int loop_grid = 0;
    int* loop_blob = nullptr;
    uint4* loop_head_tasks = nullptr;
    unsigned long long* loop_prof = nullptr;
    int loop_prof_step = -1, loop_prof_points = 0;
    // multi-token chunks (tfr_chunk.cuh): prompts and verification batches
    int chunk_tokens = CHUNK_MAX_TOKENS;  // 0: every token of a prompt is a decode step
    bool chunk_ok = false;
    std::string chunk_why;
    float *cx = nullptr, *cq = nullptr, *cattn = nullptr, *ch = nullptr, *cxn = nullptr, *clogits = nullptr, *cpart = nullptr;
    size_t cpart_floats = 0;
    unsigned char* cact = nullptr;
    size_t cact_stride = 0;
    unsigned long long* ckeys = nullptr;  // per-row, per-slice argmax keys of a verification pass
    unsigned int* ccount = nullptr;       // per-row arrival counters, zero between launches
};

struct tfr_kv {
    tfr_engine* e = nullptr;
    unsigned short *k = nullptr, *v = nullptr;
    int len = 0, max_seq = 0;
    size_t layer_stride = 0;  // elements
    // K/V exist for the softmax-attention layers only (kv.rs:8-12 keeps empty buffers for linear layers):
    // kv_slot[layer] is the layer's index into the compact arrays, -1 for a Gated-DeltaNet layer
    std::vector<int> kv_slot;
    int n_kv_layers = 0;
    // hybrid models (kv.rs:12-15): per layer the fp32 state S[n_v][128][128] and the conv history,
    // held as a ring of `kernel` slots of [channels] (see tfr_gdn.cuh)
    float *ssm = nullptr, *conv = nullptr;
    size_t ssm_stride = 0, conv_stride = 0;  // floats per layer
    long long rec_steps = 0;                 // tokens the recurrent state has absorbed
};

static bool is_hybrid(const tfr_engine* e) { return e->cfg.hybrid != 0; }
static unsigned short* kv_k(const tfr_kv* kv, int li) { return kv->k + (size_t)(kv->kv_slot[li] < 0 ? 0 : kv->kv_slot[li]) * kv->layer_stride; }
static unsigned short* kv_v(const tfr_kv* kv, int li) { return kv->v + (size_t)(kv->kv_slot[li] < 0 ? 0 : kv->kv_slot[li]) * kv->layer_stride; }
// A forward call may run: the exchange the engine is set to use has everything it needs.
static bool tp_ready(const tfr_engine* e) { return e->use_nccl ? e->nccl_ready : e->peers_wired; }
static int gdn_channels(const tfr_model_config& c) { return (2 * c.ssm_group_count + c.ssm_time_step_rank) * c.ssm_state_size; }
static int gdn_val_dim(const tfr_model_config& c) { return c.ssm_time_step_rank * c.ssm_state_size; }
static int layer_kind(const tfr_model_config& c, int i) {
    if (!c.hybrid) return LAYER_DENSE;
    const int iv = c.full_attention_interval > 0 ? c.full_attention_interval : 4;  // config.rs:186-199
    return (i + 1) % iv == 0 ? LAYER_FULL_GATED : LAYER_LINEAR;
}

static int fail(tfr_engine* e, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (e) e->err = buf;
    return code;
}

#define CU(e, call)                                                                              \
    do {                                                                                         \
        cudaError_t _r = (call);                                                                 \
        if (_r != cudaSuccess) return fail(e, TFR_E_CUDA, "%s: %s", #call, cudaGetErrorString(_r)); \
    } while (0)

static size_t raw_bytes(int type, int64_t K, int64_t N) {
    int64_t nb = K / 256;
    if (type == TFR_Q4_K) return (size_t)(N * nb * 144);
    if (type == TFR_Q6_K) return (size_t)(N * nb * 210);
    if (type == TFR_Q8_0) return (size_t)(N * nb * Q8_SUPER_BYTES);
    if (type == TFR_Q5_K) return (size_t)(N * nb * 176);
    if (type == TFR_Q5_1) return (size_t)(N * nb * 8 * 24);
    return 0;
}

template <class F>
static void configure_kernel(F f, bool dynamic) {
    if (dynamic) cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMV_SMEM_MAX);
    // one L1/shared split for every kernel of the token loop: a change of carve-out between two
    // launches drains the SMs
    cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// CUDA function attributes, occupancy answers and the stand-alone operators' scratch are per-device state: one
// process may drive several GPUs (tfr_tp_attach_pointers), so everything below is kept per device ordinal.
constexpr int TFR_MAX_DEVICES = 64;
static int current_device_slot() {
    int dev = 0;
    cudaGetDevice(&dev);
    return dev >= 0 && dev < TFR_MAX_DEVICES ? dev : 0;
}

static void configure_kernels_once() {
    static bool done[TFR_MAX_DEVICES] = {};
    const int dev = current_device_slot();
    if (done[dev]) return;
    done[dev] = true;
    configure_kernel(k_gemv<BlockQ4, EpiQkv>, true);
    configure_kernel(k_gemv<BlockQ4, EpiStore>, true);
    configure_kernel(k_gemv<BlockQ6, EpiStore>, true);
    configure_kernel(k_gemv<BlockQ4, EpiSilu>, true);
    configure_kernel(k_gemv<BlockQ8, EpiStore>, true);
    configure_kernel(k_gemv<BlockQ8, EpiLogits>, true);
    configure_kernel(k_gemv<BlockQ8, EpiAllReduce>, true);
    configure_kernel(k_gemv<BlockQ4, EpiAllReduce>, true);
    configure_kernel(k_gemv<BlockQ6, EpiAllReduce>, true);
    configure_kernel(k_gemv<BlockQ4, EpiLogits>, true);
    configure_kernel(k_gemv<BlockQ6, EpiLogits>, true);
#ifdef TFR_TEST_AIDS
    configure_kernel(k_int_dots<BlockQ8>, true);
    configure_kernel(k_int_dots<BlockQ4>, true);
    configure_kernel(k_int_dots<BlockQ6>, true);
#endif
    configure_kernel(k_gemm_q8<BlockQ4>, true);
    configure_kernel(k_gemm_q8<BlockQ6>, true);
    configure_kernel(k_gemm_q8<BlockQ8>, true);
    configure_kernel(k_gemm_mma_q6<64>, true);
    configure_kernel(k_gemm_mma_q6<16>, true);
    configure_kernel(k_gemm_splitk_finish, false);
    configure_kernel(k_gemm_mma_q4<4, true, 64>, true);
    configure_kernel(k_gemm_mma_q4<1, true, 64>, true);
    configure_kernel(k_gemm_mma_q4<4, false, 64>, true);
    configure_kernel(k_gemm_mma_q4<1, false, 64>, true);
    configure_kernel(k_gemm_mma_q4<4, true, 16>, true);
    configure_kernel(k_gemm_mma_q4<2, true, 64>, true);
    configure_kernel(k_gemm_mma_q4<2, false, 64>, true);
    configure_kernel(k_gemm_mma_q4<4, false, 16>, true);
    configure_kernel(k_attn_chunk<64>, true);
    configure_kernel(k_attn_chunk<128>, true);
    configure_kernel(k_attn_chunk<256>, true);
    configure_kernel(k_attn_chunk_mma<64>, true);
    configure_kernel(k_attn_chunk_mma<128>, true);
    configure_kernel(k_prep_rows, false);
    configure_kernel(k_attn_chunk_merge, false);
    // the attention kernel also has static shared memory: ask for exactly the dynamic part it uses
    configure_kernel(k_attn_decode<64>, false);
    configure_kernel(k_attn_decode<128>, false);
    configure_kernel(k_attn_decode<256>, false);
    configure_kernel(k_attn_decode<64, true>, false);
    configure_kernel(k_attn_decode<128, true>, false);
    configure_kernel(k_attn_decode<256, true>, false);
    cudaFuncSetAttribute(k_attn_decode<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_dyn_smem(64));
    cudaFuncSetAttribute(k_attn_decode<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_dyn_smem(128));
    cudaFuncSetAttribute(k_attn_decode<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_dyn_smem(256));
    configure_kernel(k_gdn_step, false);
    configure_kernel(k_qk_norm_rope_store, false);
    configure_kernel(k_state_advance, false);
    configure_kernel(k_add_residual, false);
    configure_kernel(k_state_begin, false);
    configure_kernel(k_state_next_prompt, false);
}

// Clusters of attention CTAs the device can hold at once for a head size and kernel instance (a cluster needs its
// SMs in one GPC with room for a CTA each); 0 when the query fails.  Cached per head size and instance.
static int attn_max_clusters(int hd, bool staged) {
    static int cache_all[TFR_MAX_DEVICES][6];
    static bool cache_init = false;
    if (!cache_init) {
        for (auto& d : cache_all)
            for (int& v : d) v = -1;
        cache_init = true;
    }
    configure_kernels_once();  // the query below asks for the kernel's opt-in dynamic shared memory
    int* cache = cache_all[current_device_slot()];
    const int slot = (hd == 64 ? 0 : hd == 128 ? 1 : 2) + (staged ? 3 : 0);
    if (cache[slot] >= 0) return cache[slot];
    const int cl = attn_cluster(staged);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(cl * 64, 1);
    cfg.blockDim = dim3(attn_threads(staged, hd));
    cfg.dynamicSmemBytes = staged ? attn_dyn_smem(hd) : 0;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cl;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t r;
    if (staged)
        r = hd == 64    ? cudaOccupancyMaxActiveClusters(&n, k_attn_decode<64, true>, &cfg)
            : hd == 128 ? cudaOccupancyMaxActiveClusters(&n, k_attn_decode<128, true>, &cfg)
                        : cudaOccupancyMaxActiveClusters(&n, k_attn_decode<256, true>, &cfg);
    else
        r = hd == 64    ? cudaOccupancyMaxActiveClusters(&n, k_attn_decode<64, false>, &cfg)
            : hd == 128 ? cudaOccupancyMaxActiveClusters(&n, k_attn_decode<128, false>, &cfg)
                        : cudaOccupancyMaxActiveClusters(&n, k_attn_decode<256, false>, &cfg);
    if (r != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    cache[slot] = n;
    return n;
}

// Splits per KV head of an instance: a multiple of its cluster size, about one CTA per SM over all KV heads, and no
// more clusters than run at the same time (a second wave would double the kernel's duration).
static int attn_splits(int sms, int n_kv, int hd, bool staged) {
    const int cl = attn_cluster(staged);
    int s = sms / n_kv / cl * cl;
    const int fit = attn_max_clusters(hd, staged) / n_kv * cl;
    if (fit >= cl && fit < s) s = fit;
    return s < cl ? cl : s;
}
// Which instance a launch takes and with how much shared memory, from the head size and the largest number of keys the
// launch can meet (the cache's capacity in the engine, pos + 1 in the operator entry points).
// Head sizes up to 128 always take the staged instance (scores and values on the tensor cores): a step of it covers 128
// keys; splits are cut at 256 keys (a second step costs less than the cluster merge a second split needs), and when no
// split can exceed 256 keys four tile stages replace the five.  Head
// size 256 takes the staged instance only where a split can exceed ATTN_LONG_MIN keys.  TFR_ATTN_REGISTER_ROUTE=1 in
// the environment keeps short caches on the register route for every head size (a test and measurement aid).
static void attn_route(AttnArgs& a, int hd, int max_keys, int s_short, int s_staged, int min_keys_short) {
    const bool long_cache = max_keys > s_short * ATTN_LONG_MIN;
    const bool mma_route = attn_staged_mma(hd) && !getenv("TFR_ATTN_REGISTER_ROUTE");
    a.staged = long_cache || mma_route;
    a.S = a.staged ? s_staged : s_short;
    const bool mma = a.staged && attn_staged_mma(hd);
    constexpr int tiles_per_split = 4;  // measured on one box: 2 tiles 718.6 tok/s, 3 715.3, 4 722.9, 5 719.0 - 723.9
    a.stages = (mma && max_keys <= s_staged * tiles_per_split * ATTN_TILE) ? tiles_per_split : 0;
    a.min_keys = mma ? tiles_per_split * ATTN_TILE : min_keys_short;
}

static int sm_count_cached() {
    static int count[TFR_MAX_DEVICES] = {};
    const int dev = current_device_slot();
    int& n = count[dev];
    if (!n) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// ------------------------------------------------------------------ Q5 -> Q8_0 conversion (host)

// IEEE f32 -> f16, round to nearest even (crates/core/src/quant.rs:26-62), and back.
static uint16_t host_f32_to_f16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000);
    const int exponent = (int)((bits >> 23) & 0xff);
    const uint32_t fraction = bits & 0x007fffffu;
    if (exponent == 255) return (uint16_t)(sign | (fraction == 0 ? 0x7c00 : 0x7e00));
    const int half_exp = exponent - 127 + 15;
    if (half_exp >= 31) return (uint16_t)(sign | 0x7c00);
    if (half_exp <= 0) {
        if (half_exp < -10) return sign;
        const uint32_t mantissa = fraction | 0x00800000u, shift = (uint32_t)(14 - half_exp);
        uint32_t rounded = mantissa >> shift;
        const uint32_t remainder = mantissa & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
        if (remainder > halfway || (remainder == halfway && (rounded & 1u))) rounded += 1;
        return (uint16_t)(sign | rounded);
    }
    uint32_t rounded = fraction + 0x00000fffu + ((fraction >> 13) & 1u);
    uint16_t out_exp = (uint16_t)half_exp;
    if (rounded & 0x00800000u) {
        rounded = 0;
        out_exp += 1;
        if (out_exp >= 31) return (uint16_t)(sign | 0x7c00);
    }
    return (uint16_t)(sign | (out_exp << 10) | (rounded >> 13));
}
static float host_f16_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// 32 fp32 values -> one Q8_0 block, load.rs:88-101: d = amax / 127, q = clamp(round half away from zero (v / d)).
static void host_q8_0_block(const float* v, uint8_t* out) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(v[i]));
    volatile float d = amax == 0.f ? 0.f : amax / 127.0f;
    const uint16_t h = host_f32_to_f16(d);
    out[0] = (uint8_t)(h & 0xff);
    out[1] = (uint8_t)(h >> 8);
    for (int i = 0; i < 32; i++) {
        int q = 0;
        if (d != 0.f) {
            volatile float r = v[i] / d;
            float rr = roundf(r);
            rr = rr < -127.f ? -127.f : (rr > 127.f ? 127.f : rr);
            q = (int)rr;
        }
        out[2 + i] = (uint8_t)(int8_t)q;
    }
}

// transcode_q5_k_to_q8_0 / transcode_q5_1_to_q8_0, load.rs:33-133.  The products and differences are kept as
// separate fp32 operations (volatile), as the reference's host code computes them.
extern "C" int tfr_transcode_to_q8_0(int src_type, const void* raw_v, size_t nbytes, void* out_v) {
    const uint8_t* raw = (const uint8_t*)raw_v;
    uint8_t* out = (uint8_t*)out_v;
    if (!raw || !out) return TFR_E_INVALID;
    if (src_type == TFR_Q5_K) {
        if (nbytes % 176) return TFR_E_INVALID;
        for (size_t b = 0; b < nbytes / 176; b++) {
            const uint8_t* blk = raw + b * 176;
            const float d = host_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8))), dmin = host_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
            const uint8_t *sc = blk + 4, *qh = blk + 16, *qs = blk + 48;
            float vals[256];
            for (int g = 0; g < 4; g++) {
                uint8_t s[2], m[2];
                for (int w = 0; w < 2; w++) {
                    const int j = 2 * g + w;
                    if (j < 4) {
                        s[w] = sc[j] & 0x3f;
                        m[w] = sc[j + 4] & 0x3f;
                    } else {
                        s[w] = (uint8_t)((sc[j + 4] & 0x0f) | ((sc[j - 4] >> 6) << 4));
                        m[w] = (uint8_t)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
                    }
                }
                volatile float scale0 = d * (float)s[0], scale1 = d * (float)s[1], off0 = dmin * (float)m[0], off1 = dmin * (float)m[1];
                const uint8_t hl = (uint8_t)(1u << (2 * g)), hh = (uint8_t)(2u << (2 * g));
                for (int l = 0; l < 32; l++) {
                    const int low = (qs[32 * g + l] & 0x0f) + ((qh[l] & hl) ? 16 : 0), high = (qs[32 * g + l] >> 4) + ((qh[l] & hh) ? 16 : 0);
                    volatile float p0 = scale0 * (float)low, p1 = scale1 * (float)high;
                    vals[64 * g + l] = p0 - off0;
                    vals[64 * g + 32 + l] = p1 - off1;
                }
            }
            for (int k = 0; k < 8; k++) host_q8_0_block(vals + 32 * k, out + (b * 8 + k) * 34);
        }
        return TFR_OK;
    }
    if (src_type == TFR_Q5_1) {
        if (nbytes % 24) return TFR_E_INVALID;
        for (size_t b = 0; b < nbytes / 24; b++) {
            const uint8_t* blk = raw + b * 24;
            const float d = host_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8))), mn = host_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
            const uint32_t qh = (uint32_t)blk[4] | ((uint32_t)blk[5] << 8) | ((uint32_t)blk[6] << 16) | ((uint32_t)blk[7] << 24);
            const uint8_t* qs = blk + 8;
            float vals[32];
            for (int j = 0; j < 16; j++) {
                const uint8_t h0 = (uint8_t)(((qh >> j) << 4) & 0x10), h1 = (uint8_t)((qh >> (j + 12)) & 0x10);
                volatile float p0 = (float)((qs[j] & 0x0f) | h0) * d, p1 = (float)((qs[j] >> 4) | h1) * d;
                vals[j] = p0 + mn;
                vals[j + 16] = p1 + mn;
            }
            host_q8_0_block(vals, out + b * 34);
        }
        return TFR_OK;
    }
    return TFR_E_UNSUPPORTED;
}

// ------------------------------------------------------------------ matrices

static int mat_create_impl(tfr_engine* e, int type, int64_t K, int64_t N, const void* bytes, size_t nbytes, int perm_hd,
                           cudaStream_t stream, tfr_mat** out) {
    if (type == TFR_Q5_K || type == TFR_Q5_1) {
        // load.rs:191-233: Q5_K / Q5_1 tensors are converted to Q8_0 once, on the host, and run on the Q8_0 kernels
        if (K <= 0 || N <= 0 || K % 256 || nbytes != raw_bytes(type, K, N))
            return fail(e, TFR_E_INVALID, "matrix byte size %zu != expected %zu", nbytes, raw_bytes(type, K, N));
        std::vector<uint8_t> src(nbytes), q8(raw_bytes(TFR_Q8_0, K, N));
        if (cudaMemcpy(src.data(), bytes, nbytes, cudaMemcpyDefault) != cudaSuccess) return fail(e, TFR_E_CUDA, "reading the tensor");
        if (tfr_transcode_to_q8_0(type, src.data(), nbytes, q8.data()) != TFR_OK) return fail(e, TFR_E_INVALID, "transcode failed");
        return mat_create_impl(e, TFR_Q8_0, K, N, q8.data(), q8.size(), perm_hd, stream, out);
    }
    if (type != TFR_Q4_K && type != TFR_Q6_K && type != TFR_Q8_0) return fail(e, TFR_E_UNSUPPORTED, "matrix type %d not supported", type);
    if (K <= 0 || N <= 0 || K % 256) return fail(e, TFR_E_INVALID, "matrix K=%lld must be a positive multiple of 256", (long long)K);
    if (nbytes != raw_bytes(type, K, N))
        return fail(e, TFR_E_INVALID, "matrix byte size %zu != expected %zu", nbytes, raw_bytes(type, K, N));
    if (perm_hd && (N % perm_hd || perm_hd % 2)) return fail(e, TFR_E_INVALID, "rope pairing head_dim %d does not divide N", perm_hd);
    configure_kernels_once();
    tfr_mat* m = new tfr_mat();
    m->m.type = type;
    m->m.K = (int)K;
    m->m.N = (int)N;
    m->m.nb = (int)(K / 256);
    m->bytes = (size_t)mat_device_bytes(type, (int)K, N);
    m->perm_hd = perm_hd;
    void* staging = nullptr;
    cudaError_t r = cudaMalloc(&m->dev, m->bytes);
    if (r == cudaSuccess) r = cudaMalloc(&staging, nbytes);
    if (r == cudaSuccess) r = cudaMemcpyAsync(staging, bytes, nbytes, cudaMemcpyDefault, stream);
    if (r == cudaSuccess) {
        const int grid = sm_count_cached() * 8;
        const size_t last_tile = (size_t)tile_bytes(type);  // zero the tail tile's unused lanes
        cudaMemsetAsync((uint8_t*)m->dev + m->bytes - last_tile, 0, last_tile, stream);
        k_repack_tiled<<<grid, 256, 0, stream>>>((const uint8_t*)staging, (uint8_t*)m->dev, type, (int)N, m->m.nb, perm_hd);
        r = cudaGetLastError();
    }
    if (r == cudaSuccess) r = cudaStreamSynchronize(stream);
    if (staging) cudaFree(staging);
    if (r != cudaSuccess) {
        if (m->dev) cudaFree(m->dev);
        delete m;
        return fail(e, TFR_E_CUDA, "matrix upload: %s", cudaGetErrorString(r));
    }
    m->m.data = (const uint8_t*)m->dev;
    *out = m;
    return TFR_OK;
}

extern "C" int tfr_mat_create(int type, int64_t K, int64_t N, const void* bytes, size_t nbytes, int perm_hd, tfr_mat** out) {
    if (!bytes || !out) return TFR_E_INVALID;
    return mat_create_impl(nullptr, type, K, N, bytes, nbytes, perm_hd, nullptr, out);
}
extern "C" void tfr_mat_free(tfr_mat* m) {
    if (!m) return;
    if (m->dev) cudaFree(m->dev);
    delete m;
}
extern "C" int64_t tfr_mat_device_bytes(const tfr_mat* m) { return m ? (int64_t)m->bytes : 0; }

// ------------------------------------------------------------------ engine lifetime

extern "C" int tfr_create(int device, tfr_engine** out) {
    if (!out) return TFR_E_INVALID;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return TFR_E_CUDA;
    if (cudaSetDevice(device) != cudaSuccess) return TFR_E_CUDA;
    tfr_engine* e = new tfr_engine();
    e->device = device;
    if (cudaGetDeviceProperties(&e->prop, device) != cudaSuccess ||
        cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreate(&e->ev0) != cudaSuccess || cudaEventCreate(&e->ev1) != cudaSuccess) {
        delete e;
        return TFR_E_CUDA;
    }
    configure_kernels_once();
    *out = e;
    return TFR_OK;
}

static void drop_graphs(tfr_engine* e) {
    if (e->g_decode) cudaGraphExecDestroy(e->g_decode);
    if (e->g_body) cudaGraphExecDestroy(e->g_body);
    e->g_decode = e->g_body = nullptr;
    e->graph_kv = nullptr;
}

extern "C" void tfr_destroy(tfr_engine* e) {
    if (!e) return;
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->stream);
    drop_graphs(e);
    if (e->nccl_comm && nccl_api()) nccl_api()->CommDestroy(e->nccl_comm);
    cudaFree(e->ypart);
    cudaFree(e->best_buf);
    if (e->comm_ipc)
        for (int r = 0; r < e->plan.tp; r++)
            if (r != e->plan.rank && e->comm.base[r]) cudaIpcCloseMemHandle(e->comm.base[r]);
    cudaFree(e->comm_local);
    for (auto& kv : e->mats) tfr_mat_free(kv.second);
    for (auto& kv : e->vecs) cudaFree(kv.second.dev);
    for (auto& L : e->layers) cudaFree(L.bias_qkv);
    void* ws[] = {e->x, e->q, e->attn, e->h, e->logits, e->partial, e->counters, e->st, e->out_tokens, e->prompt,
                  e->layer_taps, e->tap_attn, e->tap_mid, e->tap_h, e->proj, e->qgate, e->loop_layers, e->loop_bar, e->loop_best, e->loop_vec, e->cx, e->cq, e->cattn, e->ch, e->cxn, e->clogits, e->cpart, e->cact, e->ckeys, e->ccount, e->loop_blob, e->loop_head_tasks};
    for (void* p : ws) cudaFree(p);
    if (e->st_host) cudaFreeHost(e->st_host);
    if (e->out_host) cudaFreeHost(e->out_host);
    if (e->args_host) cudaFreeHost(e->args_host);
    cudaFree(e->args_dev);
    cudaEventDestroy(e->ev0);
    cudaEventDestroy(e->ev1);
    cudaStreamDestroy(e->stream);
    delete e;
}

extern "C" const char* tfr_last_error(const tfr_engine* e) { return e ? e->err.c_str() : "null engine"; }

extern "C" int tfr_device_info(const tfr_engine* e, char* name, size_t cap, int* major, int* minor, int* sms) {
    if (!e) return TFR_E_INVALID;
    if (name && cap) snprintf(name, cap, "%s", e->prop.name);
    if (major) *major = e->prop.major;
    if (minor) *minor = e->prop.minor;
    if (sms) *sms = e->prop.multiProcessorCount;
    return TFR_OK;
}

extern "C" int tfr_set_config(tfr_engine* e, const tfr_model_config* c) {
    if (!e || !c) return TFR_E_INVALID;
    if (e->finalized) return fail(e, TFR_E_INVALID, "config after finalize");
    if (c->n_layer <= 0 || c->n_embd <= 0 || c->n_embd % 256 || c->n_head <= 0 || c->n_kv_head <= 0 ||
        c->n_head % c->n_kv_head || c->n_ff <= 0 || c->n_ff % 256 || c->n_vocab <= 0)
        return fail(e, TFR_E_INVALID, "bad model configuration");
    if (c->head_dim != 64 && c->head_dim != 128 && c->head_dim != 256)
        return fail(e, TFR_E_UNSUPPORTED, "head_dim %d (supported: 64, 128, 256)", c->head_dim);
    if (c->n_head / c->n_kv_head > ATTN_REP_MAX)
        return fail(e, TFR_E_UNSUPPORTED, "more than %d query heads per KV head", ATTN_REP_MAX);
    if (c->hybrid) {
        if (c->ssm_state_size != GDN_D)
            return fail(e, TFR_E_UNSUPPORTED, "ssm.state_size %d (supported: %d)", c->ssm_state_size, GDN_D);
        if (c->ssm_conv_kernel < 2 || c->ssm_conv_kernel > GDN_MAX_KERNEL)
            return fail(e, TFR_E_UNSUPPORTED, "ssm.conv_kernel %d (supported: 2..%d)", c->ssm_conv_kernel, GDN_MAX_KERNEL);
        if (c->ssm_group_count <= 0 || c->ssm_time_step_rank <= 0) return fail(e, TFR_E_INVALID, "bad ssm head counts");
        if (c->ssm_inner_size && c->ssm_inner_size != c->ssm_time_step_rank * c->ssm_state_size)
            return fail(e, TFR_E_UNSUPPORTED, "ssm.inner_size %d != time_step_rank * state_size", c->ssm_inner_size);
        if (c->rope_dim < 0 || c->rope_dim > c->head_dim || c->rope_dim % 2) return fail(e, TFR_E_INVALID, "bad rope.dimension_count");
    }
    const int tp = c->tp_size < 1 ? 1 : c->tp_size;
    if (tp > 1) {
        if (tp > TP_MAX) return fail(e, TFR_E_UNSUPPORTED, "tp_size %d (at most %d)", tp, TP_MAX);
        if (c->tp_rank < 0 || c->tp_rank >= tp) return fail(e, TFR_E_INVALID, "tp_rank %d outside [0, %d)", c->tp_rank, tp);
        if (c->hybrid) return fail(e, TFR_E_UNSUPPORTED, "tensor parallelism covers the dense architecture only");
        if (c->n_head % tp || c->n_kv_head % tp)
            return fail(e, TFR_E_UNSUPPORTED, "tp_size %d does not divide %d query / %d KV heads", tp, c->n_head, c->n_kv_head);
        if (c->n_ff / 256 < tp || c->n_vocab < 2 * tp) return fail(e, TFR_E_UNSUPPORTED, "model too narrow for tp_size %d", tp);
    }
    e->cfg = *c;
    e->cfg.tp_size = tp;
    if (tp == 1) e->cfg.tp_rank = 0;
    TpPlan& P = e->plan;
    P.tp = tp;
    P.rank = e->cfg.tp_rank;
    P.n_head = c->n_head / tp;
    P.n_kv = c->n_kv_head / tp;
    P.nq = P.n_head * c->head_dim;
    P.nkv = P.n_kv * c->head_dim;
    P.q_lo = P.rank * P.nq;
    P.wo_b0 = P.q_lo / 256;
    P.wo_b1 = (P.q_lo + P.nq + 255) / 256;
    P.attn_off = P.q_lo - P.wo_b0 * 256;
    P.attn_width = (P.wo_b1 - P.wo_b0) * 256;
    const long long nbf = c->n_ff / 256;
    P.ff_b0 = (int)(nbf * P.rank / tp);
    P.ff_b1 = (int)(nbf * (P.rank + 1) / tp);
    P.ff = (P.ff_b1 - P.ff_b0) * 256;
    P.v0 = (int)((long long)c->n_vocab * P.rank / tp);
    P.v1 = (int)((long long)c->n_vocab * (P.rank + 1) / tp);
    e->has_cfg = true;
    return TFR_OK;
}

static bool ends_with(const std::string& s, const char* suf) {
    size_t n = strlen(suf);
    return s.size() >= n && s.compare(s.size() - n, n, suf) == 0;
}

extern "C" int tfr_upload_tensor(tfr_engine* e, const char* name, int type, int64_t n_rows, int64_t n_cols, const void* bytes,
                                 size_t nbytes) {
    if (!e || !name || !bytes) return TFR_E_INVALID;
    if (!e->has_cfg) return fail(e, TFR_E_INVALID, "tfr_set_config must precede uploads");
    if (e->finalized) return fail(e, TFR_E_INVALID, "upload after finalize");
    cudaSetDevice(e->device);
    std::string nm(name);
    if (e->mats.count(nm) || e->vecs.count(nm)) return fail(e, TFR_E_INVALID, "tensor %s uploaded twice", name);
    const TpPlan& P = e->plan;
    if (type == TFR_TYPE_F32) {
        // vectors must be F32 (load.rs:135-143)
        int64_t n = n_rows * (n_cols > 0 ? n_cols : 1);
        if (nbytes != (size_t)n * 4) return fail(e, TFR_E_INVALID, "vector %s: %zu bytes for %lld floats", name, nbytes, (long long)n);
        int64_t first = 0, keep = n;
        if (P.tp > 1) {  // biases of column-parallel projections follow their rows
            if (ends_with(nm, "attn_q.bias")) first = (int64_t)P.rank * P.nq, keep = P.nq;
            else if (ends_with(nm, "attn_k.bias") || ends_with(nm, "attn_v.bias")) first = (int64_t)P.rank * P.nkv, keep = P.nkv;
            if (first + keep > n) return fail(e, TFR_E_INVALID, "vector %s is shorter than its tensor-parallel slice", name);
        }
        VecT v;
        v.n = keep;
        CU(e, cudaMalloc(&v.dev, (size_t)keep * 4));
        CU(e, cudaMemcpy(v.dev, (const float*)bytes + first, (size_t)keep * 4, cudaMemcpyDefault));
        e->vecs[nm] = v;
        return TFR_OK;
    }
    if (P.tp > 1) {
        if (type != TFR_Q4_K && type != TFR_Q6_K && type != TFR_Q8_0) return fail(e, TFR_E_UNSUPPORTED, "matrix type %d not supported", type);
        if (n_rows <= 0 || n_cols <= 0 || n_rows % 256 || nbytes != raw_bytes(type, n_rows, n_cols))
            return fail(e, TFR_E_INVALID, "tensor %s: bad shape or byte size", name);
        const int blk = block_bytes_256(type);
        const size_t row_bytes = (size_t)(n_rows / 256) * blk;
        int64_t r0 = 0, r1 = n_cols;   // rows kept (column-parallel)
        int64_t b0 = 0, b1 = n_rows / 256;  // K blocks kept (row-parallel)
        if (ends_with(nm, "attn_q.weight")) r0 = (int64_t)P.rank * P.nq, r1 = r0 + P.nq;
        else if (ends_with(nm, "attn_k.weight") || ends_with(nm, "attn_v.weight")) r0 = (int64_t)P.rank * P.nkv, r1 = r0 + P.nkv;
        else if (ends_with(nm, "ffn_gate.weight") || ends_with(nm, "ffn_up.weight")) r0 = (int64_t)P.ff_b0 * 256, r1 = (int64_t)P.ff_b1 * 256;
        else if (nm == "output.weight") r0 = P.v0, r1 = P.v1;
        else if (ends_with(nm, "attn_output.weight")) b0 = P.wo_b0, b1 = P.wo_b1;
        else if (ends_with(nm, "ffn_down.weight")) b0 = P.ff_b0, b1 = P.ff_b1;
        if (r1 > n_cols || b1 > n_rows / 256) return fail(e, TFR_E_INVALID, "tensor %s is smaller than its tensor-parallel slice", name);
        const int perm = (ends_with(nm, "attn_q.weight") || ends_with(nm, "attn_k.weight")) ? e->cfg.head_dim : 0;
        tfr_mat* m = nullptr;
        int rc;
        if (b0 == 0 && b1 == n_rows / 256) {
            rc = mat_create_impl(e, type, n_rows, r1 - r0, (const uint8_t*)bytes + (size_t)r0 * row_bytes, (size_t)(r1 - r0) * row_bytes,
                                 perm, e->stream, &m);
        } else {
            // K-block slice of every row, gathered into a dense temporary on the device
            const size_t width = (size_t)(b1 - b0) * blk;
            void* tmp = nullptr;
            CU(e, cudaMalloc(&tmp, width * (size_t)n_cols));
            // on the engine's stream: a synchronous copy from pageable memory may return before its DMA has
            // landed, and this (non-blocking) stream would not wait for it
            cudaError_t r = cudaMemcpy2DAsync(tmp, width, (const uint8_t*)bytes + (size_t)b0 * blk, row_bytes, width, (size_t)n_cols,
                                              cudaMemcpyDefault, e->stream);
            if (r != cudaSuccess) {
                cudaFree(tmp);
                return fail(e, TFR_E_CUDA, "slicing %s: %s", name, cudaGetErrorString(r));
            }
            rc = mat_create_impl(e, type, (b1 - b0) * 256, n_cols, tmp, width * (size_t)n_cols, 0, e->stream, &m);
            cudaFree(tmp);
        }
        if (rc) return rc;
        e->mats[nm] = m;
        return TFR_OK;
    }
    // F32/F16 matrices are rejected like load.rs:15-28
    std::vector<uint8_t> converted;
    if (type == TFR_Q5_K || type == TFR_Q5_1) {
        // load.rs:191-233: Q5_K / Q5_1 tensors are converted to Q8_0 once, on the host, and run on the Q8_0 kernels
        if (n_rows <= 0 || n_cols <= 0 || n_rows % 256 || nbytes != raw_bytes(type, n_rows, n_cols))
            return fail(e, TFR_E_INVALID, "tensor %s: bad shape or byte size", name);
        std::vector<uint8_t> src(nbytes);
        CU(e, cudaMemcpy(src.data(), bytes, nbytes, cudaMemcpyDefault));
        converted.resize(raw_bytes(TFR_Q8_0, n_rows, n_cols));
        if (tfr_transcode_to_q8_0(type, src.data(), nbytes, converted.data()) != TFR_OK) return fail(e, TFR_E_INVALID, "tensor %s: transcode failed", name);
        bytes = converted.data();
        nbytes = converted.size();
        type = TFR_Q8_0;
    }
    if (is_hybrid(e) && (ends_with(nm, "attn_qkv.weight") || ends_with(nm, "attn_gate.weight") ||
                         ends_with(nm, "ssm_beta.weight") || ends_with(nm, "ssm_alpha.weight"))) {
        // the four input projections of a linear layer become one matrix at finalize
        if (type != TFR_Q4_K && type != TFR_Q6_K && type != TFR_Q8_0) return fail(e, TFR_E_UNSUPPORTED, "matrix type %d not supported", type);
        if (n_rows <= 0 || n_cols <= 0 || n_rows % 256 || nbytes != raw_bytes(type, n_rows, n_cols))
            return fail(e, TFR_E_INVALID, "tensor %s: bad shape or byte size", name);
        if (e->held.count(nm)) return fail(e, TFR_E_INVALID, "tensor %s uploaded twice", name);
        HostRaw& h = e->held[nm];
        h.type = type;
        h.K = n_rows;
        h.N = n_cols;
        h.bytes.resize(nbytes);
        CU(e, cudaMemcpy(h.bytes.data(), bytes, nbytes, cudaMemcpyDefault));  // the source may be device memory
        return TFR_OK;
    }
    // dense layers pair the RoPE partners of Q and K at upload; the hybrid's Q/K are normalised per head first
    int perm = (!is_hybrid(e) && (ends_with(nm, "attn_q.weight") || ends_with(nm, "attn_k.weight"))) ? e->cfg.head_dim : 0;
    tfr_mat* m = nullptr;
    int rc = mat_create_impl(e, type, n_rows, n_cols, bytes, nbytes, perm, e->stream, &m);
    if (rc) return rc;
    e->mats[nm] = m;
    return TFR_OK;
}

static tfr_mat* need_mat(tfr_engine* e, const std::string& n, int K, int N, int& rc) {
    auto it = e->mats.find(n);
    if (it == e->mats.end()) {
        rc = fail(e, TFR_E_INVALID, "missing tensor %s", n.c_str());
        return nullptr;
    }
    if (it->second->m.K != K || it->second->m.N != N) {
        rc = fail(e, TFR_E_INVALID, "tensor %s is %dx%d, expected %dx%d", n.c_str(), it->second->m.K, it->second->m.N, K, N);
        return nullptr;
    }
    return it->second;
}
static float* need_vec(tfr_engine* e, const std::string& n, int len, bool optional, int& rc) {
    auto it = e->vecs.find(n);
    if (it == e->vecs.end()) {
        if (!optional) rc = fail(e, TFR_E_INVALID, "missing tensor %s", n.c_str());
        return nullptr;
    }
    if (it->second.n != len) {
        rc = fail(e, TFR_E_INVALID, "tensor %s has %lld elements, expected %d", n.c_str(), (long long)it->second.n, len);
        return nullptr;
    }
    return it->second.dev;
}

// Stacks attn_qkv, attn_gate, ssm_beta and ssm_alpha of a linear layer (layer.rs:736-798 runs four
// GEMVs on the same activation) into one row-concatenated matrix [qkv | z | beta | alpha].
static int finalize_linear_layer(tfr_engine* e, int i, LayerW& L) {
    const tfr_model_config& c = e->cfg;
    const int K = c.n_embd, ch = gdn_channels(c), vd = gdn_val_dim(c), nv = c.ssm_time_step_rank;
    const std::string p = "blk." + std::to_string(i) + ".";
    const char* names[4] = {"attn_qkv.weight", "attn_gate.weight", "ssm_beta.weight", "ssm_alpha.weight"};
    const int rows[4] = {ch, vd, nv, nv};
    std::vector<uint8_t> all;
    int type = 0;
    for (int k = 0; k < 4; k++) {
        auto it = e->held.find(p + names[k]);
        if (it == e->held.end()) return fail(e, TFR_E_INVALID, "missing tensor %s%s", p.c_str(), names[k]);
        const HostRaw& h = it->second;
        if (h.K != K || h.N != rows[k])
            return fail(e, TFR_E_INVALID, "tensor %s%s is %lldx%lld, expected %dx%d", p.c_str(), names[k], (long long)h.K,
                        (long long)h.N, K, rows[k]);
        if (k == 0) type = h.type;
        if (h.type != type) type = -1;  // mixed types: one launch per matrix instead of the stacked one
        all.insert(all.end(), h.bytes.begin(), h.bytes.end());
    }
    const int total = ch + vd + 2 * nv;
    int rc = TFR_OK;
    if (type >= 0) {
        tfr_mat* m = nullptr;
        rc = mat_create_impl(e, type, K, total, all.data(), all.size(), 0, e->stream, &m);
        if (rc) return rc;
        e->mats[p + "gdn_proj"] = m;
        L.gdn_proj = m;
    } else {
        for (int k = 0; k < 4; k++) {
            const HostRaw& h = e->held[p + names[k]];
            rc = mat_create_impl(e, h.type, K, rows[k], h.bytes.data(), h.bytes.size(), 0, e->stream, &L.proj4[k]);
            if (rc) return rc;
            e->mats[p + names[k]] = L.proj4[k];
        }
    }
    L.ssm_out = need_mat(e, p + "ssm_out.weight", vd, K, rc);
    L.conv_w = need_vec(e, p + "ssm_conv1d.weight", c.ssm_conv_kernel * ch, false, rc);
    L.ssm_a = need_vec(e, p + "ssm_a", nv, false, rc);
    L.ssm_dt = need_vec(e, p + "ssm_dt.bias", nv, false, rc);
    L.ssm_norm = need_vec(e, p + "ssm_norm.weight", c.ssm_state_size, false, rc);
    return rc;
}

// ------------------------------------------------------------------ persistent decode loop: plan

template <class F>
static cudaError_t loop_configure(F f, size_t smem) {
    cudaError_t r = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (r == cudaSuccess) r = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return r;
}
static const void* loop_kernel(int hd) {
    if (hd == 64) return (const void*)k_decode_loop<64>;
    if (hd == 128) return (const void*)k_decode_loop<128>;
    return (const void*)k_decode_loop<256>;
}
static size_t loop_attn_smem(int hd) {
    return hd == 64 ? sizeof(AttnSmem<64>) : hd == 128 ? sizeof(AttnSmem<128>) : sizeof(AttnSmem<256>);
}

// Builds the persistent loop's plan after the weights are in place.  Models outside its scope keep the
// chained-kernel path; loop_why says which condition failed.
static int loop_setup(tfr_engine* e) {
    const tfr_model_config& c = e->cfg;
    const TpPlan& P = e->plan;
    e->loop_ok = false;
    auto no = [&](const char* why) {
        e->loop_why = why;
        return TFR_OK;
    };
    if (c.hybrid) return no("hybrid (Gated-DeltaNet) layers");
    if (P.tp > 1) return no("tensor parallelism");
    if (e->vocab_limit) return no("vocabulary shortlist");
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, e->device);
    if (!coop) return no("no cooperative launch on this device");
    const int G = e->prop.multiProcessorCount, K = c.n_embd, hd = c.head_dim;
    if (c.n_head / c.n_kv_head > LOOP_REP_MAX || G < P.n_kv) return no("head grouping");
    auto q46 = [](const tfr_mat* m) { return m->m.type == TFR_Q4_K || m->m.type == TFR_Q6_K; };
    if (!q46(e->head) || !q46(e->token_embd)) return no("head / embedding type");
    for (const LayerW& L : e->layers)
        if (!q46(L.wo) || !q46(L.down)) return no("attn_output / ffn_down type");
    int lpb[5] = {0, 0, 0, 0, 0};  // forced lanes per block of Q/K/V, o-proj, gate/up, down, head (0: pick)
    if (const char* env = getenv("TFR_LOOP_LPB")) sscanf(env, "%d,%d,%d,%d,%d", &lpb[0], &lpb[1], &lpb[2], &lpb[3], &lpb[4]);
    LoopArgs& a = e->loop;
    a = LoopArgs{};
    int pbuf = 4096;
    if (const char* env = getenv("TFR_LOOP_PBUF")) pbuf = std::max(1024, atoi(env));
    // sections: 0 Q/K/V, 1 o-proj Q4_K, 2 o-proj Q6_K, 3 gate/up, 4 down Q4_K, 5 down Q6_K, 6 head
    LoopPhase ph[SCHED_SECTIONS] = {};
    bool used[SCHED_SECTIONS] = {true, false, false, true, false, false, true};
    for (const LayerW& L : e->layers) {
        used[1 + (L.wo->m.type == TFR_Q6_K)] = true;
        used[4 + (L.down->m.type == TFR_Q6_K)] = true;
    }
    ph[0].job[0] = loop_job(TFR_Q4_K, P.nq, 2, 0, 0, G);
    ph[0].job[1] = loop_job(TFR_Q4_K, P.nkv, 2, P.nq / 2, 0, G);
    ph[0].job[2] = loop_job(TFR_Q6_K, P.nkv, 2, (P.nq + P.nkv) / 2, 1, G);
    for (int t = 0; t < 2; t++) {
        const int type = t ? TFR_Q6_K : TFR_Q4_K;
        ph[1 + t].job[0] = loop_job(type, K, 2, 0, 0, G);
        ph[4 + t].job[0] = loop_job(type, K, 2, 0, 0, G);
    }
    ph[3].job[0] = loop_job(TFR_Q4_K, P.ff, 1, 0, 0, G);
    ph[3].job[1] = loop_job(TFR_Q4_K, P.ff, 1, 0, 0, G);
    ph[3].zip = 1;
    const int V = e->head->m.N;
    ph[6].job[0] = loop_job(e->head->m.type, V, 2, 0, 0, G);
    const int sec_k[SCHED_SECTIONS] = {K, P.attn_width, P.attn_width, K, P.ff, P.ff, K};
    const int sec_lpb[SCHED_SECTIONS] = {lpb[0], lpb[1], lpb[1], lpb[2], lpb[3], lpb[3], lpb[4]};
    bool fits = true;
    for (int sct = 0; sct < SCHED_SECTIONS; sct++) {
        fits = fits && loop_finish_phase(ph[sct], sec_k[sct], pbuf, sec_lpb[sct]);
        a.sec_nb[sct] = sec_k[sct] / 256;
        a.sec_zip[sct] = ph[sct].zip;
    }
    LoopPlanHost plan;
    if (!fits || !loop_build_plan(ph, used, G, pbuf, plan)) return no("a phase's partial sums exceed the shared-memory buffer");
    a.blob_stride = plan.blob_stride, a.blob_chunks = plan.chunks_off, a.blob_tasks = plan.tasks_off, a.blob_sched = plan.sched_off;
    a.head_stride = plan.head_stride;
    // shared-memory map: [barriers, control, reduction scratch | plan | layer table | activation | staged fp32 vector |
    // partial sums | weight ring]; the attention scratch aliases activation .. partial sums
    const int k_act = std::max(std::max(K, P.ff), P.attn_width);
    const size_t act_b = (act_smem_bytes(k_act, false, false) + 15) & ~(size_t)15;
    const size_t xf_b = (xs_floats(K) * 4 + 15) & ~(size_t)15;
    size_t work = act_b + xf_b + (size_t)pbuf * 4;
    const size_t attn_need = std::max(loop_attn_smem(hd), (size_t)(2 * ((G / P.n_kv + 3) & ~3) + LOOP_CT) * 4);
    if (work < attn_need) work = attn_need;
    a.off_blob = LOOP_CTX_OFFSET + 256;  // barriers, control words, reduction scratch, then the context struct
    a.off_layers = (int)((a.off_blob + (size_t)plan.blob_stride * 4 + 15) & ~(size_t)15);
    a.sh_x = make_share((K + 1) / 2, G);
    a.off_own = (int)((a.off_layers + (size_t)c.n_layer * sizeof(LoopLayer) + 15) & ~(size_t)15);
    a.off_act = (int)((a.off_own + (size_t)4 * 2 * (a.sh_x.quot + 1) + 127) & ~(size_t)127);
    a.off_xf = a.off_act + (int)act_b;
    a.off_pbuf = a.off_xf + (int)xf_b;
    a.off_ring = (int)((a.off_act + work + 127) & ~(size_t)127);
    a.pbuf_floats = pbuf;
    const size_t cap = e->prop.sharedMemPerBlockOptin;
    if (cap <= (size_t)a.off_ring + 3 * LOOP_SLOT) return no("not enough shared memory for the weight ring");
    int nslot = (int)((cap - a.off_ring) / LOOP_SLOT);
    if (nslot > LOOP_MAX_SLOTS) nslot = LOOP_MAX_SLOTS;
    if (const char* env = getenv("TFR_LOOP_SLOTS")) nslot = std::max(3, std::min(nslot, atoi(env)));
    a.nslot = nslot;
    e->loop_smem = (size_t)a.off_ring + (size_t)nslot * LOOP_SLOT;
    e->loop_grid = G;
    cudaError_t r = hd == 64    ? loop_configure(k_decode_loop<64>, e->loop_smem)
                    : hd == 128 ? loop_configure(k_decode_loop<128>, e->loop_smem)
                                : loop_configure(k_decode_loop<256>, e->loop_smem);
    int per_sm = 0;
    if (r == cudaSuccess) r = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, loop_kernel(hd), LOOP_THREADS, e->loop_smem);
    if (r != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        return no("the loop kernel does not fit an SM");
    }
    // per-layer pointers
    std::vector<LoopLayer> tab(c.n_layer);
    for (int i = 0; i < c.n_layer; i++) {
        const LayerW& L = e->layers[i];
        LoopLayer& t = tab[i];
        t.wq = L.wq->m.data, t.wk = L.wk->m.data, t.wv = L.wv->m.data, t.wo = L.wo->m.data;
        t.gate = L.gate->m.data, t.up = L.up->m.data, t.down = L.down->m.data;
        t.bias_qkv = L.bias_qkv, t.attn_norm = L.attn_norm, t.ffn_norm = L.ffn_norm;
        t.o_q6 = L.wo->m.type == TFR_Q6_K, t.down_q6 = L.down->m.type == TFR_Q6_K;
    }
    CU(e, cudaMalloc(&e->loop_blob, plan.blob.size() * sizeof(int)));
    CU(e, cudaMalloc(&e->loop_head_tasks, plan.head_tasks.size() * sizeof(uint4)));
    CU(e, cudaMemcpyAsync(e->loop_blob, plan.blob.data(), plan.blob.size() * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaMemcpyAsync(e->loop_head_tasks, plan.head_tasks.data(), plan.head_tasks.size() * sizeof(uint4), cudaMemcpyHostToDevice, e->stream));
    a.blob = e->loop_blob;
    a.head_tasks = e->loop_head_tasks;
    CU(e, cudaMalloc(&e->loop_layers, tab.size() * sizeof(LoopLayer)));
    CU(e, cudaMemcpyAsync(e->loop_layers, tab.data(), tab.size() * sizeof(LoopLayer), cudaMemcpyHostToDevice, e->stream));
    CU(e, cudaStreamSynchronize(e->stream));  // tab goes out of scope
    a.attn_smax = std::max(1, G / P.n_kv);
    a.attn_min_keys = 64;
    a.attn_inline_max = 8;
    if (const char* env = getenv("TFR_LOOP_ATTN_KEYS")) a.attn_min_keys = std::max(8, atoi(env));
    if (const char* env = getenv("TFR_LOOP_ATTN_INLINE")) a.attn_inline_max = std::max(1, atoi(env));
    if (a.attn_inline_max > LOOP_INLINE_MAX) a.attn_inline_max = LOOP_INLINE_MAX;
    {
        // vectors handed between phases: q, attention output, SiLU*mul output, split partials
        const size_t n_q = (size_t)P.nq, n_h = (size_t)P.ff;
        const size_t n_p = (size_t)P.n_head * a.attn_smax * (4 + hd);
        auto up = [](size_t n) { return (n + 31) & ~(size_t)31; };
        e->loop_vec_n = 2 * up(n_q) + up(n_h) + up(n_p);
        CU(e, cudaMalloc(&e->loop_vec, e->loop_vec_n * 4));
        float* p = e->loop_vec;
        a.q = p, p += up(n_q);
        a.att = p, p += up(n_q);
        a.h = p, p += up(n_h);
        a.pc = p;
    }
    CU(e, cudaMalloc(&e->loop_bar, 8 * LOOP_BAR_STRIDE * 4));  // grid-barrier counters
    CU(e, cudaMalloc(&e->loop_best, 4 * 8));
    a.layers = e->loop_layers;
    a.n_layer = c.n_layer;
    a.K = K, a.FF = P.ff, a.nq = P.nq, a.nkv = P.nkv, a.hd = hd, a.n_head = P.n_head, a.n_kv = P.n_kv, a.V = V;
    a.rep = P.n_head / P.n_kv;
    a.hd_shift = hd == 64 ? 6 : (hd == 128 ? 7 : 8);
    a.eps = c.rms_eps, a.theta = c.rope_theta, a.attn_scale = 1.0f / sqrtf((float)hd);  // forward.rs:389
    a.embed = e->token_embd->m;
    a.head = e->head->m.data;
    a.out_norm = e->output_norm;
    a.x = e->x, a.logits = e->logits;
    a.bar = e->loop_bar;
    a.best = e->loop_best;
    a.st = e->st;
    a.out_tokens = e->out_tokens;
    a.prompt = e->prompt;
    e->loop_ok = true;
    e->loop_why.clear();
    return TFR_OK;
}

// path 0 (auto) takes the persistent loop only when the build says it is the faster schedule
constexpr bool TFR_LOOP_IS_DEFAULT = false;
static bool use_loop(const tfr_engine* e) { return e->loop_ok && (e->decode_path == 2 || (e->decode_path == 0 && TFR_LOOP_IS_DEFAULT)); }

// One launch of the persistent loop: n_headless prompt-feeding steps, then the steps TokenState asks for.
static int run_loop(tfr_engine* e, const tfr_kv* kv, int n_headless) {
    LoopArgs a = e->loop;
    a.kc = kv->k;
    a.vc = kv->v;
    a.kv_layer_stride = kv->layer_stride;
    a.layer_taps = e->layer_taps;
    a.n_headless = n_headless;
    a.prof = e->loop_prof;
    a.prof_step = e->loop_prof_step;
    a.prof_points = e->loop_prof_points;
    k_loop_reset<<<1, 256, 0, e->stream>>>(e->loop_bar, e->loop_best);
    CU(e, cudaGetLastError());
    void* params[] = {&a};
    CU(e, cudaLaunchCooperativeKernel(loop_kernel(e->cfg.head_dim), dim3(e->loop_grid), dim3(LOOP_THREADS), params, e->loop_smem,
                                      e->stream));
    e->launches += 2;
    return TFR_OK;
}

static void chunk_setup(tfr_engine* e);

extern "C" int tfr_finalize_load(tfr_engine* e) {
    if (!e || !e->has_cfg) return TFR_E_INVALID;
    if (e->finalized) return TFR_OK;
    cudaSetDevice(e->device);
    const tfr_model_config& c = e->cfg;
    const TpPlan& P = e->plan;
    // widths below are this rank's (everything when tp_size == 1)
    const int K = c.n_embd, hd = c.head_dim, nq = P.nq, nkv = P.nkv, FF = P.ff, V = c.n_vocab, Vl = P.v1 - P.v0;
    int rc = TFR_OK;
    e->token_embd = need_mat(e, "token_embd.weight", K, V, rc);
    if (rc) return rc;
    if (e->mats.count("output.weight")) {
        e->head = need_mat(e, "output.weight", K, Vl, rc);
    } else if (P.tp == 1) {
        e->head = e->token_embd;
    } else {
        // tied head: this rank's vocabulary rows are a run of whole tiles of the embedding matrix
        const long long f0 = (long long)P.v0 * (K / 256);
        if (f0 % 32) return fail(e, TFR_E_UNSUPPORTED, "tied vocabulary head: slice of rank %d does not start on a tile", P.rank);
        tfr_mat* view = new tfr_mat();
        view->m = e->token_embd->m;
        view->m.N = Vl;
        view->m.data = e->token_embd->m.data + (f0 / 32) * tile_bytes(view->m.type);
        e->mats["output.weight(view)"] = view;
        e->head = view;
    }
    if (e->vocab_limit) {
        // the head runs over rows [0, limit) plus, optionally, one more row (the end-of-sequence token)
        if (P.tp > 1) return fail(e, TFR_E_UNSUPPORTED, "vocabulary shortlist with tensor parallelism");
        if (e->vocab_limit >= V) return fail(e, TFR_E_INVALID, "vocabulary shortlist %d is not below n_vocab %d", e->vocab_limit, V);
        if (e->special_id >= V) return fail(e, TFR_E_INVALID, "shortlist: extra row %d outside the vocabulary", e->special_id);
        const tfr_mat* full = e->head;
        tfr_mat* view = new tfr_mat();
        view->m = full->m;
        view->m.N = e->vocab_limit;
        e->mats["output(shortlist)"] = view;
        e->head = view;
        if (e->special_id >= 0) {
            tfr_mat* one = new tfr_mat();
            one->m = full->m;
            one->m.N = 1;
            one->bytes = (size_t)tile_bytes(full->m.type);
            CU(e, cudaMalloc(&one->dev, one->bytes));
            CU(e, cudaMemsetAsync(one->dev, 0, one->bytes, e->stream));
            const int work = full->m.nb * 18;
            k_extract_row<<<(work + 127) / 128, 128, 0, e->stream>>>(full->m.data, (uint8_t*)one->dev, full->m.type, e->special_id, full->m.nb);
            CU(e, cudaGetLastError());
            one->m.data = (const uint8_t*)one->dev;
            e->mats["output(shortlist extra row)"] = one;
            e->head_special = one;
        }
    }
    e->output_norm = need_vec(e, "output_norm.weight", K, false, rc);
    if (rc) return rc;
    if (e->token_embd->m.type == TFR_Q8_0) return fail(e, TFR_E_UNSUPPORTED, "token_embd must be Q4_K or Q6_K (no Q8_0 embedding lookup)");
    e->layers.resize(c.n_layer);
    for (int i = 0; i < c.n_layer; i++) {
        const std::string p = "blk." + std::to_string(i) + ".";
        LayerW& L = e->layers[i];
        L.kind = layer_kind(c, i);
        L.gate = need_mat(e, p + "ffn_gate.weight", K, FF, rc);
        L.up = need_mat(e, p + "ffn_up.weight", K, FF, rc);
        L.down = need_mat(e, p + "ffn_down.weight", FF, K, rc);
        L.attn_norm = need_vec(e, p + "attn_norm.weight", K, false, rc);
        L.ffn_norm = need_vec(e, p + "ffn_norm.weight", K, true, rc);
        if (!L.ffn_norm && !rc) L.ffn_norm = need_vec(e, p + "post_attention_norm.weight", K, false, rc);  // load.rs:280-417
        if (rc) return rc;
        if (L.gate->m.type != TFR_Q4_K || L.up->m.type != TFR_Q4_K)
            return fail(e, TFR_E_UNSUPPORTED, "layer %d: ffn_gate / ffn_up must be Q4_K", i);
        if (L.kind == LAYER_LINEAR) {
            rc = finalize_linear_layer(e, i, L);
            if (rc) return rc;
            continue;
        }
        const int nq_rows = L.kind == LAYER_FULL_GATED ? 2 * nq : nq;  // fused Q|gate, deltanet.cu:144-173
        L.wq = need_mat(e, p + "attn_q.weight", K, nq_rows, rc);
        L.wk = need_mat(e, p + "attn_k.weight", K, nkv, rc);
        L.wv = need_mat(e, p + "attn_v.weight", K, nkv, rc);
        L.wo = need_mat(e, p + "attn_output.weight", P.attn_width, K, rc);
        if (rc) return rc;
        if (L.wq->m.type != TFR_Q4_K || L.wk->m.type != TFR_Q4_K)
            return fail(e, TFR_E_UNSUPPORTED, "layer %d: attn_q / attn_k must be Q4_K", i);
        if (L.wv->m.type != TFR_Q6_K) return fail(e, TFR_E_UNSUPPORTED, "layer %d: attn_v must be Q6_K", i);
        float* bq = need_vec(e, p + "attn_q.bias", nq_rows, true, rc);
        float* bk = need_vec(e, p + "attn_k.bias", nkv, true, rc);
        float* bv = need_vec(e, p + "attn_v.bias", nkv, true, rc);
        if (rc) return rc;
        if (L.kind == LAYER_FULL_GATED) {
            L.q_norm = need_vec(e, p + "attn_q_norm.weight", hd, true, rc);
            L.k_norm = need_vec(e, p + "attn_k_norm.weight", hd, true, rc);
            if (rc) return rc;
            if (!L.q_norm || !L.k_norm) return fail(e, TFR_E_UNSUPPORTED, "layer %d: attn_q_norm / attn_k_norm are required", i);
        }
        if (bq || bk || bv) {
            const int tot = nq_rows + 2 * nkv, perm = L.kind == LAYER_DENSE ? hd : 0;
            CU(e, cudaMalloc(&L.bias_qkv, (size_t)tot * 4));
            CU(e, cudaMemsetAsync(L.bias_qkv, 0, (size_t)tot * 4, e->stream));
            if (bq) k_permute_f32<<<(nq_rows + 255) / 256, 256, 0, e->stream>>>(bq, L.bias_qkv, nq_rows, perm);
            if (bk) k_permute_f32<<<(nkv + 255) / 256, 256, 0, e->stream>>>(bk, L.bias_qkv + nq_rows, nkv, perm);
            if (bv) k_permute_f32<<<(nkv + 255) / 256, 256, 0, e->stream>>>(bv, L.bias_qkv + nq_rows + nkv, nkv, 0);
            CU(e, cudaGetLastError());
        }
    }
    e->held.clear();
    // workspaces (load.rs:547-607: everything allocated once)
    const int sms = e->prop.multiProcessorCount;
    e->attn_S = attn_splits(sms, P.n_kv, hd, false);
    e->attn_S_staged = attn_splits(sms, P.n_kv, hd, true);
    CU(e, cudaMalloc(&e->x, (size_t)K * 4));
    const int vd = c.hybrid ? gdn_val_dim(c) : 0;
    CU(e, cudaMalloc(&e->q, (size_t)nq * 4));
    const int aw = P.attn_width > vd ? P.attn_width : vd;
    CU(e, cudaMalloc(&e->attn, (size_t)aw * 4));  // attention output (zero outside the local heads), or a linear layer's mixer output
    CU(e, cudaMemsetAsync(e->attn, 0, (size_t)aw * 4, e->stream));
    if (c.hybrid) {
        const int lin = gdn_channels(c) + vd + 2 * c.ssm_time_step_rank, full = 2 * nq + 2 * nkv;
        CU(e, cudaMalloc(&e->proj, (size_t)(lin > full ? lin : full) * 4));
        CU(e, cudaMalloc(&e->qgate, (size_t)nq * 4));
    }
    CU(e, cudaMalloc(&e->h, (size_t)FF * 4));
    CU(e, cudaMalloc(&e->logits, (size_t)Vl * 4));
    CU(e, cudaMalloc(&e->partial, (size_t)P.n_head * std::max(e->attn_S, e->attn_S_staged) * (2 + hd) * 4));
    CU(e, cudaMalloc(&e->counters, (size_t)P.n_kv * ATTN_CLUSTER * 4));  // one per KV head and output slice
    if (P.tp > 1) {
        e->comm.lay = tp_layout(K);
        e->comm.tp = P.tp;
        e->comm.rank = P.rank;
        e->comm.ops_per_token = 2 * c.n_layer + 1;
        CU(e, cudaMalloc(&e->comm_local, e->comm.lay.total));
        CU(e, cudaMemsetAsync(e->comm_local, 0, e->comm.lay.total, e->stream));
    }
    CU(e, cudaMalloc(&e->st, sizeof(TokenState)));
    CU(e, cudaMalloc(&e->out_tokens, (size_t)TFR_MAX_BURST * 4));
    CU(e, cudaMalloc(&e->prompt, (size_t)TFR_MAX_PROMPT * 4));
    CU(e, cudaMallocHost(&e->st_host, sizeof(TokenState)));
    CU(e, cudaMallocHost(&e->out_host, (size_t)TFR_MAX_BURST * 4));
    CU(e, cudaMalloc(&e->args_dev, 16 * sizeof(int)));  // k_state_begin reads [0..14]
    CU(e, cudaMallocHost(&e->args_host, 16 * sizeof(int)));
    CU(e, cudaMemsetAsync(e->counters, 0, (size_t)P.n_kv * ATTN_CLUSTER * 4, e->stream));
    CU(e, cudaMemsetAsync(e->st, 0, sizeof(TokenState), e->stream));
    CU(e, cudaMemsetAsync(e->logits, 0, (size_t)Vl * 4, e->stream));
    CU(e, cudaStreamSynchronize(e->stream));
    rc = loop_setup(e);
    if (rc) return rc;
    chunk_setup(e);
    if (e->decode_path == 2 && !e->loop_ok) return fail(e, TFR_E_UNSUPPORTED, "persistent decode loop unavailable: %s", e->loop_why.c_str());
    e->finalized = true;
    return TFR_OK;
}

// ------------------------------------------------------------------ KV cache

extern "C" int tfr_alloc_kv(tfr_engine* e, int max_seq, tfr_kv** out) {
    if (!e || !out || !e->finalized || max_seq <= 0) return e ? fail(e, TFR_E_INVALID, "alloc_kv: bad state or size") : TFR_E_INVALID;
    cudaSetDevice(e->device);
    tfr_kv* kv = new tfr_kv();
    kv->e = e;
    kv->max_seq = max_seq;
    kv->layer_stride = (size_t)max_seq * e->plan.nkv;
    kv->kv_slot.assign(e->cfg.n_layer, -1);
    for (int i = 0; i < e->cfg.n_layer; i++)
        if (layer_kind(e->cfg, i) != LAYER_LINEAR) kv->kv_slot[i] = kv->n_kv_layers++;
    const size_t bytes = kv->layer_stride * (size_t)(kv->n_kv_layers > 0 ? kv->n_kv_layers : 1) * 2;
    if (cudaMalloc(&kv->k, bytes) != cudaSuccess || cudaMalloc(&kv->v, bytes) != cudaSuccess) {
        cudaFree(kv->k);
        delete kv;
        cudaGetLastError();
        return fail(e, TFR_E_CUDA, "alloc_kv: out of device memory (%zu bytes x2)", bytes);
    }
    cudaMemsetAsync(kv->k, 0, bytes, e->stream);
    cudaMemsetAsync(kv->v, 0, bytes, e->stream);
    if (is_hybrid(e)) {
        const tfr_model_config& c = e->cfg;
        kv->ssm_stride = (size_t)c.ssm_time_step_rank * GDN_D * GDN_D;
        kv->conv_stride = (size_t)c.ssm_conv_kernel * gdn_channels(c);
        const size_t sb = kv->ssm_stride * c.n_layer * 4, cb = kv->conv_stride * c.n_layer * 4;
        if (cudaMalloc(&kv->ssm, sb) != cudaSuccess || cudaMalloc(&kv->conv, cb) != cudaSuccess) {
            cudaGetLastError();
            tfr_free_kv(kv);
            return fail(e, TFR_E_CUDA, "alloc_kv: out of device memory for the recurrent state (%zu bytes)", sb + cb);
        }
        cudaMemsetAsync(kv->ssm, 0, sb, e->stream);
        cudaMemsetAsync(kv->conv, 0, cb, e->stream);
    }
    cudaStreamSynchronize(e->stream);
    *out = kv;
    return TFR_OK;
}
extern "C" void tfr_free_kv(tfr_kv* kv) {
    if (!kv) return;
    if (kv->e && kv->e->graph_kv == kv) drop_graphs(kv->e);
    cudaFree(kv->k);
    cudaFree(kv->v);
    cudaFree(kv->ssm);
    cudaFree(kv->conv);
    delete kv;
}
extern "C" int tfr_kv_len(const tfr_kv* kv) { return kv ? kv->len : TFR_E_INVALID; }
extern "C" int tfr_kv_max_seq(const tfr_kv* kv) { return kv ? kv->max_seq : TFR_E_INVALID; }
extern "C" int tfr_kv_set_len(tfr_kv* kv, int len) {
    if (!kv || len < 0 || len > kv->max_seq) return TFR_E_INVALID;
    kv->len = len;
    return TFR_OK;
}
extern "C" int tfr_kv_clear(tfr_kv* kv) { return tfr_kv_set_len(kv, 0); }
extern "C" int64_t tfr_kv_bytes_per_token(const tfr_kv* kv) {
    if (!kv) return 0;
    const tfr_model_config& c = kv->e->cfg;
    (void)c;
    return (int64_t)kv->n_kv_layers * kv->e->plan.nkv * 2 * 2;  // kv.rs:36-41: full-attention layers only (this rank's KV heads)
}
extern "C" int tfr_zero_recurrent(tfr_engine* e, tfr_kv* kv) {
    if (!e || !kv || kv->e != e) return TFR_E_INVALID;
    if (!kv->ssm) return TFR_OK;  // dense models carry no recurrent state (model.rs:165-194 is a no-op for them)
    cudaSetDevice(e->device);
    CU(e, cudaMemsetAsync(kv->ssm, 0, kv->ssm_stride * e->cfg.n_layer * 4, e->stream));
    CU(e, cudaMemsetAsync(kv->conv, 0, kv->conv_stride * e->cfg.n_layer * 4, e->stream));
    CU(e, cudaStreamSynchronize(e->stream));
    kv->rec_steps = 0;
    return TFR_OK;
}

// ------------------------------------------------------------------ one token

static cudaError_t launch_attention(cudaStream_t s, const AttnArgs& a, int hd, const TokenState* st) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(a.S, a.n_kv);
    cfg.blockDim = dim3(attn_threads(a.staged != 0, hd));
    cfg.dynamicSmemBytes = a.staged ? attn_dyn_smem(hd, a.stages) : 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = attn_cluster(a.staged != 0);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gemv_pdl_enabled() ? 2 : 1;
    if (a.staged) {
        if (hd == 64) return cudaLaunchKernelEx(&cfg, k_attn_decode<64, true>, a, st);
        if (hd == 128) return cudaLaunchKernelEx(&cfg, k_attn_decode<128, true>, a, st);
        return cudaLaunchKernelEx(&cfg, k_attn_decode<256, true>, a, st);
    }
    if (hd == 64) return cudaLaunchKernelEx(&cfg, k_attn_decode<64, false>, a, st);
    if (hd == 128) return cudaLaunchKernelEx(&cfg, k_attn_decode<128, false>, a, st);
    return cudaLaunchKernelEx(&cfg, k_attn_decode<256, false>, a, st);
}

template <class Epi>
static cudaError_t launch_typed(cudaStream_t s, int grid, int type, const PrepArgs& pa, const RowJob& ja, const RowJob& jb,
                                const F32Seg& fseg, const Epi& epi, int K, TokenState* st) {
    if (type == TFR_Q4_K) return launch_gemv<BlockQ4, Epi>(s, grid, pa, ja, jb, fseg, epi, K, st);
    if (type == TFR_Q8_0) return launch_gemv<BlockQ8, Epi>(s, grid, pa, ja, jb, fseg, epi, K, st);
    return launch_gemv<BlockQ6, Epi>(s, grid, pa, ja, jb, fseg, epi, K, st);
}

// Enqueues the kernels of one decode step; returns the number of launches or a negative error.
static int record_token(tfr_engine* e, const tfr_kv* kv, bool with_head) {
    const tfr_model_config& c = e->cfg;
    const TpPlan& P = e->plan;
    const int K = c.n_embd, hd = c.head_dim, nq = P.nq, nkv = P.nkv, FF = P.ff, V = P.v1 - P.v0;
    const int cap = e->prop.multiProcessorCount;  // one 1024-thread CTA per SM
    cudaStream_t s = e->stream;
    int n = 0;
    // y = W x + y for a row-parallel matrix: plain store on one GPU, in-kernel all-reduce otherwise
    auto launch_residual = [&](const tfr_mat* w, const float* vec, int width, int op_index) -> cudaError_t {
        PrepArgs pa{};
        pa.vec = vec;
        pa.prof_id = n;
        const RowJob job = make_job(w->m, 2, cap);
        if (P.tp == 1) {
            EpiStore epi{e->x, nullptr, 2, K};
            return launch_typed(s, cap, w->m.type, pa, job, RowJob{}, F32Seg{}, epi, width, e->st);
        }
        if (e->use_nccl) {
            // comparison baseline: partial y -> ncclAllReduce -> x += y, three nodes instead of one
            EpiStore epi{e->ypart, nullptr, 0, K};
            cudaError_t r = launch_typed(s, cap, w->m.type, pa, job, RowJob{}, F32Seg{}, epi, width, e->st);
            if (r != cudaSuccess) return r;
            if (nccl_api()->AllReduce(e->ypart, e->ypart, (size_t)K, NCCL_FLOAT32, NCCL_SUM, e->nccl_comm, s) != 0) return cudaErrorUnknown;
            n += 2;
            return launch_pdl(k_add_residual, dim3((K + 255) / 256), dim3(256), 0, s, e->x, (const float*)e->ypart, K,
                              (const TokenState*)e->st);
        }
        EpiAllReduce epi{};
        epi.x = e->x;
        epi.n_rows = K;
        epi.sh = job.sh;
        epi.c = e->comm;
        epi.op_index = op_index;
        return launch_typed(s, cap, w->m.type, pa, job, RowJob{}, F32Seg{}, epi, width, e->st);
    };
    for (int li = 0; li < c.n_layer; li++) {
        const LayerW& L = e->layers[li];
        PrepArgs pn{};  // first kernel of the layer: embedding or residual stream, attn_norm, Q8
        pn.vec = li == 0 ? nullptr : e->x;
        pn.embed = e->token_embd->m;
        pn.normw = L.attn_norm;
        pn.eps = c.rms_eps;
        pn.raw_out = e->x;
        pn.prof_id = n;
        AttnArgs a{};
        a.q = e->q;
        a.kc = kv_k(kv, li);
        a.vc = kv_v(kv, li);
        a.partial = e->partial;
        a.counters = e->counters;
        a.out = e->attn + P.attn_off;
        a.gate = nullptr;
        a.n_head = P.n_head;
        a.n_kv = P.n_kv;
        // short caches never reach the long-split route: launch without its shared memory (a lighter launch)
        attn_route(a, hd, kv->max_seq, e->attn_S, e->attn_S_staged, e->attn_min_keys);
        a.scale = 1.0f / sqrtf((float)hd);  // forward.rs:389
        a.prof_id = 0;
        int mix_width = P.attn_width;       // width of the vector the output projection consumes
        const tfr_mat* wout = L.wo;
        if (L.kind == LAYER_LINEAR) {
            // 1. norm + quant + [qkv | z | beta | alpha] projections (layer.rs:736-798)
            if (L.gdn_proj) {
                EpiStore ep{e->proj, nullptr, 0, L.gdn_proj->m.N};
                if (launch_typed(s, cap, L.gdn_proj->m.type, pn, make_job(L.gdn_proj->m, 2, cap), RowJob{}, F32Seg{}, ep, K, e->st) !=
                    cudaSuccess)
                    return -1;
                n++;
            } else {
                // mixed weight types (e.g. a Q5_K attn_qkv beside a Q4_K attn_gate): one launch per matrix, as the
                // reference does (layer.rs:754-797); only the first may be the embedding / residual-writing one
                int off = 0;
                for (int k4 = 0; k4 < 4; k4++) {
                    const tfr_mat* w = L.proj4[k4];
                    PrepArgs pk = pn;
                    if (k4 > 0) {
                        pk.vec = e->x;
                        pk.raw_out = nullptr;
                    }
                    pk.prof_id = n;
                    EpiStore ep{e->proj + off, nullptr, 0, w->m.N};
                    if (launch_typed(s, cap, w->m.type, pk, make_job(w->m, 2, cap), RowJob{}, F32Seg{}, ep, K, e->st) != cudaSuccess)
                        return -1;
                    off += w->m.N;
                    n++;
                }
            }
            // 2. conv + SiLU + L2 + gated delta rule + gated RMSNorm (layer.rs:838-911)
            GdnArgs g{};
            g.proj = e->proj;
            g.conv_w = L.conv_w;
            g.conv_ring = kv->conv + (size_t)li * kv->conv_stride;
            g.state = kv->ssm + (size_t)li * kv->ssm_stride;
            g.ssm_a = L.ssm_a;
            g.ssm_dt = L.ssm_dt;
            g.norm_w = L.ssm_norm;
            g.out = e->attn;
            g.n_k = c.ssm_group_count;
            g.n_v = c.ssm_time_step_rank;
            g.kernel = c.ssm_conv_kernel;
            g.eps = c.rms_eps;
            if (launch_pdl(k_gdn_step, dim3(g.n_v), dim3(GDN_THREADS), 0, s, g, (const TokenState*)e->st) != cudaSuccess) return -1;
            n++;
            mix_width = gdn_val_dim(c);
            wout = L.ssm_out;
        } else if (L.kind == LAYER_FULL_GATED) {
            // 1. norm + quant + raw [Q|gate, K, V] (+bias)
            const RowJob jq = make_job(L.wq->m, 2, cap, 0), jk = make_job(L.wk->m, 2, cap, nq);
            F32Seg fseg{};
            fseg.m = L.wv->m;
            fseg.sh = make_share(nkv / 2, cap);
            fseg.id_base = (2 * nq + nkv) / 2;
            EpiStore ep{e->proj, L.bias_qkv, 0, 2 * nq + 2 * nkv};
            if (launch_gemv<BlockQ4, EpiStore>(s, cap, pn, jq, jk, fseg, ep, K, e->st) != cudaSuccess) return -1;
            n++;
            // 2. per-head Q/K RMSNorm + partial RoPE, Q|gate split, f16 KV store (layer.rs:386-560)
            QkNormArgs qa{};
            qa.raw = e->proj;
            qa.q_norm = L.q_norm;
            qa.k_norm = L.k_norm;
            qa.q_out = e->q;
            qa.gate_out = e->qgate;
            qa.kc = kv_k(kv, li);
            qa.vc = kv_v(kv, li);
            qa.n_head = P.n_head;
            qa.n_kv = P.n_kv;
            qa.hd = hd;
            qa.n_rot = (c.rope_dim > 0 && c.rope_dim < hd) ? c.rope_dim : hd;
            qa.theta = c.rope_theta;
            qa.eps = c.rms_eps;
            if (launch_pdl(k_qk_norm_rope_store, dim3(P.n_head + P.n_kv), dim3(256), 0, s, qa, (const TokenState*)e->st) != cudaSuccess)
                return -1;
            n++;
            // 3. attention with the sigmoid output gate (layer.rs:646-659)
            a.gate = e->qgate;
            a.prof_id = n;
            if (launch_attention(s, a, hd, e->st) != cudaSuccess) return -1;
            n++;
        } else {
            // 1. norm + quant + QKV + rope + KV store
            const RowJob jq = make_job(L.wq->m, 2, cap, 0), jk = make_job(L.wk->m, 2, cap, nq / 2);
            F32Seg fseg{};
            fseg.m = L.wv->m;
            fseg.sh = make_share(nkv / 2, cap);
            fseg.id_base = (nq + nkv) / 2;
            pn.l2_rows_a = (const unsigned char*)(kv_k(kv, li));
            pn.l2_rows_b = (const unsigned char*)(kv_v(kv, li));
            pn.l2_row_bytes = nkv * 2;
            EpiQkv epi{};
            epi.q_out = e->q;
            epi.kc = kv_k(kv, li);
            epi.vc = kv_v(kv, li);
            epi.bias = L.bias_qkv;
            epi.nq = nq;
            epi.nk = nkv;
            epi.hd = hd;
            epi.kvdim = nkv;
            epi.theta = c.rope_theta;
            if (launch_gemv<BlockQ4, EpiQkv>(s, cap, pn, jq, jk, fseg, epi, K, e->st) != cudaSuccess) return -1;
            n++;
            // 2. attention
            a.prof_id = n;
            if (launch_attention(s, a, hd, e->st) != cudaSuccess) return -1;
            n++;
        }
        auto tap = [&](float* dst, const float* src, int width) {
            return !dst || cudaMemcpyAsync(dst + (size_t)li * width, src, (size_t)width * 4, cudaMemcpyDeviceToDevice, s) == cudaSuccess;
        };
        if (!tap(e->tap_attn, e->attn, P.attn_width)) return -1;
        // output projection of the mixer + residual
        if (launch_residual(wout, e->attn, mix_width, 2 * li) != cudaSuccess) return -1;
        n++;
        if (!tap(e->tap_mid, e->x, K)) return -1;
        {  // 4. norm + quant + gate/up + silu*mul
            PrepArgs pa{};
            pa.vec = e->x;
            pa.normw = L.ffn_norm;
            pa.eps = c.rms_eps;
            pa.prof_id = n;
            EpiSilu epi{e->h};
            if (launch_gemv<BlockQ4, EpiSilu>(s, cap, pa, make_job(L.gate->m, 1, cap), make_job(L.up->m, 1, cap), F32Seg{}, epi,
                                              K, e->st) != cudaSuccess)
                return -1;
            n++;
        }
        if (!tap(e->tap_h, e->h, FF)) return -1;
        // 5. down + residual
        if (launch_residual(L.down, e->h, FF, 2 * li + 1) != cudaSuccess) return -1;
        n++;
        if (e->layer_taps &&
            cudaMemcpyAsync(e->layer_taps + (size_t)li * K, e->x, (size_t)K * 4, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
            return -1;
    }
    if (with_head) {
        PrepArgs pa{};
        pa.vec = e->x;
        pa.normw = e->output_norm;
        pa.eps = c.rms_eps;
        pa.prof_id = n;
        EpiLogits epi{};
        epi.logits = e->logits;
        epi.out_tokens = e->out_tokens;
        epi.prompt = e->prompt;
        epi.n_rows = e->vocab_limit ? e->vocab_limit + (e->head_special ? 1 : 0) : V;
        epi.special_row = e->vocab_limit;
        epi.special_id = e->head_special ? e->special_id : -1;
        epi.row_offset = P.v0;
        epi.use_tp = P.tp > 1 && !e->use_nccl;
        epi.c = e->comm;
        epi.defer_best = P.tp > 1 && e->use_nccl ? e->best_buf : nullptr;
        const RowJob extra = e->head_special ? make_job(e->head_special->m, 2, cap, e->vocab_limit / 2) : RowJob{};
        if (launch_typed(s, cap, e->head->m.type, pa, make_job(e->head->m, 2, cap), extra, F32Seg{}, epi, K, e->st) !=
            cudaSuccess)
            return -1;
        n++;
        if (epi.defer_best) {
            if (nccl_api()->AllReduce(e->best_buf, e->best_buf, 1, NCCL_UINT64, NCCL_MAX, e->nccl_comm, s) != 0) return -1;
            if (launch_pdl(k_state_advance, dim3(1), dim3(1), 0, s, e->st, (const unsigned long long*)e->best_buf, e->out_tokens,
                           (const int*)e->prompt) !=
                cudaSuccess)
                return -1;
            n += 2;
        }
    } else {
        if (launch_pdl(k_state_next_prompt, dim3(1), dim3(1), 0, s, e->st, (const int*)e->prompt,
                       P.tp > 1 ? e->comm.ops_per_token : 0) != cudaSuccess)
            return -1;
        n++;
    }
    return n;
}

static int ensure_graphs(tfr_engine* e, const tfr_kv* kv) {
    if (e->graph_kv == kv && e->g_decode && e->g_body) return TFR_OK;
    drop_graphs(e);
    for (int which = 0; which < 2; which++) {
        cudaGraph_t g = nullptr;
        CU(e, cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
        int n = record_token(e, kv, which == 0);
        cudaError_t r = cudaStreamEndCapture(e->stream, &g);
        if (n < 0 || r != cudaSuccess) {
            if (g) cudaGraphDestroy(g);
            cudaGetLastError();
            return fail(e, TFR_E_CUDA, "graph capture failed: %s", cudaGetErrorString(r));
        }
        cudaGraphExec_t ex = nullptr;
        r = cudaGraphInstantiate(&ex, g, 0);
        cudaGraphDestroy(g);
        if (r != cudaSuccess) return fail(e, TFR_E_CUDA, "graph instantiate: %s", cudaGetErrorString(r));
        if (which == 0) {
            e->g_decode = ex;
            e->nodes_decode = n;
        } else {
            e->g_body = ex;
            e->nodes_body = n;
        }
    }
    e->graph_kv = kv;
    return TFR_OK;
}

static int run_token(tfr_engine* e, const tfr_kv* kv, bool with_head) {
    if (e->use_graph) {
        CU(e, cudaGraphLaunch(with_head ? e->g_decode : e->g_body, e->stream));
        e->launches += with_head ? e->nodes_decode : e->nodes_body;
        return TFR_OK;
    }
    int n = record_token(e, kv, with_head);
    if (n < 0) return fail(e, TFR_E_CUDA, "kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    e->launches += n;
    return TFR_OK;
}


// ------------------------------------------------------------------ multi-token chunks

// Models the chunk kernels cover; everything else keeps feeding prompts by decode steps.
static void chunk_setup(tfr_engine* e) {
    const tfr_model_config& c = e->cfg;
    e->chunk_ok = false;
    auto no = [&](const char* why) { e->chunk_why = why; };
    if (c.hybrid) return no("hybrid (Gated-DeltaNet) layers");
    if (e->plan.tp > 1) return no("tensor parallelism");
    auto q468 = [](const tfr_mat* m) { return m->m.type == TFR_Q4_K || m->m.type == TFR_Q6_K || m->m.type == TFR_Q8_0; };
    if (!q468(e->head)) return no("head type");
    for (const LayerW& L : e->layers) {
        if (L.kind != LAYER_DENSE) return no("layer kind");
        if (L.wq->m.type != TFR_Q4_K || L.wk->m.type != TFR_Q4_K || L.gate->m.type != TFR_Q4_K || L.up->m.type != TFR_Q4_K)
            return no("attn_q / attn_k / ffn_gate / ffn_up type");
        if (!q468(L.wo) || !q468(L.down)) return no("attn_output / ffn_down type");
    }
    e->chunk_ok = true;
    e->chunk_why.clear();
}

static int chunk_buffers(tfr_engine* e) {
    if (e->cx) return TFR_OK;
    const TpPlan& P = e->plan;
    const int K = e->cfg.n_embd, M = CHUNK_MAX_TOKENS;
    const int kmax = std::max(std::max(K, P.ff), P.attn_width);
    e->cact_stride = (act_smem_bytes(kmax, false, false) + 255) & ~(size_t)255;
    CU(e, cudaMalloc(&e->cx, (size_t)M * K * 4));
    CU(e, cudaMalloc(&e->cxn, (size_t)M * K * 4));
    CU(e, cudaMalloc(&e->cq, (size_t)M * P.nq * 4));
    CU(e, cudaMalloc(&e->cattn, (size_t)M * P.attn_width * 4));
    CU(e, cudaMalloc(&e->ch, (size_t)M * P.ff * 4));
    CU(e, cudaMalloc(&e->cact, (size_t)M * e->cact_stride));
    CU(e, cudaMalloc(&e->clogits, (size_t)CHUNK_VERIFY_MAX * e->head->m.N * 4));
    CU(e, cudaMalloc(&e->ckeys, (size_t)CHUNK_VERIFY_MAX * ARGMAX_SLICES * 8));
    CU(e, cudaMalloc(&e->ccount, CHUNK_VERIFY_MAX * 4));
    CU(e, cudaMemset(e->ccount, 0, CHUNK_VERIFY_MAX * 4));
    e->cpart_floats = (size_t)M * P.n_head * CHUNK_ATTN_SPLITS_MAX * (2 + e->cfg.head_dim);
    CU(e, cudaMalloc(&e->cpart, e->cpart_floats * 4));
    return TFR_OK;
}

// ws / ws_floats: scratch a launch may use for partial sums (the attention partials' buffer: free between the attention
// of a layer and the next one's).
static cudaError_t launch_gemm_typed(cudaStream_t s, int grid, int type, const unsigned char* act, size_t stride, const float* xn, int M,
                                     const RowJob& ja, const RowJob& jb, const F32Seg& fseg, const ChunkEpi& epi, int K, TokenState* st,
                                     float* ws = nullptr, size_t ws_floats = 0) {
    // Q4_K projections of prompt chunks run their sub-block dots on the tensor cores (one matrix with a pair-ordered
    // epilogue, or the gate / up pair); TFR_GEMM_DP4A=1 in the environment keeps them on the dp4a kernel (a test aid)
    if (type == TFR_Q4_K && M >= GEMM_MMA_MIN_TOKENS && !fseg.m.data && (!jb.m.data || epi.kind == CEPI_SILU) && !getenv("TFR_GEMM_DP4A"))
        return launch_gemm_mma_q4(s, grid, act, stride, M, ja, jb, epi);
    if (type == TFR_Q6_K && M >= GEMM_MMA_MIN_TOKENS && !fseg.m.data && !jb.m.data && epi.kind != CEPI_SILU && !getenv("TFR_GEMM_DP4A"))
        return launch_gemm_mma_q6(s, grid, act, stride, M, ja, epi, ws, ws_floats);
    if (type == TFR_Q4_K) return launch_gemm<BlockQ4>(s, grid, act, stride, xn, M, ja, jb, fseg, epi, K, st);
    if (type == TFR_Q8_0) return launch_gemm<BlockQ8>(s, grid, act, stride, xn, M, ja, jb, fseg, epi, K, st);
    return launch_gemm<BlockQ6>(s, grid, act, stride, xn, M, ja, jb, fseg, epi, K, st);
}

// M tokens (device ids at tok) at positions pos0 .. pos0 + M - 1 through all layers: their K / V rows land in the
// cache and e->cx holds their residual streams.  all_rows: also the greedy token after every position, to
// e->out_tokens[0 .. M).  forward.rs:360-407 (forward_chunk), 292-358 (logits_for_rows).
static int forward_chunk(tfr_engine* e, const tfr_kv* kv, const int* tok, int M, int pos0, bool all_rows) {
    const tfr_model_config& c = e->cfg;
    const TpPlan& P = e->plan;
    const int K = c.n_embd, hd = c.head_dim, nq = P.nq, nkv = P.nkv, FF = P.ff, V = e->head->m.N;
    const int cap = e->prop.multiProcessorCount;
    cudaStream_t s = e->stream;
    int n = 0;
    auto prep = [&](const float* x, int ldx, int width, const float* normw, float* xn) -> cudaError_t {
        PrepRowsArgs a{x, ldx, width, normw, c.rms_eps, e->cact, e->cact_stride, xn};
        const size_t smem = normw ? (xs_floats(width) + 272) * sizeof(float) : 0;
        n++;
        return launch_pdl(k_prep_rows, dim3(M), dim3(GEMV_THREADS), smem, s, a);
    };
    auto store_epi = [&](float* out, int ldo, int rows, int use_res) {
        ChunkEpi ep{};
        ep.kind = CEPI_STORE;
        ep.out = out, ep.ldo = ldo, ep.n_rows = rows, ep.use_res = use_res;
        return ep;
    };
    k_embed_rows<<<M, 256, 0, s>>>(e->token_embd->m, tok, K, e->cx, e->st);
    if (cudaGetLastError() != cudaSuccess) return -1;
    n++;
    for (int li = 0; li < c.n_layer; li++) {
        const LayerW& L = e->layers[li];
        // 1. RMSNorm + Q8, Q/K/V (+bias) + RoPE + f16 KV rows
        if (prep(e->cx, K, K, L.attn_norm, e->cxn) != cudaSuccess) return -1;
        {
            const RowJob jq = make_job(L.wq->m, 2, cap, 0), jk = make_job(L.wk->m, 2, cap, nq / 2);
            F32Seg fseg{};
            fseg.m = L.wv->m;
            fseg.sh = make_share(nkv / 2, cap);
            fseg.id_base = (nq + nkv) / 2;
            ChunkEpi ep{};
            ep.kind = CEPI_QKV;
            ep.out = e->cq, ep.ldo = nq, ep.bias = L.bias_qkv;
            ep.kc = kv_k(kv, li), ep.vc = kv_v(kv, li);
            ep.nq = nq, ep.nk = nkv, ep.hd = hd, ep.kvdim = nkv, ep.pos0 = pos0, ep.theta = c.rope_theta;
            if (M >= GEMM_MMA_MIN_TOKENS && !getenv("TFR_GEMM_DP4A")) {
                // batches from five tokens on: the Q and K rows on the tensor cores (same integer sub-block sums, row sums
                // along k); the fp32-route V rows keep the decode kernels' arithmetic bit for bit
                if (launch_gemm_mma_q4(s, cap, e->cact, e->cact_stride, M, jq, jk, ep) != cudaSuccess) return -1;
                n++;
                if (launch_gemm<BlockQ4>(s, cap, e->cact, e->cact_stride, e->cxn, M, RowJob{}, RowJob{}, fseg, ep, K, e->st) != cudaSuccess) return -1;
            } else if (launch_gemm<BlockQ4>(s, cap, e->cact, e->cact_stride, e->cxn, M, jq, jk, fseg, ep, K, e->st) != cudaSuccess) {
                return -1;
            }
            n++;
        }
        // 2. causal attention over the cache (rows of this chunk included)
        {
            AttnChunkArgs a{};
            a.q = e->cq, a.kc = kv_k(kv, li), a.vc = kv_v(kv, li), a.out = e->cattn;
            a.M = M, a.n_head = P.n_head, a.n_kv = P.n_kv, a.pos0 = pos0, a.kvdim = nkv, a.ldq = nq;
            a.scale = 1.0f / sqrtf((float)hd);  // forward.rs:389
            const int rep = P.n_head / P.n_kv;
            // few tokens (verification batches): one query token per CTA, so that a row's serial walk over the keys is
            // a warp's only work; prompts: four tokens share every K/V tile
            // batches from five tokens on with head sizes up to 128 run on the tensor cores: 128 (token, head) rows per CTA
            const bool mma = M >= GEMM_MMA_MIN_TOKENS && attn_staged_mma(hd) && !getenv("TFR_ATTN_REGISTER_ROUTE");
            a.QT = mma ? std::max(1, ATTM_ROWS / rep) : M <= CHUNK_VERIFY_MAX ? 1 : std::max(1, ATTC_ROWS_MAX / rep);
            const int q_tiles = (M + a.QT - 1) / a.QT;
            // key splits: enough CTAs for every SM, never less than 256 keys per split
            const int blocks256 = (pos0 + M + 255) / 256;
            a.S = std::max(1, std::min(std::min(CHUNK_ATTN_SPLITS_MAX, blocks256), (2 * cap + P.n_kv * q_tiles - 1) / (P.n_kv * q_tiles)));
            a.partial = e->cpart;
            const dim3 grid(P.n_kv, q_tiles, a.S);
            const size_t smem = mma ? attn_chunk_mma_smem(hd) : attn_chunk_smem(hd);
            cudaError_t r = mma ? (hd == 64 ? launch_pdl(k_attn_chunk_mma<64>, grid, dim3(ATTC_THREADS), smem, s, a)
                                            : launch_pdl(k_attn_chunk_mma<128>, grid, dim3(ATTC_THREADS), smem, s, a))
                            : hd == 64  ? launch_pdl(k_attn_chunk<64>, grid, dim3(ATTC_THREADS), smem, s, a)
                            : hd == 128 ? launch_pdl(k_attn_chunk<128>, grid, dim3(ATTC_THREADS), smem, s, a)
                                        : launch_pdl(k_attn_chunk<256>, grid, dim3(ATTC_THREADS), smem, s, a);
            if (r != cudaSuccess) return -1;
            n++;
            if (a.S > 1) {
                if (launch_pdl(k_attn_chunk_merge, dim3(M * P.n_head), dim3(hd), 0, s, (const float*)e->cpart, e->cattn, a.S, hd, P.n_head,
                               nq) != cudaSuccess)
                    return -1;
                n++;
            }
        }
        // 3. Q8 + o-proj + residual
        if (prep(e->cattn, P.attn_width, P.attn_width, nullptr, nullptr) != cudaSuccess) return -1;
        if (launch_gemm_typed(s, cap, L.wo->m.type, e->cact, e->cact_stride, nullptr, M, make_job(L.wo->m, 2, cap), RowJob{}, F32Seg{},
                              store_epi(e->cx, K, K, 2), P.attn_width, e->st) != cudaSuccess)
            return -1;
        n++;
        // 4. RMSNorm + Q8 + gate/up + SiLU*mul
        if (prep(e->cx, K, K, L.ffn_norm, nullptr) != cudaSuccess) return -1;
        {
            ChunkEpi ep{};
            ep.kind = CEPI_SILU;
            ep.out = e->ch, ep.ldo = FF;
            if (launch_gemm_typed(s, cap, L.gate->m.type, e->cact, e->cact_stride, nullptr, M, make_job(L.gate->m, 1, cap), make_job(L.up->m, 1, cap),
                                  F32Seg{}, ep, K, e->st) != cudaSuccess)
                return -1;
            n++;
        }
        // 5. Q8 + down + residual
        if (prep(e->ch, FF, FF, nullptr, nullptr) != cudaSuccess) return -1;
        if (launch_gemm_typed(s, cap, L.down->m.type, e->cact, e->cact_stride, nullptr, M, make_job(L.down->m, 2, cap), RowJob{}, F32Seg{},
                              store_epi(e->cx, K, K, 2), FF, e->st, e->cpart, e->cpart_floats) != cudaSuccess)
            return -1;
        n++;
    }
    if (all_rows) {
        if (prep(e->cx, K, K, e->output_norm, nullptr) != cudaSuccess) return -1;
        if (launch_gemm_typed(s, cap, e->head->m.type, e->cact, e->cact_stride, nullptr, M, make_job(e->head->m, 2, cap), RowJob{},
                              F32Seg{}, store_epi(e->clogits, V, V, 0), K, e->st) != cudaSuccess)
            return -1;
        k_argmax_rows<<<dim3(M, ARGMAX_SLICES), 256, 0, s>>>(e->clogits, V, e->out_tokens, e->ckeys, e->ccount);
        if (cudaGetLastError() != cudaSuccess) return -1;
        // tfr_current_logits reports the last position's row
        if (cudaMemcpyAsync(e->logits, e->clogits + (size_t)(M - 1) * V, (size_t)V * 4, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return -1;
        n += 2;
    }
    e->launches += n;
    return TFR_OK;
}

static int begin_state(tfr_engine* e, const tfr_kv* kv, int token, int pos, int max_steps, int max_seq, const uint32_t* stops,
                       int n_stop, int force_prompt = 0) {
    int* a = e->args_host;
    // the conv ring's write slot follows the position; the offset keeps it continuous when the
    // caller moved the KV length between calls
    const int ck = is_hybrid(e) ? e->cfg.ssm_conv_kernel : 1;
    a[13] = (int)(((kv->rec_steps - pos) % ck + ck) % ck);
    a[14] = force_prompt;
    a[0] = token;
    a[1] = pos;
    a[2] = max_steps;
    a[3] = max_seq;
    a[4] = n_stop;
    for (int i = 0; i < 8; i++) a[5 + i] = i < n_stop ? (int)stops[i] : -1;
    CU(e, cudaMemcpyAsync(e->args_dev, a, 16 * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    k_state_begin<<<1, 1, 0, e->stream>>>(e->st, e->args_dev);
    CU(e, cudaGetLastError());
    e->launches += 1;
    return TFR_OK;
}

static int finish_state(tfr_engine* e, int n_tokens_out) {
    CU(e, cudaMemcpyAsync(e->st_host, e->st, sizeof(TokenState), cudaMemcpyDeviceToHost, e->stream));
    if (n_tokens_out > 0)
        CU(e, cudaMemcpyAsync(e->out_host, e->out_tokens, (size_t)n_tokens_out * 4, cudaMemcpyDeviceToHost, e->stream));
    CU(e, cudaStreamSynchronize(e->stream));
    cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1);
    if (e->st_host->err == 3) return fail(e, TFR_E_CUDA, "tensor parallelism: a peer rank did not deliver within the wait limit");
    if (e->st_host->err == 4) return fail(e, TFR_E_CUDA, "persistent decode loop: a grid-wide barrier did not complete within the wait limit");
    if (e->st_host->err == 2) return fail(e, TFR_E_CUDA, "a weight tile copy did not complete");
    if (e->st_host->err) return fail(e, TFR_E_INVALID, "device reported an invalid token id");
    return TFR_OK;
}

extern "C" int tfr_forward_greedy(tfr_engine* e, tfr_kv* kv, const uint32_t* tokens, int n, uint32_t* next_token) {
    if (!e || !kv || kv->e != e || !e->finalized) return e ? fail(e, TFR_E_INVALID, "forward_greedy: bad handle") : TFR_E_INVALID;
    if (n <= 0 || !tokens) return fail(e, TFR_E_EMPTY, "empty tokens");
    if (e->plan.tp > 1 && !tp_ready(e)) return fail(e, TFR_E_INVALID, "tensor-parallel ranks are not connected (tfr_tp_attach_*)");
    if (kv->len + n > kv->max_seq) return fail(e, TFR_E_FULL, "context full");
    if (n > TFR_MAX_PROMPT) return fail(e, TFR_E_INVALID, "more than %d tokens in one call", TFR_MAX_PROMPT);
    for (int i = 0; i < n; i++)
        if (tokens[i] >= (uint32_t)e->token_embd->m.N) return fail(e, TFR_E_INVALID, "token id %u out of range", tokens[i]);
    cudaSetDevice(e->device);
    const bool loop = use_loop(e);
    if (e->use_graph && !loop) {
        int rc = ensure_graphs(e, kv);
        if (rc) return rc;
    }
    CU(e, cudaMemcpyAsync(e->prompt, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
    // all but the last token go through the chunk kernels (weights read once per chunk); the last is a decode step
    const bool chunked = !loop && e->chunk_ok && e->chunk_tokens > 0 && n > 1;
    int rc = TFR_OK;
    if (chunked) rc = chunk_buffers(e);
    if (rc) return rc;
    rc = begin_state(e, kv, (int)tokens[chunked ? n - 1 : 0], kv->len + (chunked ? n - 1 : 0), 1, kv->max_seq + 1, nullptr, 0);
    if (rc) return rc;
    CU(e, cudaEventRecord(e->ev0, e->stream));
    if (loop) {
        rc = run_loop(e, kv, n - 1);
    } else if (chunked) {
        for (int i = 0; i < n - 1 && !rc; i += e->chunk_tokens) {
            const int M = std::min(e->chunk_tokens, n - 1 - i);
            if (forward_chunk(e, kv, e->prompt + i, M, kv->len + i, false) != TFR_OK)
                rc = fail(e, TFR_E_CUDA, "chunk kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        }
        if (!rc) rc = run_token(e, kv, true);
    } else {
        for (int i = 0; i < n && !rc; i++) rc = run_token(e, kv, i == n - 1);
    }
    if (rc) return rc;
    CU(e, cudaEventRecord(e->ev1, e->stream));
    rc = finish_state(e, 1);
    if (rc) return rc;
    kv->len += n;
    kv->rec_steps += n;
    if (next_token) *next_token = (uint32_t)e->out_host[0];
    return TFR_OK;
}

// CudaModel::forward_greedy_all, forward.rs:268-290: the caller's tokens are fed one per step (not the model's
// own predictions) and the greedy prediction after EVERY position comes back.
extern "C" int tfr_forward_greedy_all(tfr_engine* e, tfr_kv* kv, const uint32_t* tokens, int n, uint32_t* out) {
    if (!e || !kv || kv->e != e || !e->finalized || !out) return e ? fail(e, TFR_E_INVALID, "forward_greedy_all: bad argument") : TFR_E_INVALID;
    if (n <= 0 || !tokens) return fail(e, TFR_E_EMPTY, "empty tokens");
    if (e->plan.tp > 1 && !tp_ready(e)) return fail(e, TFR_E_INVALID, "tensor-parallel ranks are not connected (tfr_tp_attach_*)");
    if (kv->len + n > kv->max_seq) return fail(e, TFR_E_FULL, "context full");
    if (n > TFR_MAX_BURST) return fail(e, TFR_E_INVALID, "more than %d tokens in one call", TFR_MAX_BURST);
    for (int i = 0; i < n; i++)
        if (tokens[i] >= (uint32_t)e->token_embd->m.N) return fail(e, TFR_E_INVALID, "token id %u out of range", tokens[i]);
    cudaSetDevice(e->device);
    const bool loop = use_loop(e);
    if (e->use_graph && !loop) {
        int rc = ensure_graphs(e, kv);
        if (rc) return rc;
    }
    CU(e, cudaMemcpyAsync(e->prompt, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
    const bool chunked = !loop && e->chunk_ok && e->chunk_tokens > 0 && n > 1 && !e->vocab_limit;
    int rc = TFR_OK;
    if (chunked) {
        // one weight pass per chunk of up to CHUNK_VERIFY_MAX tokens (the reference: MAX_VERIFY_TOKENS = 9 per pass)
        rc = chunk_buffers(e);
        if (rc) return rc;
        rc = begin_state(e, kv, (int)tokens[0], kv->len, n, kv->max_seq + 1, nullptr, 0, 1);  // resets the error word
        if (rc) return rc;
        CU(e, cudaEventRecord(e->ev0, e->stream));
        for (int i = 0; i < n; i += CHUNK_VERIFY_MAX) {
            const int M = std::min(CHUNK_VERIFY_MAX, n - i);
            if (forward_chunk(e, kv, e->prompt + i, M, kv->len + i, true) != TFR_OK)
                return fail(e, TFR_E_CUDA, "chunk kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
            CU(e, cudaMemcpyAsync(e->out_host + i, e->out_tokens, (size_t)M * 4, cudaMemcpyDeviceToHost, e->stream));
        }
        CU(e, cudaEventRecord(e->ev1, e->stream));
        rc = finish_state(e, 0);
        if (rc) return rc;
        for (int i = 0; i < n; i++) out[i] = (uint32_t)e->out_host[i];
        kv->len += n;
        kv->rec_steps += n;
        return TFR_OK;
    }
    rc = begin_state(e, kv, (int)tokens[0], kv->len, n, kv->max_seq + 1, nullptr, 0, 1);
    if (rc) return rc;
    CU(e, cudaEventRecord(e->ev0, e->stream));
    if (loop) rc = run_loop(e, kv, 0);
    else
        for (int i = 0; i < n && !rc; i++) rc = run_token(e, kv, true);
    if (rc) return rc;
    CU(e, cudaEventRecord(e->ev1, e->stream));
    rc = finish_state(e, n);
    if (rc) return rc;
    for (int i = 0; i < n; i++) out[i] = (uint32_t)e->out_host[i];
    kv->len += n;
    kv->rec_steps += n;
    return TFR_OK;
}

extern "C" int tfr_decode_burst(tfr_engine* e, tfr_kv* kv, uint32_t first_token, int max_n, const uint32_t* stop_ids, int n_stop,
                                uint32_t* out, int* n_out) {
    if (!e || !kv || kv->e != e || !e->finalized || !out || !n_out)
        return e ? fail(e, TFR_E_INVALID, "decode_burst: bad argument") : TFR_E_INVALID;
    if (max_n <= 0) return fail(e, TFR_E_EMPTY, "empty tokens");
    if (e->plan.tp > 1 && !tp_ready(e)) return fail(e, TFR_E_INVALID, "tensor-parallel ranks are not connected (tfr_tp_attach_*)");
    if (n_stop < 0 || n_stop > 8) return fail(e, TFR_E_INVALID, "at most 8 stop ids");
    if (kv->len + 1 > kv->max_seq) return fail(e, TFR_E_FULL, "context full");
    if (first_token >= (uint32_t)e->token_embd->m.N) return fail(e, TFR_E_INVALID, "token id %u out of range", first_token);
    cudaSetDevice(e->device);
    int n_run = max_n < TFR_MAX_BURST ? max_n : TFR_MAX_BURST;
    if (n_run > kv->max_seq - kv->len) n_run = kv->max_seq - kv->len;
    const bool loop = use_loop(e);
    if (e->use_graph && !loop) {
        int rc = ensure_graphs(e, kv);
        if (rc) return rc;
    }
    int rc = begin_state(e, kv, (int)first_token, kv->len, n_run, kv->max_seq + 1, stop_ids, n_stop);
    if (rc) return rc;
    CU(e, cudaEventRecord(e->ev0, e->stream));
    if (loop) rc = run_loop(e, kv, 0);
    else
        for (int i = 0; i < n_run && !rc; i++) rc = run_token(e, kv, true);
    if (rc) return rc;
    CU(e, cudaEventRecord(e->ev1, e->stream));
    rc = finish_state(e, n_run);
    if (rc) return rc;
    const int produced = e->st_host->step;
    for (int i = 0; i < produced; i++) out[i] = (uint32_t)e->out_host[i];
    *n_out = produced;
    kv->len += produced;
    kv->rec_steps += produced;
    return TFR_OK;
}

extern "C" int tfr_current_logits(tfr_engine* e, float* out, int n) {
    if (!e || !out || !e->finalized || n <= 0 || n > e->cfg.n_vocab) return e ? fail(e, TFR_E_INVALID, "current_logits: bad argument") : TFR_E_INVALID;
    cudaSetDevice(e->device);
    const int active = e->vocab_limit ? e->vocab_limit + (e->head_special ? 1 : 0) : e->plan.v1;
    const int first = e->plan.v0, end = active < n ? active : n;
    if (end > first) CU(e, cudaMemcpyAsync(out + first, e->logits, (size_t)(end - first) * 4, cudaMemcpyDeviceToHost, e->stream));
    CU(e, cudaStreamSynchronize(e->stream));
    return TFR_OK;
}

extern "C" int tfr_set_vocab_shortlist(tfr_engine* e, int limit, int special_id) {
    if (!e || !e->has_cfg) return TFR_E_INVALID;
    if (e->finalized) return fail(e, TFR_E_INVALID, "set_vocab_shortlist: the model is already finalized");
    if (limit == 0) {
        e->vocab_limit = 0;
        e->special_id = -1;
        return TFR_OK;
    }
    // load.rs:301: limits below 1024 or not below n_vocab are ignored there; here they are an error
    if (limit < 1024 || limit >= e->cfg.n_vocab || (limit & 1))
        return fail(e, TFR_E_INVALID, "set_vocab_shortlist: limit %d must be even, >= 1024 and < n_vocab %d", limit, e->cfg.n_vocab);
    // load.rs:308: the extra row exists only for an id outside the shortlist
    e->vocab_limit = limit;
    e->special_id = (special_id >= limit && special_id < e->cfg.n_vocab) ? special_id : -1;
    return TFR_OK;
}
extern "C" int tfr_active_vocab(const tfr_engine* e, int* n_active, int* special_id) {
    if (!e || !e->has_cfg) return TFR_E_INVALID;
    const bool extra = e->vocab_limit && e->special_id >= 0;
    if (n_active) *n_active = e->vocab_limit ? e->vocab_limit + (extra ? 1 : 0) : e->cfg.n_vocab;
    if (special_id) *special_id = extra ? e->special_id : -1;
    return TFR_OK;
}

// ------------------------------------------------------------------ tensor-parallel wiring

extern "C" int tfr_tp_exchange_bytes(const tfr_engine* e, size_t* bytes) {
    if (!e || !bytes || !e->finalized) return TFR_E_INVALID;
    *bytes = e->plan.tp > 1 ? e->comm.lay.total : 0;
    return TFR_OK;
}
extern "C" int tfr_tp_vocab_range(const tfr_engine* e, int* first, int* end) {
    if (!e || !e->has_cfg) return TFR_E_INVALID;
    if (first) *first = e->plan.v0;
    if (end) *end = e->plan.v1;
    return TFR_OK;
}
extern "C" int tfr_tp_ipc_handle(tfr_engine* e, void* handle_out) {
    if (!e || !handle_out || !e->finalized || e->plan.tp < 2) return e ? fail(e, TFR_E_INVALID, "tp_ipc_handle: not a tensor-parallel engine") : TFR_E_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
    cudaSetDevice(e->device);
    cudaIpcMemHandle_t h;
    CU(e, cudaIpcGetMemHandle(&h, e->comm_local));
    memcpy(handle_out, &h, sizeof h);
    return TFR_OK;
}
static int tp_finish_attach(tfr_engine* e) {
    e->comm.base[e->plan.rank] = e->comm_local;
    e->peers_wired = true;
    drop_graphs(e);
    return TFR_OK;
}
extern "C" int tfr_tp_attach_ipc(tfr_engine* e, const void* handles) {
    if (!e || !handles || !e->finalized || e->plan.tp < 2) return e ? fail(e, TFR_E_INVALID, "tp_attach_ipc: not a tensor-parallel engine") : TFR_E_INVALID;
    if (e->peers_wired) return fail(e, TFR_E_INVALID, "ranks already connected");
    cudaSetDevice(e->device);
    for (int r = 0; r < e->plan.tp; r++) {
        if (r == e->plan.rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t*)handles + (size_t)r * sizeof h, sizeof h);
        void* ptr = nullptr;
        CU(e, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        e->comm.base[r] = (unsigned char*)ptr;
    }
    e->comm_ipc = true;
    return tp_finish_attach(e);
}
extern "C" int tfr_tp_local_pointer(tfr_engine* e, void** ptr) {
    if (!e || !ptr || !e->finalized || e->plan.tp < 2) return TFR_E_INVALID;
    *ptr = e->comm_local;
    return TFR_OK;
}
extern "C" int tfr_tp_attach_pointers(tfr_engine* e, void* const* bases) {
    if (!e || !bases || !e->finalized || e->plan.tp < 2) return e ? fail(e, TFR_E_INVALID, "tp_attach_pointers: not a tensor-parallel engine") : TFR_E_INVALID;
    if (e->peers_wired) return fail(e, TFR_E_INVALID, "ranks already connected");
    cudaSetDevice(e->device);
    for (int r = 0; r < e->plan.tp; r++) {
        if (r == e->plan.rank) continue;
        cudaPointerAttributes at{};
        CU(e, cudaPointerGetAttributes(&at, bases[r]));
        if (at.type != cudaMemoryTypeDevice) return fail(e, TFR_E_INVALID, "rank %d: not a device pointer", r);
        if (at.device != e->device) {
            int can = 0;
            CU(e, cudaDeviceCanAccessPeer(&can, e->device, at.device));
            if (!can) return fail(e, TFR_E_UNSUPPORTED, "device %d cannot access device %d", e->device, at.device);
            cudaError_t r2 = cudaDeviceEnablePeerAccess(at.device, 0);
            if (r2 != cudaSuccess && r2 != cudaErrorPeerAccessAlreadyEnabled) return fail(e, TFR_E_CUDA, "peer access: %s", cudaGetErrorString(r2));
            cudaGetLastError();
        }
        e->comm.base[r] = (unsigned char*)bases[r];
    }
    return tp_finish_attach(e);
}

extern "C" int tfr_tp_nccl_unique_id(void* id_out_128_bytes) {
    NcclApi* api = nccl_api();
    if (!api || !id_out_128_bytes) return TFR_E_UNSUPPORTED;
    return api->GetUniqueId(id_out_128_bytes) == 0 ? TFR_OK : TFR_E_CUDA;
}
extern "C" int tfr_tp_use_nccl(tfr_engine* e, const void* id_128_bytes) {
    if (!e || !e->finalized || e->plan.tp < 2) return e ? fail(e, TFR_E_INVALID, "tp_use_nccl: not a tensor-parallel engine") : TFR_E_INVALID;
    cudaSetDevice(e->device);
    if (!id_128_bytes) {  // back to the in-kernel exchange, which needs the peers' buffers
        if (!e->peers_wired) return fail(e, TFR_E_INVALID, "tp_use_nccl(NULL): the ranks' exchange buffers were never connected (tfr_tp_attach_*)");
        e->use_nccl = false;
        drop_graphs(e);
        return TFR_OK;
    }
    NcclApi* api = nccl_api();
    if (!api) return fail(e, TFR_E_UNSUPPORTED, "libnccl.so.2 could not be loaded");
    if (!e->nccl_comm) {
        NcclId id;
        memcpy(id.b, id_128_bytes, sizeof id.b);
        const int rc = api->CommInitRank(&e->nccl_comm, e->plan.tp, id, e->plan.rank);
        if (rc != 0) return fail(e, TFR_E_CUDA, "ncclCommInitRank: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
        CU(e, cudaMalloc(&e->ypart, (size_t)e->cfg.n_embd * 4));
        CU(e, cudaMalloc(&e->best_buf, 8));
    }
    e->use_nccl = true;
    e->nccl_ready = true;
    drop_graphs(e);
    return TFR_OK;
}

extern "C" int tfr_set_cuda_graph(tfr_engine* e, int enabled) {
    if (!e) return TFR_E_INVALID;
    e->use_graph = enabled != 0;
    if (!e->use_graph) drop_graphs(e);
    return TFR_OK;
}
extern "C" int tfr_graph_active(const tfr_engine* e) { return e && e->use_graph && e->g_decode ? 1 : 0; }
extern "C" int64_t tfr_launch_count(const tfr_engine* e) { return e ? e->launches : 0; }
extern "C" float tfr_last_device_ms(const tfr_engine* e) { return e ? e->last_ms : 0.f; }

extern "C" int tfr_set_decode_path(tfr_engine* e, int path) {
    if (!e || path < 0 || path > 2) return TFR_E_INVALID;
    if (path == 2 && e->finalized && !e->loop_ok)
        return fail(e, TFR_E_UNSUPPORTED, "persistent decode loop unavailable: %s", e->loop_why.c_str());
    e->decode_path = path;
    return TFR_OK;
}
extern "C" int tfr_set_prefill_chunk(tfr_engine* e, int tokens) {
    if (!e || tokens < 0) return TFR_E_INVALID;
    e->chunk_tokens = tokens > CHUNK_MAX_TOKENS ? CHUNK_MAX_TOKENS : tokens;
    return TFR_OK;
}
// Tokens per chunk in effect: 0 when prompts are fed by decode steps (switched off, or a model the chunk kernels do
// not cover).
extern "C" int tfr_prefill_chunk(const tfr_engine* e) { return e && e->finalized && e->chunk_ok ? e->chunk_tokens : 0; }

extern "C" int tfr_decode_path(const tfr_engine* e) {
    if (!e) return TFR_E_INVALID;
    return use_loop(e) ? 2 : 1;
}
#ifdef TFR_TEST_AIDS
extern "C" int tfr_debug_set_loop_timeline(tfr_engine* e, unsigned long long* device_buffer, int step, int points) {
    if (!e) return TFR_E_INVALID;
    e->loop_prof = device_buffer;
    e->loop_prof_step = step;
    e->loop_prof_points = device_buffer ? points : 0;
    return TFR_OK;
}

#endif  // TFR_TEST_AIDS

extern "C" int tfr_debug_read(tfr_engine* e, tfr_kv* kv, const char* what, int layer, void* out, size_t nbytes) {
    if (!e || !what || !out || !e->finalized) return TFR_E_INVALID;
    const tfr_model_config& c = e->cfg;
    const void* src = nullptr;
    size_t have = 0;
    std::string w(what);
    if (w == "x") src = e->x, have = (size_t)c.n_embd * 4;
    else if (w == "q") src = e->q, have = (size_t)c.n_head * c.head_dim * 4;
    else if (w == "attn") src = e->attn, have = (size_t)std::max(c.n_head * c.head_dim, c.hybrid ? gdn_val_dim(c) : 0) * 4;
    else if (w == "h") src = e->h, have = (size_t)c.n_ff * 4;
    else if (w == "logits") src = e->logits, have = (size_t)c.n_vocab * 4;
    else if (w == "layer_x") {
        // residual stream after every layer of the last step; the first request switches the taps on
        if (!e->layer_taps) {
            cudaSetDevice(e->device);
            CU(e, cudaMalloc(&e->layer_taps, (size_t)c.n_layer * c.n_embd * 4));
            CU(e, cudaMemset(e->layer_taps, 0, (size_t)c.n_layer * c.n_embd * 4));
            drop_graphs(e);
        }
        src = e->layer_taps, have = (size_t)c.n_layer * c.n_embd * 4;
    }
    else if (w == "layer_attn" || w == "layer_mid" || w == "layer_h") {
        // per-layer taps of the last step (dense models, chained kernels); the first request switches them on
        if (c.hybrid || e->plan.tp > 1) return fail(e, TFR_E_UNSUPPORTED, "debug_read: %s is for dense single-GPU models", what);
        if (!e->tap_attn) {
            cudaSetDevice(e->device);
            CU(e, cudaMalloc(&e->tap_attn, (size_t)c.n_layer * e->plan.attn_width * 4));
            CU(e, cudaMalloc(&e->tap_mid, (size_t)c.n_layer * c.n_embd * 4));
            CU(e, cudaMalloc(&e->tap_h, (size_t)c.n_layer * e->plan.ff * 4));
            CU(e, cudaMemset(e->tap_attn, 0, (size_t)c.n_layer * e->plan.attn_width * 4));
            CU(e, cudaMemset(e->tap_mid, 0, (size_t)c.n_layer * c.n_embd * 4));
            CU(e, cudaMemset(e->tap_h, 0, (size_t)c.n_layer * e->plan.ff * 4));
            drop_graphs(e);
        }
        if (w == "layer_attn") src = e->tap_attn, have = (size_t)c.n_layer * e->plan.attn_width * 4;
        else if (w == "layer_mid") src = e->tap_mid, have = (size_t)c.n_layer * c.n_embd * 4;
        else src = e->tap_h, have = (size_t)c.n_layer * e->plan.ff * 4;
    }
    else if (w == "proj" && e->proj) src = e->proj, have = (size_t)(gdn_channels(c) + gdn_val_dim(c) + 2 * c.ssm_time_step_rank) * 4;
    else if (w == "qgate" && e->qgate) src = e->qgate, have = (size_t)c.n_head * c.head_dim * 4;
    else if (w == "ssm_state" && kv && kv->ssm && layer >= 0 && layer < c.n_layer)
        src = kv->ssm + (size_t)layer * kv->ssm_stride, have = kv->ssm_stride * 4;
    else if (w == "conv_state" && kv && kv->conv && layer >= 0 && layer < c.n_layer) {
        // the reference's window [kernel-1][channels], oldest first (deltanet.cu:530-559), read out of the ring
        const int ck = c.ssm_conv_kernel, km1 = ck - 1, ch = gdn_channels(c);
        if (nbytes > (size_t)km1 * ch * 4) return fail(e, TFR_E_INVALID, "debug_read: conv_state holds %d floats", km1 * ch);
        std::vector<float> ring((size_t)ck * ch);
        cudaSetDevice(e->device);
        CU(e, cudaStreamSynchronize(e->stream));
        CU(e, cudaMemcpy(ring.data(), kv->conv + (size_t)layer * kv->conv_stride, ring.size() * 4, cudaMemcpyDeviceToHost));
        std::vector<float> win((size_t)km1 * ch);
        for (int k = 0; k < km1; k++) {
            const int slot = (int)(((kv->rec_steps - km1 + k) % ck + ck) % ck);
            memcpy(win.data() + (size_t)k * ch, ring.data() + (size_t)slot * ch, (size_t)ch * 4);
        }
        memcpy(out, win.data(), nbytes);
        return TFR_OK;
    }
    else if ((w == "k" || w == "v") && kv && layer >= 0 && layer < c.n_layer) {
        if (kv->kv_slot[layer] < 0) return fail(e, TFR_E_INVALID, "debug_read: layer %d is a linear-attention layer and has no K/V cache", layer);
        src = w == "k" ? kv_k(kv, layer) : kv_v(kv, layer);
        have = kv->layer_stride * 2;
    } else return fail(e, TFR_E_INVALID, "debug_read: unknown tap %s", what);
    if (nbytes > have) return fail(e, TFR_E_INVALID, "debug_read: %zu bytes requested, %zu available", nbytes, have);
    cudaSetDevice(e->device);
    CU(e, cudaStreamSynchronize(e->stream));
    CU(e, cudaMemcpy(out, src, nbytes, cudaMemcpyDeviceToHost));
    return TFR_OK;
}

// ------------------------------------------------------------------ operator level

#ifdef TFR_TEST_AIDS
// Test aid: the KV-store rounding (f32_to_f16_bits_ref) applied to n device floats.
__global__ void k_debug_f32_to_f16(const float* src, unsigned short* dst, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = f32_to_f16_bits_ref(src[i]);
}
extern "C" int tfr_debug_f32_to_f16(const float* src, uint16_t* dst, int64_t n, void* stream) {
    if (!src || !dst || n < 0) return TFR_E_INVALID;
    if (n == 0) return TFR_OK;
    k_debug_f32_to_f16<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(src, dst, (long long)n);
    return cudaGetLastError() == cudaSuccess ? TFR_OK : TFR_E_CUDA;
}

extern "C" int tfr_debug_set_timeline(unsigned long long* device_buffer) {
    return cudaMemcpyToSymbol(g_prof, &device_buffer, sizeof(device_buffer)) == cudaSuccess ? TFR_OK : TFR_E_CUDA;
}

#endif  // TFR_TEST_AIDS

// The operator entry points have no engine to keep a message in: a CUDA error is named on stderr.
static int check(cudaError_t r) {
    if (r == cudaSuccess) return TFR_OK;
    fprintf(stderr, "tarafer_b200: CUDA error: %s\n", cudaGetErrorString(r));
    return TFR_E_CUDA;
}

extern "C" int tfr_op_quantize_q8(const float* x, int n, int8_t* q8, float* d8, void* stream) {
    if (!x || !q8 || !d8 || n <= 0 || n % 32) return TFR_E_INVALID;
    const int groups = n / 32;
    k_quantize_q8<<<(groups + 7) / 8, 256, 0, (cudaStream_t)stream>>>(x, (signed char*)q8, d8, n);
    return check(cudaGetLastError());
}

extern "C" int tfr_op_gemv(const tfr_mat* w, const float* x, float* out, const float* bias, int use_res, int act_mode,
                           const float* norm_w, float eps, void* stream) {
    if (!w || !x || !out) return TFR_E_INVALID;
    if (act_mode == 1 && w->m.type != TFR_Q6_K) return TFR_E_UNSUPPORTED;
    if (w->perm_hd) return TFR_E_INVALID;  // row-permuted matrices only make sense in the fused QKV kernel
    configure_kernels_once();
    PrepArgs pa{};
    pa.vec = x;
    pa.normw = norm_w;
    pa.eps = eps;
    const int C = sm_count_cached();
    RowJob ja = make_job(w->m, 2, C);
    F32Seg fseg{};
    if (act_mode == 1) {
        ja.sh = make_share(0, C);  // every row goes through the fp32-activation route
        fseg.m = w->m;
        fseg.sh = make_share((w->m.N + 1) / 2, C);
        fseg.id_base = 0;
    }
    EpiStore epi{out, bias, use_res, w->m.N};
    return check(launch_typed((cudaStream_t)stream, C, w->m.type, pa, ja, RowJob{}, fseg, epi, w->m.K, nullptr));
}

extern "C" int tfr_op_ffn_gate_up(const tfr_mat* gate, const tfr_mat* up, const float* x, const float* norm_w, float eps, float* h,
                                  void* stream) {
    if (!gate || !up || !x || !h) return TFR_E_INVALID;
    if (gate->m.type != TFR_Q4_K || up->m.type != TFR_Q4_K || gate->m.K != up->m.K || gate->m.N != up->m.N) return TFR_E_UNSUPPORTED;
    configure_kernels_once();
    PrepArgs pa{};
    pa.vec = x;
    pa.normw = norm_w;
    pa.eps = eps;
    const int C = sm_count_cached();
    EpiSilu epi{h};
    return check(launch_gemv<BlockQ4, EpiSilu>((cudaStream_t)stream, C, pa, make_job(gate->m, 1, C), make_job(up->m, 1, C),
                                               F32Seg{}, epi, gate->m.K, nullptr));
}

extern "C" int tfr_op_ffn_block(const tfr_mat* gate, const tfr_mat* up, const tfr_mat* down, const float* x, float* h_scratch,
                                float* y, int use_res, void* stream) {
    if (!down || !y || !h_scratch || !gate || down->m.K != gate->m.N) return TFR_E_INVALID;
    int rc = tfr_op_ffn_gate_up(gate, up, x, nullptr, 0.f, h_scratch, stream);
    if (rc) return rc;
    return tfr_op_gemv(down, h_scratch, y, nullptr, use_res, 0, nullptr, 0.f, stream);
}

extern "C" int tfr_ffn_block_host(const tfr_mat* gate, const tfr_mat* up, const tfr_mat* down, const float* x_host, float* y_host) {
    if (!gate || !up || !down || !x_host || !y_host) return TFR_E_INVALID;
    const int K = gate->m.K, FF = gate->m.N, N = down->m.N;
    // device buffers of this convenience call, grown on demand, one set per device
    struct HostBlockBufs {
        float *dx = nullptr, *dh = nullptr, *dy = nullptr;
        int cap_k = 0, cap_f = 0, cap_n = 0;
    };
    static HostBlockBufs bufs[TFR_MAX_DEVICES];
    HostBlockBufs& hb = bufs[current_device_slot()];
    float *&dx = hb.dx, *&dh = hb.dh, *&dy = hb.dy;
    int &cap_k = hb.cap_k, &cap_f = hb.cap_f, &cap_n = hb.cap_n;
    if (K > cap_k || FF > cap_f || N > cap_n) {
        cudaFree(dx), cudaFree(dh), cudaFree(dy);
        if (cudaMalloc(&dx, (size_t)K * 4) != cudaSuccess || cudaMalloc(&dh, (size_t)FF * 4) != cudaSuccess ||
            cudaMalloc(&dy, (size_t)N * 4) != cudaSuccess)
            return TFR_E_CUDA;
        cap_k = K, cap_f = FF, cap_n = N;
    }
    if (cudaMemcpyAsync(dx, x_host, (size_t)K * 4, cudaMemcpyHostToDevice, nullptr) != cudaSuccess) return TFR_E_CUDA;
    int rc = tfr_op_ffn_block(gate, up, down, dx, dh, dy, 0, nullptr);
    if (rc) return rc;
    if (cudaMemcpyAsync(y_host, dy, (size_t)N * 4, cudaMemcpyDeviceToHost, nullptr) != cudaSuccess) return TFR_E_CUDA;
    return check(cudaStreamSynchronize(nullptr));
}

#ifdef TFR_TEST_AIDS
static int int_dots_impl(const tfr_mat* w, const float* x, const int8_t* q8, const float* d8, int32_t* a, int32_t* b, int8_t* q8_out,
                         void* stream) {
    if (!w || !a || w->perm_hd) return TFR_E_INVALID;
    if (w->m.type == TFR_Q4_K && !b) return TFR_E_INVALID;
    configure_kernels_once();
    const size_t smem = act_smem_bytes(w->m.K, false, false);
    const int grid = sm_count_cached();
    cudaStream_t s = (cudaStream_t)stream;
    if (w->m.type == TFR_Q4_K) k_int_dots<BlockQ4><<<grid, 256, smem, s>>>(w->m, x, (const signed char*)q8, d8, a, b, (signed char*)q8_out);
    else if (w->m.type == TFR_Q8_0) k_int_dots<BlockQ8><<<grid, 256, smem, s>>>(w->m, x, (const signed char*)q8, d8, a, b, (signed char*)q8_out);
    else k_int_dots<BlockQ6><<<grid, 256, smem, s>>>(w->m, x, (const signed char*)q8, d8, a, b, (signed char*)q8_out);
    return check(cudaGetLastError());
}
extern "C" int tfr_op_int_dots(const tfr_mat* w, const int8_t* q8, const float* d8, int32_t* a, int32_t* b, void* stream) {
    if (!q8 || !d8) return TFR_E_INVALID;
    return int_dots_impl(w, nullptr, q8, d8, a, b, nullptr, stream);
}
extern "C" int tfr_op_int_dots_x(const tfr_mat* w, const float* x, int32_t* a, int32_t* b, int8_t* q8_out, void* stream) {
    if (!x) return TFR_E_INVALID;
    return int_dots_impl(w, x, nullptr, nullptr, a, b, q8_out, stream);
}

#endif  // TFR_TEST_AIDS

static int op_attention_impl(const float* q, const uint16_t* kc, const uint16_t* vc, const float* gate, float* out, int n_head,
                             int n_kv, int head_dim, int pos, void* stream) {
    if (!q || !kc || !vc || !out || n_kv <= 0 || n_head % n_kv || n_head / n_kv > ATTN_REP_MAX || pos < 0) return TFR_E_INVALID;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return TFR_E_UNSUPPORTED;
    if (n_kv > 64) return TFR_E_UNSUPPORTED;
    configure_kernels_once();
    // scratch for the stand-alone call: partials + counters, grown on demand and kept, one set per device.
    // All calls on a device share it: calls that overlap on the GPU (different streams or threads) race on it.
    struct AttnScratch {
        float* partial = nullptr;
        unsigned int* counters = nullptr;
        size_t cap = 0;
    };
    static AttnScratch scratch[TFR_MAX_DEVICES];
    AttnScratch& sc = scratch[current_device_slot()];
    float*& partial = sc.partial;
    unsigned int*& counters = sc.counters;
    size_t& cap = sc.cap;
    AttnArgs a{};
    attn_route(a, head_dim, pos + 1, attn_splits(sm_count_cached(), n_kv, head_dim, false), attn_splits(sm_count_cached(), n_kv, head_dim, true), 64);
    const size_t need = (size_t)n_head * a.S * (2 + head_dim) * 4;
    if (need > cap || !counters) {
        cudaFree(partial);
        if (!counters) {
            if (cudaMalloc(&counters, 64 * ATTN_CLUSTER * 4) != cudaSuccess) return TFR_E_CUDA;
            cudaMemset(counters, 0, 64 * ATTN_CLUSTER * 4);
        }
        if (cudaMalloc(&partial, need) != cudaSuccess) return TFR_E_CUDA;
        cap = need;
    }
    a.q = q;
    a.kc = kc;
    a.vc = vc;
    a.partial = partial;
    a.counters = counters;
    a.out = out;
    a.n_head = n_head;
    a.n_kv = n_kv;
    a.gate = gate;
    a.scale = 1.0f / sqrtf((float)head_dim);
    a.pos = pos;
    return check(launch_attention((cudaStream_t)stream, a, head_dim, nullptr));
}

extern "C" int tfr_op_attention(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                                int head_dim, int pos, void* stream) {
    return op_attention_impl(q, kc, vc, nullptr, out, n_head, n_kv, head_dim, pos, stream);
}
extern "C" int tfr_op_attention_gated(const float* q, const uint16_t* kc, const uint16_t* vc, const float* gate, float* out,
                                      int n_head, int n_kv, int head_dim, int pos, void* stream) {
    if (!gate) return TFR_E_INVALID;
    return op_attention_impl(q, kc, vc, gate, out, n_head, n_kv, head_dim, pos, stream);
}

extern "C" int tfr_op_gdn_step(const float* proj, const float* conv_w, float* conv_ring, float* state, const float* ssm_a,
                               const float* ssm_dt, const float* norm_w, float* out, int n_k, int n_v, int state_size,
                               int kernel, int slot, float eps, void* stream) {
    if (!proj || !conv_w || !conv_ring || !state || !ssm_a || !ssm_dt || !norm_w || !out || n_k <= 0 || n_v <= 0) return TFR_E_INVALID;
    if (state_size != GDN_D || kernel < 2 || kernel > GDN_MAX_KERNEL) return TFR_E_UNSUPPORTED;
    if (slot < 0 || slot >= kernel) return TFR_E_INVALID;
    configure_kernels_once();
    GdnArgs g{};
    g.proj = proj;
    g.conv_w = conv_w;
    g.conv_ring = conv_ring;
    g.state = state;
    g.ssm_a = ssm_a;
    g.ssm_dt = ssm_dt;
    g.norm_w = norm_w;
    g.out = out;
    g.n_k = n_k;
    g.n_v = n_v;
    g.kernel = kernel;
    g.eps = eps;
    g.slot = slot;
    k_gdn_step<<<n_v, GDN_THREADS, 0, (cudaStream_t)stream>>>(g, nullptr);
    return check(cudaGetLastError());
}

extern "C" int tfr_op_qk_norm_rope_store(const float* raw, const float* q_norm, const float* k_norm, float* q_out, float* gate_out,
                                         uint16_t* kc, uint16_t* vc, int n_head, int n_kv, int head_dim, int n_rot, int pos,
                                         float theta, float eps, void* stream) {
    if (!raw || !q_out || !gate_out || !kc || !vc || n_head <= 0 || n_kv <= 0 || pos < 0) return TFR_E_INVALID;
    if (head_dim <= 0 || head_dim > 256 || n_rot < 0 || n_rot > head_dim || n_rot % 2) return TFR_E_UNSUPPORTED;
    configure_kernels_once();
    QkNormArgs a{};
    a.raw = raw;
    a.q_norm = q_norm;
    a.k_norm = k_norm;
    a.q_out = q_out;
    a.gate_out = gate_out;
    a.kc = kc;
    a.vc = vc;
    a.n_head = n_head;
    a.n_kv = n_kv;
    a.hd = head_dim;
    a.n_rot = n_rot;
    a.theta = theta;
    a.eps = eps;
    a.pos = pos;
    k_qk_norm_rope_store<<<n_head + n_kv, 256, 0, (cudaStream_t)stream>>>(a, nullptr);
    return check(cudaGetLastError());
}

// ---- flash-decode without any allocation --------------------------------------------------
//
// Some callers of this library must not allocate device memory at the moment they need
// attention: code running while a CUDA graph is being captured on another stream of the same
// context, hosts that hand the GPU a fixed memory budget at start-up and forbid later growth,
// and real-time loops where an allocator call (which may synchronise the whole device) is not
// acceptable.  For them the split-KV scratch of the decode kernel — the per-split (m, l, O)
// partials and the per-KV-head arrival counters — lives in a fixed array inside the library
// image.  Every GPU that loads the library carries these TFR_NOALLOC_SCRATCH_BYTES until exit.
constexpr size_t TFR_NOALLOC_COUNTER_BYTES = 2048;           // 64 KV heads x 8 output slices
constexpr size_t TFR_NOALLOC_SCRATCH_BYTES = 2u << 20;       // counters + partials, 2 MiB in total
static __device__ __align__(256) unsigned char g_attn_noalloc_scratch[TFR_NOALLOC_SCRATCH_BYTES];
constexpr int TFR_NOALLOC_MAX_DEVICES = 64;
static unsigned char* g_attn_noalloc_ptr[TFR_NOALLOC_MAX_DEVICES] = {};  // device address of the array, per device

extern "C" int tfr_op_attention_noalloc(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head,
                                        int n_kv, int head_dim, int pos, void* stream) {
    if (!q || !kc || !vc || !out || n_kv <= 0 || n_head % n_kv || n_head / n_kv > ATTN_REP_MAX || pos < 0) return TFR_E_INVALID;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return TFR_E_UNSUPPORTED;
    int dev = -1, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= TFR_NOALLOC_MAX_DEVICES) return TFR_E_CUDA;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return TFR_E_CUDA;
    configure_kernels_once();  // function attributes only (shared-memory carve-out): nothing is allocated
    AttnArgs a{};
    attn_route(a, head_dim, pos + 1, attn_splits(sms, n_kv, head_dim, false), attn_splits(sms, n_kv, head_dim, true), 64);
    const size_t need = (size_t)n_head * a.S * (2 + head_dim) * sizeof(float);
    if ((size_t)n_kv * ATTN_CLUSTER * sizeof(unsigned int) > TFR_NOALLOC_COUNTER_BYTES || need > TFR_NOALLOC_SCRATCH_BYTES - TFR_NOALLOC_COUNTER_BYTES) {
        fprintf(stderr,
                "tfr_op_attention_noalloc: %d heads / %d KV heads / head_dim %d need %zu bytes of split scratch; the built-in "
                "array holds %zu\n",
                n_head, n_kv, head_dim, need, TFR_NOALLOC_SCRATCH_BYTES - TFR_NOALLOC_COUNTER_BYTES);
        return TFR_E_UNSUPPORTED;
    }
    // The array's name is only a host-side handle here; the kernel needs its address on THIS device.
    // Looked up once per device, with that device current (it is: cudaGetDevice above).
    if (!g_attn_noalloc_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_attn_noalloc_scratch) != cudaSuccess || !p) return TFR_E_CUDA;
        g_attn_noalloc_ptr[dev] = (unsigned char*)p;
    }
    unsigned char* base = g_attn_noalloc_ptr[dev];
    cudaStream_t s = (cudaStream_t)stream;
    // the array keeps whatever the previous call left: the arrival counters must start at zero
    if (cudaMemsetAsync(base, 0, TFR_NOALLOC_COUNTER_BYTES, s) != cudaSuccess) return TFR_E_CUDA;
    a.q = q;
    a.kc = kc;
    a.vc = vc;
    a.counters = reinterpret_cast<unsigned int*>(base);
    a.partial = reinterpret_cast<float*>(base + TFR_NOALLOC_COUNTER_BYTES);
    a.out = out;
    a.n_head = n_head;
    a.n_kv = n_kv;
    a.scale = 1.0f / sqrtf((float)head_dim);
    a.pos = pos;
    return check(launch_attention(s, a, head_dim, nullptr));
}

extern "C" int tfr_op_qkv_rope_store(const tfr_mat* wq, const tfr_mat* wk, const tfr_mat* wv, const float* bq, const float* bk,
                                     const float* bv, const float* x, const float* norm_w, float eps, float theta, int head_dim,
                                     int pos, float* q_out, uint16_t* kc, uint16_t* vc, void* stream) {
    if (!wq || !wk || !wv || !x || !q_out || !kc || !vc) return TFR_E_INVALID;
    if (wq->perm_hd != head_dim || wk->perm_hd != head_dim || wv->perm_hd) return TFR_E_INVALID;
    if (wq->m.type != TFR_Q4_K || wk->m.type != TFR_Q4_K) return TFR_E_UNSUPPORTED;
    configure_kernels_once();
    cudaStream_t s = (cudaStream_t)stream;
    const int nq = wq->m.N, nkv = wk->m.N, tot = nq + 2 * nkv;
    float* bias = nullptr;
    if (bq || bk || bv) {
        static float* bias_buf = nullptr;
        static int bias_cap = 0;
        if (tot > bias_cap) {
            cudaFree(bias_buf);
            if (cudaMalloc(&bias_buf, (size_t)tot * 4) != cudaSuccess) return TFR_E_CUDA;
            bias_cap = tot;
        }
        bias = bias_buf;
        cudaMemsetAsync(bias, 0, (size_t)tot * 4, s);
        if (bq) k_permute_f32<<<(nq + 255) / 256, 256, 0, s>>>(bq, bias, nq, head_dim);
        if (bk) k_permute_f32<<<(nkv + 255) / 256, 256, 0, s>>>(bk, bias + nq, nkv, head_dim);
        if (bv) k_permute_f32<<<(nkv + 255) / 256, 256, 0, s>>>(bv, bias + nq + nkv, nkv, 0);
    }
    if (wv->m.type != TFR_Q6_K) return TFR_E_UNSUPPORTED;
    PrepArgs pa{};
    pa.vec = x;
    pa.normw = norm_w;
    pa.eps = eps;
    const int C = sm_count_cached();
    const RowJob jq = make_job(wq->m, 2, C, 0), jk = make_job(wk->m, 2, C, nq / 2);
    F32Seg fseg{};
    fseg.m = wv->m;
    fseg.sh = make_share(nkv / 2, C);
    fseg.id_base = (nq + nkv) / 2;
    EpiQkv epi{};
    epi.q_out = q_out;
    epi.kc = kc;
    epi.vc = vc;
    epi.bias = bias;
    epi.nq = nq;
    epi.nk = nkv;
    epi.hd = head_dim;
    epi.kvdim = nkv;
    epi.theta = theta;
    epi.pos = pos;
    return check(launch_gemv<BlockQ4, EpiQkv>(s, C, pa, jq, jk, fseg, epi, wq->m.K, nullptr));
}

#ifdef TFR_TEST_AIDS
// ------------------------------------------------------------------ synthetic quantiser (test and benchmark aid)

// One thread per 256-element super-block.  Asymmetric min/max per 32-element sub-block.
__global__ void k_synth_q4k(const float* __restrict__ w, uint8_t* __restrict__ out, long long n_blocks) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const float* x = w + b * 256;
    uint8_t* o = out + b * 144;
    float scale[8], mins[8], smax = 0.f, mmax = 0.f;
    for (int j = 0; j < 8; j++) {
        float lo = 0.f, hi = -1e30f;
        for (int i = 0; i < 32; i++) {
            lo = fminf(lo, x[32 * j + i]);
            hi = fmaxf(hi, x[32 * j + i]);
        }
        hi = fmaxf(hi, lo);
        scale[j] = (hi - lo) / 15.f;
        mins[j] = -lo;
        smax = fmaxf(smax, scale[j]);
        mmax = fmaxf(mmax, mins[j]);
    }
    const __half dh = __float2half_rn(smax / 63.f), mh = __float2half_rn(mmax / 63.f);
    const float d = __half2float(dh), dmin = __half2float(mh);
    int sc[8], mn[8];
    for (int j = 0; j < 8; j++) {
        sc[j] = d > 0.f ? min(63, max(0, (int)rintf(scale[j] / d))) : 0;
        mn[j] = dmin > 0.f ? min(63, max(0, (int)rintf(mins[j] / dmin))) : 0;
    }
    *reinterpret_cast<unsigned short*>(o) = __half_as_ushort(dh);
    *reinterpret_cast<unsigned short*>(o + 2) = __half_as_ushort(mh);
    for (int j = 0; j < 4; j++) {
        o[4 + j] = (uint8_t)(sc[j] | ((sc[j + 4] >> 4) << 6));
        o[8 + j] = (uint8_t)(mn[j] | ((mn[j + 4] >> 4) << 6));
        o[12 + j] = (uint8_t)((sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4));
    }
    for (int t = 0; t < 4; t++) {
        const float s0 = d * sc[2 * t], s1 = d * sc[2 * t + 1];
        const float o0 = dmin * mn[2 * t], o1 = dmin * mn[2 * t + 1];
        for (int l = 0; l < 32; l++) {
            const int q0 = s0 > 0.f ? min(15, max(0, (int)rintf((x[64 * t + l] + o0) / s0))) : 0;
            const int q1 = s1 > 0.f ? min(15, max(0, (int)rintf((x[64 * t + 32 + l] + o1) / s1))) : 0;
            o[16 + 32 * t + l] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

// One thread per 256-element block.  Symmetric per 16-element group.
__global__ void k_synth_q6k(const float* __restrict__ w, uint8_t* __restrict__ out, long long n_blocks) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const float* x = w + b * 256;
    uint8_t* o = out + b * 210;
    float gs[16], gmax = 0.f;
    for (int g = 0; g < 16; g++) {
        float am = 0.f;
        for (int i = 0; i < 16; i++) am = fmaxf(am, fabsf(x[16 * g + i]));
        gs[g] = am / 31.f;
        gmax = fmaxf(gmax, gs[g]);
    }
    const __half dh = __float2half_rn(gmax / 127.f);
    const float d = __half2float(dh);
    int sc[16];
    for (int g = 0; g < 16; g++) sc[g] = d > 0.f ? min(127, max(0, (int)rintf(gs[g] / d))) : 0;
    for (int i = 0; i < 192; i++) o[i] = 0;
    for (int e = 0; e < 256; e++) {
        const float step = d * sc[e >> 4];
        const int q = (step > 0.f ? min(31, max(-32, (int)rintf(x[e] / step))) : 0) + 32;
        const int n = e >> 7, r = e & 127, j = r >> 5, l = r & 31;
        const int qi = 64 * n + ((j & 1) ? 32 : 0) + l;
        o[qi] |= (uint8_t)((q & 0xF) << ((j & 2) ? 4 : 0));
        o[128 + 32 * n + l] |= (uint8_t)((q >> 4) << (2 * j));
    }
    for (int g = 0; g < 16; g++) o[192 + g] = (uint8_t)(signed char)sc[g];
    *reinterpret_cast<unsigned short*>(o + 208) = __half_as_ushort(dh);
}

extern "C" int tfr_synth_quantize(int type, const float* w, int64_t K, int64_t N, void* out, void* stream) {
    if (!w || !out || K <= 0 || K % 256 || N <= 0) return TFR_E_INVALID;
    const long long nblk = (long long)N * (K / 256);
    const int grid = (int)((nblk + 127) / 128);
    if (type == TFR_Q4_K) k_synth_q4k<<<grid, 128, 0, (cudaStream_t)stream>>>(w, (uint8_t*)out, nblk);
    else if (type == TFR_Q6_K) k_synth_q6k<<<grid, 128, 0, (cudaStream_t)stream>>>(w, (uint8_t*)out, nblk);
    else return TFR_E_UNSUPPORTED;
    return check(cudaGetLastError());
}
#endif  // TFR_TEST_AIDS
