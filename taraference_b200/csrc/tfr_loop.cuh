// Persistent decode loop: ONE cooperative kernel runs a whole burst of batch-1 decode steps.
//
// The chained-kernel path pays a kernel boundary per matrix-vector product: the successor cannot
// start its weight stream until the predecessor's CTAs have left the SM, and every CTA repeats
// the serial prologue.  Here one CTA per SM lives for the whole burst:
//
//   * the last warp is the weight streamer.  It walks the static schedule of the token (per layer:
//     Q/K/V, o-proj, gate/up, down; then the vocabulary head) and keeps a ring of shared-memory slots
//     full with bulk copies (TMA, this GPU's memory, no multicast).  The schedule does not depend on
//     any activation, so the stream never stops at a phase boundary: while the consumers wait for a
//     grid-wide hand-over, the next phases' tiles are already landing.  Lane l owns ring slot l.
//   * the other warps are consumers.  A phase is: fetch the phase's input vector, RMSNorm + Q8 it into
//     shared memory, run the block dots on the tiles as they arrive, sum rows in a fixed order, run
//     the epilogue (bias, RoPE, KV store, SiLU*mul, residual, logits + argmax), grid barrier.
//   * activations travel between CTAs as plain fp32 vectors in global memory (they stay in L2),
//     published by a grid-wide barrier (fence + arrival counters) after every phase.
//   * attention is a phase of the same kernel: CTA (kv head, split) walks its keys for all query
//     heads of the group; up to a few splits are merged by the o-proj prologue itself, more by a
//     small merge phase.
//   * position, token, step and stop state live in registers of every CTA (all CTAs compute the
//     same values from the grid-wide argmax), so a burst never touches the host.
//
// Code size is a first-order cost here.  At batch 1 a thread runs two or three block dots per layer,
// so nearly every instruction of a layer executes once per visit; measured on this part, straight-line
// code beyond about 32 KB is fetched from L2 on every pass and runs at 6 to 15 cycles per instruction
// and warp instead of 1 to 3.  Hence: one copy of every routine shared by all phases (functions kept
// out of line, the epilogue chosen by a run-time switch), loops kept rolled, one lanes-per-block
// split, state in shared memory rather than in stack frames (with nearly all of the SM's memory
// carved out for the ring, local memory misses L1).
//
// Layer schedule: crates/core/src/cuda/layer.rs:142-709, 1210-1456, 2125-2259 at n_tok = 1; token
// loop: crates/core/src/cuda/forward.rs:73-105 (the reference replays a 580-node graph and reads the
// argmax back every token).
//
// Every wait is bounded (cycle limit); on expiry the CTA records an error word, raises its abort
// flag, skips all later waits and leaves at the next token boundary; the streamer drains its copies
// before the CTA exits.
#pragma once
#include <algorithm>
#include <cstring>
#include <vector>

#include "tfr_gemv.cuh"

namespace tfr {

#ifndef TFR_LOOP_CWARPS
#define TFR_LOOP_CWARPS 23
#endif
constexpr int LOOP_CWARPS = TFR_LOOP_CWARPS;  // consumer warps; the warp after them streams weights
constexpr int LOOP_THREADS = (LOOP_CWARPS + 1) * 32;
constexpr int LOOP_CT = LOOP_CWARPS * 32;    // consumer threads (a multiple of 8: the quantiser works on groups of 8 lanes)
constexpr int LOOP_SLOT = 13824;             // 3 Q4_K tiles (13824 B) or 2 Q6_K tiles (13440 B)
constexpr int LOOP_EMPTY = 24;               // arrivals that free a slot (divisible by every tasks-per-entry count)
constexpr int LOOP_MAX_SLOTS = 16;
constexpr int LOOP_TK = 64;                  // keys per attention tile
constexpr int LOOP_REP_MAX = 8;              // query heads per KV head
constexpr int LOOP_INLINE_MAX = 4;           // most split-KV partials the o-proj prologue merges by itself
constexpr long long LOOP_SPIN_CYCLES = 1500000000ll;  // upper bound of any wait, about 0.8 s
constexpr int LOOP_BAR_STRIDE = 32;          // words between the eight grid-barrier counters (128 B apart)

enum { CTL_STOP = 0, CTL_ABORT = 1, CTL_SNAP = 2, CTL_STOPS = 8, CTL_WORDS = 16 };  // [CTL_STOPS, +8): stop ids
enum { LEPI_QKV = 0, LEPI_RESIDUAL = 1, LEPI_SILU = 2, LEPI_LOGITS = 3 };

// One matrix of a phase, spread over the CTAs in contiguous shares of `rpi` rows.
struct LoopJob {
    int type;     // TFR_Q4_K / TFR_Q6_K; 0: absent
    int N;        // rows
    int rpi;      // rows per share item: 2 (row pairs) or 1
    int id_base;  // epilogue id of the matrix's first item
    int f32;      // 1: fp32-activation route (Q6_K attn_v, kernels/gemv.cu:233-264)
    Share sh;
};

struct LoopPhase {
    LoopJob job[3];
    int K, nb;
    int lpb;   // lanes per 256-weight block on the Q8 route: 1, 2 or 4
    int rpc;   // rows per chunk (the partial-sum buffer bounds a chunk); 0: one chunk
    int zip;   // 1: job 0 and job 1 are walked together (gate / up)
};

struct LoopLayer {
    const uint8_t *wq, *wk, *wv, *wo, *gate, *up, *down;  // in the order of the schedule's matrix ids 0..6
    const float *bias_qkv, *attn_norm, *ffn_norm;
    int o_q6, down_q6;  // 1: the matrix is Q6_K (selects the phase descriptor)
};

struct LoopArgs {
    const LoopLayer* layers;
    int n_layer, K, FF, nq, nkv, hd, hd_shift, n_head, n_kv, rep, V;
    float eps, theta, attn_scale;
    Mat embed;
    const uint8_t* head;
    const float* out_norm;
    int sec_nb[7], sec_zip[7];  // per schedule section: 256-weight blocks per row, gate/up pairing
    unsigned short *kc, *vc;
    size_t kv_layer_stride;  // elements
    // vectors handed from phase to phase through global memory: residual stream, q, attention output,
    // SiLU*mul output, split-KV partials [n_head][attn_smax][4 + hd] = (m, l, -, -, O); logits for the host
    float *x, *q, *att, *h, *pc, *logits;
    Share sh_x;              // row pairs of the residual stream per CTA (the shares of o-proj and down)
    int off_own;             // shared memory: the CTA's own residual rows
    float* layer_taps;       // optional [n_layer][K]
    unsigned int* bar;       // 8 counters, LOOP_BAR_STRIDE words apart, zero at launch
    unsigned long long* best;  // [4] packed argmax keys, zero at launch
    TokenState* st;
    int* out_tokens;
    const int* prompt;
    int n_headless;          // leading steps that only feed a prompt token (no head)
    int nslot;
    int attn_min_keys, attn_smax, attn_inline_max;
    // The static plan, built on the host (loop_build_plan): per CTA one blob of `blob_stride` ints that the kernel
    // copies to shared memory at its start.  Sections: 0 Q/K/V, 1 o-proj Q4_K, 2 o-proj Q6_K, 3 gate/up, 4 down Q4_K,
    // 5 down Q6_K, 6 head.
    //   [0, 14)        per section: first ring entry, entry count       (streamer)
    //   [14, 28)       per section: first chunk, chunk count            (consumers)
    //   [blob_chunks)  ChunkDesc per chunk
    //   [blob_tasks)   TaskDesc per task of sections 0..5; the head's tasks stay in global memory (head_tasks)
    //   [blob_sched)   ring entries (uint2) of all sections
    const int* blob;
    const uint4* head_tasks;
    int blob_stride, blob_chunks, blob_tasks, blob_sched, head_stride;
    int off_blob, off_layers;  // shared-memory offsets of the blob copy and of the per-layer pointer table
    int off_act, off_xf, off_pbuf, off_ring;  // shared-memory map (bytes); attention scratch aliases [off_act, off_ring)
    int pbuf_floats;
    unsigned long long* prof;  // optional timeline: [point][cta], see loop_mark
    int prof_step, prof_points;
};

// CTA-wide state of the kernel.  It lives in SHARED memory: anything that ends up in a thread's stack frame (a
// context struct passed by reference, spilled registers) costs an L2 round trip per access here.  Every field is
// the same for all threads; thread 0 writes the per-phase fields and advances the counters between barriers.
struct LoopCtx {
    float *xf, *pbuf, *red, *own;
    unsigned long long *full, *empty;
    volatile int *issued, *ctl;
    unsigned long long* ctl_best;
    unsigned char* ring;
    unsigned char* work;        // activation | staged vector | partial sums (the attention scratch aliases it)
    const int* blob;            // this CTA's plan in shared memory
    const LoopLayer* lay;       // per-layer pointers in shared memory
    int cta, G, nslot;
    unsigned bar_k;             // grid barriers passed
    int slot, lap;              // ring cursor of the consumers: slot and use count of the next schedule entry
    int mark_id, mark_on;
    int own_row0;               // first residual row this CTA owns
    // the running layer / step (epilogues and attention read them)
    unsigned short *kc, *vc;    // layer base of the cache
    const float* bias;          // Q/K/V biases of the layer in pair order, or nullptr
    float* tap;                 // optional per-layer copy of the residual stream
    int pos;
    int at_S, at_g, at_s, at_t0, at_t1, at_active;  // this CTA's share of the step's attention
};
constexpr int LOOP_CTX_OFFSET = 1536;  // after the barriers, control words and reduction scratch
__device__ __forceinline__ int ltid() { return (int)threadIdx.x; }
__device__ __forceinline__ int llane() { return (int)threadIdx.x & 31; }
__device__ __forceinline__ int lwarp() { return (int)threadIdx.x >> 5; }

__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, %0;" ::"n"(LOOP_CT) : "memory"); }
__device__ __forceinline__ void mbar_arrive_n(unsigned long long* bar, unsigned n) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
// try_wait with a suspend-time hint: the warp is parked by the hardware until the phase completes or about `ns`
// nanoseconds have passed, instead of spinning through issue slots that the streamer and working warps need.
__device__ __forceinline__ bool mbar_try_wait_hint(unsigned long long* bar, unsigned int parity, unsigned int ns) {
    unsigned int ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_add_u32(unsigned* p, unsigned v) {
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void loop_fail(LoopCtx& c, const LoopArgs& a, int code) {
    a.st->err = code;
    c.ctl[CTL_ABORT] = 1;
    c.ctl[CTL_STOP] = 1;
}

// Timeline probe (builds with -DTFR_TEST_AIDS only): thread 0 stores the nanosecond timer at successive points of one
// decode step.
#ifdef TFR_TEST_AIDS
__device__ __noinline__ void loop_mark(LoopCtx& c, const LoopArgs& a) {
    if (ltid() == 0 && c.mark_on) {
        if (c.mark_id < a.prof_points) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            a.prof[(size_t)c.mark_id * c.G + c.cta] = t;
        }
        c.mark_id++;
    }
}
#else
__device__ __forceinline__ void loop_mark(LoopCtx&, const LoopArgs&) {}
#endif

__host__ __device__ __forceinline__ void cursor_advance(int& slot, int& lap, int n, int nslot) {
    slot += n;
    while (slot >= nslot) {
        slot -= nslot;
        lap++;
    }
}

// Flat 256-weight blocks [f0, f1) of one matrix inside one chunk of a phase, for one CTA (f0 == f1: none).
struct JobSpan {
    int f0, f1;
};
__host__ __device__ __forceinline__ JobSpan job_span(const LoopJob& j, int nb, int cta, int chunk, int rpc) {
    JobSpan v;
    v.f0 = v.f1 = 0;
    if (!j.type) return v;
    const int i0 = j.sh.begin(cta), cnt = j.sh.count(cta);
    int ra = i0 * j.rpi, rb = (i0 + cnt) * j.rpi < j.N ? (i0 + cnt) * j.rpi : j.N;
    if (rpc > 0) {
        ra += chunk * rpc;
        rb = rb < ra + rpc ? rb : ra + rpc;
    }
    if (rb <= ra) return v;
    v.f0 = ra * nb;
    v.f1 = rb * nb;
    return v;
}
__host__ __device__ __forceinline__ int span_t0(const JobSpan& v) { return v.f0 >> 5; }
__host__ __device__ __forceinline__ int span_tiles(const JobSpan& v) { return v.f1 > v.f0 ? ((v.f1 + 31) >> 5) - (v.f0 >> 5) : 0; }
__host__ __device__ __forceinline__ int type_tile_bytes(int type) { return type == TFR_Q4_K ? Q4_TILE_BYTES : Q6_TILE_BYTES; }
__host__ __device__ __forceinline__ int type_tpe(int type) { return type == TFR_Q4_K ? LOOP_SLOT / Q4_TILE_BYTES : LOOP_SLOT / Q6_TILE_BYTES; }
__host__ __device__ __forceinline__ int span_entries(const JobSpan& v, int type) {
    const int tpe = type_tpe(type);
    return (span_tiles(v) + tpe - 1) / tpe;
}
__host__ __device__ __forceinline__ int phase_chunks(const LoopPhase& ph, int cta) {
    if (ph.rpc <= 0) return 1;
    int rows = 0;
#pragma unroll
    for (int j = 0; j < 3; j++) {
        const LoopJob& jb = ph.job[j];
        if (!jb.type) continue;
        const int i0 = jb.sh.begin(cta), cnt = jb.sh.count(cta);
        const int r = ((i0 + cnt) * jb.rpi < jb.N ? (i0 + cnt) * jb.rpi : jb.N) - i0 * jb.rpi;
        rows = rows > r ? rows : r;
    }
    return (rows + ph.rpc - 1) / ph.rpc;
}

// ------------------------------------------------------------------ plan helpers (host)

inline LoopJob loop_job(int type, int N, int rpi, int id_base, int f32, int G) {
    LoopJob j{};
    j.type = type;
    j.N = N;
    j.rpi = rpi;
    j.id_base = id_base;
    j.f32 = f32;
    j.sh = make_share((N + rpi - 1) / rpi, G);
    return j;
}
// Finishes a phase descriptor: block-split and, when the CTA's block partials exceed the buffer, a chunk size.
// Most tiles a CTA's share of the job can touch (a share may straddle a tile at either end).
inline int loop_job_tiles(const LoopJob& j, int nb) {
    if (!j.type) return 0;
    const int rows = (j.sh.quot + (j.sh.rem ? 1 : 0)) * j.rpi;
    return rows ? (rows * nb + 31) / 32 + 1 : 0;
}
// Lanes per block for a phase.  A warp task costs a fixed part (descriptor, tile wait, partial store, slot release)
// plus the block dots; at batch 1 a phase is a handful of task rounds, so the split that needs the fewest dependent
// instructions on the busiest warp wins: whole blocks per lane in the large phases, halves or quarters where the
// phase has fewer tiles than the CTA has warps.
inline int loop_pick_lpb(int q8_tiles, int f32_tiles) {
    double best = 1e30;
    int pick = 1;
    for (int L = 1; L <= 4; L *= 2) {
        const int tasks = q8_tiles * L + f32_tiles * 4;
        const double rounds = (double)((tasks + LOOP_CWARPS - 1) / LOOP_CWARPS);
        const double cost = rounds * (120.0 + 300.0 / L);
        if (cost < best - 1e-9) best = cost, pick = L;
    }
    return pick;
}
inline bool loop_finish_phase(LoopPhase& ph, int K, int pbuf_floats, int lpb_forced) {
    ph.K = K;
    ph.nb = K / 256;
    int q8_tiles = 0, f32_tiles = 0, need = 0, rows_max = 0, njobs = 0, rpi = 1;
    for (int j = 0; j < 3; j++) {
        const LoopJob& jb = ph.job[j];
        if (!jb.type) continue;
        njobs++;
        (jb.f32 ? f32_tiles : q8_tiles) += loop_job_tiles(jb, ph.nb);
        const int rows = (jb.sh.quot + (jb.sh.rem ? 1 : 0)) * jb.rpi;
        need += rows * ph.nb;
        rows_max = (rows_max > rows ? rows_max : rows);
        rpi = (rpi > jb.rpi ? rpi : jb.rpi);
    }
    ph.lpb = (lpb_forced == 1 || lpb_forced == 2 || lpb_forced == 4) ? lpb_forced : loop_pick_lpb(q8_tiles, f32_tiles);
    ph.rpc = 0;
    if (need <= pbuf_floats) return true;
    if (njobs > 1 && !ph.zip) return false;  // independent matrices of one phase are not chunked
    // rows per chunk: even (row pairs) and, where it costs nothing, on tile borders
    int g = 32, a = ph.nb;
    while (a) {
        const int t = g % a;
        g = a;
        a = t;
    }
    int unit = 32 / g;
    if (unit % rpi) unit *= rpi;
    const int cap_rows = pbuf_floats / (ph.nb * njobs);
    if (cap_rows < rpi) return false;
    const int n_chunks = (rows_max + cap_rows - 1) / cap_rows;
    int rpc = (rows_max + n_chunks - 1) / n_chunks;
    rpc = (rpc + unit - 1) / unit * unit;
    if (rpc > cap_rows) rpc = cap_rows / unit * unit;
    if (rpc < rpi) rpc = cap_rows / rpi * rpi;
    ph.rpc = rpc;
    return rpc >= rpi;
}

// ------------------------------------------------------------------ weight streamer (the last warp)

__device__ __forceinline__ bool mbar_test_wait(unsigned long long* bar, unsigned int parity) {
    unsigned int ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// One ring entry of the static schedule: a run of whole tiles of one matrix.
//   x = byte offset inside the matrix / 16;  y = bytes / 16 | matrix id << 16
// matrix ids: 0 wq, 1 wk, 2 wv, 3 wo, 4 gate, 5 up, 6 down, 7 head.
constexpr int SCHED_SECTIONS = 7;
__host__ __device__ __forceinline__ uint2 sched_entry(long long byte_off, int bytes, int mat) {
    uint2 r;
    r.x = (unsigned)(byte_off >> 4);
    r.y = (unsigned)(bytes >> 4) | ((unsigned)mat << 16);
    return r;
}
// Appends the entries of one phase for one CTA in the order the consumers walk them (chunk, matrix, entry).
inline void sched_append_phase(std::vector<uint2>& out, const LoopPhase& ph, int cta, const int (&mat_ids)[3]) {
    const int nch = phase_chunks(ph, cta);
    for (int ch = 0; ch < nch; ch++)
        for (int j = 0; j < 3; j++) {
            const JobSpan v = job_span(ph.job[j], ph.nb, cta, ch, ph.rpc);
            const int type = ph.job[j].type, tpe = type_tpe(type), TB = type_tile_bytes(type);
            const int ne = span_entries(v, type), nt = span_tiles(v);
            for (int e = 0; e < ne; e++) {
                const int tiles = nt - e * tpe < tpe ? nt - e * tpe : tpe;
                out.push_back(sched_entry((long long)(span_t0(v) + e * tpe) * TB, tiles * TB, mat_ids[j]));
            }
        }
}

// One chunk of a phase for one CTA, as the consumers need it (16 ints).
struct ChunkDesc {
    int task_first, n_tasks, n_entries, pad;
    int f0[3], f1[3];   // flat block spans of the phase's matrices
    int rows[3], id0[3];  // rows of every matrix in the chunk and the epilogue id of its first item
};
// One warp task (4 ints): a tile part of 32 / lp blocks.
//   x: flat index of the part's first block      y: partial-sum index of block f is f + y
//   z: entry inside the chunk (10 bits) | tile offset in the slot / 16 (10) | matrix (2) | kind (2: 0 Q4_K, 1 Q6_K,
//      2 Q6_K fp32 route) | log2 lanes per block (2) | arrival weight (6)
//   w: x mod blocks-per-row
__host__ __device__ __forceinline__ uint4 task_desc(int f_first, int part_rel, int ent, int toff, int job, int kind, int lsh, int weight,
                                                    int b_first) {
    uint4 r;
    r.x = (unsigned)f_first;
    r.y = (unsigned)part_rel;
    r.z = (unsigned)ent | ((unsigned)(toff >> 4) << 10) | ((unsigned)job << 20) | ((unsigned)kind << 22) | ((unsigned)lsh << 24) |
          ((unsigned)weight << 26);
    r.w = (unsigned)b_first;
    return r;
}

struct LoopPlanHost {
    std::vector<int> blob;          // [G][blob_stride]
    std::vector<uint4> head_tasks;  // [G][head_stride]
    int blob_stride = 0, chunks_off = 28, tasks_off = 0, sched_off = 0, head_stride = 0;
};

// Builds every CTA's plan.  ph[sec] for the seven sections; used[sec] = false leaves a section empty (a matrix type no
// layer has).  consumer_warps only shapes nothing here: the task order is warp-count independent.
inline bool loop_build_plan(const LoopPhase (&ph)[SCHED_SECTIONS], const bool (&used)[SCHED_SECTIONS], int G, int pbuf_floats,
                            LoopPlanHost& out) {
    struct PerCta {
        std::vector<uint2> sched;
        std::vector<ChunkDesc> chunks;
        std::vector<uint4> tasks, head;
        int sec[2 * SCHED_SECTIONS], cdir[2 * SCHED_SECTIONS];
    };
    static const int mat_ids[SCHED_SECTIONS][3] = {{0, 1, 2}, {3, 3, 3}, {3, 3, 3}, {4, 5, 5}, {6, 6, 6}, {6, 6, 6}, {7, 7, 7}};
    std::vector<PerCta> all(G);
    int max_chunks = 0, max_tasks = 0, max_sched = 0, max_head = 0;
    for (int cta = 0; cta < G; cta++) {
        PerCta& pc = all[cta];
        for (int sec = 0; sec < SCHED_SECTIONS; sec++) {
            pc.sec[2 * sec] = (int)pc.sched.size();
            pc.cdir[2 * sec] = (int)pc.chunks.size();
            if (used[sec]) {
                const LoopPhase& P = ph[sec];
                sched_append_phase(pc.sched, P, cta, mat_ids[sec]);
                std::vector<uint4>& tl_out = sec == SCHED_SECTIONS - 1 ? pc.head : pc.tasks;
                const int nch = phase_chunks(P, cta);
                for (int ch = 0; ch < nch; ch++) {
                    ChunkDesc cd{};
                    cd.task_first = (int)tl_out.size();
                    int off = 0, ebase = 0;
                    for (int j = 0; j < 3; j++) {
                        const LoopJob& jb = P.job[j];
                        const JobSpan v = job_span(jb, P.nb, cta, ch, P.rpc);
                        cd.f0[j] = v.f0, cd.f1[j] = v.f1;
                        cd.rows[j] = (v.f1 - v.f0) / P.nb;
                        const int r0 = v.f0 / P.nb;
                        cd.id0[j] = jb.id_base + (P.zip ? r0 : (r0 >> 1));
                        if (v.f1 > v.f0) {
                            const int lp = jb.f32 ? 4 : P.lpb, lsh = lp == 4 ? 2 : (lp == 2 ? 1 : 0), per = 32 >> lsh;
                            const int tpe = type_tpe(jb.type), TB = type_tile_bytes(jb.type), nt = span_tiles(v);
                            const int kind = jb.f32 ? 2 : (jb.type == TFR_Q4_K ? 0 : 1);
                            for (int tl = 0; tl < nt; tl++) {
                                const int el = tl / tpe, ti = tl - el * tpe;
                                const int tiles_here = nt - el * tpe < tpe ? nt - el * tpe : tpe;
                                for (int sub = 0; sub < lp; sub++) {
                                    const int f_first = (span_t0(v) + tl) * 32 + sub * per;
                                    if (ebase + el >= 1024 || LOOP_EMPTY % (tiles_here * lp)) return false;
                                    tl_out.push_back(task_desc(f_first, off - v.f0, ebase + el, ti * TB, j, kind, lsh, LOOP_EMPTY / (tiles_here * lp),
                                                               f_first % P.nb));
                                }
                            }
                            ebase += span_entries(v, jb.type);
                        }
                        off += v.f1 - v.f0;
                    }
                    if (off > pbuf_floats) return false;
                    cd.n_tasks = (int)tl_out.size() - cd.task_first;
                    cd.n_entries = ebase;
                    pc.chunks.push_back(cd);
                }
            }
            pc.sec[2 * sec + 1] = (int)pc.sched.size() - pc.sec[2 * sec];
            pc.cdir[2 * sec + 1] = (int)pc.chunks.size() - pc.cdir[2 * sec];
        }
        max_chunks = std::max(max_chunks, (int)pc.chunks.size());
        max_tasks = std::max(max_tasks, (int)pc.tasks.size());
        max_sched = std::max(max_sched, (int)pc.sched.size());
        max_head = std::max(max_head, (int)pc.head.size());
    }
    out.chunks_off = 28;
    out.tasks_off = out.chunks_off + 16 * max_chunks;
    out.sched_off = out.tasks_off + 4 * max_tasks;
    out.blob_stride = (out.sched_off + 2 * max_sched + 3) & ~3;
    out.head_stride = max_head > 0 ? max_head : 1;
    out.blob.assign((size_t)G * out.blob_stride, 0);
    out.head_tasks.assign((size_t)G * out.head_stride, make_uint4(0u, 0u, 0u, 0u));
    for (int cta = 0; cta < G; cta++) {
        const PerCta& pc = all[cta];
        int* b = out.blob.data() + (size_t)cta * out.blob_stride;
        memcpy(b, pc.sec, sizeof pc.sec);
        memcpy(b + 14, pc.cdir, sizeof pc.cdir);
        if (!pc.chunks.empty()) memcpy(b + out.chunks_off, pc.chunks.data(), pc.chunks.size() * sizeof(ChunkDesc));
        if (!pc.tasks.empty()) memcpy(b + out.tasks_off, pc.tasks.data(), pc.tasks.size() * sizeof(uint4));
        if (!pc.sched.empty()) memcpy(b + out.sched_off, pc.sched.data(), pc.sched.size() * sizeof(uint2));
        if (!pc.head.empty()) memcpy(out.head_tasks.data() + (size_t)cta * out.head_stride, pc.head.data(), pc.head.size() * sizeof(uint4));
    }
    return true;
}

// The schedule section of a stage of layer `L`.  stage: 0 Q/K/V, 1 o-proj, 2 gate/up, 3 down, 4 head.
__host__ __device__ __forceinline__ int sched_section(int stage, const LoopLayer* L) {
    return stage == 0 ? 0 : (stage == 1 ? 1 + L->o_q6 : (stage == 2 ? 3 : (stage == 3 ? 4 + L->down_q6 : 6)));
}

// ONE lane issues the CTA's schedule entries in order: entry e goes to ring slot e mod nslot.  Per entry the lane reads
// one 8-byte descriptor from the table in shared memory, waits (parked by the hardware, bounded) for the slot's
// previous use to be released, and starts the bulk copy: a few dozen instructions, so the issue rate is far above what
// the memory system delivers.  (A lane per slot, each walking the schedule on its own, ran the walk once per entry under
// divergence and capped the stream at about a third of the memory bandwidth.)  Slots are released roughly in order,
// so waiting on them in order costs nothing.
__device__ __noinline__ void loop_streamer(LoopCtx& c, const LoopArgs& a, int n_steps) {
    if (llane() != 0) return;
    const LoopLayer* lay = c.lay;
    const int* sec = c.blob;
    const uint2* tab = reinterpret_cast<const uint2*>(c.blob + a.blob_sched);
    const int nslot = c.nslot;
    int slot = 0, lap = 0;
    bool failed = false;
#pragma unroll 1
    for (int it = 0; it < n_steps && !failed; it++) {
        const int n_stage = it < a.n_headless ? 4 * a.n_layer : 4 * a.n_layer + 1;  // prompt-feeding steps have no head
#pragma unroll 1
        for (int st = 0; st < n_stage && !failed; st++) {
            const int li = st >> 2, stage = li < a.n_layer ? (st & 3) : 4;
            const LoopLayer* L = lay + (stage == 4 ? 0 : li);
            const int sct = sched_section(stage, L);
            const uint2* en_p = tab + sec[2 * sct];
            const int len = sec[2 * sct + 1];
#pragma unroll 1
            for (int idx = 0; idx < len; idx++) {
                const uint2 en = en_p[idx];
                if (lap > 0) {
                    const unsigned par = (unsigned)((lap - 1) & 1);
                    if (!mbar_try_wait_hint(c.empty + slot, par, 1000u)) {
                        const long long t0 = clock64();
                        for (;;) {
                            if (mbar_try_wait_hint(c.empty + slot, par, 1000u)) break;
                            if (c.ctl[CTL_STOP]) {
                                failed = true;
                                break;
                            }
                            if (clock64() - t0 > LOOP_SPIN_CYCLES) {
                                loop_fail(c, a, 2);
                                failed = true;
                                break;
                            }
                        }
                        if (failed) break;
                    }
                }
                const unsigned bytes = (en.y & 0xffffu) << 4;
                const int mat = (int)(en.y >> 16);
                const uint8_t* base = mat == 7 ? a.head : reinterpret_cast<const uint8_t* const*>(L)[mat];
                fence_proxy_async();
                mbar_expect_tx(c.full + slot, bytes);
                bulk_load(c.ring + (size_t)slot * LOOP_SLOT, base + ((size_t)en.x << 4), bytes, c.full + slot);
                __threadfence_block();
                c.issued[slot] = lap + 1;
                if (++slot == nslot) {
                    slot = 0;
                    lap++;
                }
            }
        }
    }
    // every copy this lane issued and nobody consumed must have landed before the CTA's shared memory is released:
    // the last use of every slot
#pragma unroll 1
    for (int s = 0; s < nslot; s++) {
        const int last = s < slot ? lap : lap - 1;  // use count - 1 of slot s
        if (last < 0) continue;
        const long long t0 = clock64();
        while (!mbar_test_wait(c.full + s, (unsigned)(last & 1))) {
            if (clock64() - t0 > LOOP_SPIN_CYCLES) {
                a.st->err = 2;
                break;
            }
        }
    }
}

// ------------------------------------------------------------------ consumer side: waits

// Blocks until use `lap` of ring slot `s` has landed.  The issue counter is checked first: a parity wait
// alone could be satisfied by the slot's previous use.
__device__ __noinline__ void wait_entry(LoopCtx& c, const LoopArgs& a, int s, int lap) {
    if (c.ctl[CTL_ABORT]) return;
    if (c.issued[s] <= lap) {
        const long long t0 = clock64();
        while (c.issued[s] <= lap) {
            __nanosleep(200);  // leave the issue slots to the streamer and to warps that have data
            if (c.ctl[CTL_ABORT]) return;
            if (clock64() - t0 > LOOP_SPIN_CYCLES) {
                loop_fail(c, a, 2);
                return;
            }
        }
    }
    const unsigned par = (unsigned)(lap & 1);
    if (mbar_try_wait_hint(c.full + s, par, 2000u)) return;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait_hint(c.full + s, par, 2000u)) return;
        if (c.ctl[CTL_ABORT]) return;
        if (clock64() - t0 > LOOP_SPIN_CYCLES) {
            loop_fail(c, a, 2);
            return;
        }
    }
}

// Grid-wide barrier of the consumer threads of all CTAs.  Arrivals are spread over eight counters in
// different cache lines; eight lanes of warp 0 poll one counter each.  fetch != nullptr: the 64-bit
// word is read after the barrier and handed to every thread through shared memory.  The abort flag can be
// raised at any moment (by the streamer too); warp 0 takes one snapshot of it per barrier, and only that
// snapshot (loop_aborted) steers control flow, so all consumer warps of a CTA always agree.
__device__ __noinline__ unsigned long long grid_barrier(LoopCtx& c, const LoopArgs& a, const unsigned long long* fetch = nullptr) {
    cbar();
    if (lwarp() == 0) {
        if (llane() == 0) {
            c.bar_k++;
            __threadfence();
            red_add_u32(a.bar + (c.cta & 7) * LOOP_BAR_STRIDE, 1u);
        }
        __syncwarp();
        const int aborted = __shfl_sync(TFR_FULL_MASK, (int)c.ctl[CTL_ABORT], 0);  // one reading for the whole warp
        if (!aborted) {
            const int members = llane() < 8 ? (c.G - llane() + 7) >> 3 : 0;
            const unsigned target = c.bar_k * (unsigned)members;
            const unsigned* ctr = a.bar + (llane() & 7) * LOOP_BAR_STRIDE;
            const long long t0 = clock64();
            for (int spin = 0;; spin++) {
                bool ok = true;
                if (llane() < 8) ok = (int)(ld_acquire_u32(ctr) - target) >= 0;
                if (__all_sync(TFR_FULL_MASK, ok)) break;
                if ((spin & 63) == 63 && clock64() - t0 > LOOP_SPIN_CYCLES) {
                    if (llane() == 0) loop_fail(c, a, 4);
                    break;
                }
            }
        }
        if (llane() == 0) {
            if (fetch) *c.ctl_best = __ldcg(fetch);
            if (c.ctl[CTL_ABORT]) c.ctl[CTL_SNAP] = 1;
        }
    }
    cbar();
    return fetch ? *c.ctl_best : 0ull;
}
__device__ __forceinline__ bool loop_aborted(const LoopCtx& c) { return c.ctl[CTL_SNAP] != 0; }

// ------------------------------------------------------------------ partial block dots (a quarter block per lane)

// Sub-block pair `t` (64 weights) of one Q4_K block (block_dot(BlockQ4) restricted to a quarter).
__device__ __forceinline__ float q4_quarter(const uint8_t* tile, int bl, int t, const Act& act, int b, int nb) {
    const int4 wh = tile_piece<true>(tile, bl, 0);
    const unsigned s0 = (unsigned)wh.y, s1 = (unsigned)wh.z, s2 = (unsigned)wh.w;
    const unsigned sc_lo = s0 & 0x3f3f3f3fu, sc_hi = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
    const unsigned m_lo = s1 & 0x3f3f3f3fu, m_hi = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
    const int4* aq = act.q8 + b;
    const int4 a0 = aq[(4 * t) * nb], a1 = aq[(4 * t + 1) * nb], a2 = aq[(4 * t + 2) * nb], a3 = aq[(4 * t + 3) * nb];
    const int4 qa = tile_piece<true>(tile, bl, 1 + 2 * t), qb = tile_piece<true>(tile, bl, 2 + 2 * t);
    int I0 = dot16_us(qa, 0x0f0f0f0fu, a0, 0);
    I0 = dot16_us(qb, 0x0f0f0f0fu, a1, I0);
    int I1 = dot16_us(qa, 0xf0f0f0f0u, a2, 0);
    I1 = dot16_us(qb, 0xf0f0f0f0u, a3, I1);
    I1 >>= 4;
    const int sc0 = (int)(__byte_perm(sc_lo, sc_hi, 2 * t) & 0xffu), sc1 = (int)(__byte_perm(sc_lo, sc_hi, 2 * t + 1) & 0xffu);
    const int m0 = (int)(__byte_perm(m_lo, m_hi, 2 * t) & 0xffu), m1 = (int)(__byte_perm(m_lo, m_hi, 2 * t + 1) & 0xffu);
    const float2 d8 = *reinterpret_cast<const float2*>(act.d8 + 8 * b + 2 * t);
    const float2 ds = *reinterpret_cast<const float2*>(act.ds + 8 * b + 2 * t);
    const float acc = d8.x * i2f_small(I0 * sc0) + d8.y * i2f_small(I1 * sc1);
    const float accm = ds.x * i2f_small(m0) + ds.y * i2f_small(m1);
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&wh.x));
    return dd.x * acc - dd.y * accm;
}

// Group quadruple u = 2n + is of one Q6_K block (block_dot(BlockQ6) restricted to a quarter).
__device__ __forceinline__ float q6_quarter(const uint8_t* tile, int bl, int u, const Act& act, int b, int nb) {
    const int4* aq = act.q8 + b;
    const int n = u >> 1, is = u & 1;
    const int4 la = tile_piece<true>(tile, bl, 4 * n + is), lb = tile_piece<true>(tile, bl, 4 * n + 2 + is),
               h = tile_piece<true>(tile, bl, 8 + 2 * n + is);
    const int4 a0 = aq[(8 * n + is) * nb], a1 = aq[(8 * n + 2 + is) * nb], a2 = aq[(8 * n + 4 + is) * nb], a3 = aq[(8 * n + 6 + is) * nb];
    const int* sn = act.s16n + 16 * b + 8 * n + is;
    int J0 = sn[0], J1 = sn[2], J2 = sn[4], J3 = sn[6];
#define TFR_Q6W(c)                                                                                         \
    J0 = __dp4a((int)((la.c & 0x0f0f0f0f) | ((h.c << 4) & 0x30303030)), a0.c, J0);                        \
    J1 = __dp4a((int)((lb.c & 0x0f0f0f0f) | ((h.c << 2) & 0x30303030)), a1.c, J1);                        \
    J2 = __dp4a((int)((((unsigned)la.c >> 4) & 0x0f0f0f0f) | (h.c & 0x30303030)), a2.c, J2);              \
    J3 = __dp4a((int)((((unsigned)lb.c >> 4) & 0x0f0f0f0f) | (((unsigned)h.c >> 2) & 0x30303030)), a3.c, J3);
    TFR_Q6W(x) TFR_Q6W(y) TFR_Q6W(z) TFR_Q6W(w)
#undef TFR_Q6W
    // scale bytes 8n + is + {0, 2, 4, 6} of the block's sixteen
    const unsigned long long w = *reinterpret_cast<const unsigned long long*>(tile + 12 * 512 + bl * 16 + 8 * n) >> (8 * is);
    const float c0 = i2f_small((int)(signed char)(w & 0xff)), c1 = i2f_small((int)(signed char)((w >> 16) & 0xff));
    const float c2 = i2f_small((int)(signed char)((w >> 32) & 0xff)), c3 = i2f_small((int)(signed char)((w >> 48) & 0xff));
    const float4 d8 = *reinterpret_cast<const float4*>(act.d8 + 8 * b + 4 * n);
    const float acc = c0 * d8.x * i2f_small(J0) + c1 * d8.y * i2f_small(J1) + c2 * d8.z * i2f_small(J2) + c3 * d8.w * i2f_small(J3);
    const unsigned short dbits = reinterpret_cast<const unsigned short*>(tile + Q6_PIECES * 512)[bl];
    return f16_to_f32(dbits) * acc;
}

// Runs c in [4 * qq, 4 * qq + 4) (16 weights each) of one Q6_K block of a tile in shared memory against the fp32
// activation: the reference's route for a Q6_K attn_v, kernels/gemv.cu:233-264 (acc += d * scale * q * x).
__device__ __forceinline__ float q6_f32_quarter(const uint8_t* tile, int bl, int qq, const float* xf, int b) {
    const float d = f16_to_f32(reinterpret_cast<const unsigned short*>(tile + Q6_PIECES * 512)[bl]);
    float tot = 0.f;
#pragma unroll 1
    for (int cc = 0; cc < 4; cc++) {
        const int cidx = 4 * qq + cc, n = cidx >> 3, j = (cidx >> 1) & 3, is = cidx & 1;
        const int4 ql = tile_piece<true>(tile, bl, 4 * n + 2 * (j & 1) + is);
        const int4 qh = tile_piece<true>(tile, bl, 8 + 2 * n + is);
        const float sc = (float)(int)*reinterpret_cast<const signed char*>(tile + 12 * 512 + bl * 16 + 8 * n + is + 2 * j);
        const float dsc = d * sc;
        const float4* x4 = reinterpret_cast<const float4*>(xf + xs_idx(256 * b + 16 * cidx));
        const int qlw[4] = {ql.x, ql.y, ql.z, ql.w};
        const int qhw[4] = {qh.x, qh.y, qh.z, qh.w};
        const int nsh = 4 * (j >> 1), hsh = 2 * j;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float4 x = x4[k];
            const float xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int by = 0; by < 4; by++) {
                const int nib = (qlw[k] >> (8 * by + nsh)) & 0xF;
                const int hb = (qhw[k] >> (8 * by + hsh)) & 3;
                acc += dsc * (float)((nib | (hb << 4)) - 32) * xv[by];
            }
        }
        tot += acc;
    }
    return tot;
}

// ------------------------------------------------------------------ consumer side: activations

// Decodes the embedding row of `token` (kernels/embed.cu:71-131) into the staging vector c.xf and keeps the CTA's own
// rows of it.  Runs once per decode step.
__device__ __noinline__ void embed_stage(LoopCtx& c, const LoopArgs& a, int token, int n_own) {
    int tok = token;
    if (tok < 0 || tok >= a.embed.N) {
        if (ltid() == 0) a.st->err = 1;
        tok = 0;
    }
    const SrcEmbed src{a.embed, tok};
#pragma unroll 1
    for (int i = ltid(); i < a.K; i += LOOP_CT) c.xf[xs_idx(i)] = src.get(i);
    cbar();
    if (ltid() < n_own) c.own[ltid()] = c.xf[xs_idx(c.own_row0 + ltid())];
}

// One call of the Q8 quantiser (act_quantize4), out of line: every activation stage shares this copy.
__device__ __noinline__ void loop_quant4(unsigned char* work, int K, float4 x, int i4, bool on) {
    const Act act = act_carve(work, K, false, false);
    act_quantize4(act, x, i4, on, K >> 8);
}

// Elements 4 * i4 .. + 3 of the attention output merged from S <= LOOP_INLINE_MAX split-KV partials
// (kernels/attn/flash.cu:236-254: m = max m_s, alpha_s = exp(m_s - m), out = sum alpha_s O_s / max(sum alpha_s l_s, 1e-20)).
__device__ __noinline__ float4 loop_merged4(const LoopArgs& a, int i4, int S) {
    const int e = 4 * i4, h = e >> a.hd_shift, d = e - (h << a.hd_shift), po = 4 + a.hd;
    const float* hb = a.pc + (size_t)h * a.attn_smax * po;
    float2 ml[LOOP_INLINE_MAX];
    float4 o[LOOP_INLINE_MAX];
#pragma unroll
    for (int k = 0; k < LOOP_INLINE_MAX; k++) {
        ml[k] = make_float2(-1e30f, 0.f);
        o[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < S) {
            ml[k] = __ldcg(reinterpret_cast<const float2*>(hb + (size_t)k * po));
            o[k] = ldcg4(hb + (size_t)k * po + 4 + d);
        }
    }
    float m = -1e30f;
#pragma unroll
    for (int k = 0; k < LOOP_INLINE_MAX; k++) m = fmaxf(m, ml[k].x);
    float l = 0.f;
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < LOOP_INLINE_MAX; k++)
        if (k < S) {
            const float al = expf(ml[k].x - m);
            l += al * ml[k].y;
            r.x += al * o[k].x;
            r.y += al * o[k].y;
            r.z += al * o[k].z;
            r.w += al * o[k].w;
        }
    const float inv = 1.f / fmaxf(l, 1e-20f);
    return make_float4(r.x * inv, r.y * inv, r.z * inv, r.w * inv);
}

// The phase's input vector -> Q8 activation in shared memory.
//   normw != nullptr: RMSNorm first.  The raw vector comes from `src`, or is already staged in c.xf (src == nullptr:
//     the embedding row).  The sum of squares keeps the reduction shape of kernels/ops.cu:4-34 (256 strided partial
//     sums in index order, then the binary tree red[t] += red[t + s], s = 128 .. 1, replayed by one warp) so the scale,
//     and with it every int8, is bit-identical to the reference build's for the same input.  The normalised vector
//     replaces the raw one in c.xf (fp32-route rows read it).
//   normw == nullptr: the vector is quantised as it is; merge_S > 1: it is the merge of that many attention partials.
__device__ __noinline__ void loop_act(LoopCtx& c, const LoopArgs& a, const float* src, int K, const float* normw, int merge_S) {
    const int n4 = K >> 2, tid = ltid();
    if (normw) {
        float* xs = c.xf;
        float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tid < n4) w0 = __ldg(reinterpret_cast<const float4*>(normw) + tid);
        if (src) {
#pragma unroll 2
            for (int i4 = tid; i4 < n4; i4 += LOOP_CT) *reinterpret_cast<float4*>(xs + xs_idx(4 * i4)) = ldcg4(src + 4 * i4);
        }
        cbar();
        if (tid < 256) {
            float local = 0.f;
#pragma unroll 2
            for (int i = tid; i < K; i += 256) {
                const float v = xs[xs_idx(i)];
                local += v * v;
            }
            c.red[tid] = local;
            asm volatile("bar.sync 2, 256;" ::: "memory");
            if (tid < 32) {
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; k++) v[k] = c.red[tid + 32 * k];
#pragma unroll
                for (int k = 0; k < 4; k++) v[k] += v[k + 4];
                v[0] += v[2];
                v[1] += v[3];
                v[0] += v[1];
                float t = v[0];
#pragma unroll
                for (int sft = 16; sft > 0; sft >>= 1) t += __shfl_down_sync(TFR_FULL_MASK, t, sft);
                if (tid == 0) c.red[256] = rsqrtf(t / (float)K + a.eps);
            }
        }
        cbar();
        const float scale = c.red[256];
#pragma unroll 1
        for (int k0 = 0; k0 < n4; k0 += LOOP_CT) {
            const int i4 = k0 + tid;
            const bool on = i4 < n4;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on) {
                x = *reinterpret_cast<const float4*>(xs + xs_idx(4 * i4));
                const float4 w = k0 == 0 ? w0 : __ldg(reinterpret_cast<const float4*>(normw) + i4);
                x.x = x.x * scale * w.x;
                x.y = x.y * scale * w.y;
                x.z = x.z * scale * w.z;
                x.w = x.w * scale * w.w;
                *reinterpret_cast<float4*>(xs + xs_idx(4 * i4)) = x;
            }
            if (k0 + (tid & ~31) < n4) loop_quant4(c.work, K, x, i4, on);  // whole warps past the end have nothing to do
        }
    } else {
        constexpr int R = 4;  // loads in flight per thread
#pragma unroll 1
        for (int base = 0; base < n4; base += R * LOOP_CT) {
            float4 xv[R];
#pragma unroll
            for (int k = 0; k < R; k++) {
                const int i4 = base + k * LOOP_CT + tid;
                xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i4 < n4) xv[k] = merge_S > 1 ? loop_merged4(a, i4, merge_S) : ldcg4(src + 4 * i4);
            }
#pragma unroll
            for (int k = 0; k < R; k++) {
                const int i4 = base + k * LOOP_CT + tid;
                if (base + k * LOOP_CT + (tid & ~31) < n4) loop_quant4(c.work, K, xv[k], i4, i4 < n4);
            }
        }
    }
    cbar();
}

// ------------------------------------------------------------------ consumer side: row sums + epilogues

// Epilogue of one item (a row pair, or a gate/up row).  Returns the item's packed argmax key (logits) or 0.
//   LEPI_QKV: bias, neox RoPE (kernels/ops.cu:348-371), f16 KV store (kernels/ops.cu:471-486).  Pair p holds the RoPE
//     partners (i, i + hd/2) of a head (rows were re-ordered at upload); biases are stored in the same pair order.
//   LEPI_RESIDUAL: x += W act (kernels/gemv.cu:367-373, use_res = 2).  The CTA owns the same rows of the residual
//     stream in every phase that writes it, so the running value stays in shared memory (c.own).
//   LEPI_SILU: h = silu(gate . x) * (up . x), kernels/gemv.cu:2570-2574.
//   LEPI_LOGITS: logits + running argmax (kernels/ops.cu:573-599; ties resolve to the lowest index).
__device__ __noinline__ unsigned long long loop_epi(LoopCtx& c, const LoopArgs& a, int kind, int p, float x0, float x1) {
    if (kind == LEPI_SILU) {
        a.h[p] = (x0 / (1.f + __expf(-x0))) * x1;
        return 0ull;
    }
    if (kind == LEPI_RESIDUAL) {
        const int row = 2 * p, o = row - c.own_row0;
        float* tap = c.tap;
        const float v0 = x0 + c.own[o];
        c.own[o] = v0;
        a.x[row] = v0;
        if (tap) tap[row] = v0;
        if (row + 1 < a.K) {
            const float v1 = x1 + c.own[o + 1];
            c.own[o + 1] = v1;
            a.x[row + 1] = v1;
            if (tap) tap[row + 1] = v1;
        }
        return 0ull;
    }
    if (kind == LEPI_LOGITS) {
        const int row = 2 * p;
        a.logits[row] = x0;
        unsigned long long best = argmax_key(x0, row);
        if (row + 1 < a.V) {
            a.logits[row + 1] = x1;
            const unsigned long long k = argmax_key(x1, row + 1);
            best = k > best ? k : best;
        }
        return best;
    }
    const int v = 2 * p, nq = a.nq, nk = a.nkv, hd = a.hd, pos = c.pos;
    if (c.bias) {
        const float2 b = __ldg(reinterpret_cast<const float2*>(c.bias) + p);
        x0 += b.x;
        x1 += b.y;
    }
    unsigned short* dst;  // where the pair goes in the cache (k and v rows); q goes out as fp32
    int second = 1;       // distance of the pair's second element
    if (v < nq + nk) {
        const bool is_q = v < nq;
        const int vv = is_q ? v : v - nq;
        const int head = vv >> a.hd_shift, i = (vv & (hd - 1)) >> 1, half = hd >> 1;
        const float freq = powf(a.theta, -2.f * (float)i / (float)hd);
        const float ang = (float)pos * freq;
        const float cs = cosf(ang), sn = sinf(ang);
        const float y0 = x0 * cs - x1 * sn;
        const float y1 = x0 * sn + x1 * cs;
        if (is_q) {
            a.q[head * hd + i] = y0;
            a.q[head * hd + i + half] = y1;
            return 0ull;
        }
        x0 = y0;
        x1 = y1;
        dst = c.kc + (size_t)pos * nk + head * hd + i;
        second = half;
    } else {
        dst = c.vc + (size_t)pos * nk + (v - nq - nk);
    }
#pragma unroll 1
    for (int k = 0; k < 2; k++) dst[k * second] = f32_to_f16_bits_ref(k ? x1 : x0);
    return 0ull;
}

// Sums the block partials of `n_rows` rows (nb each) in a fixed order and hands every item to the epilogue.
// zip: item i = (row i of pa, row i of pb); otherwise item i = rows (2i, 2i + 1) of pa.  Rows of up to eight blocks
// are summed by groups of eight lanes (four items per warp pass), longer rows by a whole warp.
__device__ __noinline__ unsigned long long loop_reduce(LoopCtx& c, const LoopArgs& a, int kind, const float* pa, const float* pb, int n_rows,
                                                       int nb, int id0, int zip) {
    const int lane = llane(), warp = lwarp();
    const int lpr = nb <= 8 ? 8 : 32, ipw = 32 / lpr;
    const int k = lane & (lpr - 1), g = lane / lpr;
    const int items = zip ? n_rows : (n_rows + 1) >> 1;
    unsigned long long best = 0ull;
#pragma unroll 1
    for (int base = warp * ipw; base < items; base += LOOP_CWARPS * ipw) {
        const int it = base + g;
        const bool on = it < items;
        const float* ra = zip ? pa + it * nb : pa + (2 * it) * nb;
        const float* rb = zip ? pb + it * nb : ra + nb;
        const bool has_b = on && (zip || 2 * it + 1 < n_rows);
        float x = 0.f, y = 0.f;
#pragma unroll 1
        for (int i = k; i < nb; i += lpr) {
            if (on) x += ra[i];
            if (has_b) y += rb[i];
        }
#pragma unroll 1
        for (int o = lpr >> 1; o > 0; o >>= 1) {
            x += __shfl_xor_sync(TFR_FULL_MASK, x, o);
            y += __shfl_xor_sync(TFR_FULL_MASK, y, o);
        }
        if (on && k == 0) {
            const unsigned long long key = loop_epi(c, a, kind, id0 + it, x, y);
            best = key > best ? key : best;
        }
    }
    return best;
}

// ------------------------------------------------------------------ consumer side: one matrix-vector phase

// The block dots of one chunk: every warp walks its tasks (one 16-byte descriptor each), waits for the task's tile,
// runs the quarter-block dots of the task's kind, stores the block partials and releases the ring slot.  ONE copy of
// this code serves every phase.
__device__ __noinline__ void loop_dots(LoopCtx& c, const LoopArgs& a, const ChunkDesc* cd, const uint4* tl, int nb) {
    const int lane = llane(), warp = lwarp();
    const Act act = act_carve(c.work, nb << 8, false, false);
    const int n_tasks = cd->n_tasks;
    uint4 td = make_uint4(0u, 0u, 0u, 0u);
    if (warp < n_tasks) td = tl[warp];
#pragma unroll 1
    for (int task = warp; task < n_tasks; task += LOOP_CWARPS) {
        const uint4 cur = td;
        if (task + LOOP_CWARPS < n_tasks) td = tl[task + LOOP_CWARPS];  // the next descriptor travels during the dots
        const int ent = (int)(cur.z & 1023u), toff = (int)((cur.z >> 10) & 1023u) << 4, job = (int)((cur.z >> 20) & 3u);
        const int kind = (int)((cur.z >> 22) & 3u), lsh = (int)((cur.z >> 24) & 3u);
        int s = c.slot + ent, lap = c.lap;
        while (s >= c.nslot) {
            s -= c.nslot;
            lap++;
        }
        wait_entry(c, a, s, lap);
        const uint8_t* tile = c.ring + (size_t)s * LOOP_SLOT + toff;
        // 1, 2 or 4 lanes share a block: 32 >> lsh adjacent blocks per task, 4 >> lsh quarters of a block per lane
        const int dl = lane & ((32 >> lsh) - 1);
        const int q0 = (lane >> (5 - lsh)) << (2 - lsh), q1 = q0 + (4 >> lsh);
        const int f = (int)cur.x + dl;
        const int bl = f & 31;  // block inside the tile
        const bool mine = f >= cd->f0[job] && f < cd->f1[job];
        float val = 0.f;
        if (mine) {
            int b = (int)cur.w + dl;
            b = b >= nb ? b - nb : b;
            b = b >= nb ? b % nb : b;
            if (kind == 0) {
#pragma unroll 1
                for (int t = q0; t < q1; t++) val += q4_quarter(tile, bl, t, act, b, nb);
            } else if (kind == 1) {
#pragma unroll 1
                for (int t = q0; t < q1; t++) val += q6_quarter(tile, bl, t, act, b, nb);
            } else {
#pragma unroll 1
                for (int t = q0; t < q1; t++) val += q6_f32_quarter(tile, bl, t, c.xf, b);
            }
        }
        if (lsh >= 1) val += __shfl_xor_sync(TFR_FULL_MASK, val, 16);
        if (lsh == 2) val += __shfl_xor_sync(TFR_FULL_MASK, val, 8);
        if (mine && q0 == 0) c.pbuf[f + (int)cur.y] = val;
        __syncwarp();
        if (lane == 0) mbar_arrive_n(c.empty + s, cur.z >> 26);
    }
}

// One matrix-vector phase: block dots of the section's tiles as they land in the ring, row sums in a fixed order,
// epilogue `kind`.  The Q8 activation (and the staged fp32 vector for fp32-route rows) must be in shared memory.  All
// geometry comes from the CTA's plan (ChunkDesc / task descriptors).  Returns the thread's best argmax key (logits).
__device__ __noinline__ unsigned long long loop_gemv(LoopCtx& c, const LoopArgs& a, int sec, int kind) {
    const int nb = a.sec_nb[sec], zip = a.sec_zip[sec];
    const int chunk_first = c.blob[14 + 2 * sec], n_chunks = c.blob[14 + 2 * sec + 1];
    const uint4* tasks = sec == SCHED_SECTIONS - 1 ? a.head_tasks + (size_t)c.cta * a.head_stride
                                                   : reinterpret_cast<const uint4*>(c.blob + a.blob_tasks);
    unsigned long long best = 0ull;
#pragma unroll 1
    for (int ch = 0; ch < n_chunks; ch++) {
        const ChunkDesc* cd = reinterpret_cast<const ChunkDesc*>(c.blob + a.blob_chunks) + chunk_first + ch;
        loop_dots(c, a, cd, tasks + cd->task_first, nb);
        cbar();
        if (ltid() == 0) cursor_advance(c.slot, c.lap, cd->n_entries, c.nslot);  // read again after the next barrier
        if (zip) {
            const unsigned long long k = loop_reduce(c, a, kind, c.pbuf, c.pbuf + (cd->f1[0] - cd->f0[0]), cd->rows[0], nb, cd->id0[0], 1);
            best = k > best ? k : best;
        } else {
            int off = 0;
#pragma unroll 1
            for (int j = 0; j < 3; j++) {
                if (cd->rows[j] > 0) {
                    const unsigned long long k = loop_reduce(c, a, kind, c.pbuf + off, c.pbuf + off, cd->rows[j], nb, cd->id0[j], 0);
                    best = k > best ? k : best;
                }
                off += cd->f1[j] - cd->f0[j];
            }
        }
        cbar();
    }
    return best;
}

// ------------------------------------------------------------------ consumer side: attention

// Shared-memory scratch of the attention phase (aliases the activation / partial-sum area).
template <int HD>
struct AttnSmem {
    static constexpr int KROW = HD + 8;  // halfs per staged K row: 16-byte reads of 32 different rows hit 32 different banks
    float q[LOOP_REP_MAX][HD];
    float sc[LOOP_TK][LOOP_REP_MAX];
    float m[LOOP_REP_MAX], l[LOOP_REP_MAX], alpha[LOOP_REP_MAX];
    __align__(16) unsigned short k[LOOP_TK][KROW];
    __align__(16) unsigned short v[LOOP_TK][HD];
};

// This CTA's share of the step's attention: CTA = (kv head g, split s); the T keys are cut into S equal runs.
__device__ __noinline__ void attn_plan(LoopCtx& c, const LoopArgs& a, int pos) {
    const int T = pos + 1;
    int S = (T + a.attn_min_keys - 1) / a.attn_min_keys;
    S = S < 1 ? 1 : (S > a.attn_smax ? a.attn_smax : S);
    const int g = c.cta % a.n_kv, s = c.cta / a.n_kv;
    const int chunk = (T + S - 1) / S;
    const int t0 = min(T, s * chunk);
    c.pos = pos;
    c.at_S = S;
    c.at_g = g;
    c.at_s = s;
    c.at_active = s < S;
    c.at_t0 = t0;
    c.at_t1 = s < S ? min(T, t0 + chunk) : t0;
}

// Split-KV flash-decode of one (KV head, split) for all query heads of the group (kernels/attn/flash.cu:29-116;
// the reference runs one CTA per query head and split).  One split: the normalised output goes to a.att; otherwise
// (m, l, O) to the partial array.
template <int HD>
__device__ __noinline__ void loop_attention(LoopCtx& c, const LoopArgs& a) {
    if (!c.at_active) return;  // uniform over the CTA
    AttnSmem<HD>& sm = *reinterpret_cast<AttnSmem<HD>*>(c.work);
    constexpr int CPR = HD / 8;  // 16-byte chunks per row
    const int tid = ltid(), lane = llane(), warp = lwarp();
    const int rep = a.rep, g = c.at_g, t0 = c.at_t0, t1 = c.at_t1, S = c.at_S;
    constexpr int PO = 4 + HD;
    if (t1 <= t0) {
        // a split without keys still owns a partial: the neutral element of the merge
#pragma unroll 1
        for (int idx = tid; idx < rep * PO; idx += LOOP_CT) {
            const int h = idx / PO, j = idx - h * PO;
            a.pc[((size_t)(g * rep + h) * a.attn_smax + c.at_s) * PO + j] = j == 0 ? -1e30f : 0.f;
        }
        return;
    }
    const unsigned short* kc = c.kc;
    const unsigned short* vc = c.vc;
    const int kvdim = a.nkv;
#pragma unroll 1
    for (int i4 = tid; i4 < rep * HD / 4; i4 += LOOP_CT) *reinterpret_cast<float4*>(&sm.q[0][0] + 4 * i4) = ldcg4(a.q + (size_t)g * rep * HD + 4 * i4);
    if (tid < LOOP_REP_MAX) {
        sm.m[tid] = -1e30f;
        sm.l[tid] = 0.f;
    }
    // value accumulators: thread owns (head, dim pair) items idx = tid, tid + LOOP_CT, ...
    constexpr int NI = (LOOP_REP_MAX * HD / 2 + LOOP_CT - 1) / LOOP_CT;
    float2 o[NI];
#pragma unroll
    for (int i = 0; i < NI; i++) o[i] = make_float2(0.f, 0.f);
    const int n_items = rep * HD / 2;

#pragma unroll 1
    for (int tt = t0; tt < t1; tt += LOOP_TK) {
        const int tn = min(LOOP_TK, t1 - tt);
#pragma unroll 1
        for (int idx = tid; idx < LOOP_TK * CPR; idx += LOOP_CT) {
            const int row = idx / CPR, ch = idx - row * CPR;
            const int t = tt + row < t1 ? tt + row : t1 - 1;
            const size_t off = (size_t)t * kvdim + g * HD + ch * 8;
            const int n_src = tt + row < t1 ? 16 : 0;
            cp_async16(&sm.k[row][ch * 8], kc + off, n_src);
            cp_async16(&sm.v[row][ch * 8], vc + off, n_src);
        }
        cp_async_wait_all();
        cbar();
        // scores: one warp task = 32 keys x one head, a lane walks all dims of its key
#pragma unroll 1
        for (int wt = warp; wt < (LOOP_TK / 32) * rep; wt += LOOP_CWARPS) {
            const int h = wt % rep, key = (wt / rep) * 32 + lane;
            float acc = 0.f;
#pragma unroll 2
            for (int d = 0; d < HD; d += 8) {
                const int4 kr = *reinterpret_cast<const int4*>(&sm.k[key][d]);
                const float4 qa = *reinterpret_cast<const float4*>(&sm.q[h][d]), qb = *reinterpret_cast<const float4*>(&sm.q[h][d + 4]);
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kr.x)), k1 = __half22float2(*reinterpret_cast<const __half2*>(&kr.y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kr.z)), k3 = __half22float2(*reinterpret_cast<const __half2*>(&kr.w));
                acc += qa.x * k0.x + qa.y * k0.y;
                acc += qa.z * k1.x + qa.w * k1.y;
                acc += qb.x * k2.x + qb.y * k2.y;
                acc += qb.z * k3.x + qb.w * k3.y;
            }
            sm.sc[key][h] = key < tn ? acc * a.attn_scale : -1e30f;
        }
        cbar();
        // online softmax bookkeeping: warp h owns head h (LOOP_TK = 64: two keys per lane)
        if (warp < rep) {
            const float s0 = sm.sc[lane][warp], s1 = sm.sc[lane + 32][warp];
            const float tile_m = warp_max(fmaxf(s0, s1));
            const float m_old = sm.m[warp];
            const float m_new = fmaxf(m_old, tile_m);
            const float p0 = lane < tn ? expf(s0 - m_new) : 0.f;
            const float p1 = lane + 32 < tn ? expf(s1 - m_new) : 0.f;
            const float tile_l = warp_sum(p0 + p1);
            sm.sc[lane][warp] = p0;
            sm.sc[lane + 32][warp] = p1;
            if (lane == 0) {
                const float alpha = expf(m_old - m_new);
                sm.alpha[warp] = alpha;
                sm.l[warp] = sm.l[warp] * alpha + tile_l;
                sm.m[warp] = m_new;
            }
        }
        cbar();
        // values
#pragma unroll
        for (int i = 0; i < NI; i++) {
            const int idx = tid + i * LOOP_CT;
            if (idx < n_items) {
                const int h = idx / (HD / 2), dp = idx - h * (HD / 2);
                const float al = sm.alpha[h];
                float2 acc = make_float2(o[i].x * al, o[i].y * al);
#pragma unroll 2
                for (int key = 0; key < tn; key++) {
                    const float pw = sm.sc[key][h];
                    const float2 vv = __half22float2(*reinterpret_cast<const __half2*>(&sm.v[key][2 * dp]));
                    acc.x += pw * vv.x;
                    acc.y += pw * vv.y;
                }
                o[i] = acc;
            }
        }
        cbar();
    }
#pragma unroll
    for (int i = 0; i < NI; i++) {
        const int idx = tid + i * LOOP_CT;
        if (idx < n_items) {
            const int h = idx / (HD / 2), dp = idx - h * (HD / 2);
            const int hg = g * rep + h;
            if (S == 1) {
                const float inv = 1.f / fmaxf(sm.l[h], 1e-20f);
                *reinterpret_cast<float2*>(a.att + (size_t)hg * HD + 2 * dp) = make_float2(o[i].x * inv, o[i].y * inv);
            } else {
                float* base = a.pc + ((size_t)hg * a.attn_smax + c.at_s) * PO;
                *reinterpret_cast<float2*>(base + 4 + 2 * dp) = o[i];
                if (dp == 0) *reinterpret_cast<float2*>(base) = make_float2(sm.m[h], sm.l[h]);
            }
        }
    }
}

// Merge phase for many splits: CTA h < n_head merges query head h (kernels/attn/flash.cu:236-254) from the
// partials into a.att.
template <int HD>
__device__ __noinline__ void loop_attention_merge(LoopCtx& c, const LoopArgs& a, int S) {
    if (c.cta >= a.n_head) return;
    const int h = c.cta, tid = ltid();
    constexpr int PO = 4 + HD;
    const int Sp = (S + 3) & ~3;
    float* w_s = reinterpret_cast<float*>(c.work);  // [Sp] maxima, then weights
    float* l_s = w_s + Sp;                          // [Sp] sums
    float* sums = l_s + Sp;                         // [PARTS][HD]
    const float* hb = a.pc + (size_t)h * a.attn_smax * PO;
    constexpr int PARTS = LOOP_CT / HD < 1 ? 1 : LOOP_CT / HD;
#pragma unroll 1
    for (int s = tid; s < S; s += LOOP_CT) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(hb + (size_t)s * PO));
        w_s[s] = ml.x;
        l_s[s] = ml.y;
    }
    cbar();
    float m = -1e30f;
#pragma unroll 1
    for (int s = 0; s < S; s++) m = fmaxf(m, w_s[s]);
    cbar();
#pragma unroll 1
    for (int s = tid; s < S; s += LOOP_CT) w_s[s] = expf(w_s[s] - m);
    cbar();
    float l = 0.f;
#pragma unroll 1
    for (int s = 0; s < S; s++) l += w_s[s] * l_s[s];
    const int d = tid % HD, part = tid / HD;
    if (part < PARTS) {
        float acc = 0.f;
#pragma unroll 4
        for (int s = part; s < S; s += PARTS) acc += w_s[s] * __ldcg(hb + (size_t)s * PO + 4 + d);
        sums[part * HD + d] = acc;
    }
    cbar();
    if (tid < HD) {
        float acc = 0.f;
#pragma unroll 1
        for (int pp = 0; pp < PARTS; pp++) acc += sums[pp * HD + tid];
        a.att[(size_t)h * HD + tid] = acc / fmaxf(l, 1e-20f);
    }
}

// ------------------------------------------------------------------ the kernel

template <int HD>
__global__ void __launch_bounds__(LOOP_THREADS, 1) k_decode_loop(const __grid_constant__ LoopArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    LoopCtx& c = *reinterpret_cast<LoopCtx*>(smem + LOOP_CTX_OFFSET);
    if (ltid() == 0) {
        c.cta = blockIdx.x;
        c.G = gridDim.x;
        c.nslot = a.nslot;
        c.full = reinterpret_cast<unsigned long long*>(smem);
        c.empty = c.full + LOOP_MAX_SLOTS;
        c.issued = reinterpret_cast<volatile int*>(c.empty + LOOP_MAX_SLOTS);
        c.ctl = c.issued + LOOP_MAX_SLOTS;
        c.ctl_best = reinterpret_cast<unsigned long long*>(const_cast<int*>(c.ctl) + CTL_WORDS);
        c.red = reinterpret_cast<float*>(c.ctl_best + 2);
        c.work = smem + a.off_act;
        c.xf = reinterpret_cast<float*>(smem + a.off_xf);
        c.pbuf = reinterpret_cast<float*>(smem + a.off_pbuf);
        c.ring = smem + a.off_ring;
        c.blob = reinterpret_cast<const int*>(smem + a.off_blob);
        c.lay = reinterpret_cast<const LoopLayer*>(smem + a.off_layers);
        c.own = reinterpret_cast<float*>(smem + a.off_own);
        c.own_row0 = 2 * a.sh_x.begin((int)blockIdx.x);
        c.bar_k = 0;
        c.slot = 0;
        c.lap = 0;
        c.mark_id = 0;
        c.mark_on = 0;
        c.tap = nullptr;
        for (int i = 0; i < LOOP_MAX_SLOTS; i++) {
            mbar_init(c.full + i, 1);
            mbar_init(c.empty + i, LOOP_EMPTY);
            c.issued[i] = 0;
        }
        for (int i = 0; i < CTL_WORDS; i++) c.ctl[i] = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // decode state, identical in every CTA
    const TokenState* st = a.st;
    int pos = st->pos, token = st->token, step = 0, prompt_idx = st->prompt_idx;
    const int max_steps = st->max_steps, max_seq = st->max_seq, n_stop = st->n_stop, force_prompt = st->force_prompt;
    int headless = a.n_headless;

    // this CTA's plan and the per-layer pointer table -> shared memory
    {
        int* blob = reinterpret_cast<int*>(smem + a.off_blob);
        const int* src = a.blob + (size_t)c.cta * a.blob_stride;
        for (int i = ltid(); i < a.blob_stride; i += LOOP_THREADS) blob[i] = src[i];
        int* lay = reinterpret_cast<int*>(smem + a.off_layers);
        const int* lsrc = reinterpret_cast<const int*>(a.layers);
        const int lwords = a.n_layer * (int)(sizeof(LoopLayer) / 4);
        for (int i = ltid(); i < lwords; i += LOOP_THREADS) lay[i] = lsrc[i];
    }
    __syncthreads();
    if (lwarp() == LOOP_CWARPS) {
        loop_streamer(c, a, a.n_headless + max_steps);
        return;
    }

    if (ltid() < 8) c.ctl[CTL_STOPS + ltid()] = ltid() < n_stop ? st->stop_ids[ltid()] : -1;
    cbar();
    const int K = a.K;
    const int n_own = max(0, min(K, c.own_row0 + 2 * a.sh_x.count(c.cta)) - c.own_row0);
    bool done = false;
#pragma unroll 1
    for (int it = 0; !done; it++) {
        const bool with_head = headless == 0;
        if (ltid() == 0) {
            c.mark_on = a.prof != nullptr && it == a.prof_step;
            c.mark_id = 0;
            attn_plan(c, a, pos);
            if (c.cta == 0) a.best[(it + 1) & 3] = 0ull;
        }
        embed_stage(c, a, token, n_own);  // its barrier also publishes the fields above
#pragma unroll 1
        for (int li = 0; li < a.n_layer; li++) {
            const LoopLayer* L = c.lay + li;
            if (ltid() == 0) {
                c.kc = a.kc + (size_t)li * a.kv_layer_stride;
                c.vc = a.vc + (size_t)li * a.kv_layer_stride;
                c.bias = L->bias_qkv;
                c.tap = nullptr;
            }
            loop_mark(c, a);
            // ---- 1. RMSNorm + Q8 + Q/K/V (+bias) + RoPE + f16 KV store
            loop_act(c, a, li == 0 ? nullptr : a.x, K, L->attn_norm, 0);
            loop_mark(c, a);
            loop_gemv(c, a, 0, LEPI_QKV);
            loop_mark(c, a);
            grid_barrier(c, a);
            loop_mark(c, a);
            // ---- 2. attention
            loop_attention<HD>(c, a);
            loop_mark(c, a);
            grid_barrier(c, a);
            const int S = c.at_S;
            if (S > a.attn_inline_max) {
                loop_attention_merge<HD>(c, a, S);
                grid_barrier(c, a);
            }
            loop_mark(c, a);
            // ---- 3. Q8 + o-proj + residual
            loop_act(c, a, a.att, a.nq, nullptr, S <= a.attn_inline_max ? S : 1);
            loop_mark(c, a);
            loop_gemv(c, a, 1 + L->o_q6, LEPI_RESIDUAL);
            loop_mark(c, a);
            grid_barrier(c, a);
            loop_mark(c, a);
            // ---- 4. RMSNorm + Q8 + gate/up + SiLU*mul
            loop_act(c, a, a.x, K, L->ffn_norm, 0);
            loop_mark(c, a);
            loop_gemv(c, a, 3, LEPI_SILU);
            loop_mark(c, a);
            grid_barrier(c, a);
            loop_mark(c, a);
            // ---- 5. Q8 + down + residual
            if (ltid() == 0 && a.layer_taps) c.tap = a.layer_taps + (size_t)li * K;  // published by the barrier inside loop_act
            loop_act(c, a, a.h, a.FF, nullptr, 1);
            loop_mark(c, a);
            loop_gemv(c, a, 4 + L->down_q6, LEPI_RESIDUAL);
            loop_mark(c, a);
            grid_barrier(c, a);
            if (c.ctl[CTL_SNAP]) break;
        }
        if (loop_aborted(c)) break;
        if (with_head) {
            loop_mark(c, a);
            loop_act(c, a, a.x, K, a.out_norm, 0);
            unsigned long long b = loop_gemv(c, a, 6, LEPI_LOGITS);
            // CTA-wide maximum -> the grid-wide word of this step
#pragma unroll 1
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(TFR_FULL_MASK, b, o);
                b = other > b ? other : b;
            }
            unsigned long long* sb = reinterpret_cast<unsigned long long*>(c.red);
            if (llane() == 0) sb[lwarp()] = b;
            cbar();
            if (ltid() == 0) {
#pragma unroll 1
                for (int i = 1; i < LOOP_CWARPS; i++) b = sb[i] > b ? sb[i] : b;
                atomicMax(a.best + (it & 3), b);
            }
            loop_mark(c, a);
            const unsigned long long win = grid_barrier(c, a, a.best + (it & 3));
            loop_mark(c, a);
            if (loop_aborted(c)) break;
            const int tok = argmax_key_index(win);
            if (c.cta == 0 && ltid() == 0) a.out_tokens[step] = tok;
            int next = tok;
            if (force_prompt) {
                prompt_idx += 1;
                if (step + 1 < max_steps) next = a.prompt[prompt_idx];
            }
            token = next;
            pos += 1;
            step += 1;
            done = step >= max_steps || pos >= max_seq;
            for (int i = 0; i < n_stop; i++) done = done || c.ctl[CTL_STOPS + i] == tok;
        } else {
            headless -= 1;
            prompt_idx += 1;
            pos += 1;
            token = a.prompt[prompt_idx];
            if (pos >= max_seq) done = true;
        }
    }
    if (ltid() == 0) {
        c.ctl[CTL_STOP] = 1;
        if (c.cta == 0) {
            TokenState* w = a.st;
            w->pos = pos;
            w->token = token;
            w->step = step;
            w->prompt_idx = prompt_idx;
            w->done = 1;
        }
    }
}

// Zeroes the grid-barrier counters and the argmax words before a launch of k_decode_loop.
__global__ void k_loop_reset(unsigned int* bar, unsigned long long* best) {
    const int i = threadIdx.x;
    for (int j = i; j < 8 * LOOP_BAR_STRIDE; j += blockDim.x) bar[j] = 0u;
    if (i < 4) best[i] = 0ull;
}

}  // namespace tfr
