// Stage-machine decode megakernel for sm_100a: one CTA per SM, one cooperative launch for n_steps
// decode steps of up to eight sequences.
//
// What a step does is a program of mk_stage_desc records (include/mk_stage.h) in device memory.
// Every CTA has 16 consumer warps and one producer warp:
//
//   * the producer's elected lane walks the program and, for every GEMV stage, issues this CTA's weight
//     chunks (1-D bulk copies completing on mbarriers) into a shared-memory ring, in exactly the order
//     the consumer warps will ask for them.  It never looks at activations (except the routed expert
//     list), so weights of later stages land while the consumers wait at a grid barrier;
//   * a GEMV stage is cut into units: (group, K split, 16-row tile).  A CTA owns a contiguous range of
//     units; inside it each consumer warp takes whole units, converts the weight bytes to fp16 in
//     registers (bf16 stays bf16) and multiplies with `mma.sync.m16n8k16`: the weight tile is the
//     16-row A operand, the sequences are the eight B columns, so one to eight sequences cost the same
//     number of instructions.  Nothing in the GEMV needs a CTA-wide barrier: a warp waits for its own
//     chunks and releases them itself;
//   * units that add up into one output tile (K splits, routed experts) meet through a counter: each
//     writes its 16 x 8 partial tile, the last arrival adds them in a fixed order and runs the epilogue
//     (store, residual add with sums of squares for the next RMSNorm, GLU, logits + arg-max);
//   * with tensor parallelism the epilogue of a row-parallel GEMV first pushes the tile into every
//     rank's mailbox with plain peer stores (value and sequence tag in one 64-bit word), polls its own
//     mailbox and adds the ranks' tiles in rank order, so every rank holds the same bits;
//   * stages meet at a grid barrier (one atomic counter in global memory, bounded wait).
//
// Every wait is bounded: a wait that runs out records MK_ERR_TIMEOUT and its site in the status words,
// after which every wait in every CTA returns at once, the remaining stages are skipped, the producer
// waits (bounded) for its copies in flight and the kernel returns.
#pragma once
#include <cuda_fp16.h>

#include "../../include/mk_stage.h"
#include "mk_device.cuh"

namespace mks {
using namespace mk;

constexpr int SLOT_BYTES = 4352;                  // one ring slot: 8 tile steps of 512 bytes + 256 bytes of scales
constexpr int XS_BYTES = 50176;                   // staged GEMV input: 8 columns x 3072 fp16 + padding; also mixer scratch
constexpr int MAX_GROUPS = 72;                    // routed experts of one step (8 x 8) + shared / dense groups
constexpr int MISC_BYTES = 8192;
constexpr int SMEM_TOTAL = 232448;                // 227 KB
constexpr int MAX_RING_DEPTH = 4;                 // ring slots per consumer warp: 2..4, as many as the launch's input staging area leaves room for
constexpr int NS = 16 * MAX_RING_DEPTH;           // ring slots (upper bound): every consumer warp has its own
constexpr int ATTN_MAX_CHUNK = 256;               // positions per attention task (score buffer)
constexpr int MAILBOX_TILES = 1024;               // output tiles of a row-parallel GEMV one all-reduce can carry
constexpr int MAILBOX_BYTES = 2 * MAILBOX_TILES * MKS_MAX_RANKS * 128 * 8 + 2 * MKS_MAX_RANKS * MKS_MAX_BATCH * 16;
static_assert((size_t)16 * 2 * SLOT_BYTES + XS_BYTES + MISC_BYTES <= SMEM_TOTAL, "shared memory of one SM");

// wait sites (status[1])
enum { WS_FULL = 101, WS_EMPTY, WS_BARRIER, WS_ROUTE, WS_DRAIN, WS_MAILBOX, WS_KEYS };

struct Args {
    const mk_stage_desc* prog;
    int n_stages, M, n_steps;
    int* tok;
    int* pos;
    int* tokens_out;
    unsigned long long* bar;
    unsigned long long bar_base;
    int* status;
    long long spin_limit_ns;
    unsigned long long* prof;
    int tp, rank;
    unsigned long long* mailbox[MKS_MAX_RANKS];
    unsigned long long ar_base;
    const int* tokens_in;    // [n_tokens_in][M] forced inputs of the first steps, or null
    int n_tokens_in;
    const int* row_valid;    // [M] 0 = padding row, or null
    int prof_cta;            // the CTA whose timestamps go to `prof`
    int xs_bytes;            // input staging / mixer scratch area of this launch
    int ring_depth;          // ring slots per consumer warp
};

// Everything the threads of a CTA share lives in shared memory, behind the ring and the input staging
// area; what is per thread (identity, ring position) travels in registers.  A per-thread context struct
// handed to the stage functions by reference would sit in local memory: 544 threads' copies do not fit
// the few KB of L1 that the shared-memory carve-out leaves, and every field access would cost an L2 trip.
struct Shared {
    uint64_t full[NS];
    uint64_t empty[NS];
    u64 keys_s[8];                 // best key per sequence
    volatile u64 pf_pos;           // bytes of the weight stream the issuing lane has requested (read by the prefetch lane)
    unsigned long long* prof;      // this stage's timestamp row (CTA 0, last step) or null
    mk_stage_desc desc[2];         // this stage's record and the next one's
    Args A;                        // the launch arguments
    float red[16 + 17 * 8];        // block-reduction scratch
    float xinv[8];                 // factor that undoes the power-of-two scaling of a staged column
    float rstd[8];                 // 1/rms of the staged input
    int tok_s[8];
    int pos_s[8];
    int valid_s[8];                // 0: a padding row of this launch
    int r_ids[64];                 // [8][8] routed expert ids per sequence
    float r_w[64];                 // [8][8] routing weights
    float coef[MAX_GROUPS * 8];    // weight of group g for sequence m
    int glist[MAX_GROUPS];         // expert id of group g
    unsigned gmask[8];             // bitmap of the selected experts
    int n_groups;
    volatile int abort_flag;
    volatile unsigned route_seq;
    int flag;
    // dynamic shared memory: [this block | staging area of A.xs_bytes | 16 x A.ring_depth ring slots]
    __device__ __forceinline__ uint8_t* xs() { return reinterpret_cast<uint8_t*>(this) + MISC_BYTES; }
    __device__ __forceinline__ uint8_t* ring() { return reinterpret_cast<uint8_t*>(this) + MISC_BYTES + A.xs_bytes; }
};
static_assert(sizeof(Shared) <= MISC_BYTES, "the shared block fits its area");

// thread identity from the special registers: cheaper than a struct that travels through the stack
__device__ __forceinline__ int tid_() { return (int)threadIdx.x; }
__device__ __forceinline__ int warp_() { return (int)(threadIdx.x >> 5); }
__device__ __forceinline__ int lane_() { return (int)(threadIdx.x & 31); }
__device__ __forceinline__ int cta_() { return (int)blockIdx.x; }
__device__ __forceinline__ int grid_() { return (int)gridDim.x; }
struct Mut {
    uint32_t chunk_n;        // ring chunks this consumer warp has taken so far
    bool dead;               // this thread saw a wait run out
};

constexpr int PROF_FIELDS = 8;  // per stage: entered, input staged, units done, barrier passed, ring-wait ns of warp 0
__device__ __forceinline__ void prof_mark(Shared& S, int field) {
    if (S.prof && tid_() == 0) S.prof[field] = globaltimer();
}

// ---- bounded waits ---------------------------------------------------------------------------------------
struct Spin2 {
    uint32_t it = 0;
    u64 t0 = 0;
};
__device__ __noinline__ u64 spin_slow2(volatile int* abort_flag, int* status, u64 limit_ns, u64 t0, int where) {
    if (*abort_flag) return ~0ull;
    if (ld_volatile_i32(status) != 0) {
        *abort_flag = 1;
        return ~0ull;
    }
    const u64 now = globaltimer();
    if (!t0) return now;
    if (now - t0 > limit_ns) {
        if (atomicCAS(status, 0, -2) == 0) {
            status[1] = where;
            status[2] = (int)blockIdx.x;
            status[3] = (int)threadIdx.x;
        }
        __threadfence();
        *abort_flag = 1;
        return ~0ull;
    }
    return t0;
}
#define MKS_SPIN_FAIL(S, s, where) \
    ((((++(s).it) & 255u) == 0) && (((s).t0 = spin_slow2(&(S).abort_flag, (S).A.status, (u64)(S).A.spin_limit_ns, (s).t0, (where))) == ~0ull))

// Wait of a whole warp for one barrier phase.  The warp leaves together: a lane that returned alone
// would never reach the `__syncwarp` the others go on to.
__device__ __forceinline__ bool mbar_wait2(Shared& S, uint64_t* b, uint32_t parity, int where) {
    Spin2 s;
    bool fail = false;
#pragma unroll 1
    for (;;) {
        const bool ok = mbar_try_wait(b, parity);
        if (__all_sync(0xffffffffu, ok)) return true;
        if (!ok && MKS_SPIN_FAIL(S, s, where)) fail = true;
        if (__any_sync(0xffffffffu, fail)) return false;       // the abort flag is set: the stage loop stops at its next check
    }
}

__device__ __forceinline__ u64 ld_acquire_u64(const unsigned long long* p) {
    u64 v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ u64 ld_relaxed_sys_u64(const unsigned long long* p) {
    u64 v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, u64 v) {
    chaos_delay();
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Grid barrier over the consumer threads of all CTAs: one arrival per CTA on a counter that only grows.
// The arrival is a release (everything this CTA wrote before the preceding CTA barrier is visible to
// whoever observes the count), the poll an acquire; no sequentially-consistent fence is needed.
__device__ __forceinline__ void red_release_add_u64(unsigned long long* p, unsigned long long v) {
    chaos_delay();
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void grid_barrier(Shared& S, Mut& mu, const Args& A, u64& bar_n) {
    bar_n++;
    consumer_sync();
    if (tid_() == 0 && !S.abort_flag) {
        red_release_add_u64(A.bar, 1ull);
        const u64 target = A.bar_base + bar_n * (u64)grid_();
        Spin2 s;
        while (ld_acquire_u64(A.bar) < target) {
            if (MKS_SPIN_FAIL(S, s, WS_BARRIER)) break;
        }
    }
    consumer_sync();
}

// ---- conversions -----------------------------------------------------------------------------------------
// Two e2m1 values in the low byte of `b` -> f16x2 (low nibble in the low half).
__device__ __forceinline__ uint32_t cvt_e2m1x2(uint32_t b) {
    uint32_t r;
    asm("{\n .reg .b8 t;\n .reg .b16 h;\n cvt.u16.u32 h, %1;\n cvt.u8.u16 t, h;\n cvt.rn.f16x2.e2m1x2 %0, t;\n}\n" : "=r"(r) : "r"(b));
    return r;
}
// Two e4m3 values in the low 16 bits of `b` -> f16x2.
__device__ __forceinline__ uint32_t cvt_e4m3x2(uint32_t b) {
    uint32_t r;
    asm("{\n .reg .b16 h;\n cvt.u16.u32 h, %1;\n cvt.rn.f16x2.e4m3x2 %0, h;\n}\n" : "=r"(r) : "r"(b));
    return r;
}
// Two signed bytes (low 16 bits of `b`, already xor 0x80) -> f16x2: 0x6400 | u is the half 1024 + u.
__device__ __forceinline__ uint32_t cvt_s8x2(uint32_t bx, uint32_t sel) {
    const uint32_t h = __byte_perm(bx, 0x64646464u, sel);             // [0x64, b1, 0x64, b0] as two halves
    const __half2 v = *reinterpret_cast<const __half2*>(&h);
    const __half2 r = __hsub2(v, __floats2half2_rn(1152.f, 1152.f));  // 1024 + 128
    return *reinterpret_cast<const uint32_t*>(&r);
}

// (not `volatile`: the instruction has no effect beyond its outputs, and the compiler must be free to interleave
// independent accumulator chains -- a warp issues in order, and a dependent MMA behind its producer stalls it)
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
    return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float ldcg_f(const float* p) { return __ldcg(p); }

// ---- geometry of a GEMV stage (shared by producer and consumers) ----------------------------------------------
struct Gemv {
    int T, S, G, unit_steps, chunk_steps, chunk_bytes, n_chunks;
    int u0, u1;                  // this CTA's unit range; unit = (group * S + split) * T + tile (32-bit: 64-bit division costs hundreds of cycles)
};
__device__ __forceinline__ Gemv gemv_geometry(const Shared& S, const mk_stage_desc& d) {
    Gemv g;
    g.T = d.i[MKS_I_TILES];
    g.S = d.i[MKS_I_SPLITS];
    g.G = d.i[MKS_I_GROUPS] >= 0 ? d.i[MKS_I_GROUPS] : *reinterpret_cast<const volatile int*>(&S.n_groups);
    g.unit_steps = d.i[MKS_I_UNIT_STEPS];
    g.chunk_steps = d.i[MKS_I_CHUNK_STEPS];
    g.chunk_bytes = d.i[MKS_I_CHUNK_BYTES];
    g.n_chunks = g.unit_steps / g.chunk_steps;
    const unsigned P = (unsigned)(g.G * g.S), grid = (unsigned)grid_(), cta = (unsigned)cta_();
    if (P <= grid) {
        // every CTA stays inside one panel (one staged input): panel p gets the CTAs [ceil(p grid / P), ceil((p + 1) grid / P))
        // and they share its T tiles evenly.  A CTA that straddled two panels would stage its input twice and
        // keep the whole grid waiting at the stage's barrier.
        const unsigned p = cta * P / grid;
        const unsigned c0 = (p * grid + P - 1) / P, c1 = ((p + 1) * grid + P - 1) / P;
        const unsigned n = c1 - c0, k = cta - c0;
        g.u0 = (int)(p * (unsigned)g.T + (unsigned)g.T * k / n);
        g.u1 = (int)(p * (unsigned)g.T + (unsigned)g.T * (k + 1) / n);
    } else {
        const unsigned U = P * (unsigned)g.T;                      // < 2^24: U * grid fits 32 bits
        g.u0 = (int)(U * cta / grid);
        g.u1 = (int)(U * (cta + 1) / grid);
    }
    return g;
}
// Weight bytes of group `grp`: experts of a routed stage come from the routing list, the shared expert last.
__device__ __forceinline__ const uint8_t* group_weights(const Shared& S, const mk_stage_desc& d, int grp, int G) {
    const uint8_t* w = reinterpret_cast<const uint8_t*>(d.p[MKS_P_W]);
    if (d.i[MKS_I_GROUPS] >= 0) return w + (size_t)grp * d.p[MKS_P_W_GSTRIDE];
    if (d.p[MKS_P_W_SHARED] && grp == G - 1) return reinterpret_cast<const uint8_t*>(d.p[MKS_P_W_SHARED]);
    return w + (size_t)reinterpret_cast<const volatile int*>(S.glist)[grp] * d.p[MKS_P_W_GSTRIDE];
}
__device__ __forceinline__ const float* group_row_scale(const Shared& S, const mk_stage_desc& d, int grp, int G) {
    const float* s = reinterpret_cast<const float*>(d.p[MKS_P_ROW_SCALE]);
    if (!s) return nullptr;
    if (d.i[MKS_I_GROUPS] >= 0) return s + (size_t)grp * d.p[MKS_P_RS_GSTRIDE];
    if (d.p[MKS_P_W_SHARED] && grp == G - 1) return reinterpret_cast<const float*>(d.p[MKS_P_RS_SHARED]);
    return s + (size_t)S.glist[grp] * d.p[MKS_P_RS_GSTRIDE];
}

// ---- producer --------------------------------------------------------------------------------------------
// The whole producer warp walks the program.  In every round of up to 16 units lane j issues the chunks
// of the round's j-th unit (the unit consumer warp j will multiply), one 1-D bulk copy per chunk: a single
// lane needs about a quarter of a microsecond of dependent instructions per copy, which caps one SM at a few
// chunks per microsecond -- a sixth of its share of the HBM stream.
//
// Every consumer warp has its own ring_depth slots.  A slot is therefore filled and drained by the same pair
// (lane j, warp j) in strict alternation, and a waiter is never more than one phase ahead of its barrier:
// with slots shared between warps a fast warp could ask for the next-but-one phase of a slot that still
// served another warp, and a parity wait cannot tell that phase from the one before it.
__device__ __forceinline__ void prefetch_desc_l1(const mk_stage_desc* d) {
    const char* p = reinterpret_cast<const char*>(d);
    asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
    asm volatile("prefetch.global.L1 [%0];" ::"l"(p + 96));
    asm volatile("prefetch.global.L1 [%0];" ::"l"(p + 192));
    asm volatile("prefetch.global.L1 [%0];" ::"l"(p + 287));
}

// Lane j of the producer warp feeds consumer warp j and nobody else: it has its own cursor over the program
// (stage, panel, round, chunk) and never waits inside the loop.  Every turn of the warp-wide loop each lane
// looks whether the slot its next chunk goes to has been released, issues the copy if so and moves on; a lane
// whose consumer is busy (a long unit tail, a barrier) costs the others nothing.  Lanes may be in different
// rounds, panels and stages at the same time, exactly as far ahead as their own two slots allow.
struct Cursor {
    int step, si;                 // position in the program (si = -1 before the first stage)
    int T, S_, G, n_chunks, chunk_bytes, u0, u1;
    int pu, pend, r0;             // next panel start, end of the current panel's units in this CTA, next round
    int panel;
    int ch;                       // next chunk of the current unit
    const uint8_t* w;             // the current panel's units
    const uint8_t* wg;            // the current group's matrix
    const uint8_t* src;           // the current unit
    unsigned long long w_bytes;
    unsigned routes;
    bool have, done;
};

__device__ __noinline__ void producer_main(Shared& S, const Args& A) {
    const int lane = lane_();
    const u64 policy = policy_evict_first();
    const uint32_t depth = (uint32_t)A.ring_depth;
    uint32_t q = 0;              // chunks this lane has issued: chunk q of consumer warp `lane` lives in slot
                                 // lane * depth + q % depth, phase q / depth
    Cursor c;
    c.step = 0; c.si = -1; c.u0 = c.u1 = c.pu = c.pend = c.r0 = 0; c.ch = 0; c.routes = 0;
    c.have = false; c.done = lane >= NCW;
    c.T = c.S_ = c.G = 1; c.n_chunks = 1; c.chunk_bytes = 0; c.panel = 0; c.w = c.wg = c.src = nullptr; c.w_bytes = 0;
    Spin2 sp;
    bool stop = false;
#pragma unroll 1
    while (!stop) {
        bool progress = false;
        if (!c.done && !c.have) {
            // move the cursor: at most a few transitions per turn, so that the lanes stay roughly together
#pragma unroll 1
            for (int k = 0; k < 6 && !c.have && !c.done; k++) {
                if (c.r0 < c.pend) {                                   // next round of the current panel
                    const int nj = min(NCW, c.pend - c.r0);
                    if (lane < nj) {
                        c.src = c.w + (size_t)((c.r0 + lane) - c.panel * c.T) * ((size_t)c.n_chunks * c.chunk_bytes);
                        c.ch = 0;
                        c.have = true;
                    }
                    c.r0 += NCW;
                    progress = true;
                } else if (c.pu < c.u1) {                               // next panel of the current stage
                    const mk_stage_desc& d = A.prog[c.si];
                    c.panel = c.pu / c.T;
                    c.pend = min(c.u1, (c.panel + 1) * c.T);
                    const int grp = c.panel / c.S_, split = c.panel - grp * c.S_;
                    c.wg = group_weights(S, d, grp, c.G);
                    c.w = c.wg + (size_t)split * c.T * ((size_t)c.n_chunks * c.chunk_bytes);
                    c.r0 = c.pu;
                    c.pu = c.pend;
                    progress = true;
                } else {                                                // next stage
                    int nsi = c.si + 1, nstep = c.step;
                    if (nsi >= A.n_stages) {
                        nsi = 0;
                        nstep++;
                    }
                    if (nstep >= A.n_steps) {
                        c.done = true;
                        break;
                    }
                    const mk_stage_desc& d = A.prog[nsi];
                    if (d.op == MKS_OP_ROUTE && S.route_seq < c.routes + 1) break;   // the expert list is not there yet
                    if (d.op == MKS_OP_ROUTE) c.routes++;
                    c.si = nsi;
                    c.step = nstep;
                    progress = true;
                    if (d.op == MKS_OP_GEMV) {
                        const Gemv g = gemv_geometry(S, d);
                        c.T = g.T; c.S_ = g.S; c.G = g.G; c.n_chunks = g.n_chunks; c.chunk_bytes = g.chunk_bytes;
                        c.u0 = g.u0; c.u1 = g.u1;
                        c.pu = g.u0; c.pend = 0; c.r0 = 0;
                        c.w_bytes = d.p[MKS_P_W_BYTES];
                    } else {
                        c.u0 = c.u1 = c.pu = c.pend = c.r0 = 0;
                    }
                }
            }
        }
        if (c.have) {
            const int slot = lane * (int)depth + (int)(q % depth);
            const bool is_free = q < depth || mbar_try_wait(&S.empty[slot], ((q / depth) - 1) & 1);
            if (is_free) {
                // self-check: the copy must stay inside the matrix the record describes
                const size_t off = (size_t)(c.src - c.wg) + (size_t)c.ch * c.chunk_bytes;
                if (c.w_bytes && off + (size_t)c.chunk_bytes > (size_t)c.w_bytes) {
                    if (atomicCAS(S.A.status, 0, -5) == 0) {
                        S.A.status[1] = c.si;
                        S.A.status[2] = cta_();
                        S.A.status[3] = (int)(off >> 12);
                    }
                    S.abort_flag = 1;
                } else if (!S.abort_flag) {
                    mbar_expect_tx(&S.full[slot], (uint32_t)c.chunk_bytes);
                    bulk_load(S.ring() + (size_t)slot * SLOT_BYTES, c.src + (size_t)c.ch * c.chunk_bytes, (uint32_t)c.chunk_bytes,
                              &S.full[slot], policy);
                    q++;
                    c.ch++;
                    if (c.ch == c.n_chunks) c.have = false;
                    progress = true;
                }
            }
        }
        // the warp leaves together: when every lane is done, or a wait ran out somewhere
        if (__all_sync(0xffffffffu, c.done)) break;
        if (__any_sync(0xffffffffu, progress)) {
            sp.it = 0;
            sp.t0 = 0;
        } else if (lane == 0 && MKS_SPIN_FAIL(S, sp, WS_EMPTY)) {
            stop = true;
        }
        stop = __any_sync(0xffffffffu, stop || S.abort_flag != 0);
    }
    // before the CTA may exit every copy that was issued must have landed (not abortable: the copies write shared memory)
    if (lane < NCW) {
        const uint32_t first = q > depth ? q - depth : 0;
#pragma unroll 1
        for (uint32_t i = first; i < q; i++) {
            uint32_t it = 0;
            u64 t0 = 0;
            while (!mbar_try_wait(&S.full[lane * (int)depth + (int)(i % depth)], (i / depth) & 1)) {
                if (((++it) & 1023u) == 0) {
                    const u64 now = globaltimer();
                    if (!t0) t0 = now;
                    else if (now - t0 > (u64)S.A.spin_limit_ns) {
                        if (atomicCAS(S.A.status, 0, -2) == 0) S.A.status[1] = WS_DRAIN;
                        break;
                    }
                }
            }
        }
    }
}

// ---- GEMV input staging ------------------------------------------------------------------------------------
// Column stride of the staged input in bytes: a multiple of 128 plus 32, so that the eight columns'
// 8-byte fragment reads of a half warp fall into different banks.
__device__ __forceinline__ int xs_stride_bytes(int kc) { return ((kc * 2 + 127) / 128) * 128 + 32; }

// Stage columns [split * kc, (split + 1) * kc) of every sequence's input of group `grp`: normalise, round
// to bf16 (the model's activation type) and store as fp16 scaled by a power of two per column (bf16
// weights: as bf16, unscaled).  Column `m` of the staged matrix is sequence m; with two pieces column
// M + m holds what fp16 lost of sequence m, so that the products see an fp32-exact input.
//
// What matters here is the number of dependent L2 round trips (about 0.7 us each on this part), not
// bytes: the first batch of input loads, the norm weights and the sums of squares behind 1/rms are all
// requested before anything is awaited; the values go to shared memory as bf16 and are rescaled there.
constexpr int XB = 2;       // float4 groups of one batch; two batches are in flight

__device__ __noinline__ void stage_x(Shared& S, Mut& mu, const mk_stage_desc& d, int grp, int split) {
    const int kc = d.i[MKS_I_KC], fmt = d.i[MKS_I_FMT], pieces = d.i[MKS_I_PIECES], M = S.A.M;
    const int stride = xs_stride_bytes(kc);
    const bool norm = d.i[MKS_I_PROLOGUE] == MKS_P_NORM;
    const float* x = reinterpret_cast<const float*>(d.p[MKS_P_X]) + (size_t)grp * d.i[MKS_I_X_GSTRIDE] + (size_t)split * kc;
    const float* nw = reinterpret_cast<const float*>(d.p[MKS_P_NORM_W]) + (size_t)split * kc;
    const float noff = d.f[MKS_F_NORM_OFF];
    const float in_scale = d.f[MKS_F_IN_SCALE] != 0.f ? d.f[MKS_F_IN_SCALE] : 1.f;
    const int xstride = d.i[MKS_I_X_STRIDE];
    const int k4n = kc >> 2, total = M * k4n;
    int* red_i = reinterpret_cast<int*>(S.red);
    if (tid_() < MKS_MAX_BATCH) red_i[tid_()] = 0;
    // two batches in flight: the next one is requested before the current one is used, so a panel of eight
    // sequences costs one exposed round trip, not one per batch
    float4 xv[XB], xn[XB];
    auto request = [&](int base, float4 (&dst)[XB]) {
#pragma unroll
        for (int u = 0; u < XB; u++) {
            const int idx = base + u * NCT + tid_();
            if (idx < total) {
                const int m = idx / k4n, k4 = idx - m * k4n;
                dst[u] = __ldcg(reinterpret_cast<const float4*>(x + (size_t)m * xstride) + k4);
            }
        }
    };
    request(0, xv);
    if (XB * NCT < total) request(XB * NCT, xn);
    if (norm) {
        // 1/rms of every sequence from the 16-element sums of squares of the whole input vector: warp m adds up
        // sequence m's sums (all loads of a lane in flight at once, fixed order) while the other warps only wait for x
        const int K = d.i[MKS_I_K_TOTAL], n16 = K / 16;
        const float* ssq = reinterpret_cast<const float*>(d.p[MKS_P_X_SSQ]);
        if (warp_() < M) {
            const float* row = ssq + (size_t)warp_() * n16;
            float s = 0.f;
#pragma unroll 8
            for (int j = lane_(); j < n16; j += 32) s += ldcg_f(row + j);
            s = warp_sum(s);
            if (lane_() == 0) S.rstd[warp_()] = rsqrtf(s / (float)K + d.f[MKS_F_EPS]);
        }
    }
    // A bound on |input| known to the host (a normed vector cannot exceed sqrt(K) max|weight|) fixes the power-of-two
    // scale of the fp16 copy up front: the values then go to shared memory in their final form in one pass.
    const float bound = d.f[MKS_F_IN_BOUND];
    const bool fixed_scale = bound > 0.f && fmt != MKS_FMT_BF16 && pieces == 1;
    float fscale = 1.f;
    if (fixed_scale) {
        const int be = ((__float_as_int(bound) >> 23) & 0xff) - 126;          // bound < 2^be
        const int e = max(-100, min(100, 15 - be));
        fscale = __int_as_float((127 + e) << 23);
        if (tid_() < MKS_MAX_BATCH) S.xinv[tid_()] = __int_as_float((127 - e) << 23);
    }
    consumer_sync();
    prof_mark(S, 4);
#pragma unroll 1
    for (int base = 0; base < total; base += XB * NCT) {
        if (base) {
#pragma unroll
            for (int u = 0; u < XB; u++) xv[u] = xn[u];
            if (base + XB * NCT < total) request(base + XB * NCT, xn);
        }
#pragma unroll
        for (int u = 0; u < XB; u++) {
            const int idx = base + u * NCT + tid_();
            const bool live = idx < total;
            int m = 0;
            float mx = 0.f;
            if (live) {
                m = idx / k4n;
                const int k4 = idx - m * k4n;
                float v[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
                if (norm) {
                    // the norm weights are the same few KB for every sequence: after the first they come from L1
                    const float4 wv = __ldg(reinterpret_cast<const float4*>(nw) + k4);
                    const float r = S.rstd[m] * in_scale;
                    v[0] = v[0] * r * (noff + wv.x); v[1] = v[1] * r * (noff + wv.y);
                    v[2] = v[2] * r * (noff + wv.z); v[3] = v[3] * r * (noff + wv.w);
                }
                if (pieces == 2) {
                    // fp32 copy, parked in the two columns that sequence m's pieces will occupy... of sequence pair slot m
                    *reinterpret_cast<float4*>(S.xs() + (size_t)(2 * m) * stride + (size_t)k4 * 16) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                    v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
                    if (fixed_scale) {
                        const __half2 a2 = __floats2half2_rn(v[0] * fscale, v[1] * fscale), b2 = __floats2half2_rn(v[2] * fscale, v[3] * fscale);
                        *reinterpret_cast<uint2*>(S.xs() + (size_t)m * stride + (size_t)k4 * 8) =
                            make_uint2(*reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&b2));
                    } else {
                        *reinterpret_cast<uint2*>(S.xs() + (size_t)m * stride + (size_t)k4 * 8) =
                            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
                    }
                }
                mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
            }
            if (fmt != MKS_FMT_BF16 && !fixed_scale) {
                // a warp's 32 groups lie in at most two sequences
                const int m0 = __shfl_sync(0xffffffffu, m, 0);
                const float a = warp_max(live && m == m0 ? mx : 0.f), b = warp_max(live && m != m0 ? mx : 0.f);
                if (lane_() == 0) {
                    if (a > 0.f) atomicMax(&red_i[m0], __float_as_int(a));
                    if (b > 0.f) atomicMax(&red_i[min(m0 + 1, MKS_MAX_BATCH - 1)], __float_as_int(b));
                }
            }
        }
    }
    if (fixed_scale) return;                                   // staged in final form; the caller's barrier publishes it
    if (fmt == MKS_FMT_BF16) {
        if (tid_() < 8) S.xinv[tid_()] = 1.f;
        if (pieces == 2) {
            // fp32-exact inputs for bf16 weights: x = hi + lo, both bf16 (16 significant bits), no scaling needed
            consumer_sync();
            float v[16];
            int n = 0;
#pragma unroll 1
            for (int idx = tid_(); idx < M * kc && n < 16; idx += NCT, n++) {
                const int m = idx / kc, k = idx - m * kc;
                v[n] = *reinterpret_cast<const float*>(S.xs() + (size_t)(2 * m) * stride + (size_t)k * 4);
            }
            consumer_sync();
            n = 0;
#pragma unroll 1
            for (int idx = tid_(); idx < M * kc && n < 16; idx += NCT, n++) {
                const int m = idx / kc, k = idx - m * kc;
                const __nv_bfloat16 hi = __float2bfloat16_rn(v[n]);
                reinterpret_cast<__nv_bfloat16*>(S.xs() + (size_t)m * stride)[k] = hi;
                reinterpret_cast<__nv_bfloat16*>(S.xs() + (size_t)(M + m) * stride)[k] = __float2bfloat16_rn(v[n] - __bfloat162float(hi));
            }
        }
        return;
    }
    consumer_sync();
    prof_mark(S, 5);
    if (tid_() < M) {
        // a = f * 2^e with f in [0.5, 1): the exponent field gives e; scale = 2^(14 - e), built from its bits
        const int bits = red_i[tid_()];
        int e = bits > 0 && bits < 0x7f800000 ? ((bits >> 23) & 0xff) - 126 : 0;
        e = max(-100, min(100, 14 - e));
        S.red[MKS_MAX_BATCH + tid_()] = __int_as_float((127 + e) << 23);
        S.xinv[tid_()] = __int_as_float((127 - e) << 23);
        if (pieces == 2) S.xinv[M + tid_()] = __int_as_float((127 - e) << 23);
    }
    consumer_sync();
    prof_mark(S, 6);
    if (pieces == 2) {
        // at most 16 values per thread (checked by the host): read the fp32 copies, then overwrite them with the pieces
        float v[16];
        int n = 0;
#pragma unroll 1
        for (int idx = tid_(); idx < M * kc && n < 16; idx += NCT, n++) {
            const int m = idx / kc, k = idx - m * kc;
            v[n] = *reinterpret_cast<const float*>(S.xs() + (size_t)(2 * m) * stride + (size_t)k * 4) * S.red[MKS_MAX_BATCH + m];
        }
        consumer_sync();
        n = 0;
#pragma unroll 1
        for (int idx = tid_(); idx < M * kc && n < 16; idx += NCT, n++) {
            const int m = idx / kc, k = idx - m * kc;
            const __half hi = __float2half_rn(v[n]);
            reinterpret_cast<__half*>(S.xs() + (size_t)m * stride)[k] = hi;
            reinterpret_cast<__half*>(S.xs() + (size_t)(M + m) * stride)[k] = __float2half_rn(v[n] - __half2float(hi));
        }
        return;
    }
    // bf16 -> scaled fp16 in place, eight values per thread and turn
    const int k8n = kc >> 3;
#pragma unroll 1
    for (int idx = tid_(); idx < M * k8n; idx += NCT) {
        const int m = idx / k8n, k8 = idx - m * k8n;
        uint4* pq = reinterpret_cast<uint4*>(S.xs() + (size_t)m * stride) + k8;
        const uint4 q = *pq;
        const float sc = S.red[MKS_MAX_BATCH + m];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 h = __floats2half2_rn(bf_lo(w[i]) * sc, bf_hi(w[i]) * sc);
            o[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *pq = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---- tensor-parallel all-reduce of one output tile -------------------------------------------------------------
// Mailbox of a rank: [2 halves][MAILBOX_TILES][ranks][128] 64-bit words (value | tag << 32), then the key
// exchange area [2][ranks][8][2].  Each lane owns four words of the tile.
__device__ __forceinline__ bool allreduce_tile(Shared& S, Mut& mu, const Args& A, u64 seq, int tile, float (&acc)[4]) {
    const uint32_t tag = (uint32_t)seq;
    const size_t base = (((size_t)(seq & 1) * MAILBOX_TILES + tile) * MKS_MAX_RANKS);
#pragma unroll 1
    for (int r = 0; r < A.tp; r++) {
        unsigned long long* dst = A.mailbox[r] + (base + A.rank) * 128 + lane_() * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) st_relaxed_sys_u64(dst + i, ((u64)tag << 32) | __float_as_uint(acc[i]));
    }
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int r = 0; r < A.tp; r++) {
        const unsigned long long* src = A.mailbox[A.rank] + (base + r) * 128 + lane_() * 4;
        u64 w[4];
        Spin2 s;
        bool fail = false;
#pragma unroll 1
        for (;;) {                                               // the warp leaves together
            bool ok = true;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                w[i] = ld_relaxed_sys_u64(src + i);
                ok = ok && (uint32_t)(w[i] >> 32) == tag;
            }
            if (__all_sync(0xffffffffu, ok)) break;
            if (!ok && MKS_SPIN_FAIL(S, s, WS_MAILBOX)) fail = true;
            if (__any_sync(0xffffffffu, fail)) {
                mu.dead = true;
                return false;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) sum[i] += __uint_as_float((uint32_t)w[i]);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) acc[i] = sum[i];
    return true;
}

// ---- GEMV stage (consumers) ----------------------------------------------------------------------------------
// Lane (g = lane / 4, t = lane % 4) of the warp that owns a unit holds, per tile step, 8 bytes of row g
// and 8 bytes of row g + 8: the values that MMA j of the step multiplies with input columns
// k0 + 16 j + 4 t + {0, 1, 2, 3}.  Its accumulators are rows g, g + 8 x sequences 2t, 2t + 1.
struct Best2 {
    u64 k0 = 0, k1 = 0;
};

// The hot loop is a function of its own with a handful of scalar arguments: inlined into the stage function it
// shared that function's register budget (96 with 17 warps resident) and spilled inside the loop, and spilled
// registers of 544 threads do not fit the L1 that the shared-memory carve-out leaves.
struct UnitGeo {
    int n_chunks, chunk_steps;
};
template <int FMT>
__device__ __noinline__ float4 unit_steps(Shared& S, UnitGeo gm, uint32_t chunk0, const uint8_t* xcol, bool col_live, bool blocks) {
    constexpr int MMAS = FMT == MKS_FMT_MXFP4 ? 4 : (FMT == MKS_FMT_BF16 ? 1 : 2);
    const int g = lane_() >> 2, t = lane_() & 3;
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};    // two chains: consecutive MMAs never wait for each other
    float tmp[4] = {0.f, 0.f, 0.f, 0.f}, tmp2[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t depth = (uint32_t)S.A.ring_depth;
    int kstep = 0;                                            // tile step inside the unit
#pragma unroll 1
    for (int ch = 0; ch < gm.n_chunks; ch++) {
        const uint32_t qq = chunk0 + (uint32_t)ch;               // this warp's chunk counter
        const int slot = warp_() * (int)depth + (int)(qq % depth);
        if (!mbar_wait2(S, &S.full[slot], (qq / depth) & 1, WS_FULL)) break;
        const uint8_t* sl = S.ring() + (size_t)slot * SLOT_BYTES;
        const uint8_t* sc_base = sl + gm.chunk_steps * 512;
#pragma unroll 4
        for (int st = 0; st < gm.chunk_steps; st++, kstep++) {
            const uint4 wq = *reinterpret_cast<const uint4*>(sl + st * 512 + lane_() * 16);
            const uint8_t* xk = xcol + (size_t)kstep * (MMAS * 16) * 2 + t * 8;
            if (FMT == MKS_FMT_MXFP4) {
                // The conversion unit (cvt ... e2m1x2) is the scarcest pipe of this loop, so only half of the
                // values go through it.  The 32 columns of scale group 0 (MMAs 0 and 1) arrive with their bits
                // pre-arranged by the packer: every 32-bit word yields four f16x2 registers with shifts and masks
                // alone (sign at bit 15, the three magnitude bits at 11..9 of each half: the value times 2^-14,
                // which the group's scale takes back).  Scale group 1 (MMAs 2 and 3) keeps plain nibbles.
                const uint32_t scw = *reinterpret_cast<const uint32_t*>(sc_base + st * 32 + g * 4);
                float t0[4] = {0.f, 0.f, 0.f, 0.f}, t1[4] = {0.f, 0.f, 0.f, 0.f};      // scale group 0: MMAs 0, 1
                float u0[4] = {0.f, 0.f, 0.f, 0.f}, u1[4] = {0.f, 0.f, 0.f, 0.f};      // scale group 1: MMAs 2, 3
                uint2 b[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    b[j] = make_uint2(0u, 0u);
                    if (col_live) b[j] = *reinterpret_cast<const uint2*>(xk + j * 32);
                }
                {
                    const uint32_t lo = wq.x, hi = wq.z;                  // row g, row g + 8
                    uint32_t a[4];
                    a[0] = lo & 0x8E008E00u;
                    a[1] = hi & 0x8E008E00u;
                    a[2] = (lo << 3) & 0x8E008E00u;
                    a[3] = (hi << 3) & 0x8E008E00u;
                    mma_f16(t0, a, b[0].x, b[0].y);
                    a[0] = ((lo << 1) & 0x80008000u) | ((lo << 6) & 0x0E000E00u);
                    a[1] = ((hi << 1) & 0x80008000u) | ((hi << 6) & 0x0E000E00u);
                    a[2] = ((lo << 2) & 0x80008000u) | ((lo << 9) & 0x0E000E00u);
                    a[3] = ((hi << 2) & 0x80008000u) | ((hi << 9) & 0x0E000E00u);
                    mma_f16(t1, a, b[1].x, b[1].y);
                }
                {
                    const uint32_t lo = wq.y, hi = wq.w;
                    uint32_t a[4];
                    a[0] = cvt_e2m1x2(lo);
                    a[2] = cvt_e2m1x2(lo >> 8);
                    a[1] = cvt_e2m1x2(hi);
                    a[3] = cvt_e2m1x2(hi >> 8);
                    mma_f16(u0, a, b[2].x, b[2].y);
                    a[0] = cvt_e2m1x2(lo >> 16);
                    a[2] = cvt_e2m1x2(lo >> 24);
                    a[1] = cvt_e2m1x2(hi >> 16);
                    a[3] = cvt_e2m1x2(hi >> 24);
                    mma_f16(u1, a, b[3].x, b[3].y);
                }
                // e8m0 scales: bytes [row g: group 0, group 1, row g + 8: group 0, group 1]; group 0 also takes 2^14
                const float s00 = __uint_as_float(((scw & 0xFFu) + 14u) << 23), s01 = __uint_as_float(((scw >> 8) & 0xFFu) << 23);
                const float s10 = __uint_as_float((((scw >> 16) & 0xFFu) + 14u) << 23), s11 = __uint_as_float((scw >> 24) << 23);
                acc[0] = fmaf(t0[0] + t1[0], s00, acc[0]); acc[1] = fmaf(t0[1] + t1[1], s00, acc[1]);
                acc[2] = fmaf(t0[2] + t1[2], s10, acc[2]); acc[3] = fmaf(t0[3] + t1[3], s10, acc[3]);
                acc[0] = fmaf(u0[0] + u1[0], s01, acc[0]); acc[1] = fmaf(u0[1] + u1[1], s01, acc[1]);
                acc[2] = fmaf(u0[2] + u1[2], s11, acc[2]); acc[3] = fmaf(u0[3] + u1[3], s11, acc[3]);
            } else if (FMT == MKS_FMT_FP8) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const uint32_t lo = j == 0 ? wq.x : wq.y, hi = j == 0 ? wq.z : wq.w;
                    uint32_t a[4];
                    a[0] = cvt_e4m3x2(lo);
                    a[2] = cvt_e4m3x2(lo >> 16);
                    a[1] = cvt_e4m3x2(hi);
                    a[3] = cvt_e4m3x2(hi >> 16);
                    uint2 b = make_uint2(0u, 0u);
                    if (col_live) b = *reinterpret_cast<const uint2*>(xk + j * 32);
                    if (blocks) mma_f16(j == 0 ? tmp : tmp2, a, b.x, b.y);
                    else mma_f16(j == 0 ? acc : acc2, a, b.x, b.y);
                }
                if (blocks && (kstep & 3) == 3) {
                    // one scale per 128 k for rows 0-7 of the tile and one for rows 8-15 (a GLU tile pairs two matrices)
                    const float2 bs = *reinterpret_cast<const float2*>(sc_base + (st >> 2) * 8);
                    acc[0] = fmaf(tmp[0] + tmp2[0], bs.x, acc[0]); acc[1] = fmaf(tmp[1] + tmp2[1], bs.x, acc[1]);
                    acc[2] = fmaf(tmp[2] + tmp2[2], bs.y, acc[2]); acc[3] = fmaf(tmp[3] + tmp2[3], bs.y, acc[3]);
                    tmp[0] = tmp[1] = tmp[2] = tmp[3] = 0.f;
                    tmp2[0] = tmp2[1] = tmp2[2] = tmp2[3] = 0.f;
                }
            } else if (FMT == MKS_FMT_INT8) {
                const uint32_t x0 = wq.x ^ 0x80808080u, x1 = wq.y ^ 0x80808080u, x2 = wq.z ^ 0x80808080u, x3 = wq.w ^ 0x80808080u;
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const uint32_t lo = j == 0 ? x0 : x1, hi = j == 0 ? x2 : x3;
                    uint32_t a[4];
                    a[0] = cvt_s8x2(lo, 0x4140);
                    a[2] = cvt_s8x2(lo, 0x4342);
                    a[1] = cvt_s8x2(hi, 0x4140);
                    a[3] = cvt_s8x2(hi, 0x4342);
                    uint2 b = make_uint2(0u, 0u);
                    if (col_live) b = *reinterpret_cast<const uint2*>(xk + j * 32);
                    mma_f16(j == 0 ? acc : acc2, a, b.x, b.y);
                }
            } else {
                uint32_t a[4] = {wq.x, wq.z, wq.y, wq.w};                 // row g: (x, y), row g + 8: (z, w)
                uint2 b = make_uint2(0u, 0u);
                if (col_live) b = *reinterpret_cast<const uint2*>(xk);
                if (st & 1) mma_bf16(acc2, a, b.x, b.y);
                else mma_bf16(acc, a, b.x, b.y);
            }
        }
        __syncwarp();
        if (lane_() == 0) mbar_arrive(&S.empty[slot]);
    }
    return make_float4(acc[0] + acc2[0], acc[1] + acc2[1], acc[2] + acc2[2], acc[3] + acc2[3]);
}

__device__ __noinline__ void gemv_stage(Shared& S, Mut& mu, const mk_stage_desc& d, const Args& A, u64& ar_seq) {
    const Gemv gm = gemv_geometry(S, d);
    const int fmt = d.i[MKS_I_FMT], epi = d.i[MKS_I_EPILOGUE], pieces = d.i[MKS_I_PIECES];
    const int kc = d.i[MKS_I_KC];
    const int stride = xs_stride_bytes(kc);
    const int g = lane_() >> 2, t = lane_() & 3;
    const int ncols = S.A.M * pieces;
    const bool reduce_groups = d.i[MKS_I_REDUCE_GROUPS] != 0;
    const int arrivals = reduce_groups ? gm.G * gm.S : gm.S;
    const bool ar = d.i[MKS_I_ALLREDUCE] != 0 && A.tp > 1;
    if (ar) ar_seq++;
    unsigned* cnt = reinterpret_cast<unsigned*>(d.p[MKS_P_CNT]);
    float* part = reinterpret_cast<float*>(d.p[MKS_P_PART]);
    Best2 best;
#pragma unroll 1
    for (int pu = gm.u0; pu < gm.u1;) {
        const int panel = pu / gm.T;
        const int pend = min(gm.u1, (panel + 1) * gm.T);
        const int grp = (int)(panel / gm.S), split = (int)(panel % gm.S);
        consumer_sync();                                     // everybody is done reading the previous panel's input
        stage_x(S, mu, d, grp, split);
        consumer_sync();
        if (pu == gm.u0) prof_mark(S, 1);
        const float* rs = group_row_scale(S, d, grp, gm.G);
#pragma unroll 1
        for (int r0 = pu; r0 < pend; r0 += NCW) {
            const int nj = min(NCW, pend - r0);
            if (warp_() < nj && !mu.dead) {
                const int tile = (int)((r0 + warp_()) - panel * gm.T);
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const uint8_t* xcol = S.xs() + (size_t)g * stride;
                const bool live = g < ncols;
                const uint32_t chunk0 = mu.chunk_n;
                UnitGeo ug;
                ug.n_chunks = gm.n_chunks;
                ug.chunk_steps = gm.chunk_steps;
                const bool blocks = d.i[MKS_I_BLOCK_SCALES] != 0;
                float4 r;
                switch (fmt) {
                    case MKS_FMT_MXFP4: r = unit_steps<MKS_FMT_MXFP4>(S, ug, chunk0, xcol, live, blocks); break;
                    case MKS_FMT_FP8: r = unit_steps<MKS_FMT_FP8>(S, ug, chunk0, xcol, live, blocks); break;
                    case MKS_FMT_INT8: r = unit_steps<MKS_FMT_INT8>(S, ug, chunk0, xcol, live, blocks); break;
                    default: r = unit_steps<MKS_FMT_BF16>(S, ug, chunk0, xcol, live, blocks); break;
                }
                acc[0] = r.x; acc[1] = r.y; acc[2] = r.z; acc[3] = r.w;
                // undo the input scaling, fold the second piece's columns onto the first
                acc[0] *= S.xinv[2 * t]; acc[2] *= S.xinv[2 * t];
                acc[1] *= S.xinv[2 * t + 1]; acc[3] *= S.xinv[2 * t + 1];
                if (pieces == 2) {
                    // columns [0, M) + columns [M, 2M): lane t holds columns 2t, 2t + 1
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int col = 2 * t + (i & 1);
                        const int src_col = col + S.A.M;                      // the partner column, if col < M
                        const float other = __shfl_sync(0xffffffffu, acc[i], (lane_() & ~3) | ((src_col >> 1) & 3));
                        const float other1 = __shfl_sync(0xffffffffu, acc[i ^ 1], (lane_() & ~3) | ((src_col >> 1) & 3));
                        const float add = (src_col & 1) == (i & 1) ? other : other1;
                        if (col < S.A.M) acc[i] += add;
                    }
                }
                if (rs) {
                    const float s0 = rs[tile * 16 + g], s1 = rs[tile * 16 + g + 8];
                    acc[0] *= s0; acc[1] *= s0; acc[2] *= s1; acc[3] *= s1;
                }
                bool finish = true;
                const int cidx = reduce_groups ? tile : grp * gm.T + tile;
                if (arrivals > 1) {
                    const int aslot = reduce_groups ? grp * gm.S + split : split;
                    float4* pp = reinterpret_cast<float4*>(part + ((size_t)cidx * arrivals + aslot) * 128) + lane_();
                    __stcg(pp, make_float4(acc[0], acc[1], acc[2], acc[3]));
                    fence_acq_rel_gpu();
                    __syncwarp();
                    unsigned old = 0;
                    if (lane_() == 0) {
                        chaos_delay();
                        old = atomicAdd(cnt + cidx, 1u);
                        // the last arriver puts the counter back: the number of arrivals of a routed stage changes
                        // from step to step, and nobody touches the counter again before the stage's barrier
                        if (old + 1u == (unsigned)arrivals) cnt[cidx] = 0u;
                    }
                    old = __shfl_sync(0xffffffffu, old, 0);
                    finish = old + 1u == (unsigned)arrivals;
                    if (finish) {
                        fence_acq_rel_gpu();
                        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                        // eight partial tiles are requested at a time, then added in arrival-slot order
#pragma unroll 1
                        for (int a0 = 0; a0 < arrivals; a0 += 8) {
                            float4 v[8];
#pragma unroll
                            for (int u = 0; u < 8; u++)
                                if (a0 + u < arrivals)
                                    v[u] = __ldcg(reinterpret_cast<const float4*>(part + ((size_t)cidx * arrivals + a0 + u) * 128) + lane_());
#pragma unroll
                            for (int u = 0; u < 8; u++)
                                if (a0 + u < arrivals) {
                                    float c0 = 1.f, c1 = 1.f;
                                    if (reduce_groups) {
                                        c0 = S.coef[((a0 + u) / gm.S) * 8 + 2 * t];
                                        c1 = S.coef[((a0 + u) / gm.S) * 8 + 2 * t + 1];
                                    }
                                    acc[0] = fmaf(v[u].x, c0, acc[0]); acc[1] = fmaf(v[u].y, c1, acc[1]);
                                    acc[2] = fmaf(v[u].z, c0, acc[2]); acc[3] = fmaf(v[u].w, c1, acc[3]);
                                }
                        }
                    }
                } else if (reduce_groups) {
                    acc[0] *= S.coef[2 * t]; acc[2] *= S.coef[2 * t];
                    acc[1] *= S.coef[2 * t + 1]; acc[3] *= S.coef[2 * t + 1];
                }
                if (finish && ar) finish = allreduce_tile(S, mu, A, ar_seq, tile, acc);
                if (finish) {
                    // rows g, g + 8 of the tile x sequences 2t, 2t + 1
                    const int ostride = d.i[MKS_I_OUT_STRIDE];
                    const int ogrp = reduce_groups ? 0 : grp;
                    float* out = reinterpret_cast<float*>(d.p[MKS_P_OUT]) + (size_t)ogrp * d.i[MKS_I_OUT_GSTRIDE];
                    const int nvalid = d.i[MKS_I_N_VALID];
                    const int m0 = 2 * t, m1 = 2 * t + 1;
                    if (epi == MKS_E_STORE) {
                        const int ra = tile * 16 + g, rb = ra + 8;
                        if (m0 < S.A.M) {
                            if (ra < nvalid) __stcg(out + (size_t)m0 * ostride + ra, acc[0]);
                            if (rb < nvalid) __stcg(out + (size_t)m0 * ostride + rb, acc[2]);
                        }
                        if (m1 < S.A.M) {
                            if (ra < nvalid) __stcg(out + (size_t)m1 * ostride + ra, acc[1]);
                            if (rb < nvalid) __stcg(out + (size_t)m1 * ostride + rb, acc[3]);
                        }
                        float* ssq = reinterpret_cast<float*>(d.p[MKS_P_OUT_SSQ]);
                        if (ssq) {                              // the sums of squares a later norm of this vector needs (whole tiles only)
                            float q0 = acc[0] * acc[0] + acc[2] * acc[2], q1 = acc[1] * acc[1] + acc[3] * acc[3];
#pragma unroll
                            for (int o = 4; o < 32; o <<= 1) {
                                q0 += __shfl_xor_sync(0xffffffffu, q0, o);
                                q1 += __shfl_xor_sync(0xffffffffu, q1, o);
                            }
                            if (g == 0) {
                                const int ntile = nvalid / 16;
                                if (m0 < S.A.M) __stcg(ssq + (size_t)m0 * ntile + tile, q0);
                                if (m1 < S.A.M) __stcg(ssq + (size_t)m1 * ntile + tile, q1);
                            }
                        }
                    } else if (epi == MKS_E_RESID) {
                        const int ra = tile * 16 + g, rb = ra + 8;
                        float* ssq = reinterpret_cast<float*>(d.p[MKS_P_OUT_SSQ]);
                        float q0 = 0.f, q1 = 0.f;
                        if (m0 < S.A.M) {
                            const float a = ldcg_f(out + (size_t)m0 * ostride + ra) + acc[0];
                            const float b = ldcg_f(out + (size_t)m0 * ostride + rb) + acc[2];
                            __stcg(out + (size_t)m0 * ostride + ra, a);
                            __stcg(out + (size_t)m0 * ostride + rb, b);
                            q0 = a * a + b * b;
                        }
                        if (m1 < S.A.M) {
                            const float a = ldcg_f(out + (size_t)m1 * ostride + ra) + acc[1];
                            const float b = ldcg_f(out + (size_t)m1 * ostride + rb) + acc[3];
                            __stcg(out + (size_t)m1 * ostride + ra, a);
                            __stcg(out + (size_t)m1 * ostride + rb, b);
                            q1 = a * a + b * b;
                        }
                        // sum over the eight lanes that share t (the 16 rows of the tile), in a fixed order
#pragma unroll
                        for (int o = 4; o < 32; o <<= 1) {
                            q0 += __shfl_xor_sync(0xffffffffu, q0, o);
                            q1 += __shfl_xor_sync(0xffffffffu, q1, o);
                        }
                        if (g == 0 && ssq) {
                            const int ntile = nvalid / 16;
                            if (m0 < S.A.M) __stcg(ssq + (size_t)m0 * ntile + tile, q0);
                            if (m1 < S.A.M) __stcg(ssq + (size_t)m1 * ntile + tile, q1);
                        }
                    } else if (epi == MKS_E_GLU) {
                        const int r = tile * 8 + g;
                        const bool gelu = d.i[MKS_I_ACT] == MKS_ACT_GELU_TANH;
                        if (r < nvalid) {
                            if (m0 < S.A.M) __stcg(out + (size_t)m0 * ostride + r, (gelu ? gelu_tanh_f(acc[0]) : silu_f(acc[0])) * acc[2]);
                            if (m1 < S.A.M) __stcg(out + (size_t)m1 * ostride + r, (gelu ? gelu_tanh_f(acc[1]) : silu_f(acc[1])) * acc[3]);
                        }
                    } else {   // MKS_E_LOGITS
                        const float cap = d.f[MKS_F_SOFTCAP];
                        const int row_base = (int)d.p[MKS_P_ROW_BASE];
                        const int ra = tile * 16 + g, rb = ra + 8;
                        float v[4] = {acc[0], acc[1], acc[2], acc[3]};
                        if (cap > 0.f) {
#pragma unroll
                            for (int i = 0; i < 4; i++) v[i] = cap * tanhf(v[i] / cap);
                        }
                        if (m0 < S.A.M) {
                            if (ra < nvalid) { __stcg(out + (size_t)m0 * ostride + ra, v[0]); const u64 k = score_key(v[0], row_base + ra); best.k0 = k > best.k0 ? k : best.k0; }
                            if (rb < nvalid) { __stcg(out + (size_t)m0 * ostride + rb, v[2]); const u64 k = score_key(v[2], row_base + rb); best.k0 = k > best.k0 ? k : best.k0; }
                        }
                        if (m1 < S.A.M) {
                            if (ra < nvalid) { __stcg(out + (size_t)m1 * ostride + ra, v[1]); const u64 k = score_key(v[1], row_base + ra); best.k1 = k > best.k1 ? k : best.k1; }
                            if (rb < nvalid) { __stcg(out + (size_t)m1 * ostride + rb, v[3]); const u64 k = score_key(v[3], row_base + rb); best.k1 = k > best.k1 ? k : best.k1; }
                        }
                    }
                }
            }
            if (warp_() < nj) mu.chunk_n += (uint32_t)gm.n_chunks;
        }
        pu = pend;
    }
    prof_mark(S, 2);
    if (epi == MKS_E_LOGITS) {
        // best key of every sequence over this CTA's rows -> keys[m][cta]
        if (tid_() < 8) S.keys_s[tid_()] = 0;
        consumer_sync();
        if (best.k0) atomicMax(reinterpret_cast<unsigned long long*>(&S.keys_s[2 * t]), best.k0);
        if (best.k1) atomicMax(reinterpret_cast<unsigned long long*>(&S.keys_s[2 * t + 1]), best.k1);
        consumer_sync();
        u64* keys = reinterpret_cast<u64*>(d.p[MKS_P_KEYS]);
        if (tid_() < S.A.M) __stcg(reinterpret_cast<unsigned long long*>(keys + (size_t)tid_() * grid_() + cta_()), (unsigned long long)S.keys_s[tid_()]);
    }
}

}  // namespace mks
