// Persistent decode megakernel for sm_100a: one CTA per SM, one launch for many decode steps.
//
// Each CTA has one producer warp and NCW consumer warps.  The producer's elected lane walks this
// CTA's row slice of every weight matrix in execution order and streams it into a shared-memory
// ring with 1-D bulk copies that complete on mbarriers.  It never looks at activations, so the
// weights of the next ops are already in shared memory while the consumers wait for the previous
// op's outputs.  The consumers run the ops:
//
//   A  in-projection   RMSNorm prologue, GEMV, raw outputs published
//   B  mixer           Gated DeltaNet recurrence (conv1d + delta rule) or split-K attention
//   C  out-projection  gated-norm / sigmoid-gate prologue, GEMV, residual add
//   D  gate/up         RMSNorm prologue, GEMV, SwiGLU
//   E  down            GEMV, residual add
//   LM head            final RMSNorm, GEMV over the vocabulary slice, per-CTA best key
//
// Activations cross CTAs as 64-bit words carrying (epoch << 32 | fp32 bits): a reader spins on the
// word itself until it shows the epoch of the op that produces it, so one L2 round trip replaces a
// grid barrier.  A word is only rewritten by an op that transitively depends on every reader of
// the previous value, so no word is overwritten while still needed.
//
// Every wait is bounded: a wait that runs out records MK_ERR_TIMEOUT in the status words, after
// which every wait in every CTA returns at once, ops are skipped, the producer waits (bounded)
// for its copies in flight and the kernel returns.
#pragma once
#include "mk_device.cuh"

namespace mk {

constexpr int ERR_TIMEOUT = -2;

// wait sites (reported in status[1])
enum { W_FULL = 1, W_EMPTY, W_X, W_PROJ, W_MIX, W_ACT, W_LM, W_PART, W_DRAIN };

struct Smem {
    uint8_t* ring;
    uint8_t* xq;        // GEMV input as byte planes (int8 digits or bf16 pieces), or mixer scratch
    float* part_s;      // per-warp partial row sums: [NCW][T][64], or two alternating [NCW][T][32] halves when streaming
    int* bt_s;          // block table copy [max_seq / KV_BLOCK]
    float* out_s;       // small per-op scratch (attention statistics)
    float* red_s;       // block-reduction scratch, two alternating halves of up to 8 * NCW floats
    float* xown;        // fp32 master copy of the residual rows this CTA owns, [T][16]
    u64* best_s;        // [NCW] block-reduction scratch for 64-bit keys
    float* scale_s;     // per-row scales: two 128-row buffers for layer GEMVs, then the streaming ring
    float* xscale_s;    // [T] power-of-two factors that undo the fixed-point scaling of the staged inputs
    float* act_s;       // [T][DOWN_K] this CTA's SwiGLU outputs (entries past its slice stay zero)
    float* mix_s;       // [T][DOWN_K] this DeltaNet task's gated outputs (16 value columns, the rest zero)
    float* ssq_s;       // batched decoding: [sequence][NCW] per-warp sums of squares of the RMSNorm input staged last
    float* wsc_s;       // batched decoding: [NCW][sequence] inverse fixed-point scales of each warp's k-slice
    uint64_t* full;     // [ring stages]
    uint64_t* empty;    // [ring stages]
    volatile int* abort_flag;
    volatile int* quit_flag;
};

struct Ctx {
    Smem sm;
    int tid, warp, lane, cta, grid;
    uint32_t cons_n;    // ring chunks consumed so far
    uint32_t red_n;     // block reductions done so far (selects the scratch half)
    u64 limit_ns;
    int* status;
    bool dead;          // this thread saw a wait run out
    u64* prof;          // this CTA's timestamp rows for the step being profiled, or null
    u64 wait_acc;       // time consumer thread 0 spent waiting for ring chunks in the current op
    int cur_op;         // op index being traced (trace builds)
    uint32_t gemv_n;    // layer GEMVs run so far (selects the scale buffer)
};

// Per-op timestamps (enter, inputs staged, work done, outputs published), consumer thread 0 only.
__device__ __forceinline__ void prof_stamp(Ctx& c, int op, int field) {
    if (field == 0) c.cur_op = op;
    if (c.prof && c.tid == 0) {
        c.prof[(size_t)op * PROF_FIELDS + field] = globaltimer();
        if (field == 3) {
            c.prof[(size_t)op * PROF_FIELDS + 4] = c.wait_acc;
            c.wait_acc = 0;
        }
    }
}

struct Spin {
    uint32_t it = 0;
    u64 t0 = 0;
};
constexpr u64 SPIN_FAILED = ~0ull;

// Slow path of every spin loop, entered once per 256 polls.  Takes and returns the time of the
// loop's first visit by value: a `Spin` whose address went to a function that is not inlined would
// live in local memory, and every poll of every loop would then load and store it there.
__device__ __noinline__ u64 spin_slow(volatile int* abort_flag, int* status, u64 limit_ns, u64 t0, int where) {
    if (*abort_flag) return SPIN_FAILED;
    if (ld_volatile_i32(status) != 0) {
        *abort_flag = 1;
        return SPIN_FAILED;
    }
    const u64 now = globaltimer();
    if (!t0) {
        t0 = now;
    } else if (now - t0 > limit_ns) {
        if (atomicCAS(status, 0, ERR_TIMEOUT) == 0) {
            status[1] = where;
            status[2] = (int)blockIdx.x;
            status[3] = (int)threadIdx.x;
        }
        __threadfence();
        *abort_flag = 1;
        return SPIN_FAILED;
    }
    __nanosleep(40);
    return t0;
}
#define MK_SPIN_FAIL(c, s, where)          \
    ((((++(s).it) & 255u) == 0) &&         \
     (((s).t0 = spin_slow((c).sm.abort_flag, (c).status, (c).limit_ns, (s).t0, (where))) == SPIN_FAILED))

__device__ __forceinline__ void mbar_wait(Ctx& c, uint64_t* b, uint32_t parity, int where) {
    Spin s;
    while (!mbar_try_wait(b, parity)) {
        if (MK_SPIN_FAIL(c, s, where)) {
            c.dead = true;
            break;
        }
    }
}

#ifdef MK_TRACE
#define MK_MARK(c, idx) do { if ((c).prof && (c).tid == 0) (c).prof[(size_t)(c).cur_op * PROF_FIELDS + (idx)] = globaltimer(); } while (0)
#else
#define MK_MARK(c, idx) do { } while (0)
#endif

// Pause between two polls of a word that is not ready.  Thousands of threads poll the same few
// cache lines; without a pause their loads queue up in front of the store they are waiting for.
#ifndef MK_POLL_SLEEP_NS
#define MK_POLL_SLEEP_NS 0
#endif
#ifndef MK_POLL_FREE_SPINS
#define MK_POLL_FREE_SPINS 2
#endif
__device__ __forceinline__ void poll_backoff(uint32_t polls_so_far) {
    if (MK_POLL_SLEEP_NS > 0 && polls_so_far >= MK_POLL_FREE_SPINS) __nanosleep(MK_POLL_SLEEP_NS);
}

// Wait until the word shows `epoch`; returns its fp32 payload.
__device__ __forceinline__ float ll_wait(Ctx& c, const u64* p, uint32_t epoch, int where) {
    Spin s;
    u64 w = ll_load(p);
    while ((uint32_t)(w >> 32) != epoch) {
        if (MK_SPIN_FAIL(c, s, where)) {
            c.dead = true;
            break;
        }
        poll_backoff(s.it);
        w = ll_load(p);
    }
    return __uint_as_float((uint32_t)w);
}
__device__ __forceinline__ void ll_wait2(Ctx& c, const u64* p, uint32_t epoch, int where, float& a, float& b) {
    Spin s;
    u64 w0, w1;
    ll_load2(p, w0, w1);
    while ((uint32_t)(w0 >> 32) != epoch || (uint32_t)(w1 >> 32) != epoch) {
        if (MK_SPIN_FAIL(c, s, where)) {
            c.dead = true;
            break;
        }
        poll_backoff(s.it);
        ll_load2(p, w0, w1);
    }
    a = __uint_as_float((uint32_t)w0);
    b = __uint_as_float((uint32_t)w1);
}

// Wait for N word pairs at once: all loads are issued before any is checked, and only the pairs that
// are not ready are loaded again, so a thread that needs several pairs pays one round trip, not N.
template <int N>
__device__ __forceinline__ void ll_wait_pairs(Ctx& c, const u64* const (&p)[N], const uint32_t (&e)[N], float (&v)[2 * N],
                                              int where) {
    u64 w[2 * N];
#pragma unroll
    for (int i = 0; i < N; i++)
        if (p[i]) ll_load2(p[i], w[2 * i], w[2 * i + 1]);
    Spin s;
    while (true) {
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; i++)
            if (p[i] && ((uint32_t)(w[2 * i] >> 32) != e[i] || (uint32_t)(w[2 * i + 1] >> 32) != e[i])) {
                ok = false;
                ll_load2(p[i], w[2 * i], w[2 * i + 1]);
            }
        if (ok) break;
        if (MK_SPIN_FAIL(c, s, where)) {
            c.dead = true;
            break;
        }
        poll_backoff(s.it);
    }
#pragma unroll
    for (int i = 0; i < N; i++) {
        v[2 * i] = p[i] ? __uint_as_float((uint32_t)w[2 * i]) : 0.f;
        v[2 * i + 1] = p[i] ? __uint_as_float((uint32_t)w[2 * i + 1]) : 0.f;
    }
}

// The same with the addresses and epochs given as functions of the pair's index, so that a caller whose
// addresses follow from a few bases keeps no pointer array in registers.  addr(i) may be null.
template <int N, class Addr, class Epoch>
__device__ __forceinline__ void ll_wait_pairs_fn(Ctx& c, Addr&& addr, Epoch&& epoch, float (&v)[2 * N], int where) {
    u64 w[2 * N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        w[2 * i] = w[2 * i + 1] = 0;
        if (const u64* p = addr(i)) ll_load2(p, w[2 * i], w[2 * i + 1]);
    }
    Spin s;
    while (true) {
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; i++) {
            const u64* p = addr(i);
            const uint32_t e = epoch(i);
            if (p && ((uint32_t)(w[2 * i] >> 32) != e || (uint32_t)(w[2 * i + 1] >> 32) != e)) {
                ok = false;
                ll_load2(p, w[2 * i], w[2 * i + 1]);
            }
        }
        if (ok) break;
        if (MK_SPIN_FAIL(c, s, where)) {
            c.dead = true;
            break;
        }
        poll_backoff(s.it);
    }
#pragma unroll
    for (int i = 0; i < N; i++) {
        v[2 * i] = __uint_as_float((uint32_t)w[2 * i]);
        v[2 * i + 1] = __uint_as_float((uint32_t)w[2 * i + 1]);
    }
}

// A CTA that had no part in the op it now waits for arrives early.  If all of its threads polled
// right away, their loads would queue in front of the very stores they wait for.  Instead one warp
// watches 32 words spread over the buffer, at a relaxed pace, and releases the CTA when all of them
// show the epoch; the full poll that follows then finds (nearly) everything ready.
__device__ __forceinline__ void gate_on_samples(Ctx& c, const u64* buf, int nwords, uint32_t epoch) {
    if (c.warp == 0) {
        const u64* p = buf + (size_t)c.lane * (nwords / 32) + (nwords / 64);
        Spin s;
        while (true) {
            const bool ready = (uint32_t)(ll_load(p) >> 32) == epoch;
            if (__all_sync(0xffffffffu, ready)) break;
            const bool fail = MK_SPIN_FAIL(c, s, W_MIX);
            if (__any_sync(0xffffffffu, fail)) {      // leave together: the vote above needs every lane
                c.dead = true;
                break;
            }
            __nanosleep(150);
        }
    }
    consumer_sync();
}

// Geometry that depends on how many tokens one pass over the weights serves (1: plain decode,
// 2: a speculative cycle).  Four ring stages (128 KB of weights in flight per SM) measured as fast as
// six: what the ring does not take stays with the L1 cache, which the kernel's few spilled registers
// and its read-only tables need.
template <int T> struct Geo {
#ifndef MK_NS1
#define MK_NS1 4
#endif
#ifndef MK_NS2
#define MK_NS2 4
#endif
    static constexpr int NS = T == 1 ? MK_NS1 : MK_NS2;             // ring stages
    static constexpr int RING = NS * SLOT_BYTES;
    static constexpr int XQ = (T == 1 ? 3 : 7) * 2 * 3584;          // input planes: bf16 pieces of K = 3584 are the largest
    static constexpr int PART = NCW * T * 64 * 4;                   // per-warp partial sums
    static constexpr int SMEM = RING + XQ + PART + MAX_BLOCKS * 4 + 2048 + 2048;
};

// Sums and maxima over all consumer threads in one barrier, fixed order; one pair per token.
template <int T>
__device__ __forceinline__ void consumer_sum_max(Ctx& c, float (&sum)[T], float (&mx)[T]) {
    float* buf = c.sm.red_s + (c.red_n++ & 1) * (2 * T * NCW);
#pragma unroll
    for (int j = 0; j < T; j++) {
        const float a = warp_sum(sum[j]), b = warp_max(mx[j]);
        if (c.lane == 0) {
            buf[(2 * j) * NCW + c.warp] = a;
            buf[(2 * j + 1) * NCW + c.warp] = b;
        }
    }
    consumer_sync();
#pragma unroll
    for (int j = 0; j < T; j++) {
        float t = 0.f, m = 0.f;
#pragma unroll
        for (int i = 0; i < NCW; i++) {
            t += buf[(2 * j) * NCW + i];
            m = fmaxf(m, buf[(2 * j + 1) * NCW + i]);
        }
        sum[j] = t;
        mx[j] = m;
    }
}

// ---- GEMV on the tensor cores ---------------------------------------------------------------------
// A weight row is cut into 64-byte k-blocks (64 int8 or 32 bf16 weights).  Rows are stored in groups
// of up to 8, k-block major: block kb of every row of the group, then block kb + 1, ...  One 128-bit
// load per lane therefore hands a warp an 8-row x 64-byte tile in MMA operand order (lane = 4 * row +
// quarter), with no conversion and no bank conflict.  Two tiles are the 16-row A operand.
//
// The input vector is the B operand.  fp32 inputs are made exact for the tensor cores by splitting:
//   int8 weights: x * 2^s rounded to a 28-bit integer, cut into four base-128 digits (int8 planes);
//                 integer MMAs (s8 x s8 -> s32) are exact, the digits recombine in fp32;
//   bf16 weights: x = p0 + p1 + p2 with three bf16 pieces (24 significant bits); bf16 MMAs with fp32
//                 accumulation.
// Plane 4 * token + piece of the staged input is MMA column 4 * token + piece, so one MMA serves every
// plane of up to two tokens.  Each warp owns a contiguous k-slice of every row of a chunk; per-warp
// partial sums meet in shared memory.
template <bool Q8> struct Planes { static constexpr int N = Q8 ? 4 : 3; };

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Stage two consecutive inputs (elements k, k + 1) of one token into its planes (`xq` points at the
// token's first plane).  `scale` is the power of two that maps the vector's largest magnitude below
// 2^27 (int8 path only).
template <bool Q8>
__device__ __forceinline__ void stage_pair(uint8_t* xq, int rb, int k, float v0, float v1, float scale) {
    if (Q8) {
        const int a = __float2int_rn(v0 * scale), b = __float2int_rn(v1 * scale);
#pragma unroll
        for (int d = 0; d < 4; d++) {
            const int da = d < 3 ? ((a >> (7 * d)) & 127) : (a >> 21);
            const int db = d < 3 ? ((b >> (7 * d)) & 127) : (b >> 21);
            *reinterpret_cast<uint16_t*>(xq + d * rb + k) = (uint16_t)((da & 255) | ((db & 255) << 8));
        }
    } else {
#pragma unroll
        for (int d = 0; d < 3; d++) {
            const __nv_bfloat16 pa = __float2bfloat16_rn(v0), pb = __float2bfloat16_rn(v1);
            v0 -= __bfloat162float(pa);
            v1 -= __bfloat162float(pb);
            *reinterpret_cast<uint32_t*>(xq + d * rb + 2 * k) =
                (uint32_t)__bfloat16_as_ushort(pa) | ((uint32_t)__bfloat16_as_ushort(pb) << 16);
        }
    }
}

// Fixed-point scale for a vector whose largest magnitude is `mx`: 2^(26 - exponent(mx)).
__device__ __forceinline__ float fixed_scale(float mx) {
    int e = (int)((__float_as_uint(mx) >> 23) & 0xff) - 127;
    e = max(-100, min(100, e));
    return __uint_as_float((uint32_t)(127 + 26 - e) << 23);
}

// Per-row scales travel through shared memory so that the warp that finishes rows never stalls on a
// global load: `scale_prefetch` (called when an op is entered, long before its rows finish) fills the
// first 128 rows; the streaming GEMV refills its 8-chunk ring four chunks ahead.
constexpr int SCALE_BODY = 128;                 // rows per body-op buffer (two buffers, alternating)
constexpr int SCALE_RING = 8 * 32;              // streaming ring: 8 chunks of up to 32 rows
__device__ __forceinline__ void scale_prefetch(Ctx& c, const float* __restrict__ row_scale, int r0, int r1,
                                               bool stream) {
    if (!row_scale || c.warp != NCW - 1) return;
    float* dst = stream ? c.sm.scale_s + 2 * SCALE_BODY : c.sm.scale_s + (c.gemv_n & 1) * SCALE_BODY;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = (r0 + c.lane + 32 * i < r1) ? row_scale[r0 + c.lane + 32 * i] : 1.f;
#pragma unroll
    for (int i = 0; i < 4; i++) dst[c.lane + 32 * i] = v[i];
}

// MMAs of one or two 16-row blocks (rows [b0, b0 + 32) of the chunk) over this warp's k-blocks.
// Lane (g, t) holds, per block, rows g and g + 8 for MMA columns 2t and 2t + 1, i.e. two planes of
// token t / 2; after the exchange with lane t ^ 1 it holds that token's finished partial sums.
template <bool Q8>
__device__ __forceinline__ void mma_blocks(const uint8_t* buf, const uint8_t* xrow, bool xlive, int rb, int nkb, int nr,
                                           int b0, int warp, int g, int t, float (&v)[4]) {
    int n8[4];
    const uint8_t* tile[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {               // the four 8-row tiles of the two blocks
        n8[q] = max(0, min(8, nr - b0 - 8 * q));
        tile[q] = buf + (size_t)(b0 + 8 * q) * rb + g * 64 + t * 16;
    }
    int ci[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    float cf[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const bool two = nr - b0 > 16;              // the second block has rows (projections that give a CTA 7 rows have none)
    // a contiguous k-slice per warp: exactly the inputs the warp staged itself (see `stage_rmsnorm`)
    const int kb0 = nkb * warp / NCW, kb1 = nkb * (warp + 1) / NCW;
#pragma unroll 2
    for (int kb = kb0; kb < kb1; kb++) {
        uint4 w[4], x = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            w[q] = make_uint4(0, 0, 0, 0);
            if (g < n8[q]) w[q] = *reinterpret_cast<const uint4*>(tile[q] + (size_t)kb * n8[q] * 64);
        }
        if (xlive) x = *reinterpret_cast<const uint4*>(xrow + kb * 64);
#pragma unroll
        for (int b = 0; b < 2; b++) {           // two independent accumulator chains
            if (b == 1 && !two) continue;
            if (Q8) {
                mma_s8(ci[b], w[2 * b].x, w[2 * b + 1].x, w[2 * b].y, w[2 * b + 1].y, x.x, x.y);
                mma_s8(ci[b], w[2 * b].z, w[2 * b + 1].z, w[2 * b].w, w[2 * b + 1].w, x.z, x.w);
            } else {
                mma_bf16(cf[b], w[2 * b].x, w[2 * b + 1].x, w[2 * b].y, w[2 * b + 1].y, x.x, x.y);
                mma_bf16(cf[b], w[2 * b].z, w[2 * b + 1].z, w[2 * b].w, w[2 * b + 1].w, x.z, x.w);
            }
        }
    }
    const float pw0 = __uint_as_float((uint32_t)(127 + 14 * (t & 1)) << 23);       // 128^(2 * (t & 1)) for the int8 digits
    const float pw1 = pw0 * 128.f;
#pragma unroll
    for (int b = 0; b < 2; b++) {
        float lo, hi;
        if (Q8) {
            lo = (float)ci[b][0] * pw0 + (float)ci[b][1] * pw1;
            hi = (float)ci[b][2] * pw0 + (float)ci[b][3] * pw1;
        } else {
            lo = cf[b][0] + cf[b][1];
            hi = cf[b][2] + cf[b][3];
        }
        v[2 * b] = lo + __shfl_xor_sync(0xffffffffu, lo, 1);
        v[2 * b + 1] = hi + __shfl_xor_sync(0xffffffffu, hi, 1);
    }
}

// Streams this CTA's rows [r0, r1) of a matrix with `rb`-byte rows out of the ring.
//   STREAM = false  (layer GEMVs, at most 64 rows per CTA): one barrier after the last chunk, then
//                   warps 2 * token and 2 * token + 1 finish that token's rows;
//   STREAM = true   (LM head, draft head): one barrier per chunk, warp `token` finishes that token's
//                   rows of the chunk while the other warps move on.
// A finishing warp calls sink(lane, row, token, value, valid) on all of its lanes; `value` already
// carries the row's scale and the input's fixed-point scale.  A layer GEMV ends with one more barrier
// after the sink (`tail_barrier`).
template <bool Q8, int T, bool STREAM, class Sink>
__device__ __forceinline__ void gemv_mma(Ctx& c, int r0, int r1, int rb, const float* __restrict__ row_scale,
                                         Sink&& sink, bool tail_barrier = true) {
    constexpr int NS = Geo<T>::NS;
    const int rpc = SLOT_BYTES / rb;
    const int nkb = rb >> 6;
    const int g = c.lane >> 2, t = c.lane & 3;
    const uint8_t* xrow = c.sm.xq + g * rb + t * 16;                      // plane g = column g of the B operand
    const bool xlive = (g >> 2) < T && (g & 3) < Planes<Q8>::N;
    const int tok = t >> 1;                                               // token whose sums this lane ends up with
    const float* scales = STREAM ? c.sm.scale_s + 2 * SCALE_BODY : c.sm.scale_s + (c.gemv_n & 1) * SCALE_BODY;
    c.gemv_n++;
    float pend = 1.f;                            // scale fetched for the chunk four ahead (STREAM)
    int chunk = 0;
    for (int base = r0; base < r1; base += rpc, chunk++) {
        const int nr = min(rpc, r1 - base);
        const uint32_t n = c.cons_n++;
        const int slot = (int)(n % NS);
        if (STREAM && row_scale && c.warp == NCW - 1) {
            if (chunk > 0) c.sm.scale_s[2 * SCALE_BODY + ((chunk + 3) & 7) * 32 + c.lane] = pend;
            const int r = base + 4 * rpc + c.lane;
            pend = r < r1 ? row_scale[r] : 1.f;
        }
        if (c.prof && c.tid == 0) {
            const u64 t0 = globaltimer();
            mbar_wait(c, &c.sm.full[slot], (n / NS) & 1, W_FULL);
            c.wait_acc += globaltimer() - t0;
        } else {
            mbar_wait(c, &c.sm.full[slot], (n / NS) & 1, W_FULL);
        }
        const uint8_t* buf = c.sm.ring + (size_t)slot * SLOT_BYTES;
        // partial sums [warp][token][row]: 64 rows for layer GEMVs, two alternating 32-row halves when streaming
        float* part = STREAM ? c.sm.part_s + (((n & 1) * NCW + c.warp) * T + tok) * 32
                             : c.sm.part_s + (c.warp * T + tok) * 64 + (base - r0);
        if (base == r0) MK_MARK(c, 8);
        for (int b0 = 0; b0 < nr; b0 += 32) {
            float v[4];
            mma_blocks<Q8>(buf, xrow, xlive, rb, nkb, nr, b0, c.warp, g, t, v);
            if ((t & 1) == 0 && tok < T) {
#pragma unroll
                for (int q = 0; q < 4; q++)
                    if (b0 + 8 * q + g < nr) part[b0 + 8 * q + g] = v[q];
            }
        }
        __syncwarp();
        // A lane whose wait ran out never releases the slot: its copy may still be in flight, and the
        // producer must not aim a second copy at the same shared memory.
        if (c.lane == 0 && !c.dead) mbar_arrive(&c.sm.empty[slot]);
        if (STREAM) {
            consumer_sync();
            if (c.warp < T) {
                const float* pp = c.sm.part_s + ((n & 1) * NCW * T + c.warp) * 32 + c.lane;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < NCW; w++) v += pp[w * T * 32];
                const float rs = row_scale ? scales[(chunk & 7) * 32 + c.lane] : 1.f;
                sink(c.lane, base + c.lane, c.warp, v * rs * c.sm.xscale_s[c.warp], c.lane < nr);
            }
        }
    }
    if (!STREAM) {
        MK_MARK(c, 9);
        consumer_sync();
        MK_MARK(c, 10);
        if (c.warp < 2 * T) {
            const int tk = c.warp >> 1, idx = (c.warp & 1) * 32 + c.lane;
            const float* pp = c.sm.part_s + tk * 64 + idx;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < NCW; w++) v += pp[w * T * 64];
            const float rs = row_scale ? scales[idx] : 1.f;
            sink(c.lane, r0 + idx, tk, v * rs * c.sm.xscale_s[tk], idx < r1 - r0);
            MK_MARK(c, 11);
        }
        // Without a barrier here the other warps run ahead into the next op's prologue and poll for its
        // inputs; their loads then sit in this SM's memory pipeline in front of the stores the finishing
        // warps are about to issue, and every CTA's outputs reach the others later (3 % of the step).
        // A caller that follows up with a barrier of its own passes tail_barrier = false.
        if (tail_barrier) consumer_sync();
    }
}

// ---- producer ----------------------------------------------------------------------------------------
// (The reference also runs a second cursor that asks the L2 for chunks ahead of the copies,
// qwen3.5-0.8b/csrc/megakernel.cu:171-193.  Measured on B200 it gained nothing at any distance -- the ring is
// never what the consumers wait for -- and its bookkeeping in this loop cost a few per cent, so it is not here.)
template <int NS>
struct Producer {
    Ctx& c;
    u64 policy;
    uint32_t n = 0;      // chunks issued
    bool stop = false;

    __device__ Producer(Ctx& c_) : c(c_) { policy = policy_evict_first(); }

    // Issue this CTA's slice of one matrix, one ring slot at a time.
    __device__ void stream(const uint8_t* w, int rows, int unit, int row_bytes) {
        if (stop) return;
        int r0, r1;
        cta_rows(rows, unit, c.cta, c.grid, r0, r1);
        const int rpc = SLOT_BYTES / row_bytes;
        for (int base = r0; base < r1; base += rpc) {
            const int nr = min(rpc, r1 - base);
            const int slot = (int)(n % NS);
            if (n >= NS) {
                const uint32_t par = ((n / NS) - 1) & 1;
                Spin s;
                while (!mbar_try_wait(&c.sm.empty[slot], par)) {
                    if (*c.sm.quit_flag || MK_SPIN_FAIL(c, s, W_EMPTY)) {
                        stop = true;
                        return;
                    }
                }
            }
            if (*c.sm.quit_flag || *c.sm.abort_flag) {
                stop = true;
                return;
            }
            const uint32_t bytes = (uint32_t)nr * (uint32_t)row_bytes;
            mbar_expect_tx(&c.sm.full[slot], bytes);
            bulk_load(c.sm.ring + (size_t)slot * SLOT_BYTES, w + (size_t)base * row_bytes, bytes, &c.sm.full[slot],
                      policy);
            n++;
        }
    }

    // Before the CTA may exit, every copy that was issued must have landed.
    __device__ void drain() {
        const uint32_t first = n > NS ? n - NS : 0;
        for (uint32_t i = first; i < n; i++) {
            Spin s;
            s.t0 = 0;
            while (!mbar_try_wait(&c.sm.full[i % NS], (i / NS) & 1)) {
                // Not abortable by the shared flags: the copy is still writing shared memory.
                if (((++s.it) & 1023u) == 0) {
                    const u64 now = globaltimer();
                    if (!s.t0) s.t0 = now;
                    else if (now - s.t0 > c.limit_ns) {
                        if (atomicCAS(c.status, 0, ERR_TIMEOUT) == 0) c.status[1] = W_DRAIN;
                        break;
                    }
                }
            }
        }
    }
};

// The weight stream of one pass: the four GEMVs of every layer, then the LM head when its output is
// needed; a speculative cycle continues with the draft head's fusion projection, its decoder layer
// and the draft vocabulary rows.  Consumers consume exactly this sequence.
template <class S, bool Q8, int T>
__device__ void producer_main(Ctx& c, const Params& P, const Args& A) {
    Producer<Geo<T>::NS> pr(c);
    constexpr int WB = Q8 ? 1 : 2;  // bytes per weight
    auto layer = [&](const LayerP& L) {
        pr.stream(L.w_in, L.kind ? S::ATT_IN : S::GDN_IN, 1, S::HID * WB);
        if (L.kind) pr.stream(L.w_out, S::HID, 1, S::MIX * WB);
        else if (c.cta < S::GDN_TASKS) pr.stream(L.w_out, (S::HID / 16) * c.grid, S::HID / 16, 512);   // the task's column slice: 64 tiles
        pr.stream(L.w_gu, 2 * S::INTER, 2, S::HID * WB);
        pr.stream(L.w_down, (S::HID / 16) * c.grid, S::HID / 16, 16 * DOWN_K * WB);   // this CTA's column slice: 64 tiles
    };
    for (int s = 0; s < A.n_steps && !pr.stop; s++) {
        for (int l = 0; l < P.n_layers && !pr.stop; l++) layer(P.layer[l]);
        if (T == 2) {
            pr.stream(P.lm_head, P.vocab, 1, S::HID * WB);
            pr.stream(P.mtp_fc, S::HID, 1, 2 * S::HID * WB);
            layer(P.mtp);
            pr.stream(P.draft_head, P.draft_vocab, 1, S::HID * WB);
        } else if (s >= A.lm_from) {
            pr.stream(P.lm_head, P.vocab, 1, S::HID * WB);
        }
    }
    pr.drain();
}

// ---- prologues ---------------------------------------------------------------------------------------
// RMSNorm of T residual vectors into the GEMV input planes.  `x[j]` are this thread's two elements
// (2*tid, 2*tid+1) of token j.  One block reduction yields, per token, the sum of squares and the
// largest |x (1 + w)|, from which the fixed-point scale follows without a second pass.  `y` returns
// the normalised values.
template <class S, bool Q8, int T>
__device__ __forceinline__ void stage_rmsnorm(Ctx& c, const float (&x)[T][2], float2 g, float (&y)[T][2]) {
    static_assert(S::HID == 2 * NCT, "two residual elements per consumer thread");
    constexpr int RB = Q8 ? S::HID : 2 * S::HID;
    const int k = 2 * c.tid;
    float ss[T], mx[T];
#pragma unroll
    for (int j = 0; j < T; j++) {
        y[j][0] = x[j][0] * (1.0f + g.x);
        y[j][1] = x[j][1] * (1.0f + g.y);
        ss[j] = x[j][0] * x[j][0] + x[j][1] * x[j][1];
        mx[j] = fmaxf(fabsf(y[j][0]), fabsf(y[j][1]));
    }
    MK_MARK(c, 6);
    consumer_sum_max<T>(c, ss, mx);
    MK_MARK(c, 7);
#pragma unroll
    for (int j = 0; j < T; j++) {
        const float inv = rsqrtf(ss[j] * (1.0f / S::HID) + S::EPS);
        const float scale = Q8 ? fixed_scale(mx[j] * inv) : 1.0f;
        y[j][0] *= inv;
        y[j][1] *= inv;
        stage_pair<Q8>(c.sm.xq + (size_t)(4 * j) * RB, RB, k, y[j][0], y[j][1], scale);
        if (c.tid == 0) c.sm.xscale_s[j] = 1.0f / scale;
    }
    // No block barrier: a warp stages elements [64 w, 64 w + 64), which is the k-slice it multiplies;
    // the inverse scales are read after the barrier that follows the MMAs.
    __syncwarp();
}

// For inputs that need no norm: per-token fixed-point scales from this thread's largest magnitudes
// (one block reduction on the int8 path, nothing on the bf16 path) ...
template <bool Q8, int T>
__device__ __forceinline__ void block_scale(Ctx& c, float (&mx)[T], float (&scale)[T]) {
    if (Q8) {
        float dummy[T];
#pragma unroll
        for (int j = 0; j < T; j++) dummy[j] = 0.f;
        consumer_sum_max<T>(c, dummy, mx);
    }
#pragma unroll
    for (int j = 0; j < T; j++) scale[j] = Q8 ? fixed_scale(mx[j]) : 1.0f;
}
// ... and the end of a staging phase: publish the inverse scales.  The caller's threads staged 4
// consecutive inputs each, so a warp wrote exactly the k-slice it multiplies: no block barrier.
template <int T>
__device__ __forceinline__ void finish_stage(Ctx& c, const float (&scale)[T]) {
    if (c.tid == 0) {
#pragma unroll
        for (int j = 0; j < T; j++) c.sm.xscale_s[j] = 1.0f / scale[j];
    }
    __syncwarp();
}

// Embedding row of `token` -> this thread's two residual elements.
template <class S, bool Q8>
__device__ __forceinline__ void load_embedding(const Params& P, int token, int tid, float& x0, float& x1) {
    const int k = 2 * tid;
    if (Q8) {
        const uint16_t b = *reinterpret_cast<const uint16_t*>(P.embed + (size_t)token * S::HID + k);
        const float sc = P.embed_scale[token];
        x0 = (float)(int)(signed char)(b & 0xff) * sc;
        x1 = (float)(int)(signed char)(b >> 8) * sc;
    } else {
        const uint32_t b = *reinterpret_cast<const uint32_t*>(P.embed + ((size_t)token * S::HID + k) * 2);
        x0 = bf_lo(b);
        x1 = bf_hi(b);
    }
}

// ---- split-K projection of values that only this CTA holds -------------------------------------------
// `act` ([T][DOWN_K] in shared memory, zero past the CTA's slice) times the CTA's column slice of a
// matrix (S::HID / 16 tiles in fragment order out of the ring, see pack_col_slices): 1024 partial sums
// per token, published as hand-off words `out[token * tok_stride + row]`.  One MMA covers a 16-row
// tile's whole K, so results leave the registers directly: no partial sums in shared memory, no
// barrier.  Every warp derives the B fragments itself.  KM = bf16 MMAs per tile (columns / 16); the
// integer MMA always spans 32 columns.
template <class S, bool Q8, int T, int KM>
__device__ __forceinline__ void partial_cols(Ctx& c, const float* act, u64* out, size_t tok_stride, uint32_t epoch) {
    constexpr int WB = Q8 ? 1 : 2;
    constexpr int TILES = S::HID / 16, TILE_BYTES = Q8 ? 16 * DOWN_K : 16 * 16 * KM * WB, TPC = SLOT_BYTES / TILE_BYTES;
    static_assert(TPC % NCW == 0 && TILES % TPC == 0, "whole rounds of 16 tiles per ring chunk");
    const int g = c.lane >> 2, t = c.lane & 3, tok = g >> 2, piece = g & 3;
    uint32_t bf[Q8 ? 2 : 2 * KM] = {};      // B fragments of plane g = 4 * token + digit / piece
    float inv_scale[T];
#pragma unroll
    for (int j = 0; j < T; j++) {
        const float* a = act + j * DOWN_K;
        const float scale = Q8 ? fixed_scale(warp_max(fabsf(a[c.lane]))) : 1.0f;
        inv_scale[j] = 1.0f / scale;
        if (tok == j && piece < Planes<Q8>::N) {
            if (Q8) {
#pragma unroll
                for (int hf = 0; hf < 2; hf++) {
                    uint32_t pk = 0;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int q = __float2int_rn(a[16 * hf + 4 * t + i] * scale);
                        const int d = piece < 3 ? ((q >> (7 * piece)) & 127) : (q >> 21);
                        pk |= (uint32_t)(d & 255) << (8 * i);
                    }
                    bf[hf] = pk;
                }
            } else {
#pragma unroll
                for (int f = 0; f < 2 * KM; f++) {      // mma f / 2, low or high 8 columns
                    uint32_t pk = 0;
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        float v = a[16 * (f >> 1) + 8 * (f & 1) + 2 * t + i];
                        __nv_bfloat16 pb = __float2bfloat16_rn(v);
#pragma unroll
                        for (int d = 0; d < 2; d++)
                            if (d < piece) {
                                v -= __bfloat162float(pb);
                                pb = __float2bfloat16_rn(v);
                            }
                        pk |= (uint32_t)__bfloat16_as_ushort(pb) << (16 * i);
                    }
                    bf[f] = pk;
                }
            }
        }
    }
    const float pw0 = __uint_as_float((uint32_t)(127 + 14 * (t & 1)) << 23);   // 128^(2 * (t & 1)) for the int8 digits
    const float pw1 = pw0 * 128.f;
    const int otok = t >> 1;                                                     // token whose sums this lane ends up with
    const float os = inv_scale[otok < T ? otok : 0];
    u64* dst = out + (size_t)(otok < T ? otok : 0) * tok_stride;
    for (int base = 0; base < TILES; base += TPC) {
        const uint32_t n = c.cons_n++;
        const int slot = (int)(n % Geo<T>::NS);
        mbar_wait(c, &c.sm.full[slot], (n / Geo<T>::NS) & 1, W_FULL);
        const uint8_t* buf = c.sm.ring + (size_t)slot * SLOT_BYTES;
#pragma unroll
        for (int i = 0; i < TPC / NCW; i++) {
            const int tile = c.warp + NCW * i;
            const uint8_t* wt = buf + (size_t)tile * TILE_BYTES + c.lane * (Q8 ? 16 : 16 * KM);
            float lo, hi;
            if (Q8) {
                const uint4 w0 = *reinterpret_cast<const uint4*>(wt);
                int ci[4] = {0, 0, 0, 0};
                mma_s8(ci, w0.x, w0.y, w0.z, w0.w, bf[0], bf[1]);
                lo = (float)ci[0] * pw0 + (float)ci[1] * pw1;
                hi = (float)ci[2] * pw0 + (float)ci[3] * pw1;
            } else {
                float cf[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int m = 0; m < KM; m++) {
                    const uint4 w0 = *reinterpret_cast<const uint4*>(wt + 16 * m);
                    mma_bf16(cf, w0.x, w0.y, w0.z, w0.w, bf[Q8 ? 0 : 2 * m], bf[Q8 ? 1 : 2 * m + 1]);
                }
                lo = cf[0] + cf[1];
                hi = cf[2] + cf[3];
            }
            lo += __shfl_xor_sync(0xffffffffu, lo, 1);
            hi += __shfl_xor_sync(0xffffffffu, hi, 1);
            if ((t & 1) == 0 && otok < T) {
                const int row = (base + tile) * 16 + g;
                ll_store(dst + row, epoch, lo * os);
                ll_store(dst + row + 8, epoch, hi * os);
            }
        }
        __syncwarp();
        if (c.lane == 0 && !c.dead) mbar_arrive(&c.sm.empty[slot]);
    }
}

// ---- Gated DeltaNet recurrence ------------------------------------------------------------------------
// Task t < GDN_TASKS: head t / 8, value columns [16 * (t % 8), +16).  Warp w owns value column w of the
// slice; a lane holds 4 consecutive key indices of that column's state row.  With two tokens the task
// runs them one after the other: the state after the first token goes to `state_bak`, the state after
// the second to `state`, and `from_bak` says which of the two the previous cycle left valid.
template <class S, bool Q8, int T>
__device__ bool gdn_op(Ctx& c, const Params& P, const LayerP& L, int pos, uint32_t e_proj, uint32_t e_out, int op,
                       bool from_bak) {
    static_assert(S::GDN_SLICE == NCW && S::LIN_DK == 128, "one warp per value column, 4 keys per lane");
    constexpr int SL = S::LIN_DV / S::GDN_SLICE;  // slices per head
    if (c.cta >= S::GDN_TASKS) return false;
    const int h = c.cta / SL, j = c.cta % SL;
    const int vcol = j * S::GDN_SLICE + c.warp;
    constexpr int NCH = 2 * S::LIN_DK + S::GDN_SLICE;           // 272 conv channels this task needs
    constexpr int QS = NCH + 2 + S::GDN_SLICE + 6;              // per-token stride of the scratch
    float* qkv_s = reinterpret_cast<float*>(c.sm.xq);           // per token: [q 128 | k 128 | v 16 | b | a | z 16]
    float* osq = c.sm.red_s + (c.red_n++ & 1) * (2 * T * NCW);  // [token][warp] squared outputs
    const size_t soff = ((size_t)(h * S::LIN_DV + vcol) * S::LIN_DK) + 4 * c.lane;
    const float* sin = (T == 2 && from_bak) ? L.state_bak + soff : L.state + soff;
    const float4 st = *reinterpret_cast<const float4*>(sin);    // issued before the wait on purpose
    const float a_log = L.A_log[h], dt_bias = L.dt_bias[h];
    if (c.tid < NCH) {
        int ch;
        if (c.tid < S::LIN_DK) ch = h * S::LIN_DK + c.tid;
        else if (c.tid < 2 * S::LIN_DK) ch = S::LIN_QK + h * S::LIN_DK + (c.tid - S::LIN_DK);
        else ch = 2 * S::LIN_QK + h * S::LIN_DV + j * S::GDN_SLICE + (c.tid - 2 * S::LIN_DK);
        const float4 taps = *reinterpret_cast<const float4*>(L.conv_w + 4 * ch);
        // every task keeps its own history of the channels it convolves (q and k of the head are
        // duplicated across the head's 8 tasks), so nothing here is shared between CTAs
        float* hist = L.conv_hist + ((size_t)c.cta * NCH + c.tid) * CONV_RING;
        float h3 = hist[(pos - 3) & (CONV_RING - 1)];
        float h2 = hist[(pos - 2) & (CONV_RING - 1)];
        float h1 = hist[(pos - 1) & (CONV_RING - 1)];
        float cur[T];
        if (T == 1) {
            cur[0] = ll_wait(c, P.projl + ch, e_proj, W_PROJ);
        } else {
            Spin s;
            u64 w0 = ll_load(P.projl + ch), w1 = ll_load(P.projl + S::PROJ_MAX + ch);
            while ((uint32_t)(w0 >> 32) != e_proj || (uint32_t)(w1 >> 32) != e_proj) {
                if (MK_SPIN_FAIL(c, s, W_PROJ)) {
                    c.dead = true;
                    break;
                }
                if ((uint32_t)(w0 >> 32) != e_proj) w0 = ll_load(P.projl + ch);
                if ((uint32_t)(w1 >> 32) != e_proj) w1 = ll_load(P.projl + S::PROJ_MAX + ch);
            }
            cur[0] = __uint_as_float((uint32_t)w0);
            cur[T - 1] = __uint_as_float((uint32_t)w1);
        }
#pragma unroll
        for (int tk = 0; tk < T; tk++) {
            float a = h3 * taps.x;
            a = fmaf(h2, taps.y, a);
            a = fmaf(h1, taps.z, a);
            a = fmaf(cur[tk], taps.w, a);
            qkv_s[tk * QS + c.tid] = silu_f(a);
            hist[(pos + tk) & (CONV_RING - 1)] = cur[tk];
            h3 = h2; h2 = h1; h1 = cur[tk];
        }
    } else if (c.tid < NCH + 2 + S::GDN_SLICE) {
        // b, a of the head, then z of this task's value columns
        const int off = c.tid == NCH ? S::B_OFF + h
                                     : (c.tid == NCH + 1 ? S::A_OFF + h : S::Z_OFF + h * S::LIN_DV + j * S::GDN_SLICE + (c.tid - NCH - 2));
#pragma unroll
        for (int tk = 0; tk < T; tk++)
            qkv_s[tk * QS + c.tid] = ll_wait(c, P.projl + (size_t)tk * S::PROJ_MAX + off, e_proj, W_PROJ);
    }
    const float gw = L.gdn_norm[vcol];
    consumer_sync();
    prof_stamp(c, op, 1);
    float s0 = st.x, s1 = st.y, s2 = st.z, s3 = st.w;
#pragma unroll
    for (int tk = 0; tk < T; tk++) {
        const float* qs_ = qkv_s + tk * QS;
        const float4 q4 = *reinterpret_cast<const float4*>(qs_ + 4 * c.lane);
        const float4 k4 = *reinterpret_cast<const float4*>(qs_ + S::LIN_DK + 4 * c.lane);
        const float qn = warp_sum(q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w);
        const float kn = warp_sum(k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w);
        // x / max(|x|, 1e-6), and the 1/sqrt(dk) query scale
        const float qs = 0.08838834764831845f / fmaxf(sqrtf(qn), 1e-6f);
        const float ks = 1.0f / fmaxf(sqrtf(kn), 1e-6f);
        const float vval = qs_[2 * S::LIN_DK + c.warp];
        const float beta = sigmoid_f(qs_[NCH]);
        const float decay = expf(-expf(a_log) * softplus_f(qs_[NCH + 1] + dt_bias));
        const float kx = k4.x * ks, ky = k4.y * ks, kz = k4.z * ks, kw = k4.w * ks;
        s0 *= decay; s1 *= decay; s2 *= decay; s3 *= decay;
        const float recalled = warp_sum(fmaf(s3, kw, fmaf(s2, kz, fmaf(s1, ky, s0 * kx))));
        const float delta = (vval - recalled) * beta;
        s0 = fmaf(kx, delta, s0);
        s1 = fmaf(ky, delta, s1);
        s2 = fmaf(kz, delta, s2);
        s3 = fmaf(kw, delta, s3);
        float* sout = (T == 2 && tk == 0) ? L.state_bak + soff : L.state + soff;
        *reinterpret_cast<float4*>(sout) = make_float4(s0, s1, s2, s3);
        const float o = warp_sum(fmaf(s3, q4.w, fmaf(s2, q4.z, fmaf(s1, q4.y, s0 * q4.x)))) * qs;
        // The elementwise part of the gated norm (weight, silu(z)) is applied here; the head's 1 / rms
        // needs the squared outputs of the head's eight tasks and is applied by whoever sums the tasks'
        // partial out-projections: this task publishes its sum of squares beside them.
        if (c.lane == 0) {
            c.sm.mix_s[tk * DOWN_K + c.warp] = o * gw * silu_f(qs_[NCH + 2 + c.warp]);
            osq[tk * NCW + c.warp] = o * o;
        }
    }
    prof_stamp(c, op, 2);
    consumer_sync();  // the scratch aliases the GEMV input vector that the next prologue writes
    if (c.tid < T) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < NCW; w++) tot += osq[c.tid * NCW + w];
        ll_store(P.mixl + (size_t)c.tid * S::MIX + c.cta, e_out, tot);
    }
    // out-projection, split over K: this task's 16 gated outputs times its column slice -> 1024 partial sums
    partial_cols<S, Q8, T, 1>(c, c.sm.mix_s, P.partl + (size_t)c.cta * S::HID, (size_t)c.grid * S::HID, e_out);
    return true;
}

// After a launch that ends on a rejected draft the valid DeltaNet state sits in `state_bak`: copy
// this task's rows back so that the host (and the next plain launch) finds it in `state`.
template <class S>
__device__ void gdn_restore_state(Ctx& c, const Params& P) {
    constexpr int SL = S::LIN_DV / S::GDN_SLICE;
    if (c.cta >= S::GDN_TASKS) return;
    const int h = c.cta / SL, j = c.cta % SL;
    const size_t soff = ((size_t)(h * S::LIN_DV + j * S::GDN_SLICE + c.warp) * S::LIN_DK) + 4 * c.lane;
    for (int l = 0; l < P.n_layers; l++) {
        const LayerP& L = P.layer[l];
        if (L.kind != 0) continue;
        *reinterpret_cast<float4*>(L.state + soff) = *reinterpret_cast<const float4*>(L.state_bak + soff);
    }
}

// ---- attention ---------------------------------------------------------------------------------------
template <bool F32>
__device__ __forceinline__ void load8(const void* base, size_t elem, float (&v)[8]) {
    if (F32) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>((const float*)base + elem));
        const float4 b = __ldcg(reinterpret_cast<const float4*>((const float*)base + elem + 4));
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 a = __ldcg(reinterpret_cast<const uint4*>((const __nv_bfloat16*)base + elem));
        v[0] = bf_lo(a.x); v[1] = bf_hi(a.x); v[2] = bf_lo(a.y); v[3] = bf_hi(a.y);
        v[4] = bf_lo(a.z); v[5] = bf_hi(a.z); v[6] = bf_lo(a.w); v[7] = bf_hi(a.w);
    }
}
template <bool F32>
__device__ __forceinline__ float load1(const void* base, size_t elem) {
    if (F32) return __ldcg((const float*)base + elem);
    const unsigned short raw = __ldcg((const unsigned short*)base + elem);
    return __uint_as_float((uint32_t)raw << 16);
}
template <bool F32>
__device__ __forceinline__ float round_kv(float v) {
    return F32 ? v : __bfloat162float(__float2bfloat16(v));
}
template <bool F32>
__device__ __forceinline__ void store1(void* base, size_t elem, float v) {
    if (F32) ((float*)base)[elem] = v;
    else ((__nv_bfloat16*)base)[elem] = __float2bfloat16(v);
}

// Split-K decode attention over the paged cache, for T consecutive positions pos .. pos + T - 1 of one
// sequence.  Task (g, s): KV head g, positions [s * ch, min(n, (s + 1) * ch)) with n = pos + T, run by
// CTA s * NKV + g.  Token j sees positions up to pos + j.  Cached K and V rows of the task are requested
// before the task waits for its queries, so that only one memory round trip sits between the
// projection and the scores.  With one split the task publishes the normalised outputs itself;
// otherwise every task publishes (acc, m, l) partials as flag-in-data words and then merges a
// 1/nsplit share of the head group's outputs from all partials, in a fixed order.
//
// `V` says which CTAs serve the sequence and where its hand-off words and block table are: the whole
// grid and the engine's buffers for a single sequence, a group of CTAs and a slice of the buffers per
// sequence when several sequences decode side by side.
struct AttnView {
    int cta, grid;          // this CTA's index among the CTAs that serve the sequence, and their number
    const u64* projl;       // projection words of the sequence's first token slot
    u64* mixl;              // mixer output words of that slot
    u64* part;              // split partials of that slot
    const int* bt;          // the sequence's block table (shared memory)
    bool gate;              // publish o * sigmoid(gate) instead of o (otherwise the out-projection's prologue applies the gate)
};

// KU cached K rows per warp and VU cached V elements per thread are requested together before they are
// used: 1 and 8 suit the short chunks of a sequence that has the whole grid; tasks that scan 64 or more
// positions (several sequences sharing the grid) want more loads in flight.
template <class S, bool KVF32, int T, int KU = 1, int VU = 8>
__device__ bool attn_op(Ctx& c, const Params& P, const LayerP& L, const AttnView& V, int pos, uint32_t e_proj,
                        uint32_t e_out, int op) {
    static_assert(S::HD == 256 && S::QPK == 4 && NCW == 16 && S::ROT == 64, "thread mapping below");
    constexpr int NOUT = S::QPK * S::HD;        // outputs per KV head and token
    constexpr int PFV = 16;                     // V rows requested early per thread
    const int n = pos + T;
    const int max_splits = min(V.grid / S::NKV, MAX_SPLITS);
    const int ch = attn_chunk(n, max_splits);
    const int nsplit = (n + ch - 1) / ch;
    if (V.cta >= nsplit * S::NKV) return false;
    const int g = V.cta % S::NKV, sp = V.cta / S::NKV;
    const int p0 = sp * ch, p1 = min(n, p0 + ch);
    const int np = p1 - p0;

    float* q_s = reinterpret_cast<float*>(c.sm.xq);       // [T][4][256] normalised, rotated, pre-scaled queries
    float* knew_s = q_s + T * S::QPK * S::HD;             // [T][256] rows of positions pos .. pos + T - 1
    float* vnew_s = knew_s + T * S::HD;                   // [T][256]
    float* sc_s = vnew_s + T * S::HD;                     // [T][4][ch] scores, then probabilities
    float* stat_s = c.sm.out_s;                           // [T][ m[4], l[4] ]
    // sigmoid of the output gate of (token, head of the group, dim), for tasks that publish gated outputs
    auto gate_of = [&](int tk, int head, int dim) {
        if (!V.gate) return 1.0f;
        return sigmoid_f(ll_wait(c, V.projl + (size_t)tk * S::PROJ_MAX + (size_t)(g * S::QPK + head) * 2 * S::HD + S::HD + dim,
                                 e_proj, W_PROJ));
    };

    const size_t kv_head_stride = (size_t)KV_BLOCK * S::HD;
    auto kv_elem = [&](int p) -> size_t {
        const int blk = V.bt[p >> 6];
        return ((size_t)blk * S::NKV + g) * kv_head_stride + (size_t)(p & (KV_BLOCK - 1)) * S::HD;
    };
    // -- 0. request cached rows early: the K row of this warp's first position, V elements of this thread's dim
    const int d = c.tid & (S::HD - 1), hp = c.tid >> 8;
    float kpre[8], vpre[PFV];
    {
        const int p = p0 + c.warp;
#pragma unroll
        for (int i = 0; i < 8; i++) kpre[i] = 0.f;
        if (p < p1 && p < pos) load8<KVF32>(L.k_cache, kv_elem(p) + 8 * c.lane, kpre);
    }
#pragma unroll
    for (int i = 0; i < PFV; i++) {
        const int p = p0 + i;
        vpre[i] = (p < p1 && p < pos) ? load1<KVF32>(L.v_cache, kv_elem(p) + d) : 0.f;
    }

    // -- 1. q (4 heads), new k, new v of every token from the projection words; per-head RMSNorm; partial RoPE
    {
        const int hh = c.warp >> 2, qd = c.warp & 3;        // head within group, 64-wide quarter
        const int dd = qd * 64 + 2 * c.lane;
        // norm weights are requested before the wait
        const float2 qw = *reinterpret_cast<const float2*>(L.q_norm + dd);
        const float2 kw = hh == 0 ? *reinterpret_cast<const float2*>(L.k_norm + dd) : make_float2(0.f, 0.f);
        const u64* ptrs[2 * T];
        uint32_t eps[2 * T];
#pragma unroll
        for (int tk = 0; tk < T; tk++) {
            const u64* pj = V.projl + (size_t)tk * S::PROJ_MAX;
            ptrs[2 * tk] = pj + (g * S::QPK + hh) * 2 * S::HD + dd;
            ptrs[2 * tk + 1] = hh == 0 ? pj + S::ATT_K_OFF + g * S::HD + dd
                                       : (hh == 1 ? pj + S::ATT_V_OFF + g * S::HD + dd : nullptr);
            eps[2 * tk] = eps[2 * tk + 1] = e_proj;
        }
        float v4[4 * T];
        ll_wait_pairs<2 * T>(c, ptrs, eps, v4, W_PROJ);
        float* buf = c.sm.red_s + (c.red_n++ & 1) * (2 * T * NCW);      // per token: q sums [16], k sums [4]
#pragma unroll
        for (int tk = 0; tk < T; tk++) {
            const float a = v4[4 * tk], b = v4[4 * tk + 1];
            const float ka = hh == 0 ? v4[4 * tk + 2] : 0.f, kb = hh == 0 ? v4[4 * tk + 3] : 0.f;
            const float sq = warp_sum(a * a + b * b);
            const float sk = warp_sum(ka * ka + kb * kb);
            if (c.lane == 0) {
                buf[tk * 2 * NCW + c.warp] = sq;
                if (hh == 0) buf[tk * 2 * NCW + NCW + qd] = sk;
            }
        }
        consumer_sync();
#pragma unroll
        for (int tk = 0; tk < T; tk++) {
            float a = v4[4 * tk], b = v4[4 * tk + 1];
            float ka = hh == 0 ? v4[4 * tk + 2] : 0.f, kb = hh == 0 ? v4[4 * tk + 3] : 0.f;
            const float va = v4[4 * tk + 2], vb = v4[4 * tk + 3];
            const float* bq = buf + tk * 2 * NCW;
            const float qss = bq[hh * 4] + bq[hh * 4 + 1] + bq[hh * 4 + 2] + bq[hh * 4 + 3];
            const float qinv = rsqrtf(qss * (1.0f / S::HD) + S::EPS);
            a = a * qinv * (1.0f + qw.x);
            b = b * qinv * (1.0f + qw.y);
            float cs0 = 1.f, sn0 = 0.f, cs1 = 1.f, sn1 = 0.f;
            if (qd == 0) {
                const int i0 = (2 * c.lane) & 31;
                const size_t ro = (size_t)(pos + tk) * (S::ROT / 2) + i0;
                cs0 = P.rope_cos[ro]; sn0 = P.rope_sin[ro]; cs1 = P.rope_cos[ro + 1]; sn1 = P.rope_sin[ro + 1];
                // dims [0,32) live in lanes 0..15, their partners [32,64) in lanes 16..31
                const float pa = __shfl_xor_sync(0xffffffffu, a, 16), pb = __shfl_xor_sync(0xffffffffu, b, 16);
                if (c.lane < 16) { a = a * cs0 - pa * sn0; b = b * cs1 - pb * sn1; }
                else { a = a * cs0 + pa * sn0; b = b * cs1 + pb * sn1; }
            }
            float* qt = q_s + (tk * S::QPK + hh) * S::HD;
            qt[dd] = a * 0.0625f;          // 1/sqrt(256), exact
            qt[dd + 1] = b * 0.0625f;
            if (hh == 0) {
                const float kss = bq[NCW] + bq[NCW + 1] + bq[NCW + 2] + bq[NCW + 3];
                const float kinv = rsqrtf(kss * (1.0f / S::HD) + S::EPS);
                ka = ka * kinv * (1.0f + kw.x);
                kb = kb * kinv * (1.0f + kw.y);
                if (qd == 0) {
                    const float pa = __shfl_xor_sync(0xffffffffu, ka, 16), pb = __shfl_xor_sync(0xffffffffu, kb, 16);
                    if (c.lane < 16) { ka = ka * cs0 - pa * sn0; kb = kb * cs1 - pb * sn1; }
                    else { ka = ka * cs0 + pa * sn0; kb = kb * cs1 + pb * sn1; }
                }
                knew_s[tk * S::HD + dd] = round_kv<KVF32>(ka);
                knew_s[tk * S::HD + dd + 1] = round_kv<KVF32>(kb);
            }
            if (hh == 1) {
                vnew_s[tk * S::HD + dd] = round_kv<KVF32>(va);
                vnew_s[tk * S::HD + dd + 1] = round_kv<KVF32>(vb);
            }
        }
        consumer_sync();
        prof_stamp(c, op, 1);
    }
    // -- 2. append the new positions (the tasks that own them)
#pragma unroll
    for (int tk = 0; tk < T; tk++) {
        const int pn = pos + tk;
        if (pn >= p0 && pn < p1 && c.tid < S::HD) {
            const size_t e = kv_elem(pn) + c.tid;
            store1<KVF32>(L.k_cache, e, knew_s[tk * S::HD + c.tid]);
            store1<KVF32>(L.v_cache, e, vnew_s[tk * S::HD + c.tid]);
        }
    }
    // -- 3. scores: one warp per position, 8 dims per lane; token j ignores positions after pos + j
    {
        auto score = [&](int p, const float (&kk)[8]) {
#pragma unroll
            for (int tk = 0; tk < T; tk++) {
                float dsum[S::QPK];
#pragma unroll
                for (int hh = 0; hh < S::QPK; hh++) {
                    const float* qt = q_s + (tk * S::QPK + hh) * S::HD + 8 * c.lane;
                    const float4 x = *reinterpret_cast<const float4*>(qt);
                    const float4 y = *reinterpret_cast<const float4*>(qt + 4);
                    float a = x.x * kk[0];
                    a = fmaf(x.y, kk[1], a); a = fmaf(x.z, kk[2], a); a = fmaf(x.w, kk[3], a);
                    a = fmaf(y.x, kk[4], a); a = fmaf(y.y, kk[5], a); a = fmaf(y.z, kk[6], a); a = fmaf(y.w, kk[7], a);
                    dsum[hh] = warp_sum(a);
                }
                if (c.lane == 0) {
                    const bool seen = p <= pos + tk;
#pragma unroll
                    for (int hh = 0; hh < S::QPK; hh++)
                        sc_s[(tk * S::QPK + hh) * ch + (p - p0)] = seen ? dsum[hh] : -INFINITY;
                }
            }
        };
        for (int pb = p0 + c.warp; pb < p1; pb += KU * NCW) {
            float kk[KU][8];
#pragma unroll
            for (int u = 0; u < KU; u++) {
                const int p = pb + u * NCW;
                if (p >= p1) continue;
                if (p >= pos) {
#pragma unroll
                    for (int i = 0; i < 8; i++) kk[u][i] = knew_s[(p - pos) * S::HD + 8 * c.lane + i];
                } else if (p == p0 + c.warp) {
#pragma unroll
                    for (int i = 0; i < 8; i++) kk[u][i] = kpre[i];
                } else {
                    load8<KVF32>(L.k_cache, kv_elem(p) + 8 * c.lane, kk[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < KU; u++)
                if (pb + u * NCW < p1) score(pb + u * NCW, kk[u]);
        }
    }
    consumer_sync();
    // -- 4. softmax statistics: warp w < 4T handles (token w / 4, head w % 4)
    if (c.warp < T * S::QPK) {
        float* row = sc_s + c.warp * ch;
        float m = -INFINITY;
        for (int i = c.lane; i < np; i += 32) m = fmaxf(m, row[i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = c.lane; i < np; i += 32) {
            const float e = m == -INFINITY ? 0.f : __expf(row[i] - m);
            row[i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (c.lane == 0) {
            stat_s[(c.warp >> 2) * 8 + (c.warp & 3)] = m;
            stat_s[(c.warp >> 2) * 8 + S::QPK + (c.warp & 3)] = l;
        }
    }
    consumer_sync();
    // -- 5. weighted values: thread -> dim d, heads 2*hp and 2*hp+1, every token
    float acc[T][2];
#pragma unroll
    for (int tk = 0; tk < T; tk++) acc[tk][0] = acc[tk][1] = 0.f;
    {
        auto accumulate = [&](int i, float v) {
#pragma unroll
            for (int tk = 0; tk < T; tk++) {
                acc[tk][0] = fmaf(sc_s[(tk * S::QPK + 2 * hp) * ch + i], v, acc[tk][0]);
                acc[tk][1] = fmaf(sc_s[(tk * S::QPK + 2 * hp + 1) * ch + i], v, acc[tk][1]);
            }
        };
#pragma unroll
        for (int i = 0; i < PFV; i++) {
            if (i < np) {
                const int p = p0 + i;
                accumulate(i, p >= pos ? vnew_s[(p - pos) * S::HD + d] : vpre[i]);
            }
        }
        int i = PFV;
        for (; i + VU <= np; i += VU) {
            float v[VU];
#pragma unroll
            for (int u = 0; u < VU; u++) {
                const int p = p0 + i + u;
                v[u] = p >= pos ? vnew_s[(p - pos) * S::HD + d] : load1<KVF32>(L.v_cache, kv_elem(p) + d);
            }
#pragma unroll
            for (int u = 0; u < VU; u++) accumulate(i + u, v[u]);
        }
        for (; i < np; i++) {
            const int p = p0 + i;
            accumulate(i, p >= pos ? vnew_s[(p - pos) * S::HD + d] : load1<KVF32>(L.v_cache, kv_elem(p) + d));
        }
    }
    prof_stamp(c, op, 2);
    if (nsplit == 1) {
#pragma unroll
        for (int tk = 0; tk < T; tk++) {
            u64* out = V.mixl + (size_t)tk * S::MIX + (size_t)(g * S::QPK) * S::HD;
            ll_store(out + (2 * hp) * S::HD + d, e_out, acc[tk][0] / stat_s[tk * 8 + S::QPK + 2 * hp] * gate_of(tk, 2 * hp, d));
            ll_store(out + (2 * hp + 1) * S::HD + d, e_out,
                     acc[tk][1] / stat_s[tk * 8 + S::QPK + 2 * hp + 1] * gate_of(tk, 2 * hp + 1, d));
        }
        // The appended K/V rows are read by other CTAs from the next step on.  They get there only
        // through words this CTA publishes after this fence, so the fence can sit off the critical path.
        __threadfence();
        consumer_sync();  // scratch aliases the GEMV input planes that the next prologue writes
        return true;
    }
    // -- 6. partials as flag-in-data words: per token acc [4][256], then (m, l) per head
#pragma unroll
    for (int tk = 0; tk < T; tk++) {
        u64* part = V.part + (((size_t)tk * S::NKV + g) * MAX_SPLITS + sp) * S::PART_STRIDE;
        ll_store(part + (2 * hp) * S::HD + d, e_out, acc[tk][0]);
        ll_store(part + (2 * hp + 1) * S::HD + d, e_out, acc[tk][1]);
        if (c.tid < 2 * S::QPK) ll_store(part + NOUT + c.tid, e_out, stat_s[tk * 8 + (c.tid & 1) * S::QPK + (c.tid >> 1)]);
    }
    // -- 7. merge this task's share of the outputs.  `tpo` threads share one output, each takes the
    //       splits s = sub, sub + tpo, ...; a fixed shuffle tree combines them.  Token j is merged over
    //       the splits a plain step at its position would have, with that step's work split, so that a
    //       speculative cycle rounds exactly like plain decoding.
    constexpr int SPT = 4;                                   // splits per thread at most (MAX_SPLITS / 32)
#pragma unroll
    for (int tk = 0; tk < T; tk++) {
        const int ns_t = min(nsplit, (pos + tk + ch) / ch);          // splits that hold positions <= pos + tk
        if (ns_t == 1) {                                             // everything this token sees is in split 0
            if (sp == 0) {
                u64* out = V.mixl + (size_t)tk * S::MIX + (size_t)(g * S::QPK) * S::HD;
                ll_store(out + (2 * hp) * S::HD + d, e_out, acc[tk][0] / stat_s[tk * 8 + S::QPK + 2 * hp] * gate_of(tk, 2 * hp, d));
                ll_store(out + (2 * hp + 1) * S::HD + d, e_out,
                         acc[tk][1] / stat_s[tk * 8 + S::QPK + 2 * hp + 1] * gate_of(tk, 2 * hp + 1, d));
            }
            continue;
        }
        const int opc = (NOUT + ns_t - 1) / ns_t;                   // outputs per task
        int tpo = 1;
        while (tpo < 32 && 2 * tpo * opc <= NCT && tpo < ns_t) tpo *= 2;
        const int oi = c.tid / tpo, sub = c.tid % tpo;
        const int o = sp * opc + oi;
        const bool live = sp < ns_t && oi < opc && o < NOUT;
        const int h = o / S::HD;
        const u64* pg = V.part + ((size_t)tk * S::NKV + g) * MAX_SPLITS * S::PART_STRIDE;
        float mv[SPT], lv[SPT], av[SPT];
        {
            u64 wa[SPT], wm[SPT], wl[SPT];
#pragma unroll
            for (int i = 0; i < SPT; i++) {
                const int s2 = sub + i * tpo;
                wa[i] = wm[i] = wl[i] = 0;
                if (live && s2 < ns_t) {
                    const u64* ps = pg + (size_t)s2 * S::PART_STRIDE;
                    wa[i] = ll_load(ps + o);
                    ll_load2(ps + NOUT + 2 * h, wm[i], wl[i]);
                }
            }
            Spin spin;
            while (true) {
                bool ok = true;
#pragma unroll
                for (int i = 0; i < SPT; i++) {
                    const int s2 = sub + i * tpo;
                    if (live && s2 < ns_t) {
                        const u64* ps = pg + (size_t)s2 * S::PART_STRIDE;
                        if ((uint32_t)(wa[i] >> 32) != e_out) { ok = false; wa[i] = ll_load(ps + o); }
                        if ((uint32_t)(wm[i] >> 32) != e_out || (uint32_t)(wl[i] >> 32) != e_out) {
                            ok = false;
                            ll_load2(ps + NOUT + 2 * h, wm[i], wl[i]);
                        }
                    }
                }
                if (ok) break;
                if (MK_SPIN_FAIL(c, spin, W_PART)) {
                    c.dead = true;
                    break;
                }
            }
#pragma unroll
            for (int i = 0; i < SPT; i++) {
                const bool have = live && sub + i * tpo < ns_t;
                mv[i] = have ? __uint_as_float((uint32_t)wm[i]) : -INFINITY;
                lv[i] = have ? __uint_as_float((uint32_t)wl[i]) : 0.f;
                av[i] = have ? __uint_as_float((uint32_t)wa[i]) : 0.f;
            }
        }
        float M = fmaxf(fmaxf(mv[0], mv[1]), fmaxf(mv[2], mv[3]));
        for (int x = 1; x < tpo; x *= 2) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, x));
        float Ls = 0.f, Os = 0.f;
#pragma unroll
        for (int i = 0; i < SPT; i++) {
            const float w = mv[i] == -INFINITY ? 0.f : __expf(mv[i] - M);
            Ls = fmaf(lv[i], w, Ls);
            Os = fmaf(av[i], w, Os);
        }
        for (int x = 1; x < tpo; x *= 2) {
            Ls += __shfl_xor_sync(0xffffffffu, Ls, x);
            Os += __shfl_xor_sync(0xffffffffu, Os, x);
        }
        if (live && sub == 0)
            ll_store(V.mixl + (size_t)tk * S::MIX + (size_t)(g * S::QPK) * S::HD + o, e_out, Os / Ls * gate_of(tk, h, o % S::HD));
    }
    __threadfence();      // K/V append before anything this CTA publishes later (see above)
    consumer_sync();      // scratch aliases the GEMV input planes that the next prologue writes
    return true;
}

// ---- one decoder layer -----------------------------------------------------------------------------------
// Runs ops A..E of layer `L` for T tokens at positions pos .. pos + T - 1 on the residual stream `xbuf`
// (words [T][HID]).  `x` holds this thread's residual elements when `x_in_regs` (first layer: they come
// from the embedding lookup), otherwise they are awaited at epoch eA - 1.  Returns true if a wait ran out.
template <class S, bool Q8, bool KVF32, int T>
__device__ __forceinline__ bool run_layer(Ctx& c, const Params& P, const LayerP& L, u64* xbuf, uint32_t eA, int op0,
                                          int pos, float (&x)[T][2], bool x_in_regs, bool from_bak, int xr0, int xr1,
                                          float* resid_out) {
    constexpr int WB = Q8 ? 1 : 2;                       // bytes per weight
    const uint32_t eB = eA + 1, eC = eA + 2, eD = eA + 3, eE = eA + 4;
    const bool attn = L.kind != 0;
    float y[T][2];
    // ---- A: in-projection
    {
        prof_stamp(c, op0, 0);
        int r0, r1;
        cta_rows(attn ? S::ATT_IN : S::GDN_IN, 1, c.cta, c.grid, r0, r1);
        scale_prefetch(c, L.s_in, r0, r1, false);
        // the norm weights are requested before the wait so that their latency hides behind it
        const float2 nw = *reinterpret_cast<const float2*>(L.in_norm + 2 * c.tid);
        if (!x_in_regs) {
            float v[2 * T];
            const u64* base = xbuf + 2 * c.tid;
            ll_wait_pairs_fn<T>(c, [&](int j) { return base + (size_t)j * S::HID; }, [&](int) { return eA - 1; }, v, W_X);
#pragma unroll
            for (int j = 0; j < T; j++) { x[j][0] = v[2 * j]; x[j][1] = v[2 * j + 1]; }
        }
        stage_rmsnorm<S, Q8, T>(c, x, nw, y);
        prof_stamp(c, op0, 1);
        gemv_mma<Q8, T, false>(c, r0, r1, S::HID * WB, L.s_in, [&](int, int row, int tk, float v, bool ok) {
            if (ok) ll_store(P.projl + (size_t)tk * S::PROJ_MAX + row, eA, v);
        });
        prof_stamp(c, op0, 3);
    }
    // ---- B: mixer
    prof_stamp(c, op0 + 1, 0);
    const AttnView view = {c.cta, c.grid, P.projl, P.mixl, P.attn_part, c.sm.bt_s, false};
    const bool had_task = attn ? attn_op<S, KVF32, T>(c, P, L, view, pos, eA, eB, op0 + 1)
                               : gdn_op<S, Q8, T>(c, P, L, pos, eA, eB, op0 + 1, from_bak);
    prof_stamp(c, op0 + 1, 3);
    // ---- C: out-projection + residual
    if (!attn) {
        // DeltaNet: the tasks have already multiplied their outputs with their column slices.  Warp r
        // sums the 128 partial sums of owned row r, each weighted with its head's 1 / rms: lane l takes
        // tasks l, l + 32, l + 64, l + 96, whose heads' eight tasks are eight consecutive lanes.
        const int op = op0 + 2;
        prof_stamp(c, op, 0);
        static_assert(S::GDN_TASKS == 128 && S::LIN_DV / S::GDN_SLICE == 8, "four tasks per lane, eight per head");
        if (c.warp < xr1 - xr0) {
            const int row = xr0 + c.warp;
            const float rs = Q8 ? L.s_out[row] : 1.0f;           // requested before the wait
#pragma unroll
            for (int j = 0; j < T; j++) {
                const u64* psrc = P.partl + (size_t)j * c.grid * S::HID + row;
                const u64* ssrc = P.mixl + (size_t)j * S::MIX;
                u64 w[4], sw[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    w[i] = ll_load(psrc + (size_t)(c.lane + 32 * i) * S::HID);
                    sw[i] = ll_load(ssrc + c.lane + 32 * i);
                }
                Spin sp;
                while (true) {
                    bool ok = true;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        if ((uint32_t)(w[i] >> 32) != eB) { ok = false; w[i] = ll_load(psrc + (size_t)(c.lane + 32 * i) * S::HID); }
                        if ((uint32_t)(sw[i] >> 32) != eB) { ok = false; sw[i] = ll_load(ssrc + c.lane + 32 * i); }
                    }
                    if (ok) break;
                    if (MK_SPIN_FAIL(c, sp, W_MIX)) {
                        c.dead = true;
                        break;
                    }
                }
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float hs = __uint_as_float((uint32_t)sw[i]);      // sum of squares over the head: 8 lanes
                    hs += __shfl_xor_sync(0xffffffffu, hs, 1);
                    hs += __shfl_xor_sync(0xffffffffu, hs, 2);
                    hs += __shfl_xor_sync(0xffffffffu, hs, 4);
                    acc += __uint_as_float((uint32_t)w[i]) * rsqrtf(hs * (1.0f / S::LIN_DV) + S::EPS);
                }
                const float tot = warp_sum(acc);
                if (c.lane == 0) {
                    const float xn = c.sm.xown[j * 16 + c.warp] + tot * rs;
                    c.sm.xown[j * 16 + c.warp] = xn;
                    ll_store(xbuf + (size_t)j * S::HID + row, eC, xn);
                }
            }
        }
        prof_stamp(c, op, 3);
        consumer_sync();   // keep the other warps' polls for the next op behind these stores
    } else {
        const int op = op0 + 2;
        prof_stamp(c, op, 0);
        scale_prefetch(c, L.s_out, xr0, xr1, false);
        if (!had_task) gate_on_samples(c, P.mixl + (size_t)(T - 1) * S::MIX, S::MIX, eB);
        // each thread stages 4 consecutive mixer outputs; a warp covers 128 = one DeltaNet head
        const int k = 4 * c.tid;
        float m[T][4];
        const float4 gw = attn ? make_float4(0.f, 0.f, 0.f, 0.f)
                               : *reinterpret_cast<const float4*>(L.gdn_norm + (k % S::LIN_DV));
        {
            float v[8 * T];
            // pair i: token i / 4; pairs 0, 1 of a token are mixer outputs, 2, 3 the sigmoid gate or z
            const u64* mix0 = P.mixl + k;
            const u64* aux0 = P.projl + (attn ? (k / S::HD) * 2 * S::HD + S::HD + (k % S::HD) : S::Z_OFF + k);
            ll_wait_pairs_fn<4 * T>(c,
                                    [&](int i) {
                                        return ((i & 2) ? aux0 + (size_t)(i >> 2) * S::PROJ_MAX : mix0 + (size_t)(i >> 2) * S::MIX) + 2 * (i & 1);
                                    },
                                    [&](int i) { return (i & 2) ? eA : eB; }, v, W_MIX);
#pragma unroll
            for (int j = 0; j < T; j++) {
                const float* vj = v + 8 * j;
                if (attn) {
#pragma unroll
                    for (int i = 0; i < 4; i++) m[j][i] = vj[i] * sigmoid_f(vj[4 + i]);
                } else {
                    const float ss = warp_sum(vj[0] * vj[0] + vj[1] * vj[1] + vj[2] * vj[2] + vj[3] * vj[3]);
                    const float inv = rsqrtf(ss * (1.0f / S::LIN_DV) + S::EPS);
                    m[j][0] = vj[0] * inv * gw.x * silu_f(vj[4]);
                    m[j][1] = vj[1] * inv * gw.y * silu_f(vj[5]);
                    m[j][2] = vj[2] * inv * gw.z * silu_f(vj[6]);
                    m[j][3] = vj[3] * inv * gw.w * silu_f(vj[7]);
                }
            }
        }
        float mx[T], scale[T];
#pragma unroll
        for (int j = 0; j < T; j++) mx[j] = fmaxf(fmaxf(fabsf(m[j][0]), fabsf(m[j][1])), fmaxf(fabsf(m[j][2]), fabsf(m[j][3])));
        block_scale<Q8, T>(c, mx, scale);
#pragma unroll
        for (int j = 0; j < T; j++) {
            uint8_t* xq = c.sm.xq + (size_t)(4 * j) * (S::MIX * WB);
            stage_pair<Q8>(xq, S::MIX * WB, k, m[j][0], m[j][1], scale[j]);
            stage_pair<Q8>(xq, S::MIX * WB, k + 2, m[j][2], m[j][3], scale[j]);
        }
        finish_stage<T>(c, scale);
        prof_stamp(c, op, 1);
        gemv_mma<Q8, T, false>(c, xr0, xr1, S::MIX * WB, L.s_out, [&](int, int row, int tk, float v, bool ok) {
            if (ok) {
                const float xn = c.sm.xown[tk * 16 + row - xr0] + v;
                c.sm.xown[tk * 16 + row - xr0] = xn;
                ll_store(xbuf + (size_t)tk * S::HID + row, eC, xn);
            }
        });
        prof_stamp(c, op, 3);
    }
    // ---- D: gate/up + SwiGLU
    {
        const int op = op0 + 3;
        prof_stamp(c, op, 0);
        int r0, r1;
        cta_rows(2 * S::INTER, 2, c.cta, c.grid, r0, r1);
        scale_prefetch(c, L.s_gu, r0, r1, false);
        const float2 nw = *reinterpret_cast<const float2*>(L.post_norm + 2 * c.tid);
        {
            float v[2 * T];
            const u64* base = xbuf + 2 * c.tid;
            ll_wait_pairs_fn<T>(c, [&](int j) { return base + (size_t)j * S::HID; }, [&](int) { return eC; }, v, W_X);
#pragma unroll
            for (int j = 0; j < T; j++) { x[j][0] = v[2 * j]; x[j][1] = v[2 * j + 1]; }
        }
        stage_rmsnorm<S, Q8, T>(c, x, nw, y);
        prof_stamp(c, op, 1);
        gemv_mma<Q8, T, false>(c, r0, r1, S::HID * WB, L.s_gu, [&](int lane, int row, int tk, float v, bool ok) {
            // rows alternate gate, up; chunks hold whole pairs, so the partner is the next lane.  The
            // SwiGLU outputs stay in this CTA: it multiplies them with its column slice of the
            // down-projection itself.
            const float up = __shfl_down_sync(0xffffffffu, v, 1);
            if (ok && !(lane & 1)) c.sm.act_s[tk * DOWN_K + ((row - r0) >> 1)] = silu_f(v) * up;
        });
        // ---- down-projection, split over K: 1024 partial sums from this CTA's <= 32 activations
        partial_cols<S, Q8, T, DOWN_K / 16>(c, c.sm.act_s, P.partl + (size_t)c.cta * S::HID, (size_t)c.grid * S::HID, eD);
        prof_stamp(c, op, 3);
    }
    // ---- E: sum of the CTAs' partial down-projections + residual, for the rows this CTA owns
    bool failed;
    {
        const int op = op0 + 4;
        prof_stamp(c, op, 0);
        if (c.warp < xr1 - xr0) {
            const int row = xr0 + c.warp;
            const float rs = Q8 ? L.s_down[row] : 1.0f;         // requested before the wait
#pragma unroll
            for (int j = 0; j < T; j++) {
                // lane l takes CTAs l, l + 32, ...; fixed order, then the shuffle tree
                constexpr int PER = 5;                          // grids of up to 160 CTAs
                const u64* src = P.partl + (size_t)j * c.grid * S::HID + row;
                u64 w[PER];
#pragma unroll
                for (int i = 0; i < PER; i++) {
                    const int cta = c.lane + 32 * i;
                    w[i] = cta < c.grid ? ll_load(src + (size_t)cta * S::HID) : 0;
                }
                Spin sp;
                while (true) {
                    bool ok = true;
#pragma unroll
                    for (int i = 0; i < PER; i++) {
                        const int cta = c.lane + 32 * i;
                        if (cta < c.grid && (uint32_t)(w[i] >> 32) != eD) {
                            ok = false;
                            w[i] = ll_load(src + (size_t)cta * S::HID);
                        }
                    }
                    if (ok) break;
                    if (MK_SPIN_FAIL(c, sp, W_ACT)) {
                        c.dead = true;
                        break;
                    }
                }
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < PER; i++)
                    if (c.lane + 32 * i < c.grid) acc += __uint_as_float((uint32_t)w[i]);
                const float tot = warp_sum(acc);
                if (c.lane == 0) {
                    const float xn = c.sm.xown[j * 16 + c.warp] + tot * rs;
                    c.sm.xown[j * 16 + c.warp] = xn;
                    ll_store(xbuf + (size_t)j * S::HID + row, eE, xn);
                    if (resid_out) resid_out[(size_t)j * S::HID + row] = xn;
                }
            }
        }
        prof_stamp(c, op, 3);
        failed = consumer_any(c.dead);
    }
    return failed;
}

// ---- the kernel ------------------------------------------------------------------------------------------

template <class S, bool Q8, bool KVF32, int T>
__global__ void __launch_bounds__(NTHREADS, 1) decode_kernel(const __grid_constant__ Params P, const __grid_constant__ Args A) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int NS = Geo<T>::NS;
    Ctx c;
    {
        uint8_t* p = smem_raw;
        c.sm.ring = p; p += Geo<T>::RING;
        c.sm.xq = p; p += Geo<T>::XQ;
        c.sm.part_s = reinterpret_cast<float*>(p); p += Geo<T>::PART;
        c.sm.bt_s = reinterpret_cast<int*>(p); p += MAX_BLOCKS * 4;                // 2048
        c.sm.scale_s = reinterpret_cast<float*>(p); p += (2 * SCALE_BODY + SCALE_RING) * 4;   // 2048
        c.sm.out_s = reinterpret_cast<float*>(p); p += 64;                         // [T][8] attention statistics
        c.sm.red_s = reinterpret_cast<float*>(p); p += 2 * 8 * NCW * 4;            // 1024
        c.sm.xown = reinterpret_cast<float*>(p); p += 2 * 16 * 4;                  // 128
        c.sm.best_s = reinterpret_cast<u64*>(p); p += NCW * 8;                     // 128
        c.sm.full = reinterpret_cast<uint64_t*>(p); p += 6 * 8;
        c.sm.empty = reinterpret_cast<uint64_t*>(p); p += 6 * 8;
        c.sm.xscale_s = reinterpret_cast<float*>(p); p += 8;
        c.sm.abort_flag = reinterpret_cast<volatile int*>(p); p += 4;
        c.sm.quit_flag = reinterpret_cast<volatile int*>(p); p += 4;
        c.sm.act_s = reinterpret_cast<float*>(p); p += SPEC_T * DOWN_K * 4;
        c.sm.mix_s = reinterpret_cast<float*>(p); p += SPEC_T * DOWN_K * 4;
    }
    c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
    c.cta = blockIdx.x; c.grid = gridDim.x;
    c.cons_n = 0; c.red_n = 0; c.dead = false; c.prof = nullptr; c.wait_acc = 0; c.cur_op = 0; c.gemv_n = 0;
    c.limit_ns = (u64)A.spin_limit_ns;
    c.status = P.status;
    if (c.tid < SPEC_T * DOWN_K) c.sm.act_s[c.tid] = c.sm.mix_s[c.tid] = 0.f;
    if (c.tid == 0) {
        for (int i = 0; i < NS; i++) {
            mbar_init(&c.sm.full[i], 1);
            mbar_init(&c.sm.empty[i], NCW);
        }
        *c.sm.abort_flag = 0;
        *c.sm.quit_flag = 0;
        c.sm.xscale_s[0] = c.sm.xscale_s[1] = 1.0f;
        fence_barrier_init();
        fence_proxy_async();
    }
    for (int i = c.tid; i < P.max_seq / KV_BLOCK; i += NTHREADS) c.sm.bt_s[i] = P.block_table[i];
    __syncthreads();

    if (c.warp == NCW) {
        if (c.lane == 0) producer_main<S, Q8, T>(c, P, A);
        return;
    }

    // ---------------- consumers ----------------
    constexpr int WB = Q8 ? 1 : 2;                       // bytes per weight
    const int NL5 = P.n_layers * OPS_PER_LAYER;
    int xr0, xr1;                                        // residual rows this CTA owns
    cta_rows(S::HID, 1, c.cta, c.grid, xr0, xr1);
    int lr0, lr1;                                        // LM-head rows this CTA owns
    cta_rows(P.vocab, 1, c.cta, c.grid, lr0, lr1);

    // Reduce every CTA's winner stored in `slot` ([grid][2] words) at epoch `e`.
    auto reduce_key = [&](const u64* slot, uint32_t e) -> u64 {
        u64 key = 0;
        for (int i = c.tid; i < c.grid; i += NCT) {
            const float hi = ll_wait(c, slot + 2 * i, e, W_LM);
            const float lo = ll_wait(c, slot + 2 * i + 1, e, W_LM);
            const u64 k = ((u64)__float_as_uint(hi) << 32) | __float_as_uint(lo);
            key = k > key ? k : key;
        }
        key = warp_max_u64(key);
        if (c.lane == 0) c.sm.best_s[c.warp] = key;
        consumer_sync();
        u64 best = 0;
#pragma unroll
        for (int i = 0; i < NCW; i++) best = c.sm.best_s[i] > best ? c.sm.best_s[i] : best;
        consumer_sync();   // best_s is reused by the next reduction
        return best;
    };
    auto is_stop = [&](int token) {
        bool st = false;
        for (int i = 0; i < A.n_stop; i++) st |= (A.stop_ids[i] == token);
        return st;
    };
    // Embedding of `token` into this thread's residual elements and the owned master copy of token slot j.
    auto embed = [&](int token, int j, float (&xj)[2]) {
        if (token < 0 || token >= P.vocab) token = 0;    // only reachable after a failed wait
        load_embedding<S, Q8>(P, token, c.tid, xj[0], xj[1]);
        if (2 * c.tid >= xr0 && 2 * c.tid < xr1) c.sm.xown[j * 16 + 2 * c.tid - xr0] = xj[0];
        if (2 * c.tid + 1 >= xr0 && 2 * c.tid + 1 < xr1) c.sm.xown[j * 16 + 2 * c.tid + 1 - xr0] = xj[1];
    };
    // LM head over this CTA's vocabulary rows for T tokens: final RMSNorm, GEMV, optional logits dump,
    // per-CTA best key per token published at epoch eL.  `hn` returns the normalised hidden state.
    auto lm_head = [&](uint32_t eL, int op, int pos, float* logits, float (&x)[T][2], float (&hn)[T][2]) -> bool {
        prof_stamp(c, op, 0);
        scale_prefetch(c, P.lm_scale, lr0, lr1, true);
        const float2 nw = *reinterpret_cast<const float2*>(P.final_norm + 2 * c.tid);
        {
            const u64* ptrs[T];
            uint32_t eps[T];
            float v[2 * T];
#pragma unroll
            for (int j = 0; j < T; j++) { ptrs[j] = P.xl + (size_t)j * S::HID + 2 * c.tid; eps[j] = eL - 1; }
            ll_wait_pairs<T>(c, ptrs, eps, v, W_X);
#pragma unroll
            for (int j = 0; j < T; j++) { x[j][0] = v[2 * j]; x[j][1] = v[2 * j + 1]; }
        }
        stage_rmsnorm<S, Q8, T>(c, x, nw, hn);
        prof_stamp(c, op, 1);
        u64 best = 0;                                    // warp j tracks token j
        const float invT = A.inv_temperature;
        gemv_mma<Q8, T, true>(c, lr0, lr1, S::HID * WB, P.lm_scale, [&](int, int row, int tk, float v, bool ok) {
            if (!ok) return;
            if (logits) logits[(size_t)tk * P.vocab + row] = v;
            float score = v;
            if (invT != 0.f) {
                const uint32_t hsh = mk_mix32(A.seed, (uint32_t)(pos + tk), (uint32_t)row);
                const float u = ((float)(hsh >> 8) + 0.5f) * (1.0f / 16777216.0f);
                score = v * invT - __logf(-__logf(u));
            }
            const u64 key = score_key(score, row);
            best = key > best ? key : best;
        });
        if (c.warp < T) {
            best = warp_max_u64(best);
            if (c.lane == 0) {
                u64* slot = P.lml + ((size_t)c.warp * c.grid + c.cta) * 2;
                ll_store_bits(slot, eL, (uint32_t)(best >> 32));
                ll_store_bits(slot + 1, eL, (uint32_t)best);
            }
        }
        prof_stamp(c, op, 3);
        return consumer_any(c.dead);
    };

    if constexpr (T == 1) {
        // ---------------- plain decoding: one token per pass ----------------
        const int OPS = NL5 + 1;                         // epochs per step
        int steps_done = 0;
        bool stopped = false;
        u64 last_key = 0;
        for (int s = 0; s < A.n_steps; s++) {
            const uint32_t e0 = A.epoch_base + (uint32_t)s * (uint32_t)OPS;   // epoch of layer 0's op A
            const int pos = A.start_pos + s;
            c.prof = (A.prof && s == A.prof_step) ? A.prof + (size_t)c.cta * PROF_MAX_OPS * PROF_FIELDS : nullptr;
            if (c.cta == 0 && c.tid == 0 && A.step_ts) A.step_ts[s] = globaltimer();
            int token;
            if (s < A.n_forced) {
                token = A.forced[s];
            } else {
                last_key = reduce_key(P.lml, e0 - 1);        // previous step's LM-head epoch
                token = key_index(last_key);
                if (c.cta == 0 && c.tid == 0) A.tokens_out[s - 1] = last_key;
                if (is_stop(token)) {
                    stopped = true;
                    break;
                }
            }
            float x[T][2], hn[T][2];
            embed(token, 0, x[0]);
            bool failed = false;
            for (int l = 0; l < P.n_layers && !failed; l++)
                failed = run_layer<S, Q8, KVF32, T>(c, P, P.layer[l], P.xl, e0 + l * OPS_PER_LAYER, l * OPS_PER_LAYER, pos, x,
                                                    l == 0, false, xr0, xr1,
                                                    (A.resid_out && l == P.n_layers - 1) ? A.resid_out + (size_t)s * S::HID : nullptr);
            if (failed) break;
            if (s >= A.lm_from) {
                float* logits = A.logits_out ? A.logits_out + (size_t)s * P.vocab : nullptr;
                if (lm_head(e0 + (uint32_t)OPS - 1, NL5, pos, logits, x, hn)) break;
            }
            steps_done = s + 1;
        }
        // The prediction of the last step that ran (if it ran the LM head and nothing stopped us).
        if (!stopped && steps_done == A.n_steps && A.n_steps > 0 && A.n_steps - 1 >= A.lm_from) {
            const uint32_t eL = A.epoch_base + (uint32_t)A.n_steps * (uint32_t)OPS - 1;
            last_key = reduce_key(P.lml, eL);
            if (c.cta == 0 && c.tid == 0) A.tokens_out[A.n_steps - 1] = last_key;
        }
        if (c.tid == 0) *c.sm.quit_flag = 1;
        if (c.cta == 0 && c.tid == 0) {
            if (A.step_ts) A.step_ts[steps_done] = globaltimer();
            A.out_info[0] = steps_done;
            A.out_info[1] = (int)(A.epoch_base + (uint32_t)steps_done * (uint32_t)OPS);
            A.out_info[2] = A.start_pos + steps_done;
        }
    } else {
        // ---------------- speculative cycles: the pending token and a draft per pass ----------------
        // A cycle verifies [pending, draft] in one pass, emits the model's token after `pending` and,
        // if that token equals the draft, also the token after the draft.  The draft head then runs on
        // both positions (its own KV cache needs every position) and proposes the next draft from the
        // last accepted position.  Epochs per cycle: layers, LM head, fusion projection, draft layer
        // (5 ops), draft vocabulary head.
        const int OPSC = NL5 + 1 + 1 + OPS_PER_LAYER + 1;
        int pos = A.start_pos, emitted = 0, cyc = 0;
        int next_tok = A.first_tok, draft = A.first_draft;
        bool from_bak = false, done = false, failed = false;
        u64* draft_slot = P.lml + (size_t)T * c.grid * 2;
        for (;; cyc++) {
            const uint32_t e0 = A.epoch_base + (uint32_t)cyc * (uint32_t)OPSC;
            c.prof = (A.prof && cyc == A.prof_step) ? A.prof + (size_t)c.cta * PROF_MAX_OPS * PROF_FIELDS : nullptr;
            if (cyc > 0) {          // the previous cycle's draft
                const int row = key_index(reduce_key(draft_slot, e0 - 1));
                draft = (P.draft_ids && row >= 0 && row < P.draft_vocab) ? P.draft_ids[row] : row;
                if (done || failed || cyc == A.n_steps) break;
            } else if (A.n_steps == 0) {
                break;
            }
            if (c.cta == 0 && c.tid == 0 && A.step_ts) A.step_ts[cyc] = globaltimer();
            const int tok[2] = {next_tok, draft};
            float x[T][2], hn[T][2];
#pragma unroll
            for (int j = 0; j < T; j++) embed(tok[j], j, x[j]);
            for (int l = 0; l < P.n_layers && !failed; l++)
                failed = run_layer<S, Q8, KVF32, T>(c, P, P.layer[l], P.xl, e0 + l * OPS_PER_LAYER, l * OPS_PER_LAYER, pos, x,
                                                    l == 0, from_bak, xr0, xr1, nullptr);
            if (failed) { cyc++; break; }
            const uint32_t eL = e0 + NL5;
            float* logits = A.logits_out ? A.logits_out + (size_t)cyc * T * P.vocab : nullptr;
            if (lm_head(eL, NL5, pos, logits, x, hn)) { failed = true; cyc++; break; }
            // verify
            int yv[2];
            yv[0] = key_index(reduce_key(P.lml, eL));
            yv[1] = key_index(reduce_key(P.lml + (size_t)c.grid * 2, eL));
            const bool stop0 = is_stop(yv[0]);
            const int n_new = (yv[0] == tok[1] && !stop0 && emitted + 2 <= A.limit) ? 2 : 1;
            if (c.cta == 0 && c.tid == 0) {
                A.spec_out[emitted] = yv[0];
                if (n_new == 2) A.spec_out[emitted + 1] = yv[1];
                if (A.cycle_out) { A.cycle_out[2 * cyc] = n_new; A.cycle_out[2 * cyc + 1] = tok[1]; }
            }
            emitted += n_new;
            done = stop0 || (n_new == 2 && is_stop(yv[1])) || emitted >= A.limit;
            next_tok = yv[n_new - 1];
            from_bak = n_new == 1;

            // ---- draft head, op 1: u_j = fc([norm_e(embed(y_j)) | norm_h(h_j)])
            const uint32_t eF = eL + 1;
            {
                const int op = NL5 + 1;
                prof_stamp(c, op, 0);
                scale_prefetch(c, P.mtp_fc_scale, xr0, xr1, false);
                const float2 we = *reinterpret_cast<const float2*>(P.mtp_norm_e + 2 * c.tid);
                const float2 wh = *reinterpret_cast<const float2*>(P.mtp_norm_h + 2 * c.tid);
                float ev[T][2], ye[T][2], yh[T][2];
                float ss[2 * T], mx[2 * T];
#pragma unroll
                for (int j = 0; j < T; j++) {
                    int t2 = yv[j];
                    if (t2 < 0 || t2 >= P.vocab) t2 = 0;
                    load_embedding<S, Q8>(P, t2, c.tid, ev[j][0], ev[j][1]);
                    ye[j][0] = ev[j][0] * (1.0f + we.x); ye[j][1] = ev[j][1] * (1.0f + we.y);
                    yh[j][0] = hn[j][0] * (1.0f + wh.x); yh[j][1] = hn[j][1] * (1.0f + wh.y);
                    ss[2 * j] = ev[j][0] * ev[j][0] + ev[j][1] * ev[j][1];
                    ss[2 * j + 1] = hn[j][0] * hn[j][0] + hn[j][1] * hn[j][1];
                    mx[2 * j] = fmaxf(fabsf(ye[j][0]), fabsf(ye[j][1]));
                    mx[2 * j + 1] = fmaxf(fabsf(yh[j][0]), fabsf(yh[j][1]));
                }
                consumer_sum_max<2 * T>(c, ss, mx);
                constexpr int RB = 2 * S::HID * WB;
#pragma unroll
                for (int j = 0; j < T; j++) {
                    const float inv_e = rsqrtf(ss[2 * j] * (1.0f / S::HID) + S::EPS);
                    const float inv_h = rsqrtf(ss[2 * j + 1] * (1.0f / S::HID) + S::EPS);
                    const float scale = Q8 ? fixed_scale(fmaxf(mx[2 * j] * inv_e, mx[2 * j + 1] * inv_h)) : 1.0f;
                    uint8_t* xq = c.sm.xq + (size_t)(4 * j) * RB;
                    stage_pair<Q8>(xq, RB, 2 * c.tid, ye[j][0] * inv_e, ye[j][1] * inv_e, scale);
                    stage_pair<Q8>(xq, RB, S::HID + 2 * c.tid, yh[j][0] * inv_h, yh[j][1] * inv_h, scale);
                    if (c.tid == 0) c.sm.xscale_s[j] = 1.0f / scale;
                }
                consumer_sync();
                prof_stamp(c, op, 1);
                gemv_mma<Q8, T, false>(c, xr0, xr1, RB, P.mtp_fc_scale, [&](int, int row, int tk, float v, bool ok) {
                    if (ok) {
                        c.sm.xown[tk * 16 + row - xr0] = v;
                        ll_store(P.xml + (size_t)tk * S::HID + row, eF, v);
                    }
                });
                prof_stamp(c, op, 3);
            }
            // ---- draft head, ops 2..6: its decoder layer on positions pos, pos + 1 (own KV cache)
            failed = run_layer<S, Q8, KVF32, T>(c, P, P.mtp, P.xml, eF + 1, NL5 + 2, pos, x, false, false, xr0, xr1, nullptr);
            if (failed) { cyc++; break; }
            // ---- draft head, op 7: greedy choice over the draft vocabulary at the last accepted position
            {
                const uint32_t eV = eF + 1 + OPS_PER_LAYER;
                const int op = NL5 + 2 + OPS_PER_LAYER;
                prof_stamp(c, op, 0);
                int dr0, dr1;
                cta_rows(P.draft_vocab, 1, c.cta, c.grid, dr0, dr1);
                scale_prefetch(c, P.draft_scale, dr0, dr1, true);
                const float2 nw = *reinterpret_cast<const float2*>(P.mtp_norm + 2 * c.tid);
                float u[T][2], un[T][2];
                {
                    const u64* ptrs[T];
                    uint32_t eps[T];
                    float v[2 * T];
#pragma unroll
                    for (int j = 0; j < T; j++) { ptrs[j] = P.xml + (size_t)j * S::HID + 2 * c.tid; eps[j] = eV - 1; }
                    ll_wait_pairs<T>(c, ptrs, eps, v, W_X);
#pragma unroll
                    for (int j = 0; j < T; j++) { u[j][0] = v[2 * j]; u[j][1] = v[2 * j + 1]; }
                }
                stage_rmsnorm<S, Q8, T>(c, u, nw, un);
                prof_stamp(c, op, 1);
                u64 best = 0;
                const int want = n_new - 1;              // token slot whose draft counts
                gemv_mma<Q8, T, true>(c, dr0, dr1, S::HID * WB, P.draft_scale, [&](int, int row, int tk, float v, bool ok) {
                    if (!ok || tk != want) return;
                    const u64 key = score_key(v, row);
                    best = key > best ? key : best;
                });
                if (c.warp < T) {
                    best = warp_max_u64(best);
                    if (c.warp == want && c.lane == 0) {
                        ll_store_bits(draft_slot + 2 * c.cta, eV, (uint32_t)(best >> 32));
                        ll_store_bits(draft_slot + 2 * c.cta + 1, eV, (uint32_t)best);
                    }
                }
                prof_stamp(c, op, 3);
                failed = consumer_any(c.dead);
            }
            pos += n_new;
        }
        if (c.tid == 0) *c.sm.quit_flag = 1;
        if (from_bak && !failed) gdn_restore_state<S>(c, P);
        if (c.cta == 0 && c.tid == 0) {
            if (A.step_ts) A.step_ts[cyc] = globaltimer();
            A.out_info[0] = emitted;
            A.out_info[1] = (int)(A.epoch_base + (uint32_t)cyc * (uint32_t)OPSC);
            A.out_info[2] = pos;
            A.out_info[3] = next_tok;
            A.out_info[4] = draft;
            A.out_info[5] = cyc;
        }
    }
}

}  // namespace mk
