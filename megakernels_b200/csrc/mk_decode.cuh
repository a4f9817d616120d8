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
    float* part_s;      // [2][NCW][32] per-warp partial row sums of a ring chunk, alternating halves
    int* bt_s;          // block table copy [max_seq / KV_BLOCK]
    float* out_s;       // small per-op scratch (attention statistics)
    float* red_s;       // [2][2 * NCW] block-reduction scratch, alternating halves
    float* xown;        // fp32 master copy of the residual rows this CTA owns
    u64* best_s;        // [NCW] block-reduction scratch for 64-bit keys
    float* scale_s;     // per-row scales: two 128-row buffers for layer GEMVs, then the streaming ring
    float* xscale_s;    // [1] power-of-two factor that undoes the fixed-point scaling of the staged input
    uint64_t* full;     // [NSTAGE]
    uint64_t* empty;    // [NSTAGE]
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

// Slow path of every spin loop, entered once per 256 polls.
__device__ __noinline__ bool spin_slow(volatile int* abort_flag, int* status, u64 limit_ns, Spin& s, int where) {
    if (*abort_flag) return true;
    if (ld_volatile_i32(status) != 0) {
        *abort_flag = 1;
        return true;
    }
    const u64 now = globaltimer();
    if (!s.t0) {
        s.t0 = now;
    } else if (now - s.t0 > limit_ns) {
        if (atomicCAS(status, 0, ERR_TIMEOUT) == 0) {
            status[1] = where;
            status[2] = (int)blockIdx.x;
            status[3] = (int)threadIdx.x;
        }
        __threadfence();
        *abort_flag = 1;
        return true;
    }
    __nanosleep(40);
    return false;
}
#define MK_SPIN_FAIL(c, s, where) \
    ((((++(s).it) & 255u) == 0) && spin_slow((c).sm.abort_flag, (c).status, (c).limit_ns, (s), (where)))

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

// Sum and max over all consumer threads in one barrier, fixed order.
__device__ __forceinline__ void consumer_sum_max(Ctx& c, float& sum, float& mx) {
    float* buf = c.sm.red_s + (c.red_n++ & 1) * (2 * NCW);
    sum = warp_sum(sum);
    mx = warp_max(mx);
    if (c.lane == 0) {
        buf[c.warp] = sum;
        buf[NCW + c.warp] = mx;
    }
    consumer_sync();
    float t = 0.f, m = 0.f;
#pragma unroll
    for (int i = 0; i < NCW; i++) {
        t += buf[i];
        m = fmaxf(m, buf[NCW + i]);
    }
    sum = t;
    mx = m;
}

// ---- GEMV on the tensor cores ---------------------------------------------------------------------
// A weight row is cut into 64-byte k-blocks (64 int8 or 32 bf16 weights).  Rows are stored in groups
// of up to 8, k-block major: block kb of every row of the group, then block kb + 1, ...  One 128-bit
// load per lane therefore hands a warp an 8-row x 64-byte tile as the B operands of two MMAs
// (lane = 4 * row + quarter), with no conversion and no bank conflict.
//
// The input vector is the A operand.  fp32 inputs are made exact for the tensor cores by splitting:
//   int8 weights: x * 2^s rounded to a 28-bit integer, cut into four base-128 digits (int8 planes);
//                 integer MMAs (s8 x s8 -> s32) are exact, the digits recombine in fp32;
//   bf16 weights: x = p0 + p1 + p2 with three bf16 pieces (24 significant bits); bf16 MMAs with fp32
//                 accumulation.
// Plane m of the staged input is MMA row m, so one MMA handles all planes at once.  Each warp owns a
// k-slice (k-blocks warp, warp + 16, ...) of every row of the chunk; per-warp partial sums meet in
// shared memory and warp 0 finishes the rows after one barrier per chunk.
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

// Stage two consecutive inputs (elements k, k + 1) into the planes.  `scale` is the power of two that
// maps the vector's largest magnitude below 2^27 (int8 path only).
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
// Lane (g, t) returns, per block, the finished planes 2t and 2t + 1 of rows g and g + 8.
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
#pragma unroll 2
    for (int kb = warp; kb < nkb; kb += NCW) {
        uint4 w[4], x = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            w[q] = make_uint4(0, 0, 0, 0);
            if (g < n8[q]) w[q] = *reinterpret_cast<const uint4*>(tile[q] + (size_t)kb * n8[q] * 64);
        }
        if (xlive) x = *reinterpret_cast<const uint4*>(xrow + kb * 64);
#pragma unroll
        for (int b = 0; b < 2; b++) {           // two independent accumulator chains
            if (Q8) {
                mma_s8(ci[b], w[2 * b].x, w[2 * b + 1].x, w[2 * b].y, w[2 * b + 1].y, x.x, x.y);
                mma_s8(ci[b], w[2 * b].z, w[2 * b + 1].z, w[2 * b].w, w[2 * b + 1].w, x.z, x.w);
            } else {
                mma_bf16(cf[b], w[2 * b].x, w[2 * b + 1].x, w[2 * b].y, w[2 * b + 1].y, x.x, x.y);
                mma_bf16(cf[b], w[2 * b].z, w[2 * b + 1].z, w[2 * b].w, w[2 * b + 1].w, x.z, x.w);
            }
        }
    }
    const float pw0 = __uint_as_float((uint32_t)(127 + 14 * (t & 1)) << 23);       // 128^(2t) for the int8 digits
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

// Streams this CTA's rows [r0, r1) of a matrix with `rb`-byte rows out of the ring.  Two 8-row tiles
// form the 16-row A operand of an MMA, the input planes are its B operand (column n = plane n).
// Every warp owns a k-slice of all rows; per-warp partial sums meet in shared memory.
//   STREAM = false  (layer GEMVs, at most 64 rows per CTA): one barrier after the last chunk, then
//                   warps 0 and 1 finish the rows;
//   STREAM = true   (LM head): one barrier per chunk, warp 0 finishes that chunk's rows while the
//                   other warps move on.
// A finishing warp calls sink(lane, row, value, valid) on all of its lanes; `value` already carries
// the row's scale and the input's fixed-point scale.
template <bool Q8, bool STREAM, class Sink>
__device__ __forceinline__ void gemv_mma(Ctx& c, int r0, int r1, int rb, const float* __restrict__ row_scale,
                                         Sink&& sink) {
    const int rpc = SLOT_BYTES / rb;
    const int nkb = rb >> 6;
    const int g = c.lane >> 2, t = c.lane & 3;
    const uint8_t* xrow = c.sm.xq + g * rb + t * 16;
    const bool xlive = g < Planes<Q8>::N;
    const float* scales = STREAM ? c.sm.scale_s + 2 * SCALE_BODY : c.sm.scale_s + (c.gemv_n & 1) * SCALE_BODY;
    c.gemv_n++;
    float pend = 1.f;                            // scale fetched for the chunk four ahead (STREAM)
    int chunk = 0;
    for (int base = r0; base < r1; base += rpc, chunk++) {
        const int nr = min(rpc, r1 - base);
        const uint32_t n = c.cons_n++;
        const int slot = (int)(n % NSTAGE);
        if (STREAM && row_scale && c.warp == NCW - 1) {
            if (chunk > 0) c.sm.scale_s[2 * SCALE_BODY + ((chunk + 3) & 7) * 32 + c.lane] = pend;
            const int r = base + 4 * rpc + c.lane;
            pend = r < r1 ? row_scale[r] : 1.f;
        }
        if (c.prof && c.tid == 0) {
            const u64 t0 = globaltimer();
            mbar_wait(c, &c.sm.full[slot], (n / NSTAGE) & 1, W_FULL);
            c.wait_acc += globaltimer() - t0;
        } else {
            mbar_wait(c, &c.sm.full[slot], (n / NSTAGE) & 1, W_FULL);
        }
        const uint8_t* buf = c.sm.ring + (size_t)slot * SLOT_BYTES;
        // partial sums: [warp][row]; 64 rows per warp for layer GEMVs, two alternating 32-row halves when streaming
        float* part = STREAM ? c.sm.part_s + ((n & 1) * NCW + c.warp) * 32
                             : c.sm.part_s + c.warp * 64 + (base - r0);
        if (base == r0) MK_MARK(c, 8);
        for (int b0 = 0; b0 < nr; b0 += 32) {
            float v[4];
            mma_blocks<Q8>(buf, xrow, xlive, rb, nkb, nr, b0, c.warp, g, t, v);
            if (t == 0) {
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
            if (c.warp == 0) {
                const float* pp = c.sm.part_s + (n & 1) * NCW * 32 + c.lane;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < NCW; w++) v += pp[w * 32];
                const float rs = row_scale ? scales[(chunk & 7) * 32 + c.lane] : 1.f;
                sink(c.lane, base + c.lane, v * rs * *c.sm.xscale_s, c.lane < nr);
            }
        }
    }
    if (!STREAM) {
        MK_MARK(c, 9);
        consumer_sync();
        MK_MARK(c, 10);
        if (c.warp < 2) {
            const int idx = c.warp * 32 + c.lane;
            const float* pp = c.sm.part_s + idx;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < NCW; w++) v += pp[w * 64];
            const float rs = row_scale ? scales[idx] : 1.f;
            sink(c.lane, r0 + idx, v * rs * *c.sm.xscale_s, idx < r1 - r0);
            MK_MARK(c, 11);
        }
    }
}

// ---- producer ----------------------------------------------------------------------------------------
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
            const int slot = (int)(n % NSTAGE);
            if (n >= NSTAGE) {
                const uint32_t par = ((n / NSTAGE) - 1) & 1;
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
        const uint32_t first = n > NSTAGE ? n - NSTAGE : 0;
        for (uint32_t i = first; i < n; i++) {
            Spin s;
            s.t0 = 0;
            while (!mbar_try_wait(&c.sm.full[i % NSTAGE], (i / NSTAGE) & 1)) {
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

template <class S, bool Q8>
__device__ void producer_main(Ctx& c, const Params& P, const Args& A) {
    Producer pr(c);
    constexpr int WB = Q8 ? 1 : 2;  // bytes per weight
    for (int s = 0; s < A.n_steps && !pr.stop; s++) {
        for (int l = 0; l < P.n_layers && !pr.stop; l++) {
            const LayerP& L = P.layer[l];
            pr.stream(L.w_in, L.kind ? S::ATT_IN : S::GDN_IN, 1, S::HID * WB);
            pr.stream(L.w_out, S::HID, 1, S::MIX * WB);
            pr.stream(L.w_gu, 2 * S::INTER, 2, S::HID * WB);
            pr.stream(L.w_down, S::HID, 1, S::INTER * WB);
        }
        if (s >= A.lm_from) pr.stream(P.lm_head, P.vocab, 1, S::HID * WB);
    }
    pr.drain();
}

// ---- prologues ---------------------------------------------------------------------------------------
// RMSNorm of the residual stream into the GEMV input planes.  `x0`, `x1` are this thread's two
// elements (2*tid, 2*tid+1).  One block reduction yields both the sum of squares and the largest
// |x (1 + w)|, from which the fixed-point scale follows without a second pass.
template <class S, bool Q8>
__device__ __forceinline__ void stage_rmsnorm(Ctx& c, float x0, float x1, float2 g) {
    static_assert(S::HID == 2 * NCT, "two residual elements per consumer thread");
    constexpr int RB = Q8 ? S::HID : 2 * S::HID;
    const int k = 2 * c.tid;
    const float y0 = x0 * (1.0f + g.x), y1 = x1 * (1.0f + g.y);
    float ss = x0 * x0 + x1 * x1, mx = fmaxf(fabsf(y0), fabsf(y1));
    MK_MARK(c, 6);
    consumer_sum_max(c, ss, mx);
    MK_MARK(c, 7);
    const float inv = rsqrtf(ss * (1.0f / S::HID) + S::EPS);
    const float scale = Q8 ? fixed_scale(mx * inv) : 1.0f;
    stage_pair<Q8>(c.sm.xq, RB, k, y0 * inv, y1 * inv, scale);
    if (c.tid == 0) *c.sm.xscale_s = 1.0f / scale;
    consumer_sync();
}

// For inputs that need no norm: the fixed-point scale from this thread's largest magnitude (one
// block reduction on the int8 path, nothing on the bf16 path) ...
template <bool Q8>
__device__ __forceinline__ float block_scale(Ctx& c, float local_max) {
    if (!Q8) return 1.0f;
    float dummy = 0.f;
    consumer_sum_max(c, dummy, local_max);
    return fixed_scale(local_max);
}
// ... and the end of a staging phase: publish the inverse scale, make the planes visible.
__device__ __forceinline__ void finish_stage(Ctx& c, float scale) {
    if (c.tid == 0) *c.sm.xscale_s = 1.0f / scale;
    consumer_sync();
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

// ---- Gated DeltaNet recurrence ------------------------------------------------------------------------
// Task t < GDN_TASKS: head t / 8, value columns [16 * (t % 8), +16).  Warp w owns value column w of the
// slice; a lane holds 4 consecutive key indices of that column's state row.
template <class S>
__device__ bool gdn_op(Ctx& c, const Params& P, const LayerP& L, int pos, uint32_t e_proj, uint32_t e_out, int op) {
    static_assert(S::GDN_SLICE == NCW && S::LIN_DK == 128, "one warp per value column, 4 keys per lane");
    constexpr int SL = S::LIN_DV / S::GDN_SLICE;  // slices per head
    if (c.cta >= S::GDN_TASKS) return false;
    const int h = c.cta / SL, j = c.cta % SL;
    const int vcol = j * S::GDN_SLICE + c.warp;
    float* qkv_s = reinterpret_cast<float*>(c.sm.xq);   // [q 128 | k 128 | v 16 | b | a]
    float* srow = L.state + ((size_t)(h * S::LIN_DV + vcol) * S::LIN_DK) + 4 * c.lane;
    const float4 st = *reinterpret_cast<const float4*>(srow);   // issued before the wait on purpose
    const float a_log = L.A_log[h], dt_bias = L.dt_bias[h];
    constexpr int NCH = 2 * S::LIN_DK + S::GDN_SLICE;           // 272 conv channels this task needs
    if (c.tid < NCH) {
        int ch;
        if (c.tid < S::LIN_DK) ch = h * S::LIN_DK + c.tid;
        else if (c.tid < 2 * S::LIN_DK) ch = S::LIN_QK + h * S::LIN_DK + (c.tid - S::LIN_DK);
        else ch = 2 * S::LIN_QK + h * S::LIN_DV + j * S::GDN_SLICE + (c.tid - 2 * S::LIN_DK);
        const float4 taps = *reinterpret_cast<const float4*>(L.conv_w + 4 * ch);
        // every task keeps its own history of the channels it convolves (q and k of the head are
        // duplicated across the head's 8 tasks), so nothing here is shared between CTAs
        float* hist = L.conv_hist + ((size_t)c.cta * NCH + c.tid) * CONV_RING;
        const float h3 = hist[(pos - 3) & (CONV_RING - 1)];
        const float h2 = hist[(pos - 2) & (CONV_RING - 1)];
        const float h1 = hist[(pos - 1) & (CONV_RING - 1)];
        const float cur = ll_wait(c, P.projl + ch, e_proj, W_PROJ);
        float a = h3 * taps.x;
        a = fmaf(h2, taps.y, a);
        a = fmaf(h1, taps.z, a);
        a = fmaf(cur, taps.w, a);
        qkv_s[c.tid] = silu_f(a);
        hist[pos & (CONV_RING - 1)] = cur;
    } else if (c.tid < NCH + 2) {
        const int off = (c.tid == NCH ? S::B_OFF : S::A_OFF) + h;
        qkv_s[c.tid] = ll_wait(c, P.projl + off, e_proj, W_PROJ);
    }
    consumer_sync();
    prof_stamp(c, op, 1);
    const float4 q4 = *reinterpret_cast<const float4*>(qkv_s + 4 * c.lane);
    const float4 k4 = *reinterpret_cast<const float4*>(qkv_s + S::LIN_DK + 4 * c.lane);
    const float qn = warp_sum(q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w);
    const float kn = warp_sum(k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w);
    // x / max(|x|, 1e-6), and the 1/sqrt(dk) query scale
    const float qs = 0.08838834764831845f / fmaxf(sqrtf(qn), 1e-6f);
    const float ks = 1.0f / fmaxf(sqrtf(kn), 1e-6f);
    const float vval = qkv_s[2 * S::LIN_DK + c.warp];
    const float beta = sigmoid_f(qkv_s[NCH]);
    const float decay = expf(-expf(a_log) * softplus_f(qkv_s[NCH + 1] + dt_bias));
    const float kx = k4.x * ks, ky = k4.y * ks, kz = k4.z * ks, kw = k4.w * ks;
    float s0 = st.x * decay, s1 = st.y * decay, s2 = st.z * decay, s3 = st.w * decay;
    const float recalled = warp_sum(fmaf(s3, kw, fmaf(s2, kz, fmaf(s1, ky, s0 * kx))));
    const float delta = (vval - recalled) * beta;
    s0 = fmaf(kx, delta, s0);
    s1 = fmaf(ky, delta, s1);
    s2 = fmaf(kz, delta, s2);
    s3 = fmaf(kw, delta, s3);
    *reinterpret_cast<float4*>(srow) = make_float4(s0, s1, s2, s3);
    const float o = warp_sum(fmaf(s3, q4.w, fmaf(s2, q4.z, fmaf(s1, q4.y, s0 * q4.x)))) * qs;
    prof_stamp(c, op, 2);
    if (c.lane == 0) ll_store(P.mixl + h * S::LIN_DV + vcol, e_out, o);
    consumer_sync();  // the scratch aliases the GEMV input vector that the next prologue writes
    return true;
}

// ---- attention ---------------------------------------------------------------------------------------
template <bool F32> struct KvT;
template <> struct KvT<true> { typedef float type; };
template <> struct KvT<false> { typedef __nv_bfloat16 type; };

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

// Split-K decode attention over the paged cache.  Task (g, s): KV head g, positions
// [s * ch, min(n, (s + 1) * ch)), run by CTA s * NKV + g.  Cached K and V rows of the task are
// requested before the task waits for its query, so that only one memory round trip sits between
// the projection and the scores.  With one split the task publishes the normalised output itself;
// otherwise every task publishes (acc, m, l) partials as flag-in-data words and then merges a
// 1/nsplit share of the head group's outputs from all partials, in a fixed order.
template <class S, bool KVF32>
__device__ bool attn_op(Ctx& c, const Params& P, const LayerP& L, int pos, uint32_t e_proj, uint32_t e_out, int op) {
    static_assert(S::HD == 256 && S::QPK == 4 && NCW == 16 && S::ROT == 64, "thread mapping below");
    constexpr int NOUT = S::QPK * S::HD;        // outputs per KV head
    constexpr int PFK = 1, PFV = 16;            // rows prefetched per warp (K) and per thread (V)
    const int n = pos + 1;
    const int max_splits = min(c.grid / S::NKV, MAX_SPLITS);
    const int ch = attn_chunk(n, max_splits);
    const int nsplit = (n + ch - 1) / ch;
    if (c.cta >= nsplit * S::NKV) return false;
    const int g = c.cta % S::NKV, sp = c.cta / S::NKV;
    const int p0 = sp * ch, p1 = min(n, p0 + ch);
    const int np = p1 - p0;
    const bool has_new = (p1 == n);

    float* q_s = reinterpret_cast<float*>(c.sm.xq);   // [4][256] normalised, rotated, pre-scaled queries
    float* knew_s = q_s + S::QPK * S::HD;       // [256]
    float* vnew_s = knew_s + S::HD;             // [256]
    float* sc_s = vnew_s + S::HD;               // [4][ch] scores, then probabilities
    float* stat_s = c.sm.out_s;                 // [4] m, [4] l

    const size_t kv_head_stride = (size_t)KV_BLOCK * S::HD;
    auto kv_elem = [&](int p) -> size_t {
        const int blk = c.sm.bt_s[p >> 6];
        return ((size_t)blk * S::NKV + g) * kv_head_stride + (size_t)(p & (KV_BLOCK - 1)) * S::HD;
    };
    // -- 0. request cached rows early: K rows of this warp's positions, V elements of this thread's dim
    const int d = c.tid & (S::HD - 1), hp = c.tid >> 8;
    float kpre[PFK][8], vpre[PFV];
#pragma unroll
    for (int i = 0; i < PFK; i++) {
        const int p = p0 + c.warp + i * NCW;
#pragma unroll
        for (int j = 0; j < 8; j++) kpre[i][j] = 0.f;
        if (p < p1 && p != pos) load8<KVF32>(L.k_cache, kv_elem(p) + 8 * c.lane, kpre[i]);
    }
#pragma unroll
    for (int i = 0; i < PFV; i++) {
        const int p = p0 + i;
        vpre[i] = (p < p1 && p != pos) ? load1<KVF32>(L.v_cache, kv_elem(p) + d) : 0.f;
    }

    // -- 1. q (4 heads), new k, new v from the projection words; per-head RMSNorm; partial RoPE
    {
        const int hh = c.warp >> 2, qd = c.warp & 3;        // head within group, 64-wide quarter
        const int dd = qd * 64 + 2 * c.lane;
        const u64* const ptrs[2] = {P.projl + (g * S::QPK + hh) * 2 * S::HD + dd,
                                    hh == 0 ? P.projl + S::ATT_K_OFF + g * S::HD + dd
                                            : (hh == 1 ? P.projl + S::ATT_V_OFF + g * S::HD + dd : nullptr)};
        const uint32_t eps[2] = {e_proj, e_proj};
        // norm weights and rotation angles are requested before the wait
        const float2 qw = *reinterpret_cast<const float2*>(L.q_norm + dd);
        const float2 kw = hh == 0 ? *reinterpret_cast<const float2*>(L.k_norm + dd) : make_float2(0.f, 0.f);
        float cs0 = 1.f, sn0 = 0.f, cs1 = 1.f, sn1 = 0.f;
        if (qd == 0) {
            const int i0 = (2 * c.lane) & 31;
            cs0 = P.rope_cos[(size_t)pos * (S::ROT / 2) + i0];
            sn0 = P.rope_sin[(size_t)pos * (S::ROT / 2) + i0];
            cs1 = P.rope_cos[(size_t)pos * (S::ROT / 2) + i0 + 1];
            sn1 = P.rope_sin[(size_t)pos * (S::ROT / 2) + i0 + 1];
        }
        float v4[4];
        ll_wait_pairs<2>(c, ptrs, eps, v4, W_PROJ);
        float a = v4[0], b = v4[1];
        float ka = hh == 0 ? v4[2] : 0.f, kb = hh == 0 ? v4[3] : 0.f;
        const float va = v4[2], vb = v4[3];
        float* buf = c.sm.red_s + (c.red_n++ & 1) * (2 * NCW);      // q sums [16], k sums [4]
        const float sq = warp_sum(a * a + b * b);
        const float sk = warp_sum(ka * ka + kb * kb);
        if (c.lane == 0) {
            buf[c.warp] = sq;
            if (hh == 0) buf[NCW + qd] = sk;
        }
        consumer_sync();
        const float qss = buf[hh * 4] + buf[hh * 4 + 1] + buf[hh * 4 + 2] + buf[hh * 4 + 3];
        const float qinv = rsqrtf(qss * (1.0f / S::HD) + S::EPS);
        a = a * qinv * (1.0f + qw.x);
        b = b * qinv * (1.0f + qw.y);
        if (qd == 0) {
            // dims [0,32) live in lanes 0..15, their partners [32,64) in lanes 16..31
            const float pa = __shfl_xor_sync(0xffffffffu, a, 16), pb = __shfl_xor_sync(0xffffffffu, b, 16);
            if (c.lane < 16) { a = a * cs0 - pa * sn0; b = b * cs1 - pb * sn1; }
            else { a = a * cs0 + pa * sn0; b = b * cs1 + pb * sn1; }
        }
        q_s[hh * S::HD + dd] = a * 0.0625f;          // 1/sqrt(256), exact
        q_s[hh * S::HD + dd + 1] = b * 0.0625f;
        if (hh == 0) {
            const float kss = buf[NCW] + buf[NCW + 1] + buf[NCW + 2] + buf[NCW + 3];
            const float kinv = rsqrtf(kss * (1.0f / S::HD) + S::EPS);
            ka = ka * kinv * (1.0f + kw.x);
            kb = kb * kinv * (1.0f + kw.y);
            if (qd == 0) {
                const float pa = __shfl_xor_sync(0xffffffffu, ka, 16), pb = __shfl_xor_sync(0xffffffffu, kb, 16);
                if (c.lane < 16) { ka = ka * cs0 - pa * sn0; kb = kb * cs1 - pb * sn1; }
                else { ka = ka * cs0 + pa * sn0; kb = kb * cs1 + pb * sn1; }
            }
            knew_s[dd] = round_kv<KVF32>(ka);
            knew_s[dd + 1] = round_kv<KVF32>(kb);
        }
        if (hh == 1) {
            vnew_s[dd] = round_kv<KVF32>(va);
            vnew_s[dd + 1] = round_kv<KVF32>(vb);
        }
        consumer_sync();
        prof_stamp(c, op, 1);
    }
    // -- 2. append the new position (the task that owns it)
    if (has_new && c.tid < S::HD) {
        const size_t e = kv_elem(pos) + c.tid;
        store1<KVF32>(L.k_cache, e, knew_s[c.tid]);
        store1<KVF32>(L.v_cache, e, vnew_s[c.tid]);
    }
    // -- 3. scores: one warp per position, 8 dims per lane
    {
        float q[S::QPK][8];
#pragma unroll
        for (int hh = 0; hh < S::QPK; hh++) {
            const float4 x = *reinterpret_cast<const float4*>(q_s + hh * S::HD + 8 * c.lane);
            const float4 y = *reinterpret_cast<const float4*>(q_s + hh * S::HD + 8 * c.lane + 4);
            q[hh][0] = x.x; q[hh][1] = x.y; q[hh][2] = x.z; q[hh][3] = x.w;
            q[hh][4] = y.x; q[hh][5] = y.y; q[hh][6] = y.z; q[hh][7] = y.w;
        }
        auto score = [&](int p, const float (&kk)[8]) {
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                d0 = fmaf(q[0][i], kk[i], d0);
                d1 = fmaf(q[1][i], kk[i], d1);
                d2 = fmaf(q[2][i], kk[i], d2);
                d3 = fmaf(q[3][i], kk[i], d3);
            }
            d0 = warp_sum(d0); d1 = warp_sum(d1); d2 = warp_sum(d2); d3 = warp_sum(d3);
            if (c.lane == 0) {
                sc_s[0 * ch + (p - p0)] = d0;
                sc_s[1 * ch + (p - p0)] = d1;
                sc_s[2 * ch + (p - p0)] = d2;
                sc_s[3 * ch + (p - p0)] = d3;
            }
        };
#pragma unroll
        for (int i = 0; i < PFK; i++) {
            const int p = p0 + c.warp + i * NCW;
            if (p < p1) {
                if (p == pos) {
#pragma unroll
                    for (int j = 0; j < 8; j++) kpre[i][j] = knew_s[8 * c.lane + j];
                }
                score(p, kpre[i]);
            }
        }
        for (int p = p0 + c.warp + PFK * NCW; p < p1; p += NCW) {
            float kk[8];
            if (p == pos) {
#pragma unroll
                for (int j = 0; j < 8; j++) kk[j] = knew_s[8 * c.lane + j];
            } else {
                load8<KVF32>(L.k_cache, kv_elem(p) + 8 * c.lane, kk);
            }
            score(p, kk);
        }
    }
    consumer_sync();
    // -- 4. softmax statistics: warp hh < 4 handles head hh
    if (c.warp < S::QPK) {
        float* row = sc_s + c.warp * ch;
        float m = -INFINITY;
        for (int i = c.lane; i < np; i += 32) m = fmaxf(m, row[i]);
        m = warp_max(m);
        float l = 0.f;
        for (int i = c.lane; i < np; i += 32) {
            const float e = __expf(row[i] - m);
            row[i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (c.lane == 0) {
            stat_s[c.warp] = m;
            stat_s[S::QPK + c.warp] = l;
        }
    }
    consumer_sync();
    // -- 5. weighted values: thread -> dim d, heads 2*hp and 2*hp+1
    float acc0 = 0.f, acc1 = 0.f;
    {
        const float* pr0 = sc_s + (2 * hp) * ch;
        const float* pr1 = sc_s + (2 * hp + 1) * ch;
#pragma unroll
        for (int i = 0; i < PFV; i++) {
            if (i < np) {
                const float v = (p0 + i == pos) ? vnew_s[d] : vpre[i];
                acc0 = fmaf(pr0[i], v, acc0);
                acc1 = fmaf(pr1[i], v, acc1);
            }
        }
        int i = PFV;
        for (; i + 8 <= np; i += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int p = p0 + i + u;
                v[u] = (p == pos) ? vnew_s[d] : load1<KVF32>(L.v_cache, kv_elem(p) + d);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                acc0 = fmaf(pr0[i + u], v[u], acc0);
                acc1 = fmaf(pr1[i + u], v[u], acc1);
            }
        }
        for (; i < np; i++) {
            const int p = p0 + i;
            const float v = (p == pos) ? vnew_s[d] : load1<KVF32>(L.v_cache, kv_elem(p) + d);
            acc0 = fmaf(pr0[i], v, acc0);
            acc1 = fmaf(pr1[i], v, acc1);
        }
    }
    u64* out = P.mixl + (size_t)(g * S::QPK) * S::HD;
    prof_stamp(c, op, 2);
    if (nsplit == 1) {
        ll_store(out + (2 * hp) * S::HD + d, e_out, acc0 / stat_s[S::QPK + 2 * hp]);
        ll_store(out + (2 * hp + 1) * S::HD + d, e_out, acc1 / stat_s[S::QPK + 2 * hp + 1]);
        // The appended K/V row is read by other CTAs from the next step on.  They get there only
        // through words this CTA publishes after this fence, so the fence can sit off the critical path.
        __threadfence();
        consumer_sync();  // scratch aliases the GEMV input planes that the next prologue writes
        return true;
    }
    // -- 6. partials as flag-in-data words: acc [4][256], then (m, l) per head
    u64* part = P.attn_part + ((size_t)g * MAX_SPLITS + sp) * S::PART_STRIDE;
    ll_store(part + (2 * hp) * S::HD + d, e_out, acc0);
    ll_store(part + (2 * hp + 1) * S::HD + d, e_out, acc1);
    if (c.tid < 2 * S::QPK) ll_store(part + NOUT + c.tid, e_out, stat_s[(c.tid & 1) * S::QPK + (c.tid >> 1)]);
    // -- 7. merge this task's share of the outputs.  `tpo` threads share one output, each takes the
    //       splits s = sub, sub + tpo, ...; a fixed shuffle tree combines them.
    const int opc = (NOUT + nsplit - 1) / nsplit;           // outputs per task
    int tpo = 1;
    while (tpo < 32 && 2 * tpo * opc <= NCT && tpo < nsplit) tpo *= 2;
    const int oi = c.tid / tpo, sub = c.tid % tpo;
    const int o = sp * opc + oi;
    const bool live = oi < opc && o < NOUT;
    const int h = o / S::HD;
    const u64* pg = P.attn_part + (size_t)g * MAX_SPLITS * S::PART_STRIDE;
    constexpr int SPT = 4;                                   // splits per thread at most (MAX_SPLITS / 32)
    float mv[SPT], lv[SPT], av[SPT];
    {
        u64 wa[SPT], wm[SPT], wl[SPT];
#pragma unroll
        for (int i = 0; i < SPT; i++) {
            const int s2 = sub + i * tpo;
            wa[i] = wm[i] = wl[i] = 0;
            if (live && s2 < nsplit) {
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
                if (live && s2 < nsplit) {
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
            const bool have = live && sub + i * tpo < nsplit;
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
    if (live && sub == 0) ll_store(out + o, e_out, Os / Ls);
    __threadfence();      // K/V append before anything this CTA publishes later (see above)
    consumer_sync();      // scratch aliases the GEMV input planes that the next prologue writes
    return true;
}

// ---- the kernel ------------------------------------------------------------------------------------------
__constant__ Params c_params[2 * MAX_ENGINES];   // per engine handle: its block, and the variant with built-in scratch

template <class S, bool Q8, bool KVF32>
__global__ void __launch_bounds__(NTHREADS, 1) decode_kernel(const int pslot, const __grid_constant__ Args A) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const Params& P = c_params[pslot];
    Ctx c;
    {
        uint8_t* p = smem_raw;
        c.sm.ring = p; p += SMEM_RING;
        c.sm.xq = p; p += SMEM_XQ;
        c.sm.part_s = reinterpret_cast<float*>(p); p += 2 * NCW * 32 * 4;          // 4096
        c.sm.bt_s = reinterpret_cast<int*>(p); p += MAX_BLOCKS * 4;                // 2048
        c.sm.scale_s = reinterpret_cast<float*>(p); p += (2 * SCALE_BODY + SCALE_RING) * 4;   // 2048
        c.sm.out_s = reinterpret_cast<float*>(p); p += 64;
        c.sm.red_s = reinterpret_cast<float*>(p); p += 2 * 2 * NCW * 4;            // 256
        c.sm.xown = reinterpret_cast<float*>(p); p += 16 * 4;                      // 64
        c.sm.best_s = reinterpret_cast<u64*>(p); p += NCW * 8;                     // 128
        c.sm.full = reinterpret_cast<uint64_t*>(p); p += NSTAGE * 8;
        c.sm.empty = reinterpret_cast<uint64_t*>(p); p += NSTAGE * 8;
        c.sm.xscale_s = reinterpret_cast<float*>(p); p += 8;
        c.sm.abort_flag = reinterpret_cast<volatile int*>(p); p += 4;
        c.sm.quit_flag = reinterpret_cast<volatile int*>(p); p += 4;
    }
    c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
    c.cta = blockIdx.x; c.grid = gridDim.x;
    c.cons_n = 0; c.red_n = 0; c.dead = false; c.prof = nullptr; c.wait_acc = 0; c.cur_op = 0; c.gemv_n = 0;
    c.limit_ns = (u64)A.spin_limit_ns;
    c.status = P.status;
    if (c.tid == 0) {
        for (int i = 0; i < NSTAGE; i++) {
            mbar_init(&c.sm.full[i], 1);
            mbar_init(&c.sm.empty[i], NCW);
        }
        *c.sm.abort_flag = 0;
        *c.sm.quit_flag = 0;
        *c.sm.xscale_s = 1.0f;
        fence_barrier_init();
        fence_proxy_async();
    }
    for (int i = c.tid; i < P.max_seq / KV_BLOCK; i += NTHREADS) c.sm.bt_s[i] = P.block_table[i];
    __syncthreads();

    if (c.warp == NCW) {
        if (c.lane == 0) producer_main<S, Q8>(c, P, A);
        return;
    }

    // ---------------- consumers ----------------
    constexpr int WB = Q8 ? 1 : 2;                       // bytes per weight
    const int OPS = P.n_layers * OPS_PER_LAYER + 1;     // epochs per step
    int xr0, xr1;                                        // residual rows this CTA owns
    cta_rows(S::HID, 1, c.cta, c.grid, xr0, xr1);
    int lr0, lr1;                                        // LM-head rows this CTA owns
    cta_rows(P.vocab, 1, c.cta, c.grid, lr0, lr1);
    int steps_done = 0;
    bool stopped = false;
    u64 last_key = 0;

    // Reduce every CTA's LM-head winner of the step whose LM epoch is `e`.
    auto reduce_token = [&](uint32_t e) -> u64 {
        u64 key = 0;
        for (int i = c.tid; i < c.grid; i += NCT) {
            const float hi = ll_wait(c, P.lml + 2 * i, e, W_LM);
            const float lo = ll_wait(c, P.lml + 2 * i + 1, e, W_LM);
            const u64 k = ((u64)__float_as_uint(hi) << 32) | __float_as_uint(lo);
            key = k > key ? k : key;
        }
        key = warp_max_u64(key);
        if (c.lane == 0) c.sm.best_s[c.warp] = key;
        consumer_sync();
        u64 best = 0;
#pragma unroll
        for (int i = 0; i < NCW; i++) best = c.sm.best_s[i] > best ? c.sm.best_s[i] : best;
        consumer_sync();   // best_s is reused by the next LM head
        return best;
    };

    for (int s = 0; s < A.n_steps; s++) {
        const uint32_t e0 = A.epoch_base + (uint32_t)s * (uint32_t)OPS;   // epoch of layer 0's op A
        const int pos = A.start_pos + s;
        c.prof = (A.prof && s == A.prof_step) ? A.prof + (size_t)c.cta * PROF_MAX_OPS * PROF_FIELDS : nullptr;
        if (c.cta == 0 && c.tid == 0 && A.step_ts) A.step_ts[s] = globaltimer();
        int token;
        if (s < A.n_forced) {
            token = A.forced[s];
        } else {
            last_key = reduce_token(e0 - 1);             // previous step's LM-head epoch
            token = key_index(last_key);
            if (c.cta == 0 && c.tid == 0) A.tokens_out[s - 1] = last_key;
            bool is_stop = false;
            for (int i = 0; i < A.n_stop; i++) is_stop |= (A.stop_ids[i] == token);
            if (is_stop) {
                stopped = true;
                break;
            }
        }
        if (token < 0 || token >= P.vocab) token = 0;    // only reachable after a failed wait

        float x0, x1;                                    // residual elements 2*tid, 2*tid+1
        load_embedding<S, Q8>(P, token, c.tid, x0, x1);
        if (2 * c.tid >= xr0 && 2 * c.tid < xr1) c.sm.xown[2 * c.tid - xr0] = x0;
        if (2 * c.tid + 1 >= xr0 && 2 * c.tid + 1 < xr1) c.sm.xown[2 * c.tid + 1 - xr0] = x1;

        bool failed = false;
        for (int l = 0; l < P.n_layers; l++) {
            const LayerP& L = P.layer[l];
            const uint32_t eA = e0 + l * OPS_PER_LAYER, eB = eA + 1, eC = eA + 2, eD = eA + 3, eE = eA + 4;
            const bool attn = L.kind != 0;
            const int op0 = l * OPS_PER_LAYER;
            // ---- A: in-projection
            {
                prof_stamp(c, op0, 0);
                int r0, r1;
                cta_rows(attn ? S::ATT_IN : S::GDN_IN, 1, c.cta, c.grid, r0, r1);
                scale_prefetch(c, L.s_in, r0, r1, false);
                // the norm weights are requested before the wait so that their latency hides behind it
                const float2 nw = *reinterpret_cast<const float2*>(L.in_norm + 2 * c.tid);
                if (l > 0) ll_wait2(c, P.xl + 2 * c.tid, eA - 1, W_X, x0, x1);
                stage_rmsnorm<S, Q8>(c, x0, x1, nw);
                prof_stamp(c, op0, 1);
                gemv_mma<Q8, false>(c, r0, r1, S::HID * WB, L.s_in, [&](int, int row, float v, bool ok) {
                    if (ok) ll_store(P.projl + row, eA, v);
                });
                prof_stamp(c, op0, 3);
            }
            // ---- B: mixer
            prof_stamp(c, op0 + 1, 0);
            const bool had_task = attn ? attn_op<S, KVF32>(c, P, L, pos, eA, eB, op0 + 1)
                                       : gdn_op<S>(c, P, L, pos, eA, eB, op0 + 1);
            prof_stamp(c, op0 + 1, 3);
            // ---- C: out-projection + residual
            {
                const int op = op0 + 2;
                prof_stamp(c, op, 0);
                scale_prefetch(c, L.s_out, xr0, xr1, false);
                if (!had_task) gate_on_samples(c, P.mixl, S::MIX, eB);
                // each thread stages 4 consecutive mixer outputs; a warp covers 128 = one DeltaNet head
                const int k = 4 * c.tid;
                float m[4];
                const float4 gw = attn ? make_float4(0.f, 0.f, 0.f, 0.f)
                                       : *reinterpret_cast<const float4*>(L.gdn_norm + (k % S::LIN_DV));
                {
                    const u64* aux = attn ? P.projl + (k / S::HD) * 2 * S::HD + S::HD + (k % S::HD)   // sigmoid gate
                                          : P.projl + S::Z_OFF + k;                                    // z
                    const u64* const ptrs[4] = {P.mixl + k, P.mixl + k + 2, aux, aux + 2};
                    const uint32_t eps[4] = {eB, eB, eA, eA};
                    float v[8];
                    ll_wait_pairs<4>(c, ptrs, eps, v, W_MIX);
                    if (attn) {
#pragma unroll
                        for (int i = 0; i < 4; i++) m[i] = v[i] * sigmoid_f(v[4 + i]);
                    } else {
                        const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
                        const float inv = rsqrtf(ss * (1.0f / S::LIN_DV) + S::EPS);
                        m[0] = v[0] * inv * gw.x * silu_f(v[4]);
                        m[1] = v[1] * inv * gw.y * silu_f(v[5]);
                        m[2] = v[2] * inv * gw.z * silu_f(v[6]);
                        m[3] = v[3] * inv * gw.w * silu_f(v[7]);
                    }
                }
                const float scale = block_scale<Q8>(c, fmaxf(fmaxf(fabsf(m[0]), fabsf(m[1])), fmaxf(fabsf(m[2]), fabsf(m[3]))));
                stage_pair<Q8>(c.sm.xq, S::MIX * WB, k, m[0], m[1], scale);
                stage_pair<Q8>(c.sm.xq, S::MIX * WB, k + 2, m[2], m[3], scale);
                finish_stage(c, scale);
                prof_stamp(c, op, 1);
                gemv_mma<Q8, false>(c, xr0, xr1, S::MIX * WB, L.s_out, [&](int, int row, float v, bool ok) {
                    if (ok) {
                        const float xn = c.sm.xown[row - xr0] + v;
                        c.sm.xown[row - xr0] = xn;
                        ll_store(P.xl + row, eC, xn);
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
                ll_wait2(c, P.xl + 2 * c.tid, eC, W_X, x0, x1);
                stage_rmsnorm<S, Q8>(c, x0, x1, nw);
                prof_stamp(c, op, 1);
                gemv_mma<Q8, false>(c, r0, r1, S::HID * WB, L.s_gu, [&](int lane, int row, float v, bool ok) {
                    // rows alternate gate, up; chunks hold whole pairs, so the partner is the next lane
                    const float up = __shfl_down_sync(0xffffffffu, v, 1);
                    if (ok && !(lane & 1)) ll_store(P.actl + (row >> 1), eD, silu_f(v) * up);
                });
                prof_stamp(c, op, 3);
            }
            // ---- E: down-projection + residual
            {
                const int op = op0 + 4;
                prof_stamp(c, op, 0);
                scale_prefetch(c, L.s_down, xr0, xr1, false);
                float a[8];
                float mx = 0.f;
                {
                    const u64* ptrs[4];
                    const uint32_t eps[4] = {eD, eD, eD, eD};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int k = 2 * c.tid + j * 2 * NCT;
                        ptrs[j] = k < S::INTER ? P.actl + k : nullptr;
                    }
                    ll_wait_pairs<4>(c, ptrs, eps, a, W_ACT);
#pragma unroll
                    for (int j = 0; j < 8; j++) mx = fmaxf(mx, fabsf(a[j]));
                }
                const float scale = block_scale<Q8>(c, mx);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int k = 2 * c.tid + j * 2 * NCT;
                    if (k < S::INTER) stage_pair<Q8>(c.sm.xq, S::INTER * WB, k, a[2 * j], a[2 * j + 1], scale);
                }
                finish_stage(c, scale);
                prof_stamp(c, op, 1);
                const bool last = l == P.n_layers - 1;
                gemv_mma<Q8, false>(c, xr0, xr1, S::INTER * WB, L.s_down, [&](int, int row, float v, bool ok) {
                    if (ok) {
                        const float xn = c.sm.xown[row - xr0] + v;
                        c.sm.xown[row - xr0] = xn;
                        ll_store(P.xl + row, eE, xn);
                        if (A.resid_out && last) A.resid_out[(size_t)s * S::HID + row] = xn;
                    }
                });
                prof_stamp(c, op, 3);
                failed = consumer_any(c.dead);
            }
            if (failed) break;
        }
        if (failed) break;
        // ---- LM head
        if (s >= A.lm_from) {
            const uint32_t eL = e0 + (uint32_t)OPS - 1;
            const int op = P.n_layers * OPS_PER_LAYER;
            prof_stamp(c, op, 0);
            scale_prefetch(c, P.lm_scale, lr0, lr1, true);
            const float2 nw = *reinterpret_cast<const float2*>(P.final_norm + 2 * c.tid);
            ll_wait2(c, P.xl + 2 * c.tid, eL - 1, W_X, x0, x1);
            stage_rmsnorm<S, Q8>(c, x0, x1, nw);
            prof_stamp(c, op, 1);
            u64 best = 0;
            float* logits = A.logits_out ? A.logits_out + (size_t)s * P.vocab : nullptr;
            const float invT = A.inv_temperature;
            gemv_mma<Q8, true>(c, lr0, lr1, S::HID * WB, P.lm_scale, [&](int, int row, float v, bool ok) {
                if (!ok) return;
                if (logits) logits[row] = v;
                float score = v;
                if (invT != 0.f) {
                    const uint32_t hsh = mk_mix32(A.seed, (uint32_t)pos, (uint32_t)row);
                    const float u = ((float)(hsh >> 8) + 0.5f) * (1.0f / 16777216.0f);
                    score = v * invT - __logf(-__logf(u));
                }
                const u64 key = score_key(score, row);
                best = key > best ? key : best;
            });
            if (c.warp == 0) {
                best = warp_max_u64(best);
                if (c.lane == 0) {
                    ll_store_bits(P.lml + 2 * c.cta, eL, (uint32_t)(best >> 32));
                    ll_store_bits(P.lml + 2 * c.cta + 1, eL, (uint32_t)best);
                }
            }
            prof_stamp(c, op, 3);
            failed = consumer_any(c.dead);
            if (failed) break;
        }
        steps_done = s + 1;
    }
    // The prediction of the last step that ran (if it ran the LM head and nothing stopped us).
    if (!stopped && steps_done == A.n_steps && A.n_steps > 0 && A.n_steps - 1 >= A.lm_from) {
        const uint32_t eL = A.epoch_base + (uint32_t)A.n_steps * (uint32_t)OPS - 1;
        last_key = reduce_token(eL);
        if (c.cta == 0 && c.tid == 0) A.tokens_out[A.n_steps - 1] = last_key;
    }
    if (c.tid == 0) *c.sm.quit_flag = 1;
    if (c.cta == 0 && c.tid == 0) {
        if (A.step_ts) A.step_ts[steps_done] = globaltimer();
        A.out_info[0] = steps_done;
        A.out_info[1] = (int)(A.epoch_base + (uint32_t)steps_done * (uint32_t)OPS);
        A.out_info[2] = A.start_pos + steps_done;
    }
}

}  // namespace mk
