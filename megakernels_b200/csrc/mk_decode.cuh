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
    float* xs;          // GEMV input vector (permuted), or mixer scratch
    float* scale_s;     // LM-head per-row scales of this CTA
    float* out_s;       // raw row sums of a body GEMV [MAX_BODY_ROWS * 2]
    float* red_s;       // [2][NCW] block-reduction scratch, alternating halves
    float* xown;        // fp32 master copy of the residual rows this CTA owns
    u64* best_s;        // [NCW] per-warp LM-head winners
    uint64_t* full;     // [NSTAGE]
    uint64_t* empty;    // [NSTAGE]
    volatile int* abort_flag;
    volatile int* quit_flag;
    volatile int* tok_s;
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
};

// Per-op timestamps (enter, inputs staged, work done, outputs published), consumer thread 0 only.
__device__ __forceinline__ void prof_stamp(Ctx& c, int op, int field) {
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

// Pause between two polls of a word that is not ready.  Thousands of threads poll the same few
// cache lines; without a pause their loads queue up in front of the store they are waiting for.
#ifndef MK_POLL_SLEEP_NS
#define MK_POLL_SLEEP_NS 0
#endif
__device__ __forceinline__ void poll_backoff() {
    if (MK_POLL_SLEEP_NS > 0) __nanosleep(MK_POLL_SLEEP_NS);
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
        poll_backoff();
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
        poll_backoff();
        ll_load2(p, w0, w1);
    }
    a = __uint_as_float((uint32_t)w0);
    b = __uint_as_float((uint32_t)w1);
}

// Sum over all consumer threads, in a fixed order (one barrier).
__device__ __forceinline__ float consumer_sum(Ctx& c, float v) {
    float* buf = c.sm.red_s + (c.red_n++ & 1) * NCW;
    v = warp_sum(v);
    if (c.lane == 0) buf[c.warp] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < NCW; i++) t += buf[i];
    return t;
}

// ---- GEMV input vector layout --------------------------------------------------------------------
// A lane reads one 16-byte piece of a weight row at a time: 16 int8 or 8 bf16 weights.  The matching
// inputs are 4 (or 2) float4s.  Storing float4 number j of piece p at
//     (p / 32) * 32 * PIECE + j * 128 + (p % 32) * 4
// puts the j-th float4 of 32 consecutive pieces side by side, so a warp's loads are conflict-free.
template <bool Q8>
__device__ __forceinline__ int xs_index(int k) {
    constexpr int PIECE = Q8 ? 16 : 8;
    const int p = k / PIECE, r = k % PIECE;
    return (p >> 5) * (32 * PIECE) + (r >> 2) * 128 + (p & 31) * 4 + (r & 3);
}

// Partial dot products of NR weight rows (16-byte pieces [p0, p0 + np) of each) with the staged input.
template <bool Q8, int NR>
__device__ __forceinline__ void dot_rows(const uint8_t* const (&rows)[NR], const float* xs, int p0, int np, int lane,
                                         float (&acc)[NR]) {
    constexpr int PIECE = Q8 ? 16 : 8;
    float a0[NR], a1[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) a0[r] = a1[r] = 0.f;
#pragma unroll 2
    for (int i = lane; i < np; i += 32) {
        const int p = p0 + i;
        const float* xb = xs + (p >> 5) * (32 * PIECE) + (p & 31) * 4;
        uint4 w[NR];
#pragma unroll
        for (int r = 0; r < NR; r++) w[r] = *reinterpret_cast<const uint4*>(rows[r] + (size_t)p * 16);
        if (Q8) {
            const float4 x0 = *reinterpret_cast<const float4*>(xb);
            const float4 x1 = *reinterpret_cast<const float4*>(xb + 128);
            const float4 x2 = *reinterpret_cast<const float4*>(xb + 256);
            const float4 x3 = *reinterpret_cast<const float4*>(xb + 384);
#pragma unroll
            for (int r = 0; r < NR; r++) {
                a0[r] = fmaf(deq_u8<0>(w[r].x), x0.x, a0[r]);
                a1[r] = fmaf(deq_u8<1>(w[r].x), x0.y, a1[r]);
                a0[r] = fmaf(deq_u8<2>(w[r].x), x0.z, a0[r]);
                a1[r] = fmaf(deq_u8<3>(w[r].x), x0.w, a1[r]);
                a0[r] = fmaf(deq_u8<0>(w[r].y), x1.x, a0[r]);
                a1[r] = fmaf(deq_u8<1>(w[r].y), x1.y, a1[r]);
                a0[r] = fmaf(deq_u8<2>(w[r].y), x1.z, a0[r]);
                a1[r] = fmaf(deq_u8<3>(w[r].y), x1.w, a1[r]);
                a0[r] = fmaf(deq_u8<0>(w[r].z), x2.x, a0[r]);
                a1[r] = fmaf(deq_u8<1>(w[r].z), x2.y, a1[r]);
                a0[r] = fmaf(deq_u8<2>(w[r].z), x2.z, a0[r]);
                a1[r] = fmaf(deq_u8<3>(w[r].z), x2.w, a1[r]);
                a0[r] = fmaf(deq_u8<0>(w[r].w), x3.x, a0[r]);
                a1[r] = fmaf(deq_u8<1>(w[r].w), x3.y, a1[r]);
                a0[r] = fmaf(deq_u8<2>(w[r].w), x3.z, a0[r]);
                a1[r] = fmaf(deq_u8<3>(w[r].w), x3.w, a1[r]);
            }
        } else {
            const float4 x0 = *reinterpret_cast<const float4*>(xb);
            const float4 x1 = *reinterpret_cast<const float4*>(xb + 128);
#pragma unroll
            for (int r = 0; r < NR; r++) {
                a0[r] = fmaf(bf_lo(w[r].x), x0.x, a0[r]);
                a1[r] = fmaf(bf_hi(w[r].x), x0.y, a1[r]);
                a0[r] = fmaf(bf_lo(w[r].y), x0.z, a0[r]);
                a1[r] = fmaf(bf_hi(w[r].y), x0.w, a1[r]);
                a0[r] = fmaf(bf_lo(w[r].z), x1.x, a0[r]);
                a1[r] = fmaf(bf_hi(w[r].z), x1.y, a1[r]);
                a0[r] = fmaf(bf_lo(w[r].w), x1.z, a0[r]);
                a1[r] = fmaf(bf_hi(w[r].w), x1.w, a1[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r] = warp_sum(a0[r] + a1[r]);
}

// Streams this CTA's rows [r0, r1) of a [rows, K] matrix out of the ring and hands every finished
// (row, K-segment) sum to `sink(row, seg, sum)` on all lanes of the warp that computed it.
//   KSPLIT  warps that share one row (each takes a contiguous K segment); used when a CTA owns few,
//           long rows.  KSPLIT == 1 lets a warp take RPW rows at once and share the input loads.
template <int K, bool Q8, int KSPLIT, int RPW, class Sink>
__device__ __forceinline__ void gemv_stream(Ctx& c, int r0, int r1, Sink&& sink) {
    constexpr int PIECE = Q8 ? 16 : 8;
    constexpr int RB = Q8 ? K : 2 * K;          // row bytes
    constexpr int RPC = SLOT_BYTES / RB;        // rows per ring chunk
    constexpr int PPR = K / PIECE;              // pieces per row
    constexpr int PPS = PPR / KSPLIT;           // pieces per segment
    static_assert(PPR % KSPLIT == 0, "segments must be whole pieces");
    static_assert(KSPLIT == 1 || RPW == 1, "row pairing only without K split");
    static_assert(RPW == 1 || RPC % RPW == 0, "row groups must not straddle chunks");
    for (int base = r0; base < r1; base += RPC) {
        const int nr = min(RPC, r1 - base);
        const uint32_t n = c.cons_n++;
        const int slot = (int)(n % NSTAGE);
        if (c.prof && c.tid == 0) {
            const u64 t = globaltimer();
            mbar_wait(c, &c.sm.full[slot], (n / NSTAGE) & 1, W_FULL);
            c.wait_acc += globaltimer() - t;
        } else {
            mbar_wait(c, &c.sm.full[slot], (n / NSTAGE) & 1, W_FULL);
        }
        const uint8_t* buf = c.sm.ring + (size_t)slot * SLOT_BYTES;
        if (KSPLIT > 1) {
            for (int item = c.warp; item < nr * KSPLIT; item += NCW) {
                const int row = item / KSPLIT, seg = item % KSPLIT;
                const uint8_t* const rows[1] = {buf + (size_t)row * RB};
                float acc[1];
                dot_rows<Q8, 1>(rows, c.sm.xs, seg * PPS, PPS, c.lane, acc);
                sink(base + row, seg, acc[0]);
            }
        } else {
            const int nitems = (nr + RPW - 1) / RPW;
            for (int item = c.warp; item < nitems; item += NCW) {
                const uint8_t* rows[RPW];
#pragma unroll
                for (int r = 0; r < RPW; r++) rows[r] = buf + (size_t)(item * RPW + r) * RB;
                float acc[RPW];
                dot_rows<Q8, RPW>(rows, c.sm.xs, 0, PPR, c.lane, acc);
#pragma unroll
                for (int r = 0; r < RPW; r++)
                    if (item * RPW + r < nr) sink(base + item * RPW + r, 0, acc[r]);
            }
        }
        __syncwarp();
        // A lane whose wait ran out never releases the slot: its copy may still be in flight, and the
        // producer must not aim a second copy at the same shared memory.
        if (c.lane == 0 && !c.dead) mbar_arrive(&c.sm.empty[slot]);
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
// RMSNorm of the residual stream into the GEMV input vector.  `x` holds this thread's two elements
// (2*tid, 2*tid+1).
template <class S, bool Q8>
__device__ __forceinline__ void stage_rmsnorm(Ctx& c, float x0, float x1, const float* __restrict__ w) {
    static_assert(S::HID == 2 * NCT, "two residual elements per consumer thread");
    const int k = 2 * c.tid;
    const float2 g = *reinterpret_cast<const float2*>(w + k);
    const float ss = consumer_sum(c, x0 * x0 + x1 * x1);
    const float inv = rsqrtf(ss * (1.0f / S::HID) + S::EPS);
    c.sm.xs[xs_index<Q8>(k)] = x0 * inv * (1.0f + g.x);
    c.sm.xs[xs_index<Q8>(k + 1)] = x1 * inv * (1.0f + g.y);
    consumer_sync();
}

// Embedding row of `token` -> this thread's two residual elements.
template <class S, bool Q8>
__device__ __forceinline__ void load_embedding(const Params& P, int token, int tid, float& x0, float& x1) {
    const int k = 2 * tid;
    if (Q8) {
        const uint16_t b = *reinterpret_cast<const uint16_t*>(P.embed + (size_t)token * S::HID + k);
        const float sc = P.embed_scale[token];
        x0 = (float)((int)(b & 0xff) - 128) * sc;
        x1 = (float)((int)(b >> 8) - 128) * sc;
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
__device__ void gdn_op(Ctx& c, const Params& P, const LayerP& L, int pos, uint32_t e_proj, uint32_t e_out, int op) {
    static_assert(S::GDN_SLICE == NCW && S::LIN_DK == 128, "one warp per value column, 4 keys per lane");
    constexpr int SL = S::LIN_DV / S::GDN_SLICE;  // slices per head
    if (c.cta >= S::GDN_TASKS) return;
    const int h = c.cta / SL, j = c.cta % SL;
    const int vcol = j * S::GDN_SLICE + c.warp;
    float* qkv_s = c.sm.xs;                       // [q 128 | k 128 | v 16 | b | a]
    float* srow = L.state + ((size_t)(h * S::LIN_DV + vcol) * S::LIN_DK) + 4 * c.lane;
    const float4 st = *reinterpret_cast<const float4*>(srow);   // issued before the wait on purpose
    constexpr int NCH = 2 * S::LIN_DK + S::GDN_SLICE;           // 272 conv channels this task needs
    if (c.tid < NCH) {
        int ch;
        if (c.tid < S::LIN_DK) ch = h * S::LIN_DK + c.tid;
        else if (c.tid < 2 * S::LIN_DK) ch = S::LIN_QK + h * S::LIN_DK + (c.tid - S::LIN_DK);
        else ch = 2 * S::LIN_QK + h * S::LIN_DV + j * S::GDN_SLICE + (c.tid - 2 * S::LIN_DK);
        const float4 taps = *reinterpret_cast<const float4*>(L.conv_w + 4 * ch);
        float* hist = L.conv_hist + (size_t)ch * CONV_RING;
        const float h3 = __ldcg(hist + ((pos - 3) & (CONV_RING - 1)));   // written by another CTA: skip L1
        const float h2 = __ldcg(hist + ((pos - 2) & (CONV_RING - 1)));
        const float h1 = __ldcg(hist + ((pos - 1) & (CONV_RING - 1)));
        const float cur = ll_wait(c, P.projl + ch, e_proj, W_PROJ);
        float a = h3 * taps.x;
        a = fmaf(h2, taps.y, a);
        a = fmaf(h1, taps.z, a);
        a = fmaf(cur, taps.w, a);
        qkv_s[c.tid] = silu_f(a);
        if (c.tid >= 2 * S::LIN_DK || j == 0) hist[pos & (CONV_RING - 1)] = cur;
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
    const float decay = expf(-expf(L.A_log[h]) * softplus_f(qkv_s[NCH + 1] + L.dt_bias[h]));
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
    __threadfence();  // conv history of the q/k channels is read by sibling CTAs in the next steps
    if (c.lane == 0) ll_store(P.mixl + h * S::LIN_DV + vcol, e_out, o);
    consumer_sync();  // the scratch aliases the GEMV input vector that the next prologue writes
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
// [s * ch, min(n, (s + 1) * ch)), run by CTA s * NKV + g.  With one split the task publishes the
// normalised output itself; otherwise it writes (acc, m, l) partials and raises a flag, and the
// split-0 task of each KV head merges all partials in split order.
template <class S, bool KVF32>
__device__ void attn_op(Ctx& c, const Params& P, const LayerP& L, int pos, uint32_t e_proj, uint32_t e_out, int op) {
    static_assert(S::HD == 256 && S::QPK == 4 && NCW == 16 && S::ROT == 64, "thread mapping below");
    const int n = pos + 1;
    const int max_splits = min(c.grid / S::NKV, MAX_SPLITS);
    const int ch = attn_chunk(n, max_splits);
    const int nsplit = (n + ch - 1) / ch;
    if (c.cta >= nsplit * S::NKV) return;
    const int g = c.cta % S::NKV, sp = c.cta / S::NKV;
    const int p0 = sp * ch, p1 = min(n, p0 + ch);
    const bool has_new = (p1 == n);

    float* q_s = c.sm.xs;                       // [4][256] normalised, rotated, pre-scaled queries
    float* knew_s = q_s + S::QPK * S::HD;       // [256]
    float* vnew_s = knew_s + S::HD;             // [256]
    float* sc_s = vnew_s + S::HD;               // [4][ch] scores, then probabilities
    float* stat_s = c.sm.out_s;                 // [4] m, [4] l

    // -- 1. q (4 heads), new k, new v from the projection words; per-head RMSNorm; partial RoPE
    {
        const int hh = c.warp >> 2, qd = c.warp & 3;        // head within group, 64-wide quarter
        const int d = qd * 64 + 2 * c.lane;
        const int qrow = (g * S::QPK + hh) * 2 * S::HD + d;
        float a, b;
        ll_wait2(c, P.projl + qrow, e_proj, W_PROJ, a, b);
        float ka = 0.f, kb = 0.f, va = 0.f, vb = 0.f;
        if (hh == 0) ll_wait2(c, P.projl + S::ATT_K_OFF + g * S::HD + d, e_proj, W_PROJ, ka, kb);
        if (hh == 1) ll_wait2(c, P.projl + S::ATT_V_OFF + g * S::HD + d, e_proj, W_PROJ, va, vb);
        float* buf = c.sm.red_s + (c.red_n++ & 1) * NCW;    // q sums
        float* buf2 = reinterpret_cast<float*>(c.sm.best_s);   // k sums [4]; best_s is idle outside the LM head
        const float sq = warp_sum(a * a + b * b);
        const float sk = warp_sum(ka * ka + kb * kb);
        if (c.lane == 0) {
            buf[c.warp] = sq;
            if (hh == 0) buf2[qd] = sk;
        }
        consumer_sync();
        const float qss = buf[hh * 4] + buf[hh * 4 + 1] + buf[hh * 4 + 2] + buf[hh * 4 + 3];
        const float qinv = rsqrtf(qss * (1.0f / S::HD) + S::EPS);
        const float2 qw = *reinterpret_cast<const float2*>(L.q_norm + d);
        a = a * qinv * (1.0f + qw.x);
        b = b * qinv * (1.0f + qw.y);
        float cs0 = 1.f, sn0 = 0.f, cs1 = 1.f, sn1 = 0.f;
        if (qd == 0) {
            const int i0 = (2 * c.lane) & 31;
            cs0 = P.rope_cos[(size_t)pos * (S::ROT / 2) + i0];
            sn0 = P.rope_sin[(size_t)pos * (S::ROT / 2) + i0];
            cs1 = P.rope_cos[(size_t)pos * (S::ROT / 2) + i0 + 1];
            sn1 = P.rope_sin[(size_t)pos * (S::ROT / 2) + i0 + 1];
            // dims [0,32) live in lanes 0..15, their partners [32,64) in lanes 16..31
            const float pa = __shfl_xor_sync(0xffffffffu, a, 16), pb = __shfl_xor_sync(0xffffffffu, b, 16);
            if (c.lane < 16) { a = a * cs0 - pa * sn0; b = b * cs1 - pb * sn1; }
            else { a = a * cs0 + pa * sn0; b = b * cs1 + pb * sn1; }
        }
        q_s[hh * S::HD + d] = a * 0.0625f;          // 1/sqrt(256), exact
        q_s[hh * S::HD + d + 1] = b * 0.0625f;
        if (hh == 0) {
            const float kss = buf2[0] + buf2[1] + buf2[2] + buf2[3];
            const float kinv = rsqrtf(kss * (1.0f / S::HD) + S::EPS);
            const float2 kw = *reinterpret_cast<const float2*>(L.k_norm + d);
            ka = ka * kinv * (1.0f + kw.x);
            kb = kb * kinv * (1.0f + kw.y);
            if (qd == 0) {
                const float pa = __shfl_xor_sync(0xffffffffu, ka, 16), pb = __shfl_xor_sync(0xffffffffu, kb, 16);
                if (c.lane < 16) { ka = ka * cs0 - pa * sn0; kb = kb * cs1 - pb * sn1; }
                else { ka = ka * cs0 + pa * sn0; kb = kb * cs1 + pb * sn1; }
            }
            knew_s[d] = round_kv<KVF32>(ka);
            knew_s[d + 1] = round_kv<KVF32>(kb);
        }
        if (hh == 1) {
            vnew_s[d] = round_kv<KVF32>(va);
            vnew_s[d + 1] = round_kv<KVF32>(vb);
        }
        consumer_sync();
        prof_stamp(c, op, 1);
    }
    const size_t kv_head_stride = (size_t)KV_BLOCK * S::HD;
    auto kv_elem = [&](int p) -> size_t {
        const int blk = P.block_table[p >> 6];
        return ((size_t)blk * S::NKV + g) * kv_head_stride + (size_t)(p & (KV_BLOCK - 1)) * S::HD;
    };
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
        for (int p = p0 + c.warp; p < p1; p += NCW) {
            float kk[8];
            if (p == pos) {
#pragma unroll
                for (int i = 0; i < 8; i++) kk[i] = knew_s[8 * c.lane + i];
            } else {
                load8<KVF32>(L.k_cache, kv_elem(p) + 8 * c.lane, kk);
            }
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
        }
    }
    consumer_sync();
    // -- 4. softmax statistics: warp hh < 4 handles head hh
    const int np = p1 - p0;
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
    const int d = c.tid & (S::HD - 1), hp = c.tid >> 8;
    float acc0 = 0.f, acc1 = 0.f;
    {
        const float* pr0 = sc_s + (2 * hp) * ch;
        const float* pr1 = sc_s + (2 * hp + 1) * ch;
        int i = 0;
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
        __threadfence();  // the appended K/V row is read by other CTAs in later steps
        ll_store(out + (2 * hp) * S::HD + d, e_out, acc0 / stat_s[S::QPK + 2 * hp]);
        ll_store(out + (2 * hp + 1) * S::HD + d, e_out, acc1 / stat_s[S::QPK + 2 * hp + 1]);
        consumer_sync();  // scratch aliases the GEMV input vector that the next prologue writes
        return;
    }
    // -- 6. partials + flag; split 0 merges
    float* part = P.attn_part + ((size_t)g * MAX_SPLITS + sp) * S::PART_STRIDE;
    part[(2 * hp) * S::HD + d] = acc0;
    part[(2 * hp + 1) * S::HD + d] = acc1;
    if (c.tid < 2 * S::QPK) part[S::QPK * S::HD + c.tid] = stat_s[c.tid];
    __threadfence();
    consumer_sync();
    unsigned* flags = P.attn_flag + (size_t)g * MAX_SPLITS;
    if (c.tid == 0) st_relaxed_u32(flags + sp, e_out);
    if (sp != 0) return;   // (the barrier above already fenced off the scratch reads)
    for (int s2 = c.tid; s2 < nsplit; s2 += NCT) {
        Spin s;
        while (ld_relaxed_u32(flags + s2) != e_out) {
            if (MK_SPIN_FAIL(c, s, W_PART)) {
                c.dead = true;
                break;
            }
        }
    }
    __threadfence();
    consumer_sync();
    const float* pg = P.attn_part + (size_t)g * MAX_SPLITS * S::PART_STRIDE;
    float M0 = -INFINITY, M1 = -INFINITY;
    for (int s2 = 0; s2 < nsplit; s2++) {
        const float* ps = pg + (size_t)s2 * S::PART_STRIDE + S::QPK * S::HD;
        M0 = fmaxf(M0, __ldcg(ps + 2 * hp));
        M1 = fmaxf(M1, __ldcg(ps + 2 * hp + 1));
    }
    float o0 = 0.f, o1 = 0.f, l0 = 0.f, l1 = 0.f;
    for (int s2 = 0; s2 < nsplit; s2++) {
        const float* pa = pg + (size_t)s2 * S::PART_STRIDE;
        const float* ps = pa + S::QPK * S::HD;
        const float w0 = __expf(__ldcg(ps + 2 * hp) - M0), w1 = __expf(__ldcg(ps + 2 * hp + 1) - M1);
        l0 = fmaf(__ldcg(ps + S::QPK + 2 * hp), w0, l0);
        l1 = fmaf(__ldcg(ps + S::QPK + 2 * hp + 1), w1, l1);
        o0 = fmaf(__ldcg(pa + (2 * hp) * S::HD + d), w0, o0);
        o1 = fmaf(__ldcg(pa + (2 * hp + 1) * S::HD + d), w1, o1);
    }
    ll_store(out + (2 * hp) * S::HD + d, e_out, o0 / l0);
    ll_store(out + (2 * hp + 1) * S::HD + d, e_out, o1 / l1);
}

// ---- the kernel ------------------------------------------------------------------------------------------
__constant__ Params c_params[MAX_ENGINES];   // one parameter block per live engine handle

template <class S, bool Q8, bool KVF32>
__global__ void __launch_bounds__(NTHREADS, 1) decode_kernel(const int pslot, const __grid_constant__ Args A) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const Params& P = c_params[pslot];
    Ctx c;
    {
        uint8_t* p = smem_raw;
        c.sm.ring = p; p += SMEM_RING;
        c.sm.xs = reinterpret_cast<float*>(p); p += SMEM_XS;
        c.sm.scale_s = reinterpret_cast<float*>(p); p += SMEM_SCALE;
        c.sm.out_s = reinterpret_cast<float*>(p); p += 2 * MAX_BODY_ROWS * 4;      // 512
        c.sm.red_s = reinterpret_cast<float*>(p); p += 2 * NCW * 4;                // 128
        c.sm.xown = reinterpret_cast<float*>(p); p += 16 * 4;                      // 64
        c.sm.best_s = reinterpret_cast<u64*>(p); p += NCW * 8;                     // 128
        c.sm.full = reinterpret_cast<uint64_t*>(p); p += NSTAGE * 8;
        c.sm.empty = reinterpret_cast<uint64_t*>(p); p += NSTAGE * 8;
        c.sm.abort_flag = reinterpret_cast<volatile int*>(p); p += 4;
        c.sm.quit_flag = reinterpret_cast<volatile int*>(p); p += 4;
        c.sm.tok_s = reinterpret_cast<volatile int*>(p); p += 8;
    }
    c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
    c.cta = blockIdx.x; c.grid = gridDim.x;
    c.cons_n = 0; c.red_n = 0; c.dead = false; c.prof = nullptr; c.wait_acc = 0;
    c.limit_ns = (u64)A.spin_limit_ns;
    c.status = P.status;
    if (c.tid == 0) {
        for (int i = 0; i < NSTAGE; i++) {
            mbar_init(&c.sm.full[i], 1);
            mbar_init(&c.sm.empty[i], NCW);
        }
        *c.sm.abort_flag = 0;
        *c.sm.quit_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    if (c.warp == NCW) {
        if (c.lane == 0) producer_main<S, Q8>(c, P, A);
        return;
    }

    // ---------------- consumers ----------------
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
            // ---- A: in-projection
            {
                const int op = l * OPS_PER_LAYER;
                prof_stamp(c, op, 0);
                int r0, r1;
                cta_rows(attn ? S::ATT_IN : S::GDN_IN, 1, c.cta, c.grid, r0, r1);
                const int nrows = r1 - r0;
                float sc = 1.f;
                if (Q8 && c.tid < nrows) sc = L.s_in[r0 + c.tid];
                if (l > 0) ll_wait2(c, P.xl + 2 * c.tid, eA - 1, W_X, x0, x1);
                stage_rmsnorm<S, Q8>(c, x0, x1, L.in_norm);
                prof_stamp(c, op, 1);
                float* out_s = c.sm.out_s;
                gemv_stream<S::HID, Q8, 1, Q8 ? 2 : 1>(c, r0, r1, [&](int row, int, float v) {
                    if (c.lane == 0) out_s[row - r0] = v;
                });
                consumer_sync();
                prof_stamp(c, op, 2);
                if (c.tid < nrows) ll_store(P.projl + r0 + c.tid, eA, out_s[c.tid] * sc);
                prof_stamp(c, op, 3);
            }
            // ---- B: mixer
            prof_stamp(c, l * OPS_PER_LAYER + 1, 0);
            if (attn) attn_op<S, KVF32>(c, P, L, pos, eA, eB, l * OPS_PER_LAYER + 1);
            else gdn_op<S>(c, P, L, pos, eA, eB, l * OPS_PER_LAYER + 1);
            prof_stamp(c, l * OPS_PER_LAYER + 1, 3);
            // ---- C: out-projection + residual
            {
                const int op = l * OPS_PER_LAYER + 2;
                prof_stamp(c, op, 0);
                const int nrows = xr1 - xr0;
                float sc = 1.f;
                if (Q8 && c.tid < nrows) sc = L.s_out[xr0 + c.tid];
                // each thread stages 4 consecutive mixer outputs; a warp covers 128 = one DeltaNet head
                const int k = 4 * c.tid;
                float m[4];
                ll_wait2(c, P.mixl + k, eB, W_MIX, m[0], m[1]);
                ll_wait2(c, P.mixl + k + 2, eB, W_MIX, m[2], m[3]);
                if (attn) {
                    const int head = k / S::HD, d = k % S::HD;
                    float gt[4];
                    const u64* gp = P.projl + head * 2 * S::HD + S::HD + d;
                    ll_wait2(c, gp, eA, W_PROJ, gt[0], gt[1]);
                    ll_wait2(c, gp + 2, eA, W_PROJ, gt[2], gt[3]);
#pragma unroll
                    for (int i = 0; i < 4; i++) c.sm.xs[xs_index<Q8>(k + i)] = m[i] * sigmoid_f(gt[i]);
                } else {
                    float z[4];
                    ll_wait2(c, P.projl + S::Z_OFF + k, eA, W_PROJ, z[0], z[1]);
                    ll_wait2(c, P.projl + S::Z_OFF + k + 2, eA, W_PROJ, z[2], z[3]);
                    const float ss = warp_sum(m[0] * m[0] + m[1] * m[1] + m[2] * m[2] + m[3] * m[3]);
                    const float inv = rsqrtf(ss * (1.0f / S::LIN_DV) + S::EPS);
                    const float4 gw = *reinterpret_cast<const float4*>(L.gdn_norm + (k % S::LIN_DV));
                    c.sm.xs[xs_index<Q8>(k)] = m[0] * inv * gw.x * silu_f(z[0]);
                    c.sm.xs[xs_index<Q8>(k + 1)] = m[1] * inv * gw.y * silu_f(z[1]);
                    c.sm.xs[xs_index<Q8>(k + 2)] = m[2] * inv * gw.z * silu_f(z[2]);
                    c.sm.xs[xs_index<Q8>(k + 3)] = m[3] * inv * gw.w * silu_f(z[3]);
                }
                consumer_sync();
                prof_stamp(c, op, 1);
                float* out_s = c.sm.out_s;
                gemv_stream<S::MIX, Q8, 2, 1>(c, xr0, xr1, [&](int row, int seg, float v) {
                    if (c.lane == 0) out_s[(row - xr0) * 2 + seg] = v;
                });
                consumer_sync();
                prof_stamp(c, op, 2);
                if (c.tid < nrows) {
                    const float y = (out_s[2 * c.tid] + out_s[2 * c.tid + 1]) * sc;
                    const float xn = c.sm.xown[c.tid] + y;
                    c.sm.xown[c.tid] = xn;
                    ll_store(P.xl + xr0 + c.tid, eC, xn);
                }
                prof_stamp(c, op, 3);
            }
            // ---- D: gate/up + SwiGLU
            {
                const int op = l * OPS_PER_LAYER + 3;
                prof_stamp(c, op, 0);
                int r0, r1;
                cta_rows(2 * S::INTER, 2, c.cta, c.grid, r0, r1);
                const int npairs = (r1 - r0) / 2;
                float2 sc = make_float2(1.f, 1.f);
                if (Q8 && c.tid < npairs) sc = *reinterpret_cast<const float2*>(L.s_gu + r0 + 2 * c.tid);
                ll_wait2(c, P.xl + 2 * c.tid, eC, W_X, x0, x1);
                stage_rmsnorm<S, Q8>(c, x0, x1, L.post_norm);
                prof_stamp(c, op, 1);
                float* out_s = c.sm.out_s;
                gemv_stream<S::HID, Q8, 1, Q8 ? 2 : 1>(c, r0, r1, [&](int row, int, float v) {
                    if (c.lane == 0) out_s[row - r0] = v;
                });
                consumer_sync();
                prof_stamp(c, op, 2);
                if (c.tid < npairs) {
                    const float gate = out_s[2 * c.tid] * sc.x, up = out_s[2 * c.tid + 1] * sc.y;
                    ll_store(P.actl + r0 / 2 + c.tid, eD, silu_f(gate) * up);
                }
                prof_stamp(c, op, 3);
            }
            // ---- E: down-projection + residual
            {
                const int op = l * OPS_PER_LAYER + 4;
                prof_stamp(c, op, 0);
                const int nrows = xr1 - xr0;
                float sc = 1.f;
                if (Q8 && c.tid < nrows) sc = L.s_down[xr0 + c.tid];
                for (int k = 2 * c.tid; k < S::INTER; k += 2 * NCT) {
                    float a, b;
                    ll_wait2(c, P.actl + k, eD, W_ACT, a, b);
                    c.sm.xs[xs_index<Q8>(k)] = a;
                    c.sm.xs[xs_index<Q8>(k + 1)] = b;
                }
                consumer_sync();
                prof_stamp(c, op, 1);
                float* out_s = c.sm.out_s;
                constexpr int KS = Q8 ? 2 : 4;   // bf16 rows are 7 KB: 4 per chunk, so 4 warps share a row
                gemv_stream<S::INTER, Q8, KS, 1>(c, xr0, xr1, [&](int row, int seg, float v) {
                    if (c.lane == 0) out_s[(row - xr0) * KS + seg] = v;
                });
                failed = consumer_any(c.dead);
                prof_stamp(c, op, 2);
                if (c.tid < nrows) {
                    float y = 0.f;
#pragma unroll
                    for (int i = 0; i < KS; i++) y += out_s[KS * c.tid + i];
                    y *= sc;
                    const float xn = c.sm.xown[c.tid] + y;
                    c.sm.xown[c.tid] = xn;
                    ll_store(P.xl + xr0 + c.tid, eE, xn);
                    if (A.resid_out && l == P.n_layers - 1) A.resid_out[(size_t)s * S::HID + xr0 + c.tid] = xn;
                }
                prof_stamp(c, op, 3);
            }
            if (failed) break;
        }
        if (failed) break;
        // ---- LM head
        if (s >= A.lm_from) {
            const uint32_t eL = e0 + (uint32_t)OPS - 1;
            const int op = P.n_layers * OPS_PER_LAYER;
            prof_stamp(c, op, 0);
            const int nrows = lr1 - lr0;
            if (Q8) for (int i = c.tid; i < nrows; i += NCT) c.sm.scale_s[i] = P.lm_scale[lr0 + i];
            ll_wait2(c, P.xl + 2 * c.tid, eL - 1, W_X, x0, x1);
            stage_rmsnorm<S, Q8>(c, x0, x1, P.final_norm);
            prof_stamp(c, op, 1);
            u64 best = 0;
            float* logits = A.logits_out ? A.logits_out + (size_t)s * P.vocab : nullptr;
            const float invT = A.inv_temperature;
            const float* scale_s = c.sm.scale_s;
            gemv_stream<S::HID, Q8, 1, Q8 ? 2 : 1>(c, lr0, lr1, [&](int row, int, float v) {
                if (Q8) v *= scale_s[row - lr0];
                if (logits && c.lane == 0) logits[row] = v;
                float score = v;
                if (invT != 0.f) {
                    const uint32_t hsh = mk_mix32(A.seed, (uint32_t)pos, (uint32_t)row);
                    const float u = ((float)(hsh >> 8) + 0.5f) * (1.0f / 16777216.0f);
                    score = v * invT - __logf(-__logf(u));
                }
                const u64 key = score_key(score, row);
                best = key > best ? key : best;
            });
            if (c.lane == 0) c.sm.best_s[c.warp] = best;
            failed = consumer_any(c.dead);
            prof_stamp(c, op, 2);
            if (c.tid == 0) {
                u64 b = 0;
                for (int i = 0; i < NCW; i++) b = c.sm.best_s[i] > b ? c.sm.best_s[i] : b;
                ll_store_bits(P.lml + 2 * c.cta, eL, (uint32_t)(b >> 32));
                ll_store_bits(P.lml + 2 * c.cta + 1, eL, (uint32_t)b);
            }
            prof_stamp(c, op, 3);
            consumer_sync();   // best_s is read by thread 0 above before anyone reuses it
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
