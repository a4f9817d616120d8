// Batched decoding: up to eight independent sequences share every pass over the weights (int8 weights).
//
// The kernel keeps the structure of the single-sequence kernel (mk_decode.cuh): one resident CTA per
// SM, a producer lane that streams this CTA's row slices through a shared-memory ring, flag-in-data
// words between ops.  What changes:
//   * The eight sequences are the eight columns of the MMA B operand.  An input is x * 2^s rounded to a
//     signed 24-bit integer and cut into three bytes (two's complement: the top byte signed, the lower
//     two unsigned); byte d of sequence j is plane d * 8 + j, so digit d of all sequences is one
//     s8 x s8 (top) or s8 x u8 (lower) MMA.  Integer MMAs are exact; the digits recombine in fp32.
//   * Every warp owns a contiguous k-slice of the rows and stages exactly the inputs of that slice,
//     with its own power-of-two scale per pair of sequences (undone on its partial sums), so nothing
//     block-wide sits between the arrival of the inputs and the MMAs.  The 1 / rms factor of an
//     RMSNorm is applied to the finished rows from per-warp sums of squares.
//   * Every CTA stages all inputs of all sequences, so whatever can be done once is done by the op
//     that produces a value: the mixers publish gated outputs (DeltaNet: per-head RMSNorm times
//     silu(z); attention: times the sigmoid gate), and the out-projection only quantises them.
//   * A DeltaNet task is one head of one sequence (16 x sequences tasks); attention gives each
//     sequence an equal group of CTAs, each group running the single-sequence split-K op on its own
//     block table; the LM head keeps one best key per sequence.
// Sequences advance in lockstep: step s feeds position pos0[j] + s of sequence j.  A sequence whose
// prompt is shorter starts sampling earlier.  A sequence that has produced a stop token, or has run its
// n_total steps, is frozen: it keeps stepping so that the lockstep holds (the host ignores its later
// outputs), but its DeltaNet state and conv history stay as its last accepted token left them, and the
// K/V rows it appends lie beyond its valid length.  The launch ends when every sequence is frozen.
#pragma once
#include "mk_decode.cuh"

namespace mk {

constexpr int NB = 8;                       // sequences per pass = columns of one MMA
// Cached K rows a warp, and cached V elements a thread, requests together in batched attention.  More
// loads in flight (2 or 4 rows, 16 elements) measured 3 to 14 % slower per step: at 96 registers per
// thread they turn into spills, and spills are served by L2 because shared memory leaves the L1
// almost nothing.
#ifndef MK_B_KU
#define MK_B_KU 1
#endif
#ifndef MK_B_VU
#define MK_B_VU 8
#endif

struct BatchArgs {
    const int* forced;                      // [steps][NB] prompt tokens, step-major
    const int* stop_ids;
    unsigned long long* tokens_out;         // [n_steps][NB] best (score, ~id) keys of every step that ran the LM head
    float* logits_out;                      // optional [n_steps][NB][vocab]
    unsigned long long* step_ts;
    int* out_info;
    unsigned long long* prof;
    long long spin_limit_ns;
    int n_forced[NB];
    int n_total[NB];                        // steps sequence j takes part in; it is frozen afterwards
    int pos0[NB];
    int nb, n_steps, lm_from;
    unsigned epoch_base, seed;
    float inv_temperature;
    int n_stop, prof_step;
};

struct GeoB {
    static constexpr int NS = 3;                                   // ring stages: the input planes take the rest
    static constexpr int RING = NS * SLOT_BYTES;
    static constexpr int XQ = 3 * NB * 3584;                       // 24 byte planes of K = 3584 at most
    static constexpr int PL = 68;                                  // row stride of a (warp, sequence) partial-sum line: 64 rows, padded against bank conflicts
    static constexpr int PS = 36;                                  // same for the 32-row lines of the streaming GEMV
    static constexpr int PART = 2 * NCW * NB * PS * 4;             // >= NCW * NB * PL * 4
    static constexpr int MISC = 4096;
    static constexpr int SMEM = RING + XQ + PART + MAX_BLOCKS * 4 + 2048 + MISC;
};
static_assert(NCW * NB * GeoB::PL * 4 <= GeoB::PART, "layer-GEMV partial sums fit");
static_assert(GeoB::SMEM <= 232448, "shared memory of one SM");

__device__ __forceinline__ void mma_s8u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Power of two that maps a vector whose largest magnitude is `mx` below 2^22: with rounding the
// integers stay inside the signed 24-bit range.
__device__ __forceinline__ float fixed_scale24(float mx) { return fixed_scale(mx) * 0.03125f; }

// Stage inputs k, k + 1 of sequence `seq` into the three digit planes: byte d of both integers is one
// byte permute and one 16-bit store.
__device__ __forceinline__ void stage_pair_b(uint8_t* xq, int rb, int seq, int k, float v0, float v1, float scale) {
    const uint32_t a = (uint32_t)__float2int_rn(v0 * scale), b = (uint32_t)__float2int_rn(v1 * scale);
    uint8_t* p = xq + (size_t)seq * rb + k;
    *reinterpret_cast<uint16_t*>(p) = (uint16_t)__byte_perm(a, b, 0x0040);
    *reinterpret_cast<uint16_t*>(p + (size_t)NB * rb) = (uint16_t)__byte_perm(a, b, 0x0051);
    *reinterpret_cast<uint16_t*>(p + (size_t)2 * NB * rb) = (uint16_t)__byte_perm(a, b, 0x0062);
}

// Sums of eight values per lane over the warp in 9 shuffles instead of 40: every step halves the set a
// lane carries.  Returns the total of value `warp_sum8_index(lane)`; lanes that agree in their low
// three bits hold the same total.
__device__ __forceinline__ int warp_sum8_index(int lane) { return ((lane & 1) << 2) | (lane & 2) | ((lane & 4) >> 2); }
__device__ __forceinline__ float warp_sum8(const float (&v)[8], int lane) {
    float a[4], b[2], r;
    const bool b0 = lane & 1, b1 = lane & 2, b2 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float send = b0 ? v[i] : v[i + 4], keep = b0 ? v[i + 4] : v[i];
        a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const float send = b1 ? a[i] : a[i + 2], keep = b1 ? a[i + 2] : a[i];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    }
    {
        const float send = b2 ? b[0] : b[1], keep = b2 ? b[1] : b[0];
        r = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    r += __shfl_xor_sync(0xffffffffu, r, 8);
    r += __shfl_xor_sync(0xffffffffu, r, 16);
    return r;
}

// K-blocks [kb0, kb1) of a row of `nkb` 64-byte k-blocks that warp `warp` owns.
__device__ __forceinline__ void warp_kslice(int nkb, int warp, int& kb0, int& kb1) {
    kb0 = nkb * warp / NCW;
    kb1 = nkb * (warp + 1) / NCW;
}

// MMAs of one 16-row block (rows [b0, b0 + 16) of the chunk) over this warp's k-blocks, all eight
// sequences.  Lane (g, t) ends up with rows g and g + 8 of the block for sequences 2t and 2t + 1:
// v = {(g, 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)}, the warp's scale already undone.
__device__ __forceinline__ void mma_block_b(const uint8_t* buf, const uint8_t* xrow, int rb, int kb0, int kb1, int nr,
                                            int b0, int g, int t, float is0, float is1, float (&v)[4]) {
    const int n0 = max(0, min(8, nr - b0)), n1 = max(0, min(8, nr - b0 - 8));   // rows in the block's two 8-row tiles
    const uint8_t* tile0 = buf + (size_t)b0 * rb + g * 64 + t * 16;
    const uint8_t* tile1 = buf + (size_t)(b0 + 8) * rb + g * 64 + t * 16;
    int ci[3][4];
#pragma unroll
    for (int d = 0; d < 3; d++)
#pragma unroll
        for (int i = 0; i < 4; i++) ci[d][i] = 0;
#pragma unroll 2
    for (int kb = kb0; kb < kb1; kb++) {
        uint4 w0 = make_uint4(0, 0, 0, 0), w1 = make_uint4(0, 0, 0, 0), x[3];
        if (g < n0) w0 = *reinterpret_cast<const uint4*>(tile0 + (size_t)kb * n0 * 64);
        if (g < n1) w1 = *reinterpret_cast<const uint4*>(tile1 + (size_t)kb * n1 * 64);
#pragma unroll
        for (int d = 0; d < 3; d++) x[d] = *reinterpret_cast<const uint4*>(xrow + (size_t)(d * NB) * rb + kb * 64);
#pragma unroll
        for (int d = 0; d < 2; d++) {           // the unsigned lower digits
            mma_s8u8(ci[d], w0.x, w1.x, w0.y, w1.y, x[d].x, x[d].y);
            mma_s8u8(ci[d], w0.z, w1.z, w0.w, w1.w, x[d].z, x[d].w);
        }
        mma_s8(ci[2], w0.x, w1.x, w0.y, w1.y, x[2].x, x[2].y);
        mma_s8(ci[2], w0.z, w1.z, w0.w, w1.w, x[2].z, x[2].w);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float f = fmaf((float)ci[2][i], 65536.f, fmaf((float)ci[1][i], 256.f, (float)ci[0][i]));
        v[i] = f * ((i & 1) ? is1 : is0);
    }
}

// Streams this CTA's rows [r0, r1) of a matrix with `rb`-byte int8 rows out of the ring, for every
// sequence.  The warp has staged its k-slice of the planes and left the inverse scale of each pair of
// sequences in `wsc_s`.
//   STREAM = false  (layer GEMVs, at most 64 rows per CTA): one barrier after the last chunk, then
//                   warps 2j and 2j + 1 finish sequence j's rows, then one more barrier (the partial
//                   sums and scales are free again);
//   STREAM = true   (LM head): one barrier per chunk, warp j finishes sequence j's rows of the chunk.
//   rms             the input was x (1 + w) of an RMSNorm: the finishing warps multiply by the
//                   1 / rms factor that follows from the per-warp sums of squares in `ssq_s`.
// sink(lane, row, sequence, value, valid) runs on all lanes of a finishing warp.  A layer GEMV
// returns whether any consumer thread has seen a wait run out.
template <class S, bool STREAM, class Sink>
__device__ __forceinline__ bool gemv_b(Ctx& c, int r0, int r1, int rb, const float* __restrict__ row_scale, bool rms,
                                       Sink&& sink) {
    constexpr int NS = GeoB::NS, PL = GeoB::PL, PS = GeoB::PS;
    const int rpc = SLOT_BYTES / rb;
    int kb0, kb1;
    warp_kslice(rb >> 6, c.warp, kb0, kb1);
    const int g = c.lane >> 2, t = c.lane & 3;
    const uint8_t* xrow = c.sm.xq + (size_t)g * rb + t * 16;             // plane d * 8 + g = column g of digit d
    const float is0 = c.sm.wsc_s[c.warp * 4 + t], is1 = is0;             // columns 2t, 2t + 1 are sequence pair t
    const float* scales = STREAM ? c.sm.scale_s + 2 * SCALE_BODY : c.sm.scale_s + (c.gemv_n & 1) * SCALE_BODY;
    c.gemv_n++;
    auto post_factor = [&](int j) {
        const float* q = c.sm.ssq_s + j * NCW;
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < NCW; w++) a += q[w];
        return rsqrtf(a * (1.0f / S::HID) + S::EPS);
    };
    float pend = 1.f, postf = 1.f;
    bool any_dead = false;
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
        // partial sums [warp][sequence][row]
        float* part = STREAM ? c.sm.part_s + (size_t)(((n & 1) * NCW + c.warp) * NB) * PS
                             : c.sm.part_s + (size_t)(c.warp * NB) * PL + (base - r0);
        constexpr int STR = STREAM ? PS : PL;
        for (int b0 = 0; b0 < nr; b0 += 16) {
            float v[4];
            mma_block_b(buf, xrow, rb, kb0, kb1, nr, b0, g, t, is0, is1, v);
            const int row = b0 + g;
            if (row < nr) {
                part[(2 * t) * STR + row] = v[0];
                part[(2 * t + 1) * STR + row] = v[1];
            }
            if (row + 8 < nr) {
                part[(2 * t) * STR + row + 8] = v[2];
                part[(2 * t + 1) * STR + row + 8] = v[3];
            }
        }
        __syncwarp();
        // A lane whose wait ran out never releases the slot: its copy may still be in flight.
        if (c.lane == 0 && !c.dead) mbar_arrive(&c.sm.empty[slot]);
        if (STREAM) {
            consumer_sync();
            if (c.warp < NB) {
                const float* pp = c.sm.part_s + (size_t)((n & 1) * NCW * NB + c.warp) * PS + c.lane;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < NCW; w++) v += pp[(size_t)w * NB * PS];
                if (chunk == 0 && rms) postf = post_factor(c.warp);
                const float rs = row_scale ? scales[(chunk & 7) * 32 + c.lane] : 1.f;
                sink(c.lane, base + c.lane, c.warp, v * rs * postf, c.lane < nr);
            }
        }
    }
    if (!STREAM) {
        any_dead = consumer_any(c.dead);
        {
            const int j = c.warp >> 1, idx = (c.warp & 1) * 32 + c.lane;
            const float* pp = c.sm.part_s + (size_t)j * PL + idx;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < NCW; w++) v += pp[(size_t)w * NB * PL];
            if (rms) v *= post_factor(j);
            const float rs = row_scale ? scales[idx] : 1.f;
            sink(c.lane, r0 + idx, j, v * rs, idx < r1 - r0);
        }
        consumer_sync();
    }
    return any_dead;
}

// RMSNorm input of every sequence, warp-local: this thread's elements 2 tid, 2 tid + 1 of x (1 + w)
// go into the planes of the warp's 64-element k-slice with one scale for all sequences; the warp's
// sums of squares go to `ssq_s`.
template <class S>
__device__ __forceinline__ void stage_rms_b(Ctx& c, const float (&x)[NB][2], float2 g) {
    static_assert(S::HID == 2 * NCT, "two residual elements per consumer thread");
    const int k = 2 * c.tid;
    float ss[NB], mx = 0.f;
#pragma unroll
    for (int j = 0; j < NB; j++) {
        ss[j] = x[j][0] * x[j][0] + x[j][1] * x[j][1];
        mx = fmaxf(mx, fmaxf(fabsf(x[j][0] * (1.0f + g.x)), fabsf(x[j][1] * (1.0f + g.y))));
    }
    const float scale = fixed_scale24(warp_max(mx));
#pragma unroll
    for (int j = 0; j < NB; j++) stage_pair_b(c.sm.xq, S::HID, j, k, x[j][0] * (1.0f + g.x), x[j][1] * (1.0f + g.y), scale);
    const float tot = warp_sum8(ss, c.lane);
    if (c.lane < 8) c.sm.ssq_s[warp_sum8_index(c.lane) * NCW + c.warp] = tot;
    if (c.lane < 4) c.sm.wsc_s[c.warp * 4 + c.lane] = 1.0f / scale;
    __syncwarp();
}

// Residual elements 2 tid, 2 tid + 1 of every live sequence at `epoch`.
template <class S>
__device__ __forceinline__ void wait_residual_b(Ctx& c, const u64* xbuf, uint32_t epoch, int nb, float (&x)[NB][2]) {
    float v[2 * NB];
    const u64* base = xbuf + 2 * c.tid;
    ll_wait_pairs_fn<NB>(c, [&](int j) { return j < nb ? base + (size_t)j * S::HID : nullptr; },
                         [&](int) { return epoch; }, v, W_X);
#pragma unroll
    for (int j = 0; j < NB; j++) { x[j][0] = v[2 * j]; x[j][1] = v[2 * j + 1]; }
}

// ---- Gated DeltaNet recurrence, every sequence ---------------------------------------------------------
// Task t < 16 * sequences: head t % 16 of sequence t / 16, all 128 value columns (warp w owns columns
// 8w .. 8w + 7; a lane holds 4 consecutive key indices of each).  One CTA sees the whole head, so the
// gated per-head RMSNorm (norm weight, silu(z)) is applied here, once, instead of by every CTA's
// out-projection prologue.  A sequence in `frozen` (it has produced a stop token or run its steps)
// still gets outputs, so that nothing downstream stalls, but its state and history stay as the last
// accepted token left them.
template <class S>
__device__ bool gdn_batch(Ctx& c, const Params& P, const LayerP& L, const BatchArgs& A, int step, unsigned frozen,
                          uint32_t e_proj, uint32_t e_out, int op) {
    static_assert(S::LIN_DK == 128 && S::LIN_DV == 128 && NCW == 16, "8 value columns per warp, 4 keys per lane");
    if (c.cta >= S::LIN_H * A.nb) return false;
    const int q = c.cta / S::LIN_H, h = c.cta % S::LIN_H;
    const bool keep = !((frozen >> q) & 1u);
    const int pos = A.pos0[q] + step;
    constexpr int NCH = 2 * S::LIN_DK + S::LIN_DV;              // 384 conv channels of the head: q | k | v
    float* qkv_s = reinterpret_cast<float*>(c.sm.xq);           // [q 128 | k 128 | v 128 | z 128 | b | a]
    float4* st_s = reinterpret_cast<float4*>(c.sm.xq + 4096);   // [value column][lane]: the head's 64 KB of state
    float* red = c.sm.red_s + (c.red_n++ & 1) * (2 * NCW);
    static_assert(4096 + S::LIN_DV * 32 * 16 <= GeoB::XQ, "mixer scratch fits the plane area");
    const u64* proj = P.projl + (size_t)q * S::PROJ_MAX;
    float* state = L.state + (size_t)q * S::LIN_H * S::LIN_DV * S::LIN_DK + (size_t)h * S::LIN_DV * S::LIN_DK;
    // The state rows are requested before the wait, as asynchronous copies into shared memory, so that
    // they cost no registers while the projection is awaited.
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int vcol = c.warp * 8 + i;
        cp_async16(st_s + vcol * 32 + c.lane, state + (size_t)vcol * S::LIN_DK + 4 * c.lane);
    }
    cp_async_commit();
    const float a_log = L.A_log[h], dt_bias = L.dt_bias[h];
    if (c.tid < NCH) {
        const int ch = (c.tid >> 7) * S::LIN_QK + h * S::LIN_DK + (c.tid & 127);   // q, k and v blocks are 2048 channels each
        const float4 taps = *reinterpret_cast<const float4*>(L.conv_w + 4 * ch);
        float* hist = L.conv_hist_b + (((size_t)q * S::LIN_H + h) * NCH + c.tid) * CONV_RING;
        const float h3 = hist[(pos - 3) & (CONV_RING - 1)];
        const float h2 = hist[(pos - 2) & (CONV_RING - 1)];
        const float h1 = hist[(pos - 1) & (CONV_RING - 1)];
        const float cur = ll_wait(c, proj + ch, e_proj, W_PROJ);
        float a = h3 * taps.x;
        a = fmaf(h2, taps.y, a);
        a = fmaf(h1, taps.z, a);
        a = fmaf(cur, taps.w, a);
        qkv_s[c.tid] = silu_f(a);
        if (keep) hist[pos & (CONV_RING - 1)] = cur;
    } else {
        const int i = c.tid - NCH;                               // 128 threads: z of the head, and b, a
        qkv_s[NCH + i] = ll_wait(c, proj + S::Z_OFF + h * S::LIN_DV + i, e_proj, W_PROJ);
        if (i < 2) qkv_s[NCH + S::LIN_DV + i] = ll_wait(c, proj + (i == 0 ? S::B_OFF : S::A_OFF) + h, e_proj, W_PROJ);
    }
    cp_async_wait_all();                                        // this thread's own copies
    consumer_sync();
    prof_stamp(c, op, 1);
    const float4 q4 = *reinterpret_cast<const float4*>(qkv_s + 4 * c.lane);
    const float4 k4 = *reinterpret_cast<const float4*>(qkv_s + S::LIN_DK + 4 * c.lane);
    const float qn = warp_sum(q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w);
    const float kn = warp_sum(k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w);
    // x / max(|x|, 1e-6), and the 1/sqrt(dk) query scale
    const float qs = 0.08838834764831845f / fmaxf(sqrtf(qn), 1e-6f);
    const float ks = 1.0f / fmaxf(sqrtf(kn), 1e-6f);
    const float beta = sigmoid_f(qkv_s[NCH + S::LIN_DV]);
    const float decay = expf(-expf(a_log) * softplus_f(qkv_s[NCH + S::LIN_DV + 1] + dt_bias));
    const float kx = k4.x * ks, ky = k4.y * ks, kz = k4.z * ks, kw = k4.w * ks;
    // Two passes over the state rows in shared memory rather than 32 registers of state per lane.
    float rec[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float4 sv = st_s[(c.warp * 8 + i) * 32 + c.lane];
        rec[i] = fmaf(sv.w * decay, kw, fmaf(sv.z * decay, kz, fmaf(sv.y * decay, ky, sv.x * decay * kx)));
    }
    // what the decayed state recalls for k, per column: lane l ends up with column warp_sum8_index(l)
    const float recalled = warp_sum8(rec, c.lane);
    const int mine = warp_sum8_index(c.lane);
    const float delta_mine = (qkv_s[2 * S::LIN_DK + c.warp * 8 + mine] - recalled) * beta;
    float out[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        // column i's delta sits in the lanes whose index maps to i: lane ((i & 1) << 2) | (i & 2) | ((i & 4) >> 2)
        const float delta = __shfl_sync(0xffffffffu, delta_mine, ((i & 1) << 2) | (i & 2) | ((i & 4) >> 2));
        float4 sv = st_s[(c.warp * 8 + i) * 32 + c.lane];
        sv.x = fmaf(kx, delta, sv.x * decay);
        sv.y = fmaf(ky, delta, sv.y * decay);
        sv.z = fmaf(kz, delta, sv.z * decay);
        sv.w = fmaf(kw, delta, sv.w * decay);
        if (keep) *reinterpret_cast<float4*>(state + (size_t)(c.warp * 8 + i) * S::LIN_DK + 4 * c.lane) = sv;
        out[i] = fmaf(sv.w, q4.w, fmaf(sv.z, q4.z, fmaf(sv.y, q4.y, sv.x * q4.x)));
    }
    const float o = warp_sum8(out, c.lane) * qs;                 // output of column `mine`
    // per-head RMSNorm over the 128 columns: lanes 0..7 of the 16 warps hold them
    const float osq = warp_sum(c.lane < 8 ? o * o : 0.f);
    if (c.lane == 0) red[c.warp] = osq;
    consumer_sync();
    if (c.lane < 8) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < NCW; w++) tot += red[w];
        const float inv = rsqrtf(tot * (1.0f / S::LIN_DV) + S::EPS);
        const int vcol = c.warp * 8 + mine;
        const float m = o * inv * L.gdn_norm[vcol] * silu_f(qkv_s[NCH + vcol]);
        ll_store(P.mixl + (size_t)q * S::MIX + h * S::LIN_DV + vcol, e_out, m);
    }
    prof_stamp(c, op, 2);
    consumer_sync();  // the scratch aliases the GEMV input planes that the next prologue writes
    return true;
}

// The weight stream of the batched kernel: the four GEMVs of every layer, then the LM head from
// step `lm_from` on.
template <class S>
__device__ void producer_batch(Ctx& c, const Params& P, const BatchArgs& A) {
    Producer<GeoB::NS> pr(c);
    for (int s = 0; s < A.n_steps && !pr.stop; s++) {
        for (int l = 0; l < P.n_layers && !pr.stop; l++) {
            const LayerP& L = P.layer[l];
            pr.stream(L.w_in, L.kind ? S::ATT_IN : S::GDN_IN, 1, S::HID);
            pr.stream(L.kind ? L.w_out : L.w_out_rows, S::HID, 1, S::MIX);
            pr.stream(L.w_gu, 2 * S::INTER, 2, S::HID);
            pr.stream(L.w_down_rows, S::HID, 1, S::INTER);
        }
        if (s >= A.lm_from) pr.stream(P.lm_head, P.vocab, 1, S::HID);
    }
    pr.drain();
}

// One decoder layer for every live sequence (ops A..E as in `run_layer`).  `x` holds this thread's
// residual elements when `x_in_regs` (first layer), otherwise they are awaited at epoch eA - 1.
template <class S, bool KVF32>
__device__ __forceinline__ bool run_layer_b(Ctx& c, const Params& P, const LayerP& L, const BatchArgs& A, int step,
                                            unsigned frozen, uint32_t eA, int op0, float (&x)[NB][2], bool x_in_regs, int xr0, int xr1) {
    const uint32_t eB = eA + 1, eC = eA + 2, eD = eA + 3, eE = eA + 4;
    const bool attn = L.kind != 0;
    const int nb = A.nb;
    // ---- A: in-projection
    {
        prof_stamp(c, op0, 0);
        int r0, r1;
        cta_rows(attn ? S::ATT_IN : S::GDN_IN, 1, c.cta, c.grid, r0, r1);
        scale_prefetch(c, L.s_in, r0, r1, false);
        const float2 nw = *reinterpret_cast<const float2*>(L.in_norm + 2 * c.tid);
        if (!x_in_regs) wait_residual_b<S>(c, P.xl, eA - 1, nb, x);
        stage_rms_b<S>(c, x, nw);
        prof_stamp(c, op0, 1);
        gemv_b<S, false>(c, r0, r1, S::HID, L.s_in, true, [&](int, int row, int j, float v, bool ok) {
            if (ok && j < nb) ll_store(P.projl + (size_t)j * S::PROJ_MAX + row, eA, v);
        });
        prof_stamp(c, op0, 3);
    }
    // ---- B: mixer
    prof_stamp(c, op0 + 1, 0);
    bool had_task = false;
    if (attn) {
        // sequence q is served by CTAs [q * per, (q + 1) * per)
        const int per = c.grid / nb, q = c.cta / per;
        if (q < nb) {
            const AttnView view = {c.cta - q * per, per, P.projl + (size_t)q * S::PROJ_MAX, P.mixl + (size_t)q * S::MIX,
                                   P.attn_part + (size_t)q * S::NKV * MAX_SPLITS * S::PART_STRIDE,
                                   c.sm.bt_s + q * (P.max_seq / KV_BLOCK), true};
            had_task = attn_op<S, KVF32, 1, MK_B_KU, MK_B_VU>(c, P, L, view, A.pos0[q] + step, eA, eB, op0 + 1);
        }
    } else {
        had_task = gdn_batch<S>(c, P, L, A, step, frozen, eA, eB, op0 + 1);
    }
    prof_stamp(c, op0 + 1, 3);
    // ---- C: out-projection + residual
    {
        const int op = op0 + 2;
        prof_stamp(c, op, 0);
        scale_prefetch(c, L.s_out, xr0, xr1, false);
        if (!had_task) gate_on_samples(c, P.mixl + (size_t)(nb - 1) * S::MIX, S::MIX, eB);
        // a lane stages 4 consecutive (already gated) mixer outputs of every sequence: the warp's 128 are its k-slice
        const int k = 4 * c.tid;
#pragma unroll 1
        for (int jj = 0; jj < NB; jj += 4) {        // four sequences per round: 8 word pairs in flight
            float v[16];
            const u64* mix0 = P.mixl + (size_t)jj * S::MIX + k;
            ll_wait_pairs_fn<8>(c,
                                [&](int i) -> const u64* {
                                    if (jj + (i >> 1) >= nb) return nullptr;
                                    return mix0 + (size_t)(i >> 1) * S::MIX + 2 * (i & 1);
                                },
                                [&](int) { return eB; }, v, W_MIX);
#pragma unroll
            for (int u = 0; u < 2; u++) {           // one scale per pair of sequences
                float mx = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(v[8 * u + i]));
                const float scale = fixed_scale24(warp_max(mx));
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    stage_pair_b(c.sm.xq, S::MIX, jj + 2 * u + i, k, v[8 * u + 4 * i], v[8 * u + 4 * i + 1], scale);
                    stage_pair_b(c.sm.xq, S::MIX, jj + 2 * u + i, k + 2, v[8 * u + 4 * i + 2], v[8 * u + 4 * i + 3], scale);
                }
                if (c.lane == 0) c.sm.wsc_s[c.warp * 4 + (jj >> 1) + u] = 1.0f / scale;
            }
        }
        __syncwarp();
        prof_stamp(c, op, 1);
        gemv_b<S, false>(c, xr0, xr1, S::MIX, L.s_out, false, [&](int, int row, int j, float v, bool ok) {
            if (ok && j < nb) {
                const float xn = c.sm.xown[j * 16 + row - xr0] + v;
                c.sm.xown[j * 16 + row - xr0] = xn;
                ll_store(P.xl + (size_t)j * S::HID + row, eC, xn);
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
        wait_residual_b<S>(c, P.xl, eC, nb, x);
        stage_rms_b<S>(c, x, nw);
        prof_stamp(c, op, 1);
        gemv_b<S, false>(c, r0, r1, S::HID, L.s_gu, true, [&](int lane, int row, int j, float v, bool ok) {
            // rows alternate gate, up; chunks hold whole pairs, so the partner is the next lane
            const float up = __shfl_down_sync(0xffffffffu, v, 1);
            if (ok && j < nb && !(lane & 1)) ll_store(P.actl + (size_t)j * S::INTER + (row >> 1), eD, silu_f(v) * up);
        });
        prof_stamp(c, op, 3);
    }
    // ---- E: down-projection + residual
    bool failed;
    {
        const int op = op0 + 4;
        prof_stamp(c, op, 0);
        scale_prefetch(c, L.s_down, xr0, xr1, false);
        // the warp stages the inputs of the k-blocks it multiplies (3 or 4): pairs e0 + 2 lane + 64 i
        int kb0, kb1;
        warp_kslice(S::INTER / 64, c.warp, kb0, kb1);
        const int e0 = kb0 * 64, e1 = kb1 * 64;
        const int np = (e1 - e0) / 64;                           // 3 or 4 pairs per lane and sequence
        // Two sequences per round (8 word pairs in flight).  Keeping the next round's loads in flight
        // while this one is staged measured slower: the registers it takes end up as spills.
#pragma unroll 1
        for (int jj = 0; jj < NB; jj += 2) {
            float v[16];
            const u64* act0 = P.actl + (size_t)jj * S::INTER + e0 + 2 * c.lane;
            ll_wait_pairs_fn<8>(c,
                                [&](int i) -> const u64* {
                                    if (jj + (i >> 2) >= nb || (i & 3) >= np) return nullptr;
                                    return act0 + (size_t)(i >> 2) * S::INTER + 64 * (i & 3);
                                },
                                [&](int) { return eD; }, v, W_ACT);
            float mx = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) mx = fmaxf(mx, fabsf(v[i]));
            const float scale = fixed_scale24(warp_max(mx));        // one scale for the pair of sequences
#pragma unroll
            for (int u = 0; u < 2; u++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int k = e0 + 2 * c.lane + 64 * i;
                    if (k < e1) stage_pair_b(c.sm.xq, S::INTER, jj + u, k, v[8 * u + 2 * i], v[8 * u + 2 * i + 1], scale);
                }
            if (c.lane == 0) c.sm.wsc_s[c.warp * 4 + (jj >> 1)] = 1.0f / scale;
        }
        __syncwarp();
        prof_stamp(c, op, 1);
        failed = gemv_b<S, false>(c, xr0, xr1, S::INTER, L.s_down, false, [&](int, int row, int j, float v, bool ok) {
            if (ok && j < nb) {
                const float xn = c.sm.xown[j * 16 + row - xr0] + v;
                c.sm.xown[j * 16 + row - xr0] = xn;
                ll_store(P.xl + (size_t)j * S::HID + row, eE, xn);
            }
        });
        prof_stamp(c, op, 3);
    }
    return failed;
}

// ---- the kernel ------------------------------------------------------------------------------------------
template <class S, bool KVF32>
__global__ void __launch_bounds__(NTHREADS, 1) batch_kernel(const __grid_constant__ Params P, const __grid_constant__ BatchArgs A) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    constexpr int NS = GeoB::NS;
    Ctx c;
    {
        uint8_t* p = smem_raw;
        c.sm.ring = p; p += GeoB::RING;
        c.sm.xq = p; p += GeoB::XQ;
        c.sm.part_s = reinterpret_cast<float*>(p); p += GeoB::PART;
        c.sm.bt_s = reinterpret_cast<int*>(p); p += MAX_BLOCKS * 4;
        c.sm.scale_s = reinterpret_cast<float*>(p); p += (2 * SCALE_BODY + SCALE_RING) * 4;    // 2048
        c.sm.out_s = reinterpret_cast<float*>(p); p += 64;
        c.sm.red_s = reinterpret_cast<float*>(p); p += 2 * 8 * NCW * 4;                        // 1024
        c.sm.xown = reinterpret_cast<float*>(p); p += NB * 16 * 4;                             // 512
        c.sm.best_s = reinterpret_cast<u64*>(p); p += NCW * 8;                                 // 128
        c.sm.ssq_s = reinterpret_cast<float*>(p); p += NB * NCW * 4;                           // 512
        c.sm.wsc_s = reinterpret_cast<float*>(p); p += NB * NCW * 4;                           // 512
        c.sm.full = reinterpret_cast<uint64_t*>(p); p += 6 * 8;
        c.sm.empty = reinterpret_cast<uint64_t*>(p); p += 6 * 8;
        c.sm.xscale_s = reinterpret_cast<float*>(p); p += 8;
        c.sm.abort_flag = reinterpret_cast<volatile int*>(p); p += 4;
        c.sm.quit_flag = reinterpret_cast<volatile int*>(p); p += 4;
    }
    c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
    c.cta = blockIdx.x; c.grid = gridDim.x;
    c.cons_n = 0; c.red_n = 0; c.dead = false; c.prof = nullptr; c.wait_acc = 0; c.cur_op = 0; c.gemv_n = 0;
    c.limit_ns = (u64)A.spin_limit_ns;
    c.status = P.status;
    const int nb = A.nb;
    if (c.tid == 0) {
        for (int i = 0; i < NS; i++) {
            mbar_init(&c.sm.full[i], 1);
            mbar_init(&c.sm.empty[i], NCW);
        }
        *c.sm.abort_flag = 0;
        *c.sm.quit_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    for (int i = c.tid; i < nb * (P.max_seq / KV_BLOCK); i += NTHREADS) c.sm.bt_s[i] = P.block_table[i];
    __syncthreads();

    if (c.warp == NCW) {
        if (c.lane == 0) producer_batch<S>(c, P, A);
        return;
    }

    // ---------------- consumers ----------------
    const int NL5 = P.n_layers * OPS_PER_LAYER;
    const int OPS = NL5 + 1;                             // epochs per step
    int xr0, xr1;                                        // residual rows this CTA owns
    cta_rows(S::HID, 1, c.cta, c.grid, xr0, xr1);
    int lr0, lr1;                                        // LM-head rows this CTA owns
    cta_rows(P.vocab, 1, c.cta, c.grid, lr0, lr1);

    // Every sequence's winner over all CTAs' keys at epoch `e`, into best_s[sequence].
    auto reduce_keys = [&](uint32_t e) {
        if (c.tid < NB) c.sm.best_s[c.tid] = 0;
        consumer_sync();
        for (int idx = c.tid; idx < nb * c.grid; idx += NCT) {
            const u64* slot = P.lml + 2 * (size_t)idx;            // [sequence][cta][2]
            float hi, lo;
            ll_wait2(c, slot, e, W_LM, hi, lo);
            const u64 k = ((u64)__float_as_uint(hi) << 32) | __float_as_uint(lo);
            atomicMax(reinterpret_cast<unsigned long long*>(&c.sm.best_s[idx / c.grid]), k);
        }
        consumer_sync();
    };
    auto is_stop = [&](int token) {
        bool st = false;
        for (int i = 0; i < A.n_stop; i++) st |= (A.stop_ids[i] == token);
        return st;
    };

    int steps_done = 0;
    unsigned done_mask = 0;                              // frozen sequences: stop token produced, or all their steps run
    const unsigned all_mask = (1u << nb) - 1u;
    bool stopped = false;
    int tok[NB];
#pragma unroll
    for (int j = 0; j < NB; j++) tok[j] = 0;
    for (int s = 0; s < A.n_steps; s++) {
        const uint32_t e0 = A.epoch_base + (uint32_t)s * (uint32_t)OPS;
        c.prof = (A.prof && s == A.prof_step) ? A.prof + (size_t)c.cta * PROF_MAX_OPS * PROF_FIELDS : nullptr;
        if (c.cta == 0 && c.tid == 0 && A.step_ts) A.step_ts[s] = globaltimer();
        const bool have_keys = s > 0 && s - 1 >= A.lm_from;
        if (have_keys) reduce_keys(e0 - 1);
#pragma unroll
        for (int j = 0; j < NB; j++) {
            if (j < nb) {
                if (have_keys) {
                    const u64 key = c.sm.best_s[j];
                    if (c.cta == 0 && c.tid == 0) A.tokens_out[(size_t)(s - 1) * NB + j] = key;
                    if (s >= A.n_forced[j]) {
                        tok[j] = key_index(key);
                        if (is_stop(tok[j])) done_mask |= 1u << j;
                    }
                }
                if (s < A.n_forced[j]) tok[j] = A.forced[(size_t)s * NB + j];
            }
        }
        if (have_keys) consumer_sync();                  // best_s is reused by the next reduction
#pragma unroll
        for (int j = 0; j < NB; j++)
            if (j < nb && s >= A.n_total[j]) done_mask |= 1u << j;
        if (done_mask == all_mask) {
            stopped = true;
            break;
        }
        float x[NB][2];
#pragma unroll
        for (int j = 0; j < NB; j++) {
            x[j][0] = x[j][1] = 0.f;
            if (j < nb) {
                int t = tok[j];
                if (t < 0 || t >= P.vocab) t = 0;        // only reachable after a failed wait
                load_embedding<S, true>(P, t, c.tid, x[j][0], x[j][1]);
                if (2 * c.tid >= xr0 && 2 * c.tid < xr1) c.sm.xown[j * 16 + 2 * c.tid - xr0] = x[j][0];
                if (2 * c.tid + 1 >= xr0 && 2 * c.tid + 1 < xr1) c.sm.xown[j * 16 + 2 * c.tid + 1 - xr0] = x[j][1];
            }
        }
        bool failed = false;
        for (int l = 0; l < P.n_layers && !failed; l++)
            failed = run_layer_b<S, KVF32>(c, P, P.layer[l], A, s, done_mask, e0 + l * OPS_PER_LAYER, l * OPS_PER_LAYER, x, l == 0,
                                           xr0, xr1);
        if (failed) break;
        if (s >= A.lm_from) {
            // LM head: final RMSNorm, GEMV, optional logits dump, per-CTA best key per sequence at epoch eL
            const uint32_t eL = e0 + (uint32_t)OPS - 1;
            prof_stamp(c, NL5, 0);
            scale_prefetch(c, P.lm_scale, lr0, lr1, true);
            const float2 nw = *reinterpret_cast<const float2*>(P.final_norm + 2 * c.tid);
            wait_residual_b<S>(c, P.xl, eL - 1, nb, x);
            stage_rms_b<S>(c, x, nw);
            prof_stamp(c, NL5, 1);
            u64 best = 0;                                // warp j tracks sequence j
            const float invT = A.inv_temperature;
            float* logits = A.logits_out ? A.logits_out + (size_t)s * NB * P.vocab : nullptr;
            gemv_b<S, true>(c, lr0, lr1, S::HID, P.lm_scale, true, [&](int, int row, int j, float v, bool ok) {
                if (!ok || j >= nb) return;
                if (logits) logits[(size_t)j * P.vocab + row] = v;
                float score = v;
                if (invT != 0.f) {
                    const uint32_t hsh = mk_mix32(A.seed + (uint32_t)j * 0x9E3779B9u, (uint32_t)(A.pos0[j] + s), (uint32_t)row);
                    const float u = ((float)(hsh >> 8) + 0.5f) * (1.0f / 16777216.0f);
                    score = v * invT - __logf(-__logf(u));
                }
                const u64 key = score_key(score, row);
                best = key > best ? key : best;
            });
            if (c.warp < nb) {
                best = warp_max_u64(best);
                if (c.lane == 0) {
                    u64* slot = P.lml + ((size_t)c.warp * c.grid + c.cta) * 2;
                    ll_store_bits(slot, eL, (uint32_t)(best >> 32));
                    ll_store_bits(slot + 1, eL, (uint32_t)best);
                }
            }
            prof_stamp(c, NL5, 3);
            if (consumer_any(c.dead)) break;
        }
        steps_done = s + 1;
    }
    // The predictions of the last step that ran (if it ran the LM head and nothing stopped us).
    if (!stopped && steps_done == A.n_steps && A.n_steps > 0 && A.n_steps - 1 >= A.lm_from) {
        reduce_keys(A.epoch_base + (uint32_t)A.n_steps * (uint32_t)OPS - 1);
        if (c.cta == 0 && c.tid < nb) A.tokens_out[(size_t)(A.n_steps - 1) * NB + c.tid] = c.sm.best_s[c.tid];
    }
    if (c.tid == 0) *c.sm.quit_flag = 1;
    if (c.cta == 0 && c.tid == 0) {
        if (A.step_ts) A.step_ts[steps_done] = globaltimer();
        A.out_info[0] = steps_done;
        A.out_info[1] = (int)(A.epoch_base + (uint32_t)steps_done * (uint32_t)OPS);
        A.out_info[2] = (int)done_mask;
    }
}

}  // namespace mk
