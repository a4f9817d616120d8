// The non-GEMV stages of the stage-machine megakernel (embedding + token choice, Gated DeltaNet,
// attention, expert routing) and the kernel itself.  See mk_stage.cuh for the execution model.
#pragma once
#include "mk_stage.cuh"

namespace mks {

constexpr size_t MAILBOX_KEY_WORDS = (size_t)2 * MAILBOX_TILES * MKS_MAX_RANKS * 128;   // key exchange area starts here

// ---- token choice ----------------------------------------------------------------------------------------------
// Every sequence's arg-max over the keys the LM head's CTAs left in `keys` ([M][grid]); with tensor
// parallelism each rank's CTA 0 pushes its best key into every rank's mailbox and every CTA takes the
// maximum over ranks (a key carries the vocabulary row, so equal scores go to the lowest id on every rank).
__device__ void choose_tokens(Shared& S, Mut& mu, const Args& A, const u64* keys, uint32_t tag, int vocab) {
    if (warp_() < S.A.M) {
        const int m = warp_();
        u64 key = 0;
#pragma unroll 1
        for (int i = lane_(); i < grid_(); i += 32) {
            const u64 k = __ldcg(reinterpret_cast<const unsigned long long*>(keys + (size_t)m * grid_() + i));
            key = k > key ? k : key;
        }
        key = warp_max_u64(key);
        if (A.tp > 1) {
            if (cta_() == 0 && lane_() < A.tp) {
                unsigned long long* dst = A.mailbox[lane_()] + MAILBOX_KEY_WORDS + ((size_t)A.rank * MKS_MAX_BATCH + m) * 2;
                st_relaxed_sys_u64(dst, ((u64)tag << 32) | (uint32_t)(key >> 32));
                st_relaxed_sys_u64(dst + 1, ((u64)tag << 32) | (uint32_t)key);
            }
            const unsigned long long* src = A.mailbox[A.rank] + MAILBOX_KEY_WORDS + ((size_t)min(lane_(), A.tp - 1) * MKS_MAX_BATCH + m) * 2;
            Spin2 s;
            bool fail = false;
            u64 hi = 0, lo = 0;
#pragma unroll 1
            for (;;) {
                hi = ld_relaxed_sys_u64(src);
                lo = ld_relaxed_sys_u64(src + 1);
                const bool ok = (uint32_t)(hi >> 32) == tag && (uint32_t)(lo >> 32) == tag;
                if (__all_sync(0xffffffffu, ok)) break;
                if (!ok && MKS_SPIN_FAIL(S, s, WS_KEYS)) fail = true;
                if (__any_sync(0xffffffffu, fail)) {
                    mu.dead = true;
                    break;
                }
            }
            key = warp_max_u64(((hi & 0xffffffffull) << 32) | (lo & 0xffffffffull));
        }
        if (lane_() == 0) S.tok_s[m] = max(0, min(vocab - 1, key_index(key)));
    }
}

// ---- embedding ---------------------------------------------------------------------------------------------------
__device__ __noinline__ void embed_stage(Shared& S, Mut& mu, const mk_stage_desc& d, const Args& A, int step, uint32_t tag) {
    const int H = d.i[MKS_I_HIDDEN], vocab = d.i[MKS_I_VOCAB];
    if (step > 0 && d.i[MKS_I_KEYS_VALID] && d.p[MKS_P_E_KEYS]) {
        choose_tokens(S, mu, A, reinterpret_cast<const u64*>(d.p[MKS_P_E_KEYS]), tag, vocab);
        consumer_sync();
        if (cta_() == 0 && tid_() < S.A.M) {
            A.tok[tid_()] = S.tok_s[tid_()];
            if (A.tokens_out) A.tokens_out[(size_t)(step - 1) * S.A.M + tid_()] = S.tok_s[tid_()];
        }
    } else {
        if (tid_() < S.A.M) S.tok_s[tid_()] = max(0, min(vocab - 1, A.tok[tid_()]));
        consumer_sync();
    }
    if (step < A.n_tokens_in) {
        // a prompt position: the given token replaces the choice (which tokens_out still records)
        if (tid_() < S.A.M) S.tok_s[tid_()] = max(0, min(vocab - 1, __ldg(A.tokens_in + (size_t)step * S.A.M + tid_())));
        consumer_sync();
    }
    const __nv_bfloat16* table = reinterpret_cast<const __nv_bfloat16*>(d.p[MKS_P_TABLE]);
    float* h = reinterpret_cast<float*>(d.p[MKS_P_H]);
    float* ssq = reinterpret_cast<float*>(d.p[MKS_P_H_SSQ]);
    const float scale = d.f[MKS_F_SCALE];
    const int ng = H / 16;
    const int g0 = ng * cta_() / grid_(), g1 = ng * (cta_() + 1) / grid_();
    const int n = g1 - g0;
#pragma unroll 1
    for (int idx = tid_(); idx < n * S.A.M; idx += NCT) {
        const int m = idx / n, grp = g0 + idx % n;
        const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)S.tok_s[m] * H + grp * 16);
        const uint4 a = __ldg(src), b = __ldg(src + 1);
        const uint32_t wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        float q = 0.f;
        float* dst = h + (size_t)m * H + grp * 16;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float lo = bf_lo(wv[i]), hi = bf_hi(wv[i]);
            if (scale != 0.f) {
                lo = bf16_round(lo * scale);
                hi = bf16_round(hi * scale);
            }
            __stcg(dst + 2 * i, lo);
            __stcg(dst + 2 * i + 1, hi);
            q += lo * lo + hi * hi;
        }
        __stcg(ssq + (size_t)m * ng + grp, q);
    }
}

// ---- Gated DeltaNet ------------------------------------------------------------------------------------------------
// One task = one value head of one sequence, run by a whole CTA: 384 threads compute the causal conv1d
// (+ SiLU) of the head's q, k and v channels, the 16 warps each own 8 rows of the 128 x 128 state
// ([v][k], fp32): decay, delta-rule update and output row by row, then the head's gated RMSNorm.
// The conv history is a ring of four inputs per channel indexed by position & 3: this step's input
// goes to one slot while the other three are read, so tasks that share q/k channels never collide.
__device__ __noinline__ void gdn_stage(Shared& S, Mut& mu, const mk_stage_desc& d) {
    const int nkh = d.i[MKS_I_NKH], nvh = d.i[MKS_I_NVH], rep = nvh / nkh;
    const int key_dim = nkh * 128, conv_dim = d.i[MKS_I_CONV_DIM];
    const int q_off = d.i[MKS_I_Q_OFF], k_off = d.i[MKS_I_K_OFF], v_off = d.i[MKS_I_V_OFF], z_off = d.i[MKS_I_Z_OFF];
    const int b_off = d.i[MKS_I_B_OFF], a_off = d.i[MKS_I_A_OFF];
    const float* Y = reinterpret_cast<const float*>(d.p[MKS_P_Y]);
    float* Y2 = reinterpret_cast<float*>(d.p[MKS_P_Y2]);
    const float* convw = reinterpret_cast<const float*>(d.p[MKS_P_CONV_W]);
    const float* A_log = reinterpret_cast<const float*>(d.p[MKS_P_A_LOG]);
    const float* dt_bias = reinterpret_cast<const float*>(d.p[MKS_P_DT_BIAS]);
    const float* normw = reinterpret_cast<const float*>(d.p[MKS_P_GDN_NORM]);
    float* conv_state = reinterpret_cast<float*>(d.p[MKS_P_CONV_STATE]);
    float* ssm = reinterpret_cast<float*>(d.p[MKS_P_SSM_STATE]);
    const bool conv_bf16 = d.i[MKS_I_CONV_BF16] != 0, clamp = d.i[MKS_I_L2_CLAMP] != 0;
    const float eps = d.f[MKS_F_EPS];
    float* sm = reinterpret_cast<float*>(S.xs());          // q[128] k[128] v[128] o[128] scalars[8]
    float* scal = sm + 512;
    const int ntask = S.A.M * nvh;
#pragma unroll 1
    for (int task = cta_(); task < ntask; task += grid_()) {
        const int m = task / nvh, h = task % nvh, kh = h / rep;
        if (!S.valid_s[m]) continue;                           // a padding row keeps its state (uniform over the CTA)
        const int pos = S.pos_s[m];
        const float* y = Y + (size_t)m * d.i[MKS_I_Y_STRIDE];
        float* S = ssm + ((size_t)(m * nvh + h) * 128) * 128;
        float4 st[8];
#pragma unroll
        for (int r = 0; r < 8; r++) st[r] = __ldcg(reinterpret_cast<const float4*>(S + (size_t)(8 * warp_() + r) * 128) + lane_());
        if (tid_() < 384) {
            const int part = tid_() >> 7, i = tid_() & 127;
            const int ch = part == 0 ? kh * 128 + i : (part == 1 ? key_dim + kh * 128 + i : 2 * key_dim + h * 128 + i);
            const int ycol = part == 0 ? q_off + kh * 128 + i : (part == 1 ? k_off + kh * 128 + i : v_off + h * 128 + i);
            const float xnew = ldcg_f(y + ycol);
            const float4 cw = __ldg(reinterpret_cast<const float4*>(convw) + ch);          // taps, oldest first
            float* hist = conv_state + ((size_t)m * conv_dim + ch) * 4;
            const float h3 = ldcg_f(hist + ((pos - 3) & 3)), h2 = ldcg_f(hist + ((pos - 2) & 3)), h1 = ldcg_f(hist + ((pos - 1) & 3));
            float acc = h3 * cw.x;
            acc = fmaf(h2, cw.y, acc);
            acc = fmaf(h1, cw.z, acc);
            acc = fmaf(xnew, cw.w, acc);
            if (part == 2 || h % rep == 0) __stcg(hist + (pos & 3), conv_bf16 ? bf16_round(xnew) : xnew);
            sm[tid_()] = acc * sigmoid_f(acc);
        }
        consumer_sync();
        if (warp_() < 2) {
            const float* v = sm + warp_() * 128;
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) s = fmaf(v[lane_() + 32 * i], v[lane_() + 32 * i], s);
            s = warp_sum(s);
            if (lane_() == 0) {
                const float inv = clamp ? 1.f / fmaxf(sqrtf(s), eps) : 1.f / sqrtf(s + eps);
                scal[warp_()] = warp_() == 0 ? inv * 0.08838834764831845f : inv;             // q also takes 128^-0.5
            }
        } else if (warp_() == 2 && lane_() == 0) {
            const float b = ldcg_f(y + b_off + h), a = ldcg_f(y + a_off + h);
            scal[2] = sigmoid_f(b);
            scal[3] = expf(-expf(A_log[h]) * softplus_f(a + dt_bias[h]));
        }
        consumer_sync();
        {
            const float qs = scal[0], ks = scal[1], beta = scal[2], dec = scal[3];
            const float4 kq = reinterpret_cast<const float4*>(sm + 128)[lane_()];
            const float4 qq = reinterpret_cast<const float4*>(sm)[lane_()];
            const float k0 = kq.x * ks, k1 = kq.y * ks, k2 = kq.z * ks, k3 = kq.w * ks;
            const float q0 = qq.x * qs, q1 = qq.y * qs, q2 = qq.z * qs, q3 = qq.w * qs;
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const int vrow = 8 * warp_() + r;
                float4 s4 = st[r];
                s4.x *= dec; s4.y *= dec; s4.z *= dec; s4.w *= dec;
                float kv = fmaf(s4.x, k0, fmaf(s4.y, k1, fmaf(s4.z, k2, s4.w * k3)));
                kv = warp_sum(kv);
                const float delta = (sm[256 + vrow] - kv) * beta;
                s4.x = fmaf(delta, k0, s4.x); s4.y = fmaf(delta, k1, s4.y);
                s4.z = fmaf(delta, k2, s4.z); s4.w = fmaf(delta, k3, s4.w);
                float o = fmaf(s4.x, q0, fmaf(s4.y, q1, fmaf(s4.z, q2, s4.w * q3)));
                o = warp_sum(o);
                __stcg(reinterpret_cast<float4*>(S + (size_t)vrow * 128) + lane_(), s4);
                if (lane_() == 0) sm[384 + vrow] = o;
            }
        }
        consumer_sync();
        if (warp_() == 0) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) s = fmaf(sm[384 + lane_() + 32 * i], sm[384 + lane_() + 32 * i], s);
            s = warp_sum(s);
            if (lane_() == 0) scal[4] = rsqrtf(s / 128.f + eps);
        }
        consumer_sync();
        if (tid_() < 128) {
            const float z = ldcg_f(y + z_off + h * 128 + tid_());
            __stcg(Y2 + (size_t)m * d.i[MKS_I_Y2_STRIDE] + h * 128 + tid_(), sm[384 + tid_()] * scal[4] * normw[tid_()] * (z * sigmoid_f(z)));
        }
        consumer_sync();
    }
}

// ---- attention ---------------------------------------------------------------------------------------------------
// One task = one chunk of cached positions of one KV head of one sequence, run by a whole CTA:
//   1. the KV head's query heads are normed, rotated and kept in shared memory; the task whose chunk ends
//      at the new position also norms / rotates the new K and V rows and writes them to the paged cache;
//   2. the warps share the chunk's positions and write scaled scores [head][position];
//   3. per head the chunk's maximum and sum; 4. the warps share the head dimension and add up P x V;
//   5. the chunk's (acc, max, sum) goes to global memory; the last chunk to arrive merges all of them,
//      applies the output gate and writes the mixer output.
template <bool KVF32>
__device__ __forceinline__ void load8(const void* row, int elem, float (&v)[8]) {
    if (KVF32) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(row) + elem));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(row) + elem) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 a = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(row) + elem));
        v[0] = bf_lo(a.x); v[1] = bf_hi(a.x); v[2] = bf_lo(a.y); v[3] = bf_hi(a.y);
        v[4] = bf_lo(a.z); v[5] = bf_hi(a.z); v[6] = bf_lo(a.w); v[7] = bf_hi(a.w);
    }
}

// RMS-norm (optional), rotate and round one head vector; one warp.  `dst` receives HD <= 512 floats.  All of a
// lane's loads are requested before the first is used (one L2 round trip for the vector, one for the weights).
__device__ __noinline__ void head_prepare(Shared& S, Mut& mu, const float* src, float* dst, int HD, const float* nw, float norm_off, bool do_norm,
                                          float eps, const float* cs, const float* sn, int pairs, int pair_dist, bool round_bf16) {
    float v[16], w[16];
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int i = lane_() + 32 * j;
        v[j] = i < HD ? ldcg_f(src + i) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int i = lane_() + 32 * j;
        w[j] = nw && i < HD ? norm_off + __ldg(nw + i) : 1.f;
    }
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 16; j++)
        if (lane_() + 32 * j < HD) s = fmaf(v[j], v[j], s);
    s = warp_sum(s);
    const float r = do_norm ? rsqrtf(s / (float)HD + eps) : 1.f;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int i = lane_() + 32 * j;
        if (i < HD) dst[i] = v[j] * r * w[j];
    }
    __syncwarp();
    if (cs) {
#pragma unroll 1
        for (int i = lane_(); i < pairs; i += 32) {
            const float a = dst[i], b = dst[i + pair_dist], co = cs[i], si = sn[i];
            dst[i] = a * co - b * si;
            dst[i + pair_dist] = b * co + a * si;
        }
        __syncwarp();
    }
    if (round_bf16)
#pragma unroll 1
        for (int i = lane_(); i < HD; i += 32) dst[i] = bf16_round(dst[i]);
    __syncwarp();
}

// Latency, not bandwidth, decides this stage (a task reads a few hundred KB): every loop over cached positions
// asks for several rows before it uses the first, the page-table lookups are done once per task into shared
// memory, and the merge first turns the chunks' (max, sum) pairs into weights in shared memory.
constexpr int ATTN_MAX_CHUNKS = 256;      // split records per (sequence, kv head)

template <bool KVF32>
__device__ __noinline__ void attn_stage(Shared& S, Mut& mu, const mk_stage_desc& d) {
    const int NQ = d.i[MKS_I_NQ], NKV = d.i[MKS_I_NKV], HD = d.i[MKS_I_HD], ROT = d.i[MKS_I_ROT];
    const int QPK = NQ / NKV, CP = d.i[MKS_I_CHUNK_POS], window = d.i[MKS_I_WINDOW], maxpages = d.i[MKS_I_MAX_PAGES];
    const int kvb = d.i[MKS_I_KV_BLOCK] > 0 ? d.i[MKS_I_KV_BLOCK] : 64, kvb_shift = 31 - __clz(kvb);
    const bool own_layout = d.i[MKS_I_KV_S_PAGE] == 0;
    const uint32_t kv_s_page = own_layout ? (uint32_t)(NKV * kvb * HD) : (uint32_t)d.i[MKS_I_KV_S_PAGE];
    const uint32_t kv_s_head = own_layout ? (uint32_t)(kvb * HD) : (uint32_t)d.i[MKS_I_KV_S_HEAD];
    const uint32_t kv_s_pos = own_layout ? (uint32_t)HD : (uint32_t)d.i[MKS_I_KV_S_POS];
    const int pairs = d.i[MKS_I_ROPE_PAIRS], pair_dist = ROT == HD ? HD / 2 : ROT / 2;
    const int q_off = d.i[MKS_I_A_Q_OFF], q_hs = d.i[MKS_I_A_Q_HSTRIDE], gate_off = d.i[MKS_I_A_GATE_OFF];
    const int k_off = d.i[MKS_I_A_K_OFF], v_off = d.i[MKS_I_A_V_OFF];
    const float* Y = reinterpret_cast<const float*>(d.p[MKS_P_A_Y]);
    float* Y2 = reinterpret_cast<float*>(d.p[MKS_P_A_Y2]);
    const float* qn = reinterpret_cast<const float*>(d.p[MKS_P_Q_NORM]);
    const float* kn = reinterpret_cast<const float*>(d.p[MKS_P_K_NORM]);
    uint8_t* kc = reinterpret_cast<uint8_t*>(d.p[MKS_P_K_CACHE]);
    uint8_t* vc = reinterpret_cast<uint8_t*>(d.p[MKS_P_V_CACHE]);
    const int* bt = reinterpret_cast<const int*>(d.p[MKS_P_BLOCK_TABLE]);
    const float* cosT = reinterpret_cast<const float*>(d.p[MKS_P_ROPE_COS]);
    const float* sinT = reinterpret_cast<const float*>(d.p[MKS_P_ROPE_SIN]);
    float* part = reinterpret_cast<float*>(d.p[MKS_P_A_PART]);
    unsigned* cnt = reinterpret_cast<unsigned*>(d.p[MKS_P_A_CNT]);
    const float eps = d.f[MKS_F_EPS], scale = d.f[MKS_F_SCALE];
    const float norm_off = d.i[MKS_I_NORM_PLAIN] ? 0.f : 1.f;
    const bool q_bf16 = d.i[MKS_I_Q_BF16] != 0;
    const int esz = KVF32 ? 4 : 2;
    const int rec = (QPK * (HD + 2) + 3) & ~3;                 // floats of one chunk's partial record (whole float4s: QPK may be odd)
    const int max_chunks = d.i[MKS_I_MAX_CHUNKS];
    // this CTA's rows behind the partial records: [16 warps][QPK][128] sums of the P x V pieces
    float* scratch = part + (size_t)S.A.M * NKV * max_chunks * rec + (size_t)cta_() * NCW * QPK * 128;
    // shared scratch
    float* q_s = reinterpret_cast<float*>(S.xs());             // [QPK][HD]
    float* kn_s = q_s + QPK * HD;                              // [HD] the new K row
    float* vn_s = kn_s + HD;                                   // [HD] the new V row
    float* sc_s = vn_s + HD;                                   // [QPK][CP] scores, then probabilities
    float* wn_s = sc_s + QPK * CP;                             // [QPK][chunks] merge weights
    float* stat_s = wn_s + QPK * ATTN_MAX_CHUNKS;              // [QPK][2]
    uint32_t* row_s = reinterpret_cast<uint32_t*>(stat_s + 2 * QPK);   // [CP] element offset of each position's cache row
    // chunks per sequence: the longest context decides the task grid
    int maxn = 1;
#pragma unroll 1
    for (int m = 0; m < S.A.M; m++) {
        const int n = S.pos_s[m] + 1;
        maxn = max(maxn, window ? min(n, window) : n);
    }
    const int NCH = (maxn + CP - 1) / CP;
    const int ntask = S.A.M * NKV * NCH;
#pragma unroll 1
    for (int task = cta_(); task < ntask; task += grid_()) {
        const int ch = task % NCH, kvh = (task / NCH) % NKV, m = task / (NCH * NKV);
        if (!S.valid_s[m]) continue;                           // a padding row reads and writes no KV (uniform over the CTA)
        const int pos = S.pos_s[m], n = pos + 1;
        const int lo = window ? max(0, n - window) : 0;
        const int first = lo + ch * CP;
        if (first >= n) continue;                              // uniform over the CTA
        const int last = min(first + CP, n), np = last - first;
        const int nch = (n - lo + CP - 1) / CP;
        const float* y = Y + (size_t)m * d.i[MKS_I_A_Y_STRIDE];
        const float* cs = cosT + (size_t)pos * pairs;
        const float* sn = sinT + (size_t)pos * pairs;
        const bool has_new = last == n;
        const int ncached = has_new ? np - 1 : np;             // positions of the chunk that come from the cache
        // 1. queries (warps 0..QPK-1), new K (warp QPK), new V (warp QPK + 1), cache row offsets (the other warps)
        if (warp_() < QPK) {
            const int hq = kvh * QPK + warp_();
            head_prepare(S, mu, y + q_off + (size_t)hq * q_hs, q_s + warp_() * HD, HD, qn, norm_off, true, eps, cs, sn, pairs, pair_dist, q_bf16);
        } else if (has_new && warp_() == QPK) {
            head_prepare(S, mu, y + k_off + (size_t)kvh * HD, kn_s, HD, kn, norm_off, true, eps, cs, sn, pairs, pair_dist, !KVF32);
        } else if (has_new && warp_() == QPK + 1) {
            const float* vsrc = v_off >= 0 ? y + v_off + (size_t)kvh * HD : y + k_off + (size_t)kvh * HD;
            head_prepare(S, mu, vsrc, vn_s, HD, nullptr, 0.f, d.i[MKS_I_V_NORM] != 0, eps, nullptr, nullptr, 0, 0, !KVF32);
        } else if (warp_() >= QPK + 2) {
#pragma unroll 1
            for (int i = tid_() - (QPK + 2) * 32; i < np; i += NCT - (QPK + 2) * 32) {
                const int p = first + i;
                const int page = __ldg(bt + (size_t)m * maxpages + (p >> kvb_shift));
                const uint32_t off = (uint32_t)page * kv_s_page + (uint32_t)kvh * kv_s_head + (uint32_t)(p & (kvb - 1)) * kv_s_pos;
                row_s[i] = off;
                // touch every cache block of the chunk once now: the weight stream between two attention stages has
                // pushed the cache's pages out of the TLBs, and the first touch of a page costs several microseconds.
                // (One line per block, not the rows themselves: an SM retires about one L2 prefetch per 25 cycles, and
                // asking for all 8 lines of all 580 rows of a batch-8 chunk took 60 us.)
                if (i < ncached && (i == 0 || (p & (kvb - 1)) == 0)) {
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(kc + (size_t)off * esz));
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(vc + (size_t)off * esz));
                }
            }
        }
        consumer_sync();
        if (has_new && warp_() >= QPK && warp_() < QPK + 2) {
            // append the new row to the paged cache
            const float* srcv = warp_() == QPK ? kn_s : vn_s;
            uint8_t* dst = (warp_() == QPK ? kc : vc) + (size_t)row_s[np - 1] * esz;
#pragma unroll 1
            for (int i = lane_(); i < HD; i += 32) {
                if (KVF32) reinterpret_cast<float*>(dst)[i] = srcv[i];
                else reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(srcv[i]);
            }
        }
        prof_mark(S, 4);
        // 2. scores: a warp takes every 16th position, four of them per turn, a lane 8 dims of every 256 of the K row.
        //    The four rows are requested before the first is used; the 4 x 8 (position, head) partial dots of a lane
        //    are summed over the warp by a transposing butterfly (31 shuffles instead of 160) that leaves sum l in lane l.
#pragma unroll 1
        for (int i0 = warp_(); i0 < np; i0 += NCW * 4) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = 0.f;
#pragma unroll 1
            for (int e = lane_() * 8; e < HD; e += 256) {
                float kv[4][8];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int i = i0 + u * NCW;
                    if (i < ncached) {
                        load8<KVF32>(kc + (size_t)row_s[i] * esz, e, kv[u]);
                    } else {
#pragma unroll
                        for (int x = 0; x < 8; x++) kv[u][x] = i < np ? kn_s[e + x] : 0.f;     // the new row, or past the chunk
                    }
                }
#pragma unroll
                for (int hq = 0; hq < 8; hq++) {
                    if (hq < QPK) {
                        const float4 qa = *reinterpret_cast<const float4*>(q_s + hq * HD + e);
                        const float4 qb = *reinterpret_cast<const float4*>(q_s + hq * HD + e + 4);
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            float a = v[u * 8 + hq];
                            a = fmaf(qa.x, kv[u][0], a); a = fmaf(qa.y, kv[u][1], a); a = fmaf(qa.z, kv[u][2], a); a = fmaf(qa.w, kv[u][3], a);
                            a = fmaf(qb.x, kv[u][4], a); a = fmaf(qb.y, kv[u][5], a); a = fmaf(qb.z, kv[u][6], a); a = fmaf(qb.w, kv[u][7], a);
                            v[u * 8 + hq] = a;
                        }
                    }
                }
            }
#pragma unroll
            for (int o = 16, n = 16; o; o >>= 1, n >>= 1) {
                const bool up = (lane_() & o) != 0;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (j < n) {
                        const float send = up ? v[j] : v[j + n], keep = up ? v[j + n] : v[j];
                        v[j] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                    }
                }
            }
            {
                const int u = lane_() >> 3, hq = lane_() & 7, i = i0 + u * NCW;
                if (hq < QPK && i < np) sc_s[hq * CP + i] = v[0] * scale;
            }
        }
        consumer_sync();
        prof_mark(S, 5);
        // 3. per head: maximum, exponentials, sum
        if (warp_() < QPK) {
            float* sc = sc_s + warp_() * CP;
            float mx = -3.0e38f;
#pragma unroll 1
            for (int i = lane_(); i < np; i += 32) mx = fmaxf(mx, sc[i]);
            mx = warp_max(mx);
            float l = 0.f;
#pragma unroll 1
            for (int i = lane_(); i < np; i += 32) {
                const float ex = __expf(sc[i] - mx);
                sc[i] = ex;
                l += ex;
            }
            l = warp_sum(l);
            if (lane_() == 0) {
                stat_s[2 * warp_()] = mx;
                stat_s[2 * warp_() + 1] = l;
            }
        }
        consumer_sync();
        // 4. P x V: warp = (128-dim piece of the head, residue class of the positions), lane = 4 dims; a lane keeps
        //    its four outputs of every query head and asks for PB rows before it uses the first.  The warps of a piece
        //    then leave their sums in this CTA's scratch rows and every thread adds a few outputs in warp order.
        float* prec = part + ((size_t)(m * NKV + kvh) * max_chunks + ch) * rec;
        {
            constexpr int PB = KVF32 ? 4 : 8;
            const int ndc = HD / 128, nres = NCW / ndc;
            const int dc = warp_() % ndc, res = warp_() / ndc;
            const int e0 = dc * 128 + lane_() * 4;
            float acc[8][4];
#pragma unroll
            for (int hq = 0; hq < 8; hq++) acc[hq][0] = acc[hq][1] = acc[hq][2] = acc[hq][3] = 0.f;
#pragma unroll 1
            for (int i0 = res; i0 < ncached; i0 += nres * PB) {
                float vv[PB][4];
#pragma unroll
                for (int u = 0; u < PB; u++) {
                    const int i = i0 + u * nres;
                    vv[u][0] = vv[u][1] = vv[u][2] = vv[u][3] = 0.f;
                    if (i < ncached) {
                        const uint8_t* row = vc + (size_t)row_s[i] * esz;
                        if (KVF32) {
                            const float4 q4 = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(row) + e0));
                            vv[u][0] = q4.x; vv[u][1] = q4.y; vv[u][2] = q4.z; vv[u][3] = q4.w;
                        } else {
                            const uint2 q2 = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(row) + e0));
                            vv[u][0] = bf_lo(q2.x); vv[u][1] = bf_hi(q2.x); vv[u][2] = bf_lo(q2.y); vv[u][3] = bf_hi(q2.y);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < PB; u++) {
                    const int i = min(i0 + u * nres, ncached - 1);          // rows past the end were read as zeros
#pragma unroll
                    for (int hq = 0; hq < 8; hq++) {
                        if (hq < QPK) {
                            const float w = sc_s[hq * CP + i];
                            acc[hq][0] = fmaf(w, vv[u][0], acc[hq][0]); acc[hq][1] = fmaf(w, vv[u][1], acc[hq][1]);
                            acc[hq][2] = fmaf(w, vv[u][2], acc[hq][2]); acc[hq][3] = fmaf(w, vv[u][3], acc[hq][3]);
                        }
                    }
                }
            }
            if (has_new && res == 0) {
#pragma unroll
                for (int hq = 0; hq < 8; hq++) {
                    if (hq < QPK) {
                        const float w = sc_s[hq * CP + np - 1];
                        acc[hq][0] = fmaf(w, vn_s[e0], acc[hq][0]); acc[hq][1] = fmaf(w, vn_s[e0 + 1], acc[hq][1]);
                        acc[hq][2] = fmaf(w, vn_s[e0 + 2], acc[hq][2]); acc[hq][3] = fmaf(w, vn_s[e0 + 3], acc[hq][3]);
                    }
                }
            }
            float* mine = scratch + ((size_t)warp_() * QPK) * 128 + lane_() * 4;
#pragma unroll
            for (int hq = 0; hq < 8; hq++)
                if (hq < QPK) __stcg(reinterpret_cast<float4*>(mine + hq * 128), make_float4(acc[hq][0], acc[hq][1], acc[hq][2], acc[hq][3]));
            fence_acq_rel_gpu();
            consumer_sync();
#pragma unroll 1
            for (int idx = tid_(); idx < QPK * (HD / 4); idx += NCT) {
                const int hq = idx / (HD / 4), dd = (idx - hq * (HD / 4)) * 4;
                const float* src = scratch + ((size_t)(dd >> 7) * QPK + hq) * 128 + (dd & 127);    // warp (residue 0, piece dd / 128)
                float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                for (int r = 0; r < nres; r++) {
                    const float4 t4 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)r * ndc * QPK * 128));
                    o.x += t4.x; o.y += t4.y; o.z += t4.z; o.w += t4.w;
                }
                __stcg(reinterpret_cast<float4*>(prec + hq * HD + dd), o);
            }
        }
        if (tid_() < 2 * QPK) __stcg(prec + QPK * HD + tid_(), stat_s[tid_()]);
        // 5. arrival; the last chunk merges
        fence_acq_rel_gpu();
        consumer_sync();
        prof_mark(S, 6);
        if (tid_() == 0) {
            chaos_delay();
            const unsigned old = atomicAdd(cnt + m * NKV + kvh, 1u);
            const int is_last = (int)(old + 1u == (unsigned)nch);
            if (is_last) {
                cnt[m * NKV + kvh] = 0u;
                fence_acq_rel_gpu();
            }
            S.flag = is_last;
        }
        consumer_sync();
        if (S.flag) {
            const float* pbase = part + ((size_t)(m * NKV + kvh) * max_chunks) * rec;
            // weights of the chunks: w[hq][j] = exp(max_j - max) / sum_j' exp(max_j' - max) l_j'
#pragma unroll 1
            for (int i = tid_(); i < QPK * nch; i += NCT) {
                const int hq = i / nch, j = i - hq * nch;
                wn_s[hq * ATTN_MAX_CHUNKS + j] = ldcg_f(pbase + (size_t)j * rec + QPK * HD + 2 * hq);
            }
            consumer_sync();
            if (warp_() < QPK) {
                float* w = wn_s + warp_() * ATTN_MAX_CHUNKS;
                float mx = -3.0e38f;
#pragma unroll 1
                for (int j = lane_(); j < nch; j += 32) mx = fmaxf(mx, w[j]);
                mx = warp_max(mx);
                float den = 0.f;
#pragma unroll 1
                for (int j = lane_(); j < nch; j += 32) {
                    const float ex = __expf(w[j] - mx);
                    w[j] = ex;
                    den += ex * ldcg_f(pbase + (size_t)j * rec + QPK * HD + 2 * warp_() + 1);
                }
                den = warp_sum(den);
                __syncwarp();
#pragma unroll 1
                for (int j = lane_(); j < nch; j += 32) w[j] = w[j] / den;
            }
            consumer_sync();
#pragma unroll 1
            for (int idx = tid_(); idx < QPK * (HD / 4); idx += NCT) {
                const int hq = idx / (HD / 4), dd = (idx - hq * (HD / 4)) * 4;
                const float* w = wn_s + hq * ATTN_MAX_CHUNKS;
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll 8
                for (int j = 0; j < nch; j++) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(pbase + (size_t)j * rec + hq * HD + dd));
                    o0 = fmaf(w[j], v.x, o0); o1 = fmaf(w[j], v.y, o1); o2 = fmaf(w[j], v.z, o2); o3 = fmaf(w[j], v.w, o3);
                }
                const int hfull = kvh * QPK + hq;
                if (gate_off >= 0) {
                    const float4 g = __ldcg(reinterpret_cast<const float4*>(y + q_off + (size_t)hfull * q_hs + gate_off + dd));
                    o0 *= sigmoid_f(g.x); o1 *= sigmoid_f(g.y); o2 *= sigmoid_f(g.z); o3 *= sigmoid_f(g.w);
                }
                __stcg(reinterpret_cast<float4*>(Y2 + (size_t)m * d.i[MKS_I_A_Y2_STRIDE] + (size_t)hfull * HD + dd), make_float4(o0, o1, o2, o3));
            }
        }
        consumer_sync();
    }
}

// ---- expert routing ------------------------------------------------------------------------------------------------
// Every CTA builds the same tables from the router logits: per sequence the top-k experts (ties to the
// lower id) and their weights, the list of distinct experts in ascending id (the groups of the routed
// GEMV stages) and coef[group][sequence], the weight with which a group's product enters a sequence.
__device__ __noinline__ void route_stage(Shared& S, Mut& mu, const mk_stage_desc& d) {
    const int E = d.i[MKS_I_EXPERTS], topk = d.i[MKS_I_TOPK], stride = d.i[MKS_I_LOGIT_STRIDE], kind = d.i[MKS_I_ROUTE_KIND];
    const float* logits = reinterpret_cast<const float*>(d.p[MKS_P_LOGITS]);
    const float* pes = reinterpret_cast<const float*>(d.p[MKS_P_EXPERT_SCALE]);
    if (tid_() < 8) S.gmask[tid_()] = 0u;
#pragma unroll 1
    for (int i = tid_(); i < MAX_GROUPS * 8; i += NCT) S.coef[i] = 0.f;
    consumer_sync();
    if (warp_() < S.A.M && S.valid_s[warp_()]) {              // a padding row selects no expert
        const int m = warp_();
        float v[8];
        bool used[8];
        const int per = E / 32;                                   // 8 (256 experts) or 4 (128)
#pragma unroll
        for (int i = 0; i < 8; i++) {
            v[i] = i < per ? ldcg_f(logits + (size_t)m * stride + lane_() + 32 * i) : 0.f;
            used[i] = i >= per;
        }
        float top0 = 0.f, wsum = 0.f, myw = 0.f;
#pragma unroll 1
        for (int k = 0; k < topk; k++) {
            u64 best = 0;
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (!used[i]) {
                    const u64 key = score_key(v[i], lane_() + 32 * i);
                    best = key > best ? key : best;
                }
            best = warp_max_u64(best);
            int id = key_index(best);
            id = max(0, min(E - 1, id));
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (lane_() + 32 * i == id) used[i] = true;
            float mine = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (i == (id >> 5)) mine = v[i];
            const float sc = __shfl_sync(0xffffffffu, mine, id & 31);
            if (k == 0) top0 = sc;
            const float w = __expf(sc - top0);
            wsum += w;
            if (lane_() == k) myw = w;
            if (lane_() == 0) {
                S.r_ids[m * 8 + k] = id;
                atomicOr(&S.gmask[id >> 5], 1u << (id & 31));
            }
        }
        if (lane_() < topk) {
            const int id = S.r_ids[m * 8 + lane_()];
            S.r_w[m * 8 + lane_()] = myw / wsum * (kind == 1 && pes ? pes[id] : 1.f);
            int* ids_out = reinterpret_cast<int*>(d.p[MKS_P_ROUTE_OUT]);
            if (ids_out && cta_() == 0) ids_out[m * topk + lane_()] = id;
        }
    }
    consumer_sync();
    auto rank_of = [&](int id) {
        int r = 0;
#pragma unroll 1
        for (int w = 0; w < (id >> 5); w++) r += __popc(S.gmask[w]);
        return r + __popc(S.gmask[id >> 5] & ((1u << (id & 31)) - 1u));
    };
    if (tid_() < E && (S.gmask[tid_() >> 5] >> (tid_() & 31)) & 1u) S.glist[rank_of(tid_())] = tid_();
    if (warp_() < S.A.M && S.valid_s[warp_()] && lane_() < topk) S.coef[rank_of(S.r_ids[warp_() * 8 + lane_()]) * 8 + warp_()] = S.r_w[warp_() * 8 + lane_()];
    int U = 0;
#pragma unroll 1
    for (int w = 0; w < 8; w++) U += __popc(S.gmask[w]);
    if (kind == 0 && tid_() < S.A.M) S.coef[U * 8 + tid_()] = sigmoid_f(ldcg_f(logits + (size_t)tid_() * stride + E));   // the shared expert's gate
    consumer_sync();
    if (tid_() == 0) {
        S.n_groups = kind == 0 ? U + 1 : U;
        __threadfence_block();
        S.route_seq = S.route_seq + 1;
    }
    consumer_sync();
}

// ---- element-wise residual / sandwich-norm step ------------------------------------------------------------------
// out[m][i] = (base[m][i] + a[m][i] rstd_a[m] (off + w_a[i]) [+ b[m][i] rstd_b[m] (off + w_b[i])]) * scale, and the sums
// of squares of the result per 16 elements.  rstd comes from the 16-element sums of squares the producing GEMV stage
// left (every CTA adds them up itself, in a fixed order); a CTA then takes a slice of the 16-element groups.
__device__ __noinline__ void vec_stage(Shared& S, Mut& mu, const mk_stage_desc& d) {
    const int N = d.i[MKS_I_VEC_N], ng = N / 16, M = S.A.M;
    if (N == 0) return;                                        // an empty stage: its barrier only
    const float* base = reinterpret_cast<const float*>(d.p[MKS_P_VEC_BASE]);
    const float* a = reinterpret_cast<const float*>(d.p[MKS_P_VEC_A]);
    const float* b = reinterpret_cast<const float*>(d.p[MKS_P_VEC_B]);
    const float* wa = reinterpret_cast<const float*>(d.p[MKS_P_VEC_A_W]);
    const float* wb = reinterpret_cast<const float*>(d.p[MKS_P_VEC_B_W]);
    float* out = reinterpret_cast<float*>(d.p[MKS_P_VEC_OUT]);
    float* out_ssq = reinterpret_cast<float*>(d.p[MKS_P_VEC_OUT_SSQ]);
    const float eps = d.f[MKS_F_EPS], off = d.f[MKS_F_NORM_OFF];
    const float scale = d.f[MKS_F_SCALE] != 0.f ? d.f[MKS_F_SCALE] : 1.f;
    // warps 0..M-1: rstd of a; warps 8..8+M-1: rstd of b
    {
        const int m = warp_() & 7;
        const bool second = warp_() >= 8;
        const float* ssq = reinterpret_cast<const float*>(d.p[second ? MKS_P_VEC_B_SSQ : MKS_P_VEC_A_SSQ]);
        if (m < M && (!second || b)) {
            float s = 0.f;
#pragma unroll 4
            for (int j = lane_(); j < ng; j += 32) s += ldcg_f(ssq + (size_t)m * ng + j);
            s = warp_sum(s);
            if (lane_() == 0) S.red[(second ? 8 : 0) + m] = rsqrtf(s / (float)N + eps);
        }
    }
    consumer_sync();
    const int g0 = ng * cta_() / grid_(), g1 = ng * (cta_() + 1) / grid_();
    const int n = g1 - g0;
#pragma unroll 1
    for (int idx0 = 0; idx0 < n * M * 4; idx0 += NCT) {
        // four threads share a 16-element group: each takes a float4 and the group's sum of squares is shuffled together
        // (every lane of a warp takes part in the shuffles; the ones past the end carry zeros)
        const int idx = idx0 + tid_();
        const bool live = idx < n * M * 4;
        const int q4 = idx & 3, gi = live ? idx >> 2 : 0;
        const int m = gi / n, grp = g0 + gi - m * n;
        const size_t o = (size_t)m * N + grp * 16 + q4 * 4;
        float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            const float4 av = __ldcg(reinterpret_cast<const float4*>(a + o));
            const float4 aw = __ldg(reinterpret_cast<const float4*>(wa + grp * 16 + q4 * 4));
            const float ra = S.red[m];
            r = make_float4(av.x * ra * (off + aw.x), av.y * ra * (off + aw.y), av.z * ra * (off + aw.z), av.w * ra * (off + aw.w));
            if (b) {
                const float4 bv = __ldcg(reinterpret_cast<const float4*>(b + o));
                const float4 bw = __ldg(reinterpret_cast<const float4*>(wb + grp * 16 + q4 * 4));
                const float rb = S.red[8 + m];
                r.x += bv.x * rb * (off + bw.x); r.y += bv.y * rb * (off + bw.y); r.z += bv.z * rb * (off + bw.z); r.w += bv.w * rb * (off + bw.w);
            }
            if (base) {
                const float4 hv = __ldcg(reinterpret_cast<const float4*>(base + o));
                r.x += hv.x; r.y += hv.y; r.z += hv.z; r.w += hv.w;
            }
            r.x *= scale; r.y *= scale; r.z *= scale; r.w *= scale;
            __stcg(reinterpret_cast<float4*>(out + o), r);
        }
        float q = r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w;
        q += __shfl_xor_sync(0xffffffffu, q, 1);
        q += __shfl_xor_sync(0xffffffffu, q, 2);
        if (live && out_ssq && q4 == 0) __stcg(out_ssq + (size_t)m * ng + grp, q);
    }
}

// ---- the kernel ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHREADS, 1) stage_kernel(const __grid_constant__ Args A_in) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Shared& S = *reinterpret_cast<Shared*>(smem_raw);
    Mut mu;
    mu.chunk_n = 0; mu.dead = false;
    {
        // the launch arguments, once, into shared memory
        constexpr int ARG_WORDS = (int)(sizeof(Args) / 4);
        const uint32_t* src = reinterpret_cast<const uint32_t*>(&A_in);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&S.A);
        if (tid_() < ARG_WORDS) dst[tid_()] = src[tid_()];
    }
    if (tid_() == 0) S.prof = nullptr;
    if (tid_() == 0) {
#pragma unroll 1
        for (int i = 0; i < NS; i++) {
            mbar_init(&S.full[i], 1);
            mbar_init(&S.empty[i], 1);
        }
        S.abort_flag = 0;
        S.route_seq = 0;
        S.n_groups = 0;
        S.pf_pos = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (tid_() < 8) {
        S.xinv[tid_()] = 1.f;
        S.rstd[tid_()] = 1.f;
        S.tok_s[tid_()] = 0;
        S.pos_s[tid_()] = tid_() < A_in.M ? A_in.pos[tid_()] : 0;
        S.valid_s[tid_()] = tid_() < A_in.M && (!A_in.row_valid || A_in.row_valid[tid_()] != 0);
    }
    __syncthreads();
    const Args& A = S.A;

    if (warp_() == NCW) {
        producer_main(S, A);
        return;
    }
    // stage records travel through shared memory: the next one is requested while the current stage runs
    constexpr int DESC_WORDS = (int)(sizeof(mk_stage_desc) / 4);
    if (tid_() < DESC_WORDS) reinterpret_cast<uint32_t*>(&S.desc[0])[tid_()] = __ldg(reinterpret_cast<const uint32_t*>(&A.prog[0]) + tid_());
    int cur = 0;

    u64 bar_n = 0, ar_seq = A.ar_base;
    bool failed = false;
#pragma unroll 1
    for (int step = 0; step < A.n_steps && !failed; step++) {
        if (tid_() < S.A.M) S.pos_s[tid_()] = A.pos[tid_()] + (S.valid_s[tid_()] ? step : 0);
        consumer_sync();
#pragma unroll 1
        for (int si = 0; si < A.n_stages; si++) {
            if (consumer_any(mu.dead || S.abort_flag != 0)) {
                failed = true;
                break;
            }
            const mk_stage_desc& d = S.desc[cur];
            uint32_t next_word = 0;
            if (tid_() < DESC_WORDS) next_word = __ldg(reinterpret_cast<const uint32_t*>(&A.prog[si + 1 < A.n_stages ? si + 1 : 0]) + tid_());
            if (tid_() == 0) {
                // prof_cta >= 0: that CTA's rows [stage][8]; prof_cta < 0: every CTA's rows [cta][stage][8]
                if (A.prof && step == A.n_steps - 1 && (A.prof_cta < 0 || cta_() == A.prof_cta))
                    S.prof = A.prof + ((A.prof_cta < 0 ? (size_t)cta_() * A.n_stages : 0) + si) * PROF_FIELDS;
                else
                    S.prof = nullptr;
            }
            prof_mark(S, 0);
            switch (d.op) {
                case MKS_OP_EMBED: embed_stage(S, mu, d, A, step, (uint32_t)(A.bar_base / grid_() + bar_n) + 1u); break;
                case MKS_OP_GEMV: gemv_stage(S, mu, d, A, ar_seq); break;
                case MKS_OP_GDN: gdn_stage(S, mu, d); break;
                case MKS_OP_ATTN:
                    if (d.i[MKS_I_KV_F32]) attn_stage<true>(S, mu, d);
                    else attn_stage<false>(S, mu, d);
                    break;
                case MKS_OP_ROUTE: route_stage(S, mu, d); break;
                case MKS_OP_VEC: vec_stage(S, mu, d); break;
                default: break;
            }
            if (d.op != MKS_OP_GEMV) prof_mark(S, 2);
            const bool barrier = !(d.flags & MKS_FLAG_NO_BARRIER);
            if (tid_() < DESC_WORDS) reinterpret_cast<uint32_t*>(&S.desc[cur ^ 1])[tid_()] = next_word;
            if (barrier) grid_barrier(S, mu, A, bar_n);
            else consumer_sync();
            cur ^= 1;
            prof_mark(S, 3);
        }
    }
    // the choice after the last step, and the positions (the program's first stage names the key buffer)
    const mk_stage_desc& d0 = A.prog[0];
    if (!failed && d0.op == MKS_OP_EMBED && d0.i[MKS_I_KEYS_VALID] && d0.p[MKS_P_E_KEYS]) {
        choose_tokens(S, mu, A, reinterpret_cast<const u64*>(d0.p[MKS_P_E_KEYS]), (uint32_t)(A.bar_base / grid_() + bar_n) + 1u, d0.i[MKS_I_VOCAB]);
        consumer_sync();
        if (cta_() == 0 && tid_() < S.A.M) {
            A.tok[tid_()] = S.tok_s[tid_()];
            if (A.tokens_out) A.tokens_out[(size_t)(A.n_steps - 1) * S.A.M + tid_()] = S.tok_s[tid_()];
        }
    }
    if (!failed && cta_() == 0 && tid_() < S.A.M && S.valid_s[tid_()]) A.pos[tid_()] = A.pos[tid_()] + A.n_steps;
}

}  // namespace mks
