// C ABI of the decode megakernel (declarations and reference citations: include/mk_b200.h).
// Host code only assembles the parameter block from raw device addresses and launches; it never
// allocates device memory.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>

#include "../../include/mk_b200.h"
#include "mk_decode.cuh"
#include "mk_batch.cuh"

using namespace mk;

struct mk_engine {
    mk_model_desc desc;
    int n_sm;
    bool params_set;
    bool static_only;    // the parameter block came without hand-off buffers: only mk_launch_static may run
    Params host;         // the parameter block; every launch passes it to the kernel by value
};

static thread_local char g_err[512] = "";
static std::mutex g_mu;

static int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}
// text behind mk_last_error() for the library's other translation units
int mk_set_error(int code, const char* text) {
    snprintf(g_err, sizeof g_err, "%s", text);
    return code;
}
#define MK_CUDA(call)                                                                      \
    do {                                                                                   \
        cudaError_t err__ = (call);                                                        \
        if (err__ != cudaSuccess)                                                          \
            return fail(MK_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(err__));   \
    } while (0)

template <class T>
static T as_ptr(int64_t v) { return reinterpret_cast<T>(static_cast<uintptr_t>(v)); }
template <class T>
static T as_ptr(uint64_t v) { return reinterpret_cast<T>(static_cast<uintptr_t>(v)); }

static void fill_layer(LayerP& L, const int64_t* f) {
    L.w_in = as_ptr<const uint8_t*>(f[MK_L_W_IN]);
    L.w_out = as_ptr<const uint8_t*>(f[MK_L_W_OUT]);
    L.w_gu = as_ptr<const uint8_t*>(f[MK_L_W_GU]);
    L.w_down = as_ptr<const uint8_t*>(f[MK_L_W_DOWN]);
    L.w_down_rows = as_ptr<const uint8_t*>(f[MK_L_W_DOWN_ROWS]);
    L.w_out_rows = as_ptr<const uint8_t*>(f[MK_L_W_OUT_ROWS]);
    L.s_in = as_ptr<const float*>(f[MK_L_S_IN]);
    L.s_out = as_ptr<const float*>(f[MK_L_S_OUT]);
    L.s_gu = as_ptr<const float*>(f[MK_L_S_GU]);
    L.s_down = as_ptr<const float*>(f[MK_L_S_DOWN]);
    L.in_norm = as_ptr<const float*>(f[MK_L_IN_NORM]);
    L.post_norm = as_ptr<const float*>(f[MK_L_POST_NORM]);
    L.conv_w = as_ptr<const float*>(f[MK_L_CONV_W]);
    L.A_log = as_ptr<const float*>(f[MK_L_A_LOG]);
    L.dt_bias = as_ptr<const float*>(f[MK_L_DT_BIAS]);
    L.gdn_norm = as_ptr<const float*>(f[MK_L_GDN_NORM]);
    L.conv_hist = as_ptr<float*>(f[MK_L_CONV_HIST]);
    L.conv_hist_b = as_ptr<float*>(f[MK_L_CONV_HIST_B]);
    L.state = as_ptr<float*>(f[MK_L_STATE]);
    L.state_bak = as_ptr<float*>(f[MK_L_STATE_BAK]);
    L.q_norm = as_ptr<const float*>(f[MK_L_Q_NORM]);
    L.k_norm = as_ptr<const float*>(f[MK_L_K_NORM]);
    L.k_cache = as_ptr<void*>(f[MK_L_K_CACHE]);
    L.v_cache = as_ptr<void*>(f[MK_L_V_CACHE]);
    L.kind = f[MK_L_KIND];
}

// Pointers a layer of the given kind must carry (non-null, 16-byte aligned where bulk-copied).
static const char* check_layer(const LayerP& L, bool q8) {
    auto bad16 = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
    if (bad16(L.w_in) || bad16(L.w_out) || bad16(L.w_gu) || bad16(L.w_down)) return "weight matrix null or not 16-byte aligned";
    if (q8 && (!L.s_in || !L.s_out || !L.s_gu || !L.s_down)) return "int8 layer without scales";
    if (!L.in_norm || !L.post_norm) return "norm weights missing";
    if (L.kind == 0) {
        if (!L.conv_w || !L.A_log || !L.dt_bias || !L.gdn_norm || !L.conv_hist || !L.state) return "DeltaNet layer field missing";
        if (bad16(L.state) || bad16(L.conv_w) || bad16(L.gdn_norm)) return "DeltaNet state/conv/norm not 16-byte aligned";
    } else if (L.kind == 1) {
        if (!L.q_norm || !L.k_norm || bad16(L.k_cache) || bad16(L.v_cache)) return "attention layer field missing or misaligned";
    } else {
        return "unknown layer kind";
    }
    return nullptr;
}

extern "C" int mk_create(const mk_model_desc* d, mk_engine** out) {
    if (!d || !out) return fail(MK_ERR_BADARG, "mk_create: null argument");
    if (d->shape != MK_SHAPE_QWEN35_08B) return fail(MK_ERR_UNSUPPORTED, "mk_create: unknown shape %d", d->shape);
    if (d->n_layers < 1 || d->n_layers > MAX_LAYERS) return fail(MK_ERR_BADARG, "mk_create: n_layers %d out of [1, %d]", d->n_layers, MAX_LAYERS);
    if (d->quant != MK_QUANT_BF16 && d->quant != MK_QUANT_INT8) return fail(MK_ERR_UNSUPPORTED, "mk_create: quant %d", d->quant);
    if (d->kv_dtype != MK_KV_BF16 && d->kv_dtype != MK_KV_F32) return fail(MK_ERR_UNSUPPORTED, "mk_create: kv_dtype %d", d->kv_dtype);
    if (d->vocab < 1 || d->max_seq < 1 || d->max_seq % KV_BLOCK) return fail(MK_ERR_BADARG, "mk_create: vocab %d / max_seq %d (must be a multiple of %d)", d->vocab, d->max_seq, KV_BLOCK);
    if (d->max_seq > MAX_BLOCKS * KV_BLOCK) return fail(MK_ERR_BADARG, "mk_create: max_seq %d exceeds %d", d->max_seq, MAX_BLOCKS * KV_BLOCK);
    if (d->max_batch < 0 || d->max_batch > MK_MAX_BATCH) return fail(MK_ERR_BADARG, "mk_create: max_batch %d out of [0, %d]", d->max_batch, (int)MK_MAX_BATCH);
    if ((int64_t)(d->max_batch > 1 ? d->max_batch : 1) * (d->max_seq / KV_BLOCK) > MAX_BLOCKS)
        return fail(MK_ERR_BADARG, "mk_create: %d sequences of %d positions need more than %d KV pages", d->max_batch, d->max_seq, MAX_BLOCKS);
    int n_sm = 0;
    MK_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, d->device));
    if (d->grid < 0 || d->grid > n_sm) return fail(MK_ERR_BADARG, "mk_create: grid %d exceeds the %d SMs (every CTA must be resident)", d->grid, n_sm);
    mk_engine* e = new mk_engine();
    e->desc = *d;
    if (e->desc.grid == 0) e->desc.grid = n_sm;
    e->n_sm = n_sm;
    e->params_set = false;
    e->static_only = false;
    memset(&e->host, 0, sizeof e->host);
    *out = e;
    return MK_OK;
}

extern "C" int mk_destroy(mk_engine* e) {
    if (!e) return MK_OK;
    delete e;
    return MK_OK;
}

extern "C" int mk_set_params(mk_engine* e, const int64_t* layers, int64_t n_layer_values, const int64_t* mtp,
                             int64_t n_mtp_values, const int64_t* g, int64_t n_global_values) {
    if (!e || !layers || !g) return fail(MK_ERR_BADARG, "mk_set_params: null argument");
    if (n_layer_values != (int64_t)e->desc.n_layers * MK_LAYER_FIELDS)
        return fail(MK_ERR_BADARG, "bad layer pointer count: got %lld, want %d x %d", (long long)n_layer_values, e->desc.n_layers, (int)MK_LAYER_FIELDS);
    if (mtp && n_mtp_values != MK_LAYER_FIELDS) return fail(MK_ERR_BADARG, "bad MTP layer pointer count: %lld", (long long)n_mtp_values);
    if (n_global_values != MK_GLOBAL_FIELDS) return fail(MK_ERR_BADARG, "bad global pointer count: got %lld, want %d", (long long)n_global_values, (int)MK_GLOBAL_FIELDS);
    const bool q8 = e->desc.quant == MK_QUANT_INT8;
    Params& p = e->host;
    memset(&p, 0, sizeof p);
    for (int l = 0; l < e->desc.n_layers; l++) {
        fill_layer(p.layer[l], layers + (size_t)l * MK_LAYER_FIELDS);
        if (const char* why = check_layer(p.layer[l], q8)) return fail(MK_ERR_BADARG, "layer %d: %s", l, why);
    }
    if (mtp) {
        fill_layer(p.mtp, mtp);
        if (p.mtp.kind != 1) return fail(MK_ERR_BADARG, "MTP layer must be a gated-attention layer");
        if (const char* why = check_layer(p.mtp, q8)) return fail(MK_ERR_BADARG, "MTP layer: %s", why);
    }
    p.embed = as_ptr<const uint8_t*>(g[MK_G_EMBED]);
    p.embed_scale = as_ptr<const float*>(g[MK_G_EMBED_SCALE]);
    p.lm_head = as_ptr<const uint8_t*>(g[MK_G_LM_HEAD]);
    p.lm_scale = as_ptr<const float*>(g[MK_G_LM_SCALE]);
    p.final_norm = as_ptr<const float*>(g[MK_G_FINAL_NORM]);
    p.rope_cos = as_ptr<const float*>(g[MK_G_ROPE_COS]);
    p.rope_sin = as_ptr<const float*>(g[MK_G_ROPE_SIN]);
    p.xl = as_ptr<unsigned long long*>(g[MK_G_XL]);
    p.projl = as_ptr<unsigned long long*>(g[MK_G_PROJL]);
    p.mixl = as_ptr<unsigned long long*>(g[MK_G_MIXL]);
    p.actl = as_ptr<unsigned long long*>(g[MK_G_ACTL]);
    p.lml = as_ptr<unsigned long long*>(g[MK_G_LML]);
    p.attn_part = as_ptr<unsigned long long*>(g[MK_G_ATTN_PART]);
    p.block_table = as_ptr<const int*>(g[MK_G_BLOCK_TABLE]);
    p.status = as_ptr<int*>(g[MK_G_STATUS]);
    p.mtp_fc = as_ptr<const uint8_t*>(g[MK_G_MTP_FC]);
    p.mtp_fc_scale = as_ptr<const float*>(g[MK_G_MTP_FC_SCALE]);
    p.mtp_norm_e = as_ptr<const float*>(g[MK_G_MTP_NORM_E]);
    p.mtp_norm_h = as_ptr<const float*>(g[MK_G_MTP_NORM_H]);
    p.mtp_norm = as_ptr<const float*>(g[MK_G_MTP_NORM]);
    p.draft_head = as_ptr<const uint8_t*>(g[MK_G_DRAFT_HEAD]);
    p.draft_scale = as_ptr<const float*>(g[MK_G_DRAFT_SCALE]);
    p.draft_ids = as_ptr<const int*>(g[MK_G_DRAFT_IDS]);
    p.xml = as_ptr<unsigned long long*>(g[MK_G_XML]);
    p.partl = as_ptr<unsigned long long*>(g[MK_G_PARTL]);
    p.n_layers = e->desc.n_layers;
    p.vocab = e->desc.vocab;
    p.max_seq = e->desc.max_seq;
    p.draft_vocab = e->desc.draft_vocab;
    auto bad16 = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
    if (bad16(p.embed) || bad16(p.lm_head)) return fail(MK_ERR_BADARG, "embedding / LM head null or not 16-byte aligned");
    if (q8 && (!p.embed_scale || !p.lm_scale)) return fail(MK_ERR_BADARG, "int8 embedding / LM head without scales");
    if (!p.final_norm || !p.rope_cos || !p.rope_sin) return fail(MK_ERR_BADARG, "final norm / RoPE tables missing");
    // A host that may not allocate passes none of the hand-off buffers: mk_launch_static brings its own.
    const bool no_handoff = !p.xl && !p.projl && !p.mixl && !p.actl && !p.lml && !p.partl && !p.attn_part;
    if (!no_handoff) {
        if (bad16(p.xl) || bad16(p.projl) || bad16(p.mixl) || bad16(p.lml) || bad16(p.partl))
            return fail(MK_ERR_BADARG, "activation word buffers null or not 16-byte aligned (all of them, or none for a static-only engine)");
        // the MLP activation words are a hand-off of the batched kernel only: mk_launch_batch refuses an engine without them
        if (p.actl != nullptr && bad16(p.actl)) return fail(MK_ERR_BADARG, "MLP activation words not 16-byte aligned");
        if (!p.attn_part) return fail(MK_ERR_BADARG, "attention scratch missing");
    }
    if (!p.block_table || !p.status) return fail(MK_ERR_BADARG, "block table / status missing");
    e->static_only = no_handoff;
    e->params_set = true;
    return MK_OK;
}

typedef void (*kernel_fn)(const Params, const Args);
static_assert(sizeof(Params) + sizeof(Args) + 64 <= 32764, "the parameter block travels as a kernel argument");
static_assert(Geo<1>::SMEM <= SMEM_BYTES && Geo<2>::SMEM <= SMEM_BYTES, "MK_Q_SMEM_BYTES reports the largest kernel");

// Dynamic shared memory of the kernel variant: what is not requested stays with the L1 cache.
static int kernel_smem(bool spec) { return spec ? Geo<2>::SMEM : Geo<1>::SMEM; }

static kernel_fn pick_kernel(const mk_model_desc& d, bool spec = false) {
    const bool q8 = d.quant == MK_QUANT_INT8, f32 = d.kv_dtype == MK_KV_F32;
    if (spec) {
        if (q8) return f32 ? decode_kernel<Qwen35_08B, true, true, 2> : decode_kernel<Qwen35_08B, true, false, 2>;
        return f32 ? decode_kernel<Qwen35_08B, false, true, 2> : decode_kernel<Qwen35_08B, false, false, 2>;
    }
    if (q8) return f32 ? decode_kernel<Qwen35_08B, true, true, 1> : decode_kernel<Qwen35_08B, true, false, 1>;
    return f32 ? decode_kernel<Qwen35_08B, false, true, 1> : decode_kernel<Qwen35_08B, false, false, 1>;
}

extern "C" int mk_launch(mk_engine* e, const mk_launch_args* a, void* stream) {
    if (!e || !a) return fail(MK_ERR_BADARG, "mk_launch: null argument");
    if (!e->params_set) return fail(MK_ERR_BADARG, "mk_launch: mk_set_params has not succeeded on this engine");
    if (e->static_only) return fail(MK_ERR_BADARG, "mk_launch: this engine was given no hand-off buffers; only mk_launch_static can run it");
    const bool spec = a->spec != 0;
    if (spec) {
        // n_steps counts cycles; a cycle feeds two positions and may emit two tokens
        const Params& p = e->host;
        if (e->desc.draft_vocab < 1 || !p.mtp_fc || !p.draft_head || !p.xml || !p.mtp.w_in || !p.mtp_norm_e || !p.mtp_norm_h || !p.mtp_norm)
            return fail(MK_ERR_BADARG, "mk_launch: speculative cycles need the draft head's parameters (mk_set_params with an MTP record)");
        if (a->n_steps < 1 || a->limit < 1 || !a->spec_out || !a->out_info) return fail(MK_ERR_BADARG, "mk_launch: need n_steps >= 1 cycles, limit >= 1 and spec_out / out_info");
        if (a->first_tok < 0 || a->first_tok >= e->desc.vocab || a->first_draft < 0 || a->first_draft >= e->desc.vocab)
            return fail(MK_ERR_BADARG, "mk_launch: pending token or draft outside the vocabulary");
        if (a->start_pos < 0 || (int64_t)a->start_pos + 2 * (int64_t)a->n_steps + 1 > e->desc.max_seq)
            return fail(MK_ERR_BADARG, "mk_launch: sequence would exceed max_seq=%d", e->desc.max_seq);
    } else {
        if (a->n_forced < 1 || a->n_steps < a->n_forced || !a->forced) return fail(MK_ERR_BADARG, "mk_launch: need 1 <= n_forced <= n_steps and a token list");
        if (a->start_pos < 0 || (int64_t)a->start_pos + a->n_steps > e->desc.max_seq)
            return fail(MK_ERR_BADARG, "mk_launch: sequence would exceed max_seq=%d", e->desc.max_seq);
        if (a->lm_from < 0 || a->lm_from > a->n_steps) return fail(MK_ERR_BADARG, "mk_launch: lm_from out of range");
        // a step past the prompt reduces the previous step's LM-head keys: that step must have run the LM head
        if (a->n_steps > a->n_forced && a->lm_from > a->n_forced - 1)
            return fail(MK_ERR_BADARG, "mk_launch: lm_from %d > n_forced - 1 = %d while %d steps feed predicted tokens", a->lm_from, a->n_forced - 1, a->n_steps - a->n_forced);
        if (!a->tokens_out || !a->out_info) return fail(MK_ERR_BADARG, "mk_launch: tokens_out / out_info missing");
    }
    if (a->n_stop < 0 || (a->n_stop > 0 && !a->stop_ids)) return fail(MK_ERR_BADARG, "mk_launch: stop ids missing");
    const int grid = a->grid > 0 ? a->grid : e->desc.grid;
    if (grid != e->desc.grid) return fail(MK_ERR_BADARG, "mk_launch: grid %d, but the weights are packed for %d CTAs", grid, e->desc.grid);
    // per-CTA ownership limits of the kernel's shared-memory staging
    if ((Qwen35_08B::GDN_IN + grid - 1) / grid > MAX_BODY_ROWS || (Qwen35_08B::HID + grid - 1) / grid > 16 || grid > Qwen35_08B::HID)
        return fail(MK_ERR_BADARG, "mk_launch: grid %d too small or too large for this shape", grid);
    if (grid < Qwen35_08B::GDN_TASKS) return fail(MK_ERR_BADARG, "mk_launch: grid %d < %d DeltaNet tasks", grid, (int)Qwen35_08B::GDN_TASKS);
    const int last_pos = a->start_pos + (spec ? 2 * a->n_steps + 1 : a->n_steps);
    if (attn_chunk(last_pos, grid / Qwen35_08B::NKV < MAX_SPLITS ? grid / Qwen35_08B::NKV : MAX_SPLITS) > MAX_CHUNK_POS)
        return fail(MK_ERR_BADARG, "mk_launch: context of %d positions is too long for %d CTAs", last_pos, grid);
    const uint64_t ops = (uint64_t)e->desc.n_layers * OPS_PER_LAYER + 1 + (spec ? 2 + OPS_PER_LAYER : 0);
    if ((uint64_t)a->epoch_base + ops * (uint64_t)a->n_steps >= 0xFFFFFF00ull || a->epoch_base == 0)
        return fail(MK_ERR_BADARG, "mk_launch: epoch counter exhausted or zero; reset the engine");

    Args A;
    memset(&A, 0, sizeof A);
    A.forced = as_ptr<const int*>(a->forced);
    A.stop_ids = as_ptr<const int*>(a->stop_ids);
    A.tokens_out = as_ptr<unsigned long long*>(a->tokens_out);
    A.logits_out = as_ptr<float*>(a->logits_out);
    A.resid_out = as_ptr<float*>(a->resid_out);
    A.step_ts = as_ptr<unsigned long long*>(a->step_ts);
    A.out_info = as_ptr<int*>(a->out_info);
    A.prof = as_ptr<unsigned long long*>(a->prof);
    A.spec_out = as_ptr<int*>(a->spec_out);
    A.cycle_out = as_ptr<int*>(a->cycle_out);
    A.spin_limit_ns = a->spin_limit_ns > 0 ? a->spin_limit_ns : 2000000000ll;
    A.n_forced = a->n_forced;
    A.n_steps = a->n_steps;
    A.lm_from = a->lm_from;
    A.start_pos = a->start_pos;
    A.epoch_base = a->epoch_base;
    A.seed = a->seed;
    A.inv_temperature = a->inv_temperature;
    A.n_stop = a->n_stop;
    A.prof_step = a->prof_step;
    A.spec = a->spec;
    A.first_tok = a->first_tok;
    A.first_draft = a->first_draft;
    A.limit = a->limit;

    MK_CUDA(cudaSetDevice(e->desc.device));
    kernel_fn fn = pick_kernel(e->desc, spec);
    MK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kernel_smem(spec)));
    void* kargs[] = {&e->host, &A};
    MK_CUDA(cudaLaunchCooperativeKernel((const void*)fn, dim3(grid), dim3(NTHREADS), kargs, kernel_smem(spec),
                                        static_cast<cudaStream_t>(stream)));
    return MK_OK;
}

// ---- launch without caller-provided scratch ---------------------------------------------------------
// The hand-off words of the kernel in an array that is part of the library image.  In host code the
// array's name is only a stand-in for the symbol: its device address comes from cudaGetSymbolAddress,
// once per device, and is what the kernel's parameter block receives.
static __device__ __align__(256) unsigned char g_static_scratch[MK_STATIC_SCRATCH_BYTES];
static constexpr int MAX_DEVICES = 64;
static std::atomic<unsigned char*> g_static_addr[MAX_DEVICES] = {};

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

extern "C" int mk_launch_static(mk_engine* e, const mk_launch_args* a, void* stream) {
    if (!e || !a) return fail(MK_ERR_BADARG, "mk_launch_static: null argument");
    if (!e->params_set) return fail(MK_ERR_BADARG, "mk_launch_static: mk_set_params has not succeeded on this engine");
    if (a->spec) return fail(MK_ERR_UNSUPPORTED, "mk_launch_static: speculative cycles are not built into this library yet");
    if (a->n_forced < 1 || a->n_steps < a->n_forced || !a->forced) return fail(MK_ERR_BADARG, "mk_launch_static: need 1 <= n_forced <= n_steps and a token list");
    if (a->start_pos < 0 || (int64_t)a->start_pos + a->n_steps > e->desc.max_seq)
        return fail(MK_ERR_BADARG, "mk_launch_static: sequence would exceed max_seq=%d", e->desc.max_seq);
    if (a->lm_from < 0 || a->lm_from > a->n_steps) return fail(MK_ERR_BADARG, "mk_launch_static: lm_from out of range");
    if (a->n_steps > a->n_forced && a->lm_from > a->n_forced - 1)
        return fail(MK_ERR_BADARG, "mk_launch_static: lm_from %d > n_forced - 1 = %d while predicted tokens are fed", a->lm_from, a->n_forced - 1);
    if (!a->tokens_out || !a->out_info) return fail(MK_ERR_BADARG, "mk_launch_static: tokens_out / out_info missing");
    if (a->n_stop < 0 || (a->n_stop > 0 && !a->stop_ids)) return fail(MK_ERR_BADARG, "mk_launch_static: stop ids missing");
    const int grid = a->grid > 0 ? a->grid : e->desc.grid;
    if (grid != e->desc.grid) return fail(MK_ERR_BADARG, "mk_launch_static: grid %d, but the weights are packed for %d CTAs", grid, e->desc.grid);
    if ((Qwen35_08B::GDN_IN + grid - 1) / grid > MAX_BODY_ROWS || (Qwen35_08B::HID + grid - 1) / grid > 16 || grid > Qwen35_08B::HID ||
        grid < Qwen35_08B::GDN_TASKS)
        return fail(MK_ERR_BADARG, "mk_launch_static: grid %d too small or too large for this shape", grid);
    if (attn_chunk(a->start_pos + a->n_steps, grid / Qwen35_08B::NKV < MAX_SPLITS ? grid / Qwen35_08B::NKV : MAX_SPLITS) > MAX_CHUNK_POS)
        return fail(MK_ERR_BADARG, "mk_launch_static: context of %d positions is too long for %d CTAs", a->start_pos + a->n_steps, grid);
    const uint64_t ops = (uint64_t)e->desc.n_layers * OPS_PER_LAYER + 1;
    if ((uint64_t)a->epoch_base + ops * (uint64_t)a->n_steps >= 0xFFFFFF00ull || a->epoch_base == 0)
        return fail(MK_ERR_BADARG, "mk_launch_static: epoch counter exhausted or zero; reset the engine");
    const int dev = e->desc.device;
    if (dev < 0 || dev >= MAX_DEVICES) return fail(MK_ERR_BADARG, "mk_launch_static: device ordinal %d", dev);

    // layout of the hand-off words inside the array
    typedef Qwen35_08B S;
    size_t off = 0;
    const size_t o_xl = off;    off = align256(off + sizeof(unsigned long long) * S::HID);
    const size_t o_proj = off;  off = align256(off + sizeof(unsigned long long) * S::PROJ_MAX);
    const size_t o_mix = off;   off = align256(off + sizeof(unsigned long long) * S::MIX);
    const size_t o_act = off;   off = align256(off + sizeof(unsigned long long) * S::INTER);
    const size_t o_lml = off;   off = align256(off + sizeof(unsigned long long) * 2 * (size_t)grid);
    const size_t o_part = off;  off = align256(off + sizeof(unsigned long long) * (size_t)S::NKV * MAX_SPLITS * S::PART_STRIDE);
    const size_t o_partl = off; off = align256(off + sizeof(unsigned long long) * (size_t)grid * S::HID);
    if (off > MK_STATIC_SCRATCH_BYTES)
        return fail(MK_ERR_BADARG, "mk_launch_static: this shape and a grid of %d CTAs need %zu bytes of hand-off words, the built-in array holds %u",
                    grid, off, (unsigned)MK_STATIC_SCRATCH_BYTES);

    MK_CUDA(cudaSetDevice(dev));
    if (!g_static_addr[dev].load(std::memory_order_acquire)) {
        // set-up, once per device, with that device current
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_static_addr[dev].load(std::memory_order_relaxed)) {
            void* p = nullptr;
            MK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
            if (!p) return fail(MK_ERR_CUDA, "mk_launch_static: the built-in array has no device address");
            g_static_addr[dev].store(static_cast<unsigned char*>(p), std::memory_order_release);
        }
    }
    unsigned char* base = g_static_addr[dev].load(std::memory_order_acquire);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the engine's parameter block with the hand-off words redirected into the array
    Params p = e->host;
    p.xl = reinterpret_cast<unsigned long long*>(base + o_xl);
    p.projl = reinterpret_cast<unsigned long long*>(base + o_proj);
    p.mixl = reinterpret_cast<unsigned long long*>(base + o_mix);
    p.actl = reinterpret_cast<unsigned long long*>(base + o_act);
    p.lml = reinterpret_cast<unsigned long long*>(base + o_lml);
    p.attn_part = reinterpret_cast<unsigned long long*>(base + o_part);
    p.partl = reinterpret_cast<unsigned long long*>(base + o_partl);
    // the array keeps the previous call's words (and their epochs): everything must start at zero
    MK_CUDA(cudaMemsetAsync(base, 0, off, st));

    Args A;
    memset(&A, 0, sizeof A);
    A.forced = as_ptr<const int*>(a->forced);
    A.stop_ids = as_ptr<const int*>(a->stop_ids);
    A.tokens_out = as_ptr<unsigned long long*>(a->tokens_out);
    A.logits_out = as_ptr<float*>(a->logits_out);
    A.resid_out = as_ptr<float*>(a->resid_out);
    A.step_ts = as_ptr<unsigned long long*>(a->step_ts);
    A.out_info = as_ptr<int*>(a->out_info);
    A.prof = as_ptr<unsigned long long*>(a->prof);
    A.spin_limit_ns = a->spin_limit_ns > 0 ? a->spin_limit_ns : 2000000000ll;
    A.n_forced = a->n_forced;
    A.n_steps = a->n_steps;
    A.lm_from = a->lm_from;
    A.start_pos = a->start_pos;
    A.epoch_base = a->epoch_base;
    A.seed = a->seed;
    A.inv_temperature = a->inv_temperature;
    A.n_stop = a->n_stop;
    A.prof_step = a->prof_step;
    kernel_fn fn = pick_kernel(e->desc);
    MK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kernel_smem(false)));
    void* kargs[] = {&p, &A};
    MK_CUDA(cudaLaunchCooperativeKernel((const void*)fn, dim3(grid), dim3(NTHREADS), kargs, kernel_smem(false), st));
    return MK_OK;
}

// ---- batched decoding ---------------------------------------------------------------------------------
static_assert(MK_MAX_BATCH == NB, "header and kernel agree on the batch width");
typedef void (*batch_kernel_fn)(const Params, const BatchArgs);

extern "C" int mk_launch_batch(mk_engine* e, const mk_batch_args* a, void* stream) {
    typedef Qwen35_08B S;
    if (!e || !a) return fail(MK_ERR_BADARG, "mk_launch_batch: null argument");
    if (!e->params_set) return fail(MK_ERR_BADARG, "mk_launch_batch: mk_set_params has not succeeded on this engine");
    if (e->static_only) return fail(MK_ERR_BADARG, "mk_launch_batch: this engine was given no hand-off buffers; only mk_launch_static can run it");
    if (e->desc.quant != MK_QUANT_INT8) return fail(MK_ERR_UNSUPPORTED, "mk_launch_batch: batched decoding is built for int8 weights only");
    if (a->batch < 1 || a->batch > NB) return fail(MK_ERR_BADARG, "mk_launch_batch: batch %d out of [1, %d]", a->batch, NB);
    if (a->batch > (e->desc.max_batch > 1 ? e->desc.max_batch : 1))
        return fail(MK_ERR_BADARG, "mk_launch_batch: batch %d, but the engine's buffers were sized for %d sequence(s) (mk_model_desc.max_batch)",
                    a->batch, e->desc.max_batch > 1 ? e->desc.max_batch : 1);
    if (a->n_steps < 1 || !a->forced || !a->tokens_out || !a->out_info) return fail(MK_ERR_BADARG, "mk_launch_batch: need n_steps >= 1, a token list, tokens_out and out_info");
    if (!e->host.actl) return fail(MK_ERR_BADARG, "mk_launch_batch: the engine was given no MLP activation words (MK_G_ACTL)");
    if ((int64_t)a->batch * (e->desc.max_seq / KV_BLOCK) > MAX_BLOCKS)
        return fail(MK_ERR_BADARG, "mk_launch_batch: %d sequences of %d positions need more than %d KV pages", a->batch, e->desc.max_seq, MAX_BLOCKS);
    int min_forced = 1 << 30, last_pos = 0;
    for (int j = 0; j < a->batch; j++) {
        if (a->n_forced[j] < 1 || a->n_forced[j] > a->n_total[j] || a->n_total[j] > a->n_steps)
            return fail(MK_ERR_BADARG, "mk_launch_batch: sequence %d: need 1 <= n_forced <= n_total <= n_steps", j);
        if (a->pos0[j] < 0 || (int64_t)a->pos0[j] + a->n_steps > e->desc.max_seq)
            return fail(MK_ERR_BADARG, "mk_launch_batch: sequence %d would exceed max_seq=%d", j, e->desc.max_seq);
        min_forced = a->n_forced[j] < min_forced ? a->n_forced[j] : min_forced;
        last_pos = a->pos0[j] + a->n_steps > last_pos ? a->pos0[j] + a->n_steps : last_pos;
    }
    if (a->lm_from < 0 || a->lm_from > min_forced - 1) return fail(MK_ERR_BADARG, "mk_launch_batch: lm_from must lie in [0, min n_forced - 1]");
    if (a->n_stop < 0 || (a->n_stop > 0 && !a->stop_ids)) return fail(MK_ERR_BADARG, "mk_launch_batch: stop ids missing");
    const int grid = e->desc.grid;
    if ((S::GDN_IN + grid - 1) / grid > MAX_BODY_ROWS || (S::HID + grid - 1) / grid > 16 || grid > S::HID || grid < S::GDN_TASKS)
        return fail(MK_ERR_BADARG, "mk_launch_batch: grid %d too small or too large for this shape", grid);
    const int per = grid / a->batch;                     // CTAs that serve one sequence's attention
    if (per < S::NKV) return fail(MK_ERR_BADARG, "mk_launch_batch: grid %d too small for %d sequences", grid, a->batch);
    if (attn_chunk(last_pos, per / S::NKV < MAX_SPLITS ? per / S::NKV : MAX_SPLITS) > MAX_CHUNK_POS)
        return fail(MK_ERR_BADARG, "mk_launch_batch: context of %d positions is too long for %d CTAs per sequence", last_pos, per);
    const uint64_t ops = (uint64_t)e->desc.n_layers * OPS_PER_LAYER + 1;
    if ((uint64_t)a->epoch_base + ops * (uint64_t)a->n_steps >= 0xFFFFFF00ull || a->epoch_base == 0)
        return fail(MK_ERR_BADARG, "mk_launch_batch: epoch counter exhausted or zero; reset the engine");
    for (int l = 0; l < e->desc.n_layers; l++)
        if ((e->host.layer[l].kind == 0 && (!e->host.layer[l].conv_hist_b || !e->host.layer[l].w_out_rows)) || !e->host.layer[l].w_down_rows)
            return fail(MK_ERR_BADARG, "mk_launch_batch: layer %d lacks the batched kernel's buffers (MK_L_CONV_HIST_B, MK_L_W_OUT_ROWS, MK_L_W_DOWN_ROWS)", l);

    BatchArgs A;
    memset(&A, 0, sizeof A);
    A.forced = as_ptr<const int*>(a->forced);
    A.stop_ids = as_ptr<const int*>(a->stop_ids);
    A.tokens_out = as_ptr<unsigned long long*>(a->tokens_out);
    A.logits_out = as_ptr<float*>(a->logits_out);
    A.step_ts = as_ptr<unsigned long long*>(a->step_ts);
    A.out_info = as_ptr<int*>(a->out_info);
    A.prof = as_ptr<unsigned long long*>(a->prof);
    A.spin_limit_ns = a->spin_limit_ns > 0 ? a->spin_limit_ns : 2000000000ll;
    for (int j = 0; j < NB; j++) {
        A.n_forced[j] = j < a->batch ? a->n_forced[j] : 0;
        A.n_total[j] = j < a->batch ? a->n_total[j] : 0;
        A.pos0[j] = j < a->batch ? a->pos0[j] : 0;
    }
    A.nb = a->batch;
    A.n_steps = a->n_steps;
    A.lm_from = a->lm_from;
    A.epoch_base = a->epoch_base;
    A.seed = a->seed;
    A.inv_temperature = a->inv_temperature;
    A.n_stop = a->n_stop;
    A.prof_step = a->prof_step;

    MK_CUDA(cudaSetDevice(e->desc.device));
    batch_kernel_fn fn = e->desc.kv_dtype == MK_KV_F32 ? batch_kernel<S, true> : batch_kernel<S, false>;
    MK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, GeoB::SMEM));
    void* kargs[] = {&e->host, &A};
    MK_CUDA(cudaLaunchCooperativeKernel((const void*)fn, dim3(grid), dim3(NTHREADS), kargs, GeoB::SMEM,
                                        static_cast<cudaStream_t>(stream)));
    return MK_OK;
}

extern "C" int mk_status(mk_engine* e, int32_t* where) {
    if (!e || !e->params_set) return fail(MK_ERR_BADARG, "mk_status: engine has no parameters");
    MK_CUDA(cudaSetDevice(e->desc.device));
    MK_CUDA(cudaDeviceSynchronize());
    int st[4] = {0, 0, 0, 0};
    MK_CUDA(cudaMemcpy(st, e->host.status, sizeof st, cudaMemcpyDeviceToHost));
    if (where) *where = st[1];
    if (st[0] != 0) return fail(MK_ERR_TIMEOUT, "a device-side wait ran out (site %d, CTA %d, thread %d)", st[1], st[2], st[3]);
    return MK_OK;
}

extern "C" int64_t mk_query(int what) {
    switch (what) {
        case MK_Q_SMEM_BYTES: return SMEM_BYTES;
        case MK_Q_N_THREADS: return NTHREADS;
        case MK_Q_CONV_RING: return CONV_RING;
        case MK_Q_KV_BLOCK: return KV_BLOCK;
        case MK_Q_MAX_SPLITS: return MAX_SPLITS;
        case MK_Q_PART_STRIDE: return Qwen35_08B::PART_STRIDE;
        case MK_Q_OPS_PER_LAYER: return OPS_PER_LAYER;
        case MK_Q_PROF_MAX_OPS: return PROF_MAX_OPS;
        case MK_Q_PROF_FIELDS: return PROF_FIELDS;
        case MK_Q_SPEC_T: return SPEC_T;
        case MK_Q_MAX_LAYERS: return MAX_LAYERS;
        case MK_Q_LAYER_FIELDS: return MK_LAYER_FIELDS;
        case MK_Q_GLOBAL_FIELDS: return MK_GLOBAL_FIELDS;
        case MK_Q_SLOT_BYTES: return SLOT_BYTES;
        case MK_Q_STAGES: return Geo<1>::NS;
        case MK_Q_MAX_LM_ROWS: return MAX_LM_ROWS;
        case MK_Q_MAX_BATCH: return NB;
        case MK_Q_BATCH_SMEM_BYTES: return GeoB::SMEM;
        default: return -1;
    }
}

// ---- bandwidth probe ---------------------------------------------------------------------------------
namespace mk {

__global__ void __launch_bounds__(512) bw_plain_kernel(const uint4* __restrict__ src, long long n16, unsigned* sink) {
    unsigned acc = 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n16; i += 4 * stride) {
        const uint4 a = __ldcs(src + i), b = __ldcs(src + i + stride), c2 = __ldcs(src + i + 2 * stride),
                    d = __ldcs(src + i + 3 * stride);
        acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c2.x ^ c2.y ^ c2.z ^ c2.w ^ d.x ^ d.y ^ d.z ^ d.w;
    }
    for (; i < n16; i += stride) {
        const uint4 a = __ldcs(src + i);
        acc ^= a.x ^ a.y ^ a.z ^ a.w;
    }
    if (acc == 0x9E3779B9u) atomicAdd(sink, 1u);   // keeps the loads alive; practically never true
}

// The decode kernel's own ring: one elected producer lane issues bulk copies, consumer warps read
// every 16-byte piece once.  Waits are bounded by an iteration cap.
__global__ void __launch_bounds__(NTHREADS, 1) bw_ring_kernel(const uint8_t* __restrict__ src, long long bytes,
                                                              unsigned* sink) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* ring = smem_raw;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (NSTAGE * SLOT_BYTES));
    uint64_t* empty = full + NSTAGE;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < NSTAGE; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], NCW); }
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();
    const long long nchunk = bytes / SLOT_BYTES;
    const long long c0 = nchunk * blockIdx.x / gridDim.x, c1 = nchunk * (blockIdx.x + 1) / gridDim.x;
    constexpr unsigned SPIN_CAP = 1u << 24;
    if (warp == NCW) {
        if (lane != 0) return;
        const u64 pol = policy_evict_first();
        uint32_t n = 0;
        bool ok = true;
        for (long long ch = c0; ch < c1 && ok; ch++, n++) {
            const int slot = (int)(n % NSTAGE);
            if (n >= NSTAGE) {
                unsigned it = 0;
                while (!mbar_try_wait(&empty[slot], ((n / NSTAGE) - 1) & 1))
                    if (++it > SPIN_CAP) { ok = false; break; }
                if (!ok) break;
            }
            mbar_expect_tx(&full[slot], SLOT_BYTES);
            bulk_load(ring + (size_t)slot * SLOT_BYTES, src + ch * SLOT_BYTES, SLOT_BYTES, &full[slot], pol);
        }
        const uint32_t first = n > NSTAGE ? n - NSTAGE : 0;
        for (uint32_t i = first; i < n; i++) {
            unsigned it = 0;
            while (!mbar_try_wait(&full[i % NSTAGE], (i / NSTAGE) & 1))
                if (++it > SPIN_CAP) break;
        }
        return;
    }
    unsigned acc = 0;
    uint32_t n = 0;
    for (long long ch = c0; ch < c1; ch++, n++) {
        const int slot = (int)(n % NSTAGE);
        unsigned it = 0;
        bool ok = true;
        while (!mbar_try_wait(&full[slot], (n / NSTAGE) & 1))
            if (++it > SPIN_CAP) { ok = false; break; }
        if (!ok) break;
        const uint4* p = reinterpret_cast<const uint4*>(ring + (size_t)slot * SLOT_BYTES);
        for (int i = tid; i < SLOT_BYTES / 16; i += NCT) {
            const uint4 a = p[i];
            acc ^= a.x ^ a.y ^ a.z ^ a.w;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
    }
    if (acc == 0x9E3779B9u) atomicAdd(sink, 1u);
}

}  // namespace mk

extern "C" int mk_bw_probe(uint64_t src, int64_t bytes, int mode, uint64_t sink, int device, void* stream) {
    if (!src || !sink || bytes < SLOT_BYTES || (src & 15)) return fail(MK_ERR_BADARG, "mk_bw_probe: bad buffer");
    MK_CUDA(cudaSetDevice(device));
    int n_sm = 0;
    MK_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (mode == 0) {
        bw_plain_kernel<<<n_sm * 4, 512, 0, st>>>(as_ptr<const uint4*>(src), bytes / 16, as_ptr<unsigned*>(sink));
    } else if (mode == 1) {
        const int smem = (NSTAGE * SLOT_BYTES) + 2 * NSTAGE * 8;
        MK_CUDA(cudaFuncSetAttribute(bw_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        bw_ring_kernel<<<n_sm, NTHREADS, smem, st>>>(as_ptr<const uint8_t*>(src), bytes, as_ptr<unsigned*>(sink));
    } else {
        return fail(MK_ERR_BADARG, "mk_bw_probe: mode %d", mode);
    }
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

extern "C" int mk_plan_rows(int rows, int unit, int cta, int grid, int* r0, int* r1) {
    if (rows < 0 || unit < 1 || grid < 1 || cta < 0 || cta >= grid || rows % unit || !r0 || !r1)
        return fail(MK_ERR_BADARG, "mk_plan_rows: bad arguments");
    cta_rows(rows, unit, cta, grid, *r0, *r1);
    return MK_OK;
}

extern "C" int mk_plan_attn_chunk(int n, int max_splits) {
    if (n < 1 || max_splits < 1) return fail(MK_ERR_BADARG, "mk_plan_attn_chunk: bad arguments");
    return attn_chunk(n, max_splits);
}

extern "C" const char* mk_last_error(void) { return g_err; }
