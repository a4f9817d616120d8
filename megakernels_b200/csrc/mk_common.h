// Constants and parameter blocks shared by the host API and the device kernel.
#pragma once
#include <stdint.h>

namespace mk {

// ---- execution shape -------------------------------------------------------------------------
constexpr int NCW = 16;                   // consumer warps per CTA
constexpr int NCT = NCW * 32;             // consumer threads
constexpr int NTHREADS = NCT + 32;        // + one producer warp
constexpr int SLOT_BYTES = 32768;         // one ring slot: 32/16/9 int8 rows or 16/8/4 bf16 rows of K = 1024/2048/3584
constexpr int NSTAGE = 6;                 // ring depth of the bandwidth probe: 192 KB in flight per SM (the decode kernels choose their own)
constexpr int MAX_LAYERS = 64;
constexpr int KV_BLOCK = 64;              // positions per KV page
constexpr int CONV_RING = 8;              // conv history slots, indexed by position & 7
constexpr int MAX_SPLITS = 128;           // attention split-K chunks per KV head (buffer sizing)
constexpr int MAX_CHUNK_POS = 448;        // positions one attention task scans at most
constexpr int MAX_LM_ROWS = 1 << 20;      // LM-head rows one CTA can own (no per-CTA staging limits it)
constexpr int MAX_BODY_ROWS = 64;         // rows of a layer GEMV one CTA can own
constexpr int OPS_PER_LAYER = 5;
#ifdef MK_TRACE
constexpr int PROF_FIELDS = 12;         // + fine-grained marks of a trace build
#else
constexpr int PROF_FIELDS = 6;          // enter, staged, done, published, ring-wait ns, spare
#endif
constexpr int PROF_MAX_OPS = MAX_LAYERS * OPS_PER_LAYER + 8;
constexpr int SPEC_T = 2;
constexpr int DOWN_K = 32;                  // columns of a CTA's down-projection slice (its SwiGLU outputs, padded)

// ---- the 0.8B hybrid shape --------------------------------------------------------------------
struct Qwen35_08B {
    static constexpr int HID = 1024, INTER = 3584;
    static constexpr int LIN_H = 16, LIN_DK = 128, LIN_DV = 128, CONV_K = 4;
    static constexpr int LIN_QK = LIN_H * LIN_DK, LIN_V = LIN_H * LIN_DV;
    static constexpr int CONV_DIM = 2 * LIN_QK + LIN_V;            // 6144
    static constexpr int Z_OFF = CONV_DIM, B_OFF = Z_OFF + LIN_V, A_OFF = B_OFF + LIN_H;
    static constexpr int GDN_IN = A_OFF + LIN_H;                   // 8224 rows: qkv | z | b | a
    static constexpr int GDN_SLICE = 16;                           // value columns per recurrence task
    static constexpr int GDN_TASKS = LIN_H * (LIN_DV / GDN_SLICE); // 128
    static constexpr int NQ = 8, NKV = 2, HD = 256, ROT = 64, QPK = NQ / NKV;
    static constexpr int ATT_K_OFF = NQ * 2 * HD, ATT_V_OFF = ATT_K_OFF + NKV * HD;
    static constexpr int ATT_IN = ATT_V_OFF + NKV * HD;            // 5120 rows: per-head [q|gate], k, v
    static constexpr int MIX = NQ * HD;                            // 2048 = mixer output width (== LIN_V)
    static constexpr int PROJ_MAX = GDN_IN;
    static constexpr int PART_STRIDE = QPK * HD + 2 * QPK;         // per split: acc[4][256], m[4], l[4]
    static constexpr float EPS = 1e-6f;
};

constexpr int MAX_BLOCKS = 512;                                    // KV pages per sequence (max_seq <= 32768)
constexpr int SMEM_BYTES = NSTAGE * SLOT_BYTES + 3 * 2 * 3584 + NCW * 64 * 4 + MAX_BLOCKS * 4 + 2048 + 2048;   // upper bound of the single-sequence kernels' dynamic shared memory

// ---- device-side parameter block (one per engine, passed to every launch as a kernel argument) ---
struct LayerP {
    const uint8_t* w_in;
    const uint8_t* w_out;
    const uint8_t* w_gu;
    const uint8_t* w_down;        // single-sequence kernels: column slices per CTA in fragment order (pack_down_cols)
    const uint8_t* w_down_rows;   // batched kernel: row slices per CTA (pack_rows)
    const uint8_t* w_out_rows;    // batched kernel, DeltaNet layers: row slices (single-sequence kernels: w_out holds column slices per task)
    const float* s_in;
    const float* s_out;
    const float* s_gu;
    const float* s_down;
    const float* in_norm;
    const float* post_norm;
    const float* conv_w;
    const float* A_log;
    const float* dt_bias;
    const float* gdn_norm;
    float* conv_hist;
    float* conv_hist_b;   // batched decoding: [sequence][head][q 128 | k 128 | v 128][CONV_RING]
    float* state;
    float* state_bak;
    const float* q_norm;
    const float* k_norm;
    void* k_cache;
    void* v_cache;
    long long kind;
};

struct Params {
    LayerP layer[MAX_LAYERS];
    LayerP mtp;
    const uint8_t* embed;
    const float* embed_scale;
    const uint8_t* lm_head;
    const float* lm_scale;
    const float* final_norm;
    const float* rope_cos;
    const float* rope_sin;
    unsigned long long* xl;
    unsigned long long* projl;
    unsigned long long* mixl;
    unsigned long long* actl;
    unsigned long long* lml;
    unsigned long long* attn_part;
    const int* block_table;
    int* status;
    const uint8_t* mtp_fc;
    const float* mtp_fc_scale;
    const float* mtp_norm_e;
    const float* mtp_norm_h;
    const float* mtp_norm;
    const uint8_t* draft_head;
    const float* draft_scale;
    const int* draft_ids;
    unsigned long long* xml;
    unsigned long long* partl;    // [token][cta][hidden] partial down-projection sums
    int n_layers, vocab, max_seq, draft_vocab;
};

struct Args {
    const int* forced;
    const int* stop_ids;
    unsigned long long* tokens_out;
    float* logits_out;
    float* resid_out;
    unsigned long long* step_ts;
    int* out_info;
    unsigned long long* prof;
    int* spec_out;
    int* cycle_out;
    long long spin_limit_ns;
    int n_forced, n_steps, lm_from, start_pos;
    unsigned epoch_base, seed;
    float inv_temperature;
    int n_stop, prof_step;
    int spec, first_tok, first_draft, limit;
};

// Row range of a GEMV that one CTA owns.  `unit` rows stay together (2 for gate/up pairs).
// Producer and consumers both call this, so they agree on the chunk sequence.
__host__ __device__ inline void cta_rows(int rows, int unit, int cta, int grid, int& r0, int& r1) {
    const long long units = rows / unit;
    r0 = (int)(units * cta / grid) * unit;
    r1 = (int)(units * (cta + 1) / grid) * unit;
}

// Attention split geometry for `n` cached positions (the new one included): positions per task.
// Small chunks give many CTAs work when the context is short; the chunk grows in page-aligned
// steps once tasks would outnumber `max_splits`.  A chunk never straddles a KV page.
__host__ __device__ inline int attn_chunk(int n, int max_splits) {
    int ch = 16;
    while ((n + ch - 1) / ch > max_splits) ch = ch < KV_BLOCK ? ch * 2 : ch + KV_BLOCK;
    return ch;
}

}  // namespace mk
