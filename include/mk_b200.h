/* mk_b200.h -- C ABI of the B200 (sm_100a) persistent decode megakernel.
 *
 * One cooperative launch runs every layer of one or many decode steps of a hybrid
 * Gated-DeltaNet / gated-attention decoder, the LM head and the sampling rule.  The caller owns
 * every device buffer and passes raw device addresses; the library keeps only a small host-side
 * handle that holds the pointer tables.
 *
 * Each entry point names the reference interface it replaces, by the file's path in the
 * reference project (SamuelReeder/megakernels).  Nothing here throws: every function returns an
 * int status (MK_OK or a negative MK_ERR_*), and mk_last_error() gives the text of the last failure
 * on the calling thread.
 */
#ifndef MK_B200_H
#define MK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    MK_OK = 0,
    MK_ERR_BADARG = -1,       /* a count, size or pointer failed validation; nothing was launched */
    MK_ERR_TIMEOUT = -2,      /* a device-side wait ran out; results of that launch are garbage    */
    MK_ERR_CUDA = -3,         /* a CUDA runtime call failed; see mk_last_error()                   */
    MK_ERR_UNSUPPORTED = -4   /* shape / option combination that this build has no kernel for      */
};

enum { MK_QUANT_BF16 = 0, MK_QUANT_INT8 = 1 };
enum { MK_KV_BF16 = 0, MK_KV_F32 = 1 };
enum { MK_SHAPE_QWEN35_08B = 1 };

/* Field order of one layer's pointer record (MK_LAYER_FIELDS int64 values per layer).
 * Replaces the 18-field record of qwen3.5-0.8b/csrc/binding.cpp:18-37. */
enum {
    /* the four matrices are in the kernel's tile layout (megakernels_b200/pack.py), int8 or bf16 */
    MK_L_W_IN = 0,      /* DeltaNet: [qkv|z|b|a rows, hidden]; attention: [per-head q|gate, k, v rows, hidden] */
    MK_L_W_OUT,         /* [hidden, 2048]                                                     */
    MK_L_W_GU,          /* [2*intermediate, hidden], rows interleaved gate0, up0, gate1, ...  */
    MK_L_W_DOWN,        /* [hidden, intermediate]                                             */
    MK_L_S_IN, MK_L_S_OUT, MK_L_S_GU, MK_L_S_DOWN, /* fp32 per-row scales (int8 only, else 0) */
    MK_L_IN_NORM,       /* fp32 [hidden]                                                      */
    MK_L_POST_NORM,     /* fp32 [hidden]                                                      */
    MK_L_CONV_W,        /* fp32 [conv_dim, 4]                                                 */
    MK_L_A_LOG,         /* fp32 [heads]                                                       */
    MK_L_DT_BIAS,       /* fp32 [heads]                                                       */
    MK_L_GDN_NORM,      /* fp32 [v_dim]                                                       */
    MK_L_CONV_HIST,     /* fp32 [128 tasks, 272 channels, MK_CONV_RING]: per recurrence task, ring by position & 7 */
    MK_L_STATE,         /* fp32 [heads, v_dim, k_dim]                                         */
    MK_L_STATE_BAK,     /* same shape; spare copy used by speculative cycles                  */
    MK_L_Q_NORM,        /* fp32 [head_dim]                                                    */
    MK_L_K_NORM,        /* fp32 [head_dim]                                                    */
    MK_L_K_CACHE,       /* paged: [n_blocks, kv_heads, MK_KV_BLOCK, head_dim], bf16 or fp32   */
    MK_L_V_CACHE,
    MK_L_KIND,          /* 0 = Gated DeltaNet, 1 = gated full attention (a value, not a pointer) */
    MK_L_CONV_HIST_B,   /* fp32 [batch, 16 heads, 384 channels, 8]: conv history of batched decoding (0 if unused) */
    MK_L_W_OUT_ROWS,    /* DeltaNet layers: out-projection in the row-slice layout, the batched kernel's copy (0 if unused) */
    MK_L_W_DOWN_ROWS,   /* down-projection in the row-slice layout of the other matrices: the batched kernel's copy (0 if unused) */
    MK_LAYER_FIELDS
};

/* Field order of the model-wide pointer record (MK_GLOBAL_FIELDS int64 values).
 * Replaces the 20-entry list of qwen3.5-0.8b/csrc/binding.cpp:47-66. */
enum {
    MK_G_EMBED = 0,     /* token embedding table, plain row-major [vocab, hidden], int8 or bf16 */
    MK_G_EMBED_SCALE,   /* fp32 [vocab] (int8) or 0                                            */
    MK_G_LM_HEAD,       /* LM head [vocab, hidden] in the kernel's tile layout                 */
    MK_G_LM_SCALE,
    MK_G_FINAL_NORM,    /* fp32 [hidden]                                                       */
    MK_G_ROPE_COS,      /* fp32 [max_seq, rotary_dim/2]                                        */
    MK_G_ROPE_SIN,
    MK_G_XL,            /* u64 [tokens, hidden]        residual stream, (epoch<<32)|fp32 words */
    MK_G_PROJL,         /* u64 [tokens, in_rows_max]   input-projection output                 */
    MK_G_MIXL,          /* u64 [tokens, 2048]          mixer (DeltaNet / attention) output     */
    MK_G_ACTL,          /* u64 [tokens, intermediate]  MLP activation: mk_launch_batch only (0: never batched) */
    MK_G_LML,           /* u64 [tokens, grid, 2]       per-CTA LM-head winners                 */
    MK_G_ATTN_PART,     /* u64 [tokens, kv_heads, MK_MAX_SPLITS, MK_PART_STRIDE] split partials, flag-in-data words */
    MK_G_BLOCK_TABLE,   /* int32 [max_seq / MK_KV_BLOCK]: logical KV block -> physical block   */
    MK_G_STATUS,        /* int32 [4]: [0] error code of the first wait that ran out, [1] where */
    MK_G_MTP_FC, MK_G_MTP_FC_SCALE, MK_G_MTP_NORM_E, MK_G_MTP_NORM_H, MK_G_MTP_NORM,
    MK_G_DRAFT_HEAD, MK_G_DRAFT_SCALE, MK_G_DRAFT_IDS,
    MK_G_XML,           /* u64 [tokens, hidden] MTP residual stream                            */
    MK_G_PARTL,         /* u64 [tokens, grid, hidden] partial down-projection sums of every CTA */
    MK_GLOBAL_FIELDS
};

typedef struct mk_model_desc {
    int32_t shape;        /* MK_SHAPE_*                                        */
    int32_t n_layers;     /* <= MK_MAX_LAYERS                                  */
    int32_t vocab;
    int32_t max_seq;
    int32_t quant;        /* MK_QUANT_*                                        */
    int32_t kv_dtype;     /* MK_KV_*                                           */
    int32_t draft_vocab;  /* rows of the draft head (0: no MTP head)           */
    int32_t device;       /* CUDA device ordinal                               */
    int32_t grid;         /* CTAs the weights were packed for (0: one per SM)  */
    int32_t max_batch;    /* sequences the per-sequence buffers were sized for (0 or 1: one);
                             mk_launch_batch refuses a larger batch                     */
} mk_model_desc;

/* Per-launch arguments.  Replaces `Args` of qwen3.5-0.8b/csrc/megakernel.h:134-161 and the 26
 * scalars of `launch` in csrc/binding.cpp:73-105; fields keep the reference's meaning. */
typedef struct mk_launch_args {
    uint64_t forced;         /* int32[n_forced] tokens fed at steps [0, n_forced)              */
    int32_t n_forced;
    int32_t n_steps;         /* n_forced + n_generate - 1                                      */
    int32_t lm_from;         /* first step that runs the LM head                               */
    int32_t start_pos;
    uint32_t epoch_base;     /* epoch of the launch's first op; the host carries it across launches */
    uint32_t seed;
    float inv_temperature;   /* 0 => greedy                                                    */
    int32_t n_stop;
    uint64_t stop_ids;       /* int32[n_stop]                                                  */
    uint64_t tokens_out;     /* u64[n_steps] (ordered score << 32) | ~id; zeroed by the caller */
    uint64_t logits_out;     /* optional fp32 [n_steps, vocab]                                 */
    uint64_t resid_out;      /* optional fp32 [n_steps, hidden]: residual after the last layer */
    uint64_t step_ts;        /* optional u64 [n_steps + 1]: GPU nanosecond timer per step      */
    uint64_t out_info;       /* int32[8]: steps run, next epoch, pos, pending, draft, cycles   */
    uint64_t prof;           /* optional u64 [grid, MK_PROF_MAX_OPS, MK_PROF_FIELDS]           */
    int32_t prof_step;
    int32_t grid;            /* CTAs; 0 = one per SM                                           */
    int64_t spin_limit_ns;   /* bound on every device-side wait; 0 = library default (2 s)    */
    /* speculative cycles (spec = 1; n_steps counts cycles, each verifies the pending token and one draft;
     * needs the MTP record and draft-head fields of mk_set_params; qwen3.5-0.8b/csrc/megakernel.cu:1196-1276) */
    int32_t spec;
    int32_t first_tok;
    int32_t first_draft;
    int32_t limit;
    uint64_t spec_out;       /* int32[limit]                                                   */
    uint64_t cycle_out;      /* optional int32[n_steps, 2]                                     */
} mk_launch_args;

typedef struct mk_engine mk_engine;

/* Create / destroy a handle.  The reference keeps its parameter block in one process-wide
 * __constant__ symbol (qwen3.5-0.8b/csrc/megakernel.cu:22,1280-1283), so two engines alias; here the
 * handle owns its block and every launch passes it to the kernel by value, so any number of engines
 * can live side by side. */
int mk_create(const mk_model_desc* desc, mk_engine** out);
int mk_destroy(mk_engine* e);

/* Replaces `set_params` (qwen3.5-0.8b/csrc/binding.cpp:39-71).  `layers` holds
 * n_layers * MK_LAYER_FIELDS values, `mtp` MK_LAYER_FIELDS values or NULL, `globals`
 * MK_GLOBAL_FIELDS values; the counts are checked (MK_ERR_BADARG). */
int mk_set_params(mk_engine* e, const int64_t* layers, int64_t n_layer_values, const int64_t* mtp,
                  int64_t n_mtp_values, const int64_t* globals, int64_t n_global_values);

/* Replaces `launch` (qwen3.5-0.8b/csrc/binding.cpp:73-105, csrc/megakernel.cu:1291-1309).
 * Asynchronous on `stream` (a cudaStream_t, 0 for the default stream). */
int mk_launch(mk_engine* e, const mk_launch_args* args, void* stream);

/* Same launch as mk_launch, for a host that cannot give the kernel freshly allocated scratch.
 *
 * No counterpart in the reference.  Some callers must not allocate device memory: a serving
 * process whose memory pool has already claimed the whole device, a plug-in that is called at a
 * point where the host forbids allocation, a real-time loop that may not take the allocator's
 * lock.  For them the activation hand-off words of the kernel (the buffers a normal engine passes
 * as MK_G_XL, MK_G_PROJL, MK_G_MIXL, MK_G_ACTL, MK_G_LML, MK_G_ATTN_PART and MK_G_PARTL) live in one array that
 * is compiled into the library, MK_STATIC_SCRATCH_BYTES (4 MiB) per GPU that loads it, held until the
 * process exits.  The caller still passes every input and output (weights, state, KV cache, status
 * words, the launch arguments); this function calls no cudaMalloc / cudaFree and no allocating
 * library routine.
 *
 *  - The first call on a device looks up the array's device address and caches it; make that first
 *    call outside any stream capture.
 *  - Such a host need not own hand-off buffers at all: mk_set_params accepts an engine whose MK_G_XL, MK_G_PROJL,
 *    MK_G_MIXL, MK_G_ACTL, MK_G_LML, MK_G_ATTN_PART and MK_G_PARTL are all 0 (all of them, or none).  mk_launch
 *    and mk_launch_batch refuse that engine with MK_ERR_BADARG; mk_launch_static runs it.
 *  - A grid or shape whose hand-off words do not fit the array is refused with MK_ERR_BADARG.
 *  - Every call clears the array on `stream` before the kernel runs, because all calls (of all
 *    engines) share it and it keeps what the last call wrote.  Two calls that overlap on the GPU
 *    (different streams, or different engines at once) therefore race: serialise them. */
#define MK_STATIC_SCRATCH_BYTES (4u << 20)
int mk_launch_static(mk_engine* e, const mk_launch_args* args, void* stream);

/* Batched decoding: up to MK_MAX_BATCH independent sequences share every pass over the weights
 * (int8 engines only).  The reference's 0.8B kernel decodes one sequence per launch; its batched
 * engines are the gfx942 ones, whose `Engine.step(tok[M])` (qwen3.8-27b-gfx942/mk/runner.py:202-213)
 * takes one token per sequence and step.  Here the whole generation of all sequences is one launch,
 * like mk_launch: step s feeds position pos0[j] + s of sequence j, first the sequence's prompt tokens
 * (forced, n_forced[j] of them), then its own greedy or sampled choices.
 *
 * The engine's buffers are those of mk_set_params with every per-sequence buffer `batch` times as
 * large, sequence-major: the hand-off words (MK_G_XL, MK_G_PROJL, MK_G_MIXL, MK_G_ACTL [batch, width],
 * MK_G_LML [batch, grid, 2], MK_G_ATTN_PART [batch, kv_heads, MK_Q_MAX_SPLITS, MK_Q_PART_STRIDE]), the
 * DeltaNet state (MK_L_STATE [batch, 16, 128, 128]) and the batched conv history (MK_L_CONV_HIST_B: a
 * DeltaNet task here is one head of one sequence, so the history is kept per head, not per task of
 * MK_L_CONV_HIST) of every layer, and MK_G_BLOCK_TABLE [batch, max_seq / 64] with page
 * numbers into one pool per layer (batch * max_seq / 64 <= 512 pages).  A sequence that has produced a
 * stop id, or has run its n_total steps, keeps stepping until all have (its outputs are to be
 * ignored), but its DeltaNet state and conv history stay as its last accepted token left them. */
#define MK_MAX_BATCH 8
typedef struct mk_batch_args {
    uint64_t forced;                 /* int32[max n_forced, MK_MAX_BATCH], step-major                 */
    int32_t n_forced[MK_MAX_BATCH];  /* prompt tokens of each sequence, >= 1                          */
    int32_t n_total[MK_MAX_BATCH];   /* steps each sequence takes part in (n_forced + n_generate - 1) */
    int32_t pos0[MK_MAX_BATCH];      /* position of each sequence's first token in this launch        */
    int32_t batch;                   /* live sequences, 1..MK_MAX_BATCH                               */
    int32_t n_steps;
    int32_t lm_from;                 /* first step that runs the LM head: <= min n_forced - 1         */
    uint32_t epoch_base;
    uint32_t seed;                   /* sequence j samples with seed + j * 0x9E3779B9                 */
    float inv_temperature;
    int32_t n_stop;
    int32_t prof_step;
    uint64_t stop_ids;
    uint64_t tokens_out;             /* u64[n_steps, MK_MAX_BATCH] keys of every step from lm_from on */
    uint64_t logits_out;             /* optional fp32 [n_steps, MK_MAX_BATCH, vocab]                  */
    uint64_t step_ts;                /* optional u64 [n_steps + 1]                                    */
    uint64_t out_info;               /* int32[8]: steps run, next epoch, bit mask of stopped sequences */
    uint64_t prof;
    int64_t spin_limit_ns;
} mk_batch_args;
int mk_launch_batch(mk_engine* e, const mk_batch_args* args, void* stream);

/* Replaces `watchdog_fired` (qwen3.5-0.8b/csrc/megakernel.cu:1284-1289): synchronises the device,
 * reads the status words of the last launch and returns MK_OK or MK_ERR_TIMEOUT.  Unlike the
 * reference, waits are bounded in every build, not only with -DMK_WATCHDOG. */
int mk_status(mk_engine* e, int32_t* where);

/* Replaces the module constants exported at qwen3.5-0.8b/csrc/binding.cpp:107-121. */
enum {
    MK_Q_SMEM_BYTES = 0, MK_Q_N_THREADS, MK_Q_CONV_RING, MK_Q_KV_BLOCK, MK_Q_MAX_SPLITS, MK_Q_PART_STRIDE,
    MK_Q_OPS_PER_LAYER, MK_Q_PROF_MAX_OPS, MK_Q_PROF_FIELDS, MK_Q_SPEC_T, MK_Q_MAX_LAYERS, MK_Q_LAYER_FIELDS,
    MK_Q_GLOBAL_FIELDS, MK_Q_SLOT_BYTES, MK_Q_STAGES, MK_Q_MAX_LM_ROWS, MK_Q_MAX_BATCH, MK_Q_BATCH_SMEM_BYTES
};
int64_t mk_query(int what);

/* Streams `bytes` from `src` through every SM once with plain 128-bit loads (mode 0) or with the
 * kernel's own bulk-copy ring (mode 1) and writes one checksum word to `sink`; the measured
 * bandwidth is the denominator sanity check.  Replaces common/bw.cu:10-17,42-83. */
int mk_bw_probe(uint64_t src, int64_t bytes, int mode, uint64_t sink, int device, void* stream);

/* The kernel's work partition, exposed so that packers and tests can reproduce it on the host:
 * rows [*r0, *r1) of a `rows`-row matrix that CTA `cta` of `grid` owns (`unit` rows stay together),
 * and the number of cached positions one attention task scans for a context of `n` positions.
 * Restates `block_slice` (qwen3.5-0.8b/csrc/megakernel.cu:118-121) and `attn_split` (:732-753). */
int mk_plan_rows(int rows, int unit, int cta, int grid, int* r0, int* r1);
int mk_plan_attn_chunk(int n, int max_splits);

const char* mk_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
