/* mk_stage.h -- C ABI of the stage-machine decode megakernel for the large hybrid shapes
 * (27B dense MXFP4, 35B-A3B FP8 MoE, 26B-A4B FP8 sliding-window MoE) on B200 (sm_100a).
 *
 * One cooperative launch runs `n_steps` whole decode steps for M <= 8 sequences: embedding, every
 * layer, the LM head and the greedy choice.  What a step does is a *program*: an array of
 * mk_stage_desc records in device memory that the host builds once per model (the Python packages
 * megakernels_b200.qwen27b / qwen35b / gemma26b do it).  Every CTA walks the program; a producer
 * warp streams the weight chunks of every GEMV stage into a shared-memory ring ahead of the
 * consumers, which run the stages and meet at a grid barrier after each one.
 *
 * It replaces `launch(tab_ptr, glob_ptr, nlayers, stream)` of the reference's gfx942 engines
 * (qwen3.8-27b-gfx942/mk/kernel.py:478, its pointer tables kernel.py:63-108 and runner.py:113-196;
 * the same interface in qwen3.6-35b-a3b-gfx942/mk and gemma4-26b-a4b-gfx942/mk): there the stage
 * list is compiled into the kernel and the tables carry pointers, here the table carries the stages.
 *
 * Conventions as in mk_b200.h: the caller owns every device buffer and passes raw addresses, every
 * function returns MK_OK or a negative MK_ERR_*, mk_last_error() has the text, nothing throws, every
 * device-side wait is bounded (MK_ERR_TIMEOUT through the status words).
 */
#ifndef MK_STAGE_H
#define MK_STAGE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- stage kinds --------------------------------------------------------------------------------- */
enum {
    MKS_OP_EMBED = 1,   /* token choice of the previous step, embedding rows -> residual stream   */
    MKS_OP_GEMV = 2,    /* dequantising matrix-vector products on the tensor cores                */
    MKS_OP_GDN = 3,     /* Gated DeltaNet: causal conv1d, delta-rule state update, gated RMSNorm  */
    MKS_OP_ATTN = 4,    /* split-K flash-decode attention over a paged bf16/fp32 KV cache         */
    MKS_OP_ROUTE = 5,   /* top-k expert routing tables (CTA-local, identical in every CTA)        */
    MKS_OP_VEC = 6      /* out = (base + rms(a) w_a [+ rms(b) w_b]) * F_SCALE over the hidden vector: the residual /
                           sandwich-norm steps of the 26B model (gemma4-26b-a4b-gfx942/mk/reference.py:296-307) */
};

/* flags */
enum {
    MKS_FLAG_NO_BARRIER = 1   /* the next stage does not read this one's outputs: no grid barrier      */
};

/* weight formats of a GEMV stage: bytes per 16-row x k tile step are 512 in every format */
enum {
    MKS_FMT_BF16 = 0,    /* 16 k per step                                                          */
    MKS_FMT_MXFP4 = 1,   /* e2m1, one e8m0 scale per 32 k; 64 k per step                           */
    MKS_FMT_FP8 = 2,     /* e4m3; optional fp32 scale per 128 k (block scaled) and / or per row; 32 k per step */
    MKS_FMT_INT8 = 3     /* signed bytes, fp32 scale per row; 32 k per step                        */
};

/* GEMV input (prologue) */
enum {
    MKS_P_PLAIN = 0,     /* x = src                                                                */
    MKS_P_NORM = 1       /* x = src * rsqrt(mean(src^2) + eps) * (norm_off + norm_w)               */
};

/* GEMV output (epilogue) */
enum {
    MKS_E_STORE = 0,     /* out[group][m][row] = y                                                 */
    MKS_E_RESID = 1,     /* h[m][row] += y, and the sum of squares of each 16-row group of h       */
    MKS_E_GLU = 2,       /* rows pair up inside a tile (row r: gate, row r + 8: up): out = act(gate) * up */
    MKS_E_LOGITS = 3     /* logits[m][row] = y (optionally soft-capped) and the running arg-max    */
};

enum { MKS_ACT_SILU = 0, MKS_ACT_GELU_TANH = 1 };

/* ---- integer fields i[] of a stage record -------------------------------------------------------- */
enum {
    /* GEMV */
    MKS_I_FMT = 0,
    MKS_I_TILES,         /* 16-row tiles per group                                                 */
    MKS_I_SPLITS,        /* K splits                                                               */
    MKS_I_GROUPS,        /* matrices of the stage (experts); -1: the routed list (+ the shared expert if P_W_SHARED) */
    MKS_I_UNIT_STEPS,    /* tile steps per (tile, split) unit                                      */
    MKS_I_CHUNK_STEPS,   /* tile steps per ring chunk                                              */
    MKS_I_CHUNK_BYTES,   /* bytes of a chunk in HBM: steps * 512 + scales, multiple of 16          */
    MKS_I_KC,            /* input columns per split                                                */
    MKS_I_PROLOGUE,
    MKS_I_EPILOGUE,
    MKS_I_N_VALID,       /* output rows per group that exist (the last tile may be padding)        */
    MKS_I_X_STRIDE,      /* input: elements between sequences                                      */
    MKS_I_X_GSTRIDE,     /* input: elements between groups (0: every group reads the same vector)  */
    MKS_I_OUT_STRIDE,    /* output: elements between sequences                                     */
    MKS_I_OUT_GSTRIDE,   /* output: elements between groups                                        */
    MKS_I_REDUCE_GROUPS, /* 1: the groups' products add up (routing coefficients) into one output  */
    MKS_I_ALLREDUCE,     /* 1: sum over tensor-parallel ranks before the epilogue                  */
    MKS_I_ACT,           /* MKS_ACT_* of E_GLU                                                     */
    MKS_I_K_TOTAL,       /* columns of the whole input vector (the mean of P_NORM divides by it)    */
    MKS_I_BLOCK_SCALES,  /* FP8: fp32 scales per 128 k inside each chunk (0: none)                 */
    MKS_I_PIECES,        /* 1: input rounded to bf16 (the model dtype); 2: hi + lo pieces, fp16 (bf16 for bf16 weights):
                            inputs exact to 16+ bits, two MMA columns per sequence, M <= 4       */
    MKS_I_GEMV_END,

    /* EMBED */
    MKS_I_HIDDEN = 0,    /* residual width                                                         */
    MKS_I_VOCAB,
    MKS_I_KEYS_VALID,    /* 1: later steps take their token from the arg-max keys of the LM head   */

    /* GDN */
    MKS_I_NKH = 0, MKS_I_NVH, MKS_I_Q_OFF, MKS_I_K_OFF, MKS_I_V_OFF, MKS_I_Z_OFF, MKS_I_B_OFF, MKS_I_A_OFF,
    MKS_I_CONV_DIM,      /* channels of the conv state (q | k | v)                                 */
    MKS_I_Y_STRIDE,      /* in-projection output: elements between sequences                       */
    MKS_I_Y2_STRIDE,     /* mixer output: elements between sequences                               */
    MKS_I_CONV_BF16,     /* 1: conv history holds bf16-rounded values                              */
    MKS_I_L2_CLAMP,      /* 1: l2norm divides by max(norm, eps) (0.8B decoder); 0: rsqrt(sum + eps) */

    /* ATTN */
    MKS_I_NQ = 0, MKS_I_NKV, MKS_I_HD, MKS_I_ROT,   /* q heads, kv heads (of this rank), head dim, rotated dims */
    MKS_I_A_Q_OFF,       /* per head: [q | gate] (gated) or [q] at Q_OFF + head * Q_HEAD_STRIDE     */
    MKS_I_A_Q_HSTRIDE, MKS_I_A_GATE_OFF,   /* gate offset inside a head record, -1: no output gate */
    MKS_I_A_K_OFF, MKS_I_A_V_OFF,          /* V_OFF = -1: V is the raw k projection (k_eq_v)       */
    MKS_I_A_Y_STRIDE, MKS_I_A_Y2_STRIDE,
    MKS_I_WINDOW,        /* sliding window (0: full attention)                                     */
    MKS_I_CHUNK_POS,     /* positions per split task                                               */
    MKS_I_MAX_PAGES,     /* columns of the block table                                             */
    MKS_I_KV_F32,        /* 1: fp32 KV cache, 0: bf16                                              */
    MKS_I_NORM_PLAIN,    /* 1: q/k norm weight is the factor itself (Gemma), 0: 1 + w              */
    MKS_I_V_NORM,        /* 1: V is RMS-normed without weight (Gemma)                              */
    MKS_I_ROPE_PAIRS,    /* cos/sin table columns (angle pairs); pair d rotates dims (d, d + HD/2) when ROT == HD, else (d, d + ROT/2) */
    MKS_I_Q_BF16,        /* 1: q rounded to bf16 before QK^T                                       */
    MKS_I_MAX_CHUNKS,    /* split records per (sequence, kv head) in A_PART                        */
    MKS_I_KV_BLOCK,      /* positions per cache page, a power of two (0: 64)                        */
    MKS_I_KV_S_PAGE, MKS_I_KV_S_HEAD, MKS_I_KV_S_POS,   /* element strides of the paged cache between pages, kv heads and
                            positions (all 0: [page][kv head][64][head dim]); a serving stack's layout, e.g.
                            [page][position][kv head][head dim], is strides (block * heads * dim, dim, heads * dim)
                            (qwen3.8-27b-gfx942/mk/kernel.py:15-27) */

    /* ROUTE */
    MKS_I_EXPERTS = 0, MKS_I_TOPK, MKS_I_LOGIT_STRIDE,
    MKS_I_ROUTE_KIND,    /* 0: weights = softmax over the selected logits, shared-expert gate = sigmoid(logit[EXPERTS]);
                            1: softmax over all experts, top-k renormalised, times per_expert_scale  */

    /* VEC */
    MKS_I_VEC_N = 0,     /* elements per sequence (a multiple of 16; 0: an empty stage, its barrier only) */

    MKS_I_COUNT = 30
};

/* ---- float fields f[] ---------------------------------------------------------------------------- */
enum {
    MKS_F_EPS = 0,
    MKS_F_NORM_OFF,      /* 1 for zero-centred norm weights (x * (1 + w)), 0 for plain ones        */
    MKS_F_SOFTCAP,       /* E_LOGITS: cap * tanh(y / cap) if > 0                                   */
    MKS_F_SCALE,         /* EMBED: embedding scale (0: none); ATTN: score scale; VEC: factor on the result (0: none) */
    MKS_F_IN_SCALE,      /* P_NORM: extra factor on the normed input (router of the 26B model)     */
    MKS_F_IN_BOUND,      /* > 0: no staged input value exceeds it in magnitude (the host knows: a normed vector is at most
                            sqrt(K) max|weight|); lets the kernel fix the fp16 scale without a pass over the values */
    MKS_F_COUNT = 8
};

/* ---- pointer fields p[] -------------------------------------------------------------------------- */
enum {
    /* GEMV */
    MKS_P_W = 0,         /* weights of group 0 in the tile layout (megakernels_b200/stage/pack.py)  */
    MKS_P_W_GSTRIDE,     /* bytes between groups / experts (a value, not a pointer)                */
    MKS_P_W_SHARED,      /* routed stages: the shared expert's matrix, appended as the last group  */
    MKS_P_ROW_SCALE,     /* fp32 [groups][rows] or 0                                               */
    MKS_P_RS_GSTRIDE,    /* elements between groups in ROW_SCALE (a value)                         */
    MKS_P_RS_SHARED,
    MKS_P_X,             /* fp32 input                                                             */
    MKS_P_X_SSQ,         /* fp32 [M][K/16] sums of squares of the input (P_NORM)                   */
    MKS_P_NORM_W,        /* fp32 [K]                                                               */
    MKS_P_OUT,
    MKS_P_OUT_SSQ,       /* E_RESID: fp32 [M][N/16]                                                */
    MKS_P_CNT,           /* u32 arrival counters, one per output tile (per group unless REDUCE_GROUPS) */
    MKS_P_PART,          /* fp32 partial tiles [counter][arrival][16 x 8]                          */
    MKS_P_KEYS,          /* E_LOGITS: u64 [M][grid] best (score, ~row) key of every CTA            */
    MKS_P_ROW_BASE,      /* E_LOGITS: first vocabulary row of this rank (a value)                  */
    MKS_P_W_BYTES,       /* bytes of one group's matrix (a value; 0: unchecked): a copy that would leave it
                            is not issued, the launch ends with status -5                          */

    /* EMBED */
    MKS_P_TABLE = 0,     /* bf16 [vocab][hidden]                                                   */
    MKS_P_H,             /* fp32 [M][hidden] residual stream                                       */
    MKS_P_H_SSQ,         /* fp32 [M][hidden / 16]                                                  */
    MKS_P_E_KEYS,        /* the LM head's key buffer                                               */

    /* GDN */
    MKS_P_Y = 0,         /* in-projection output, fp32 [M][...]                                    */
    MKS_P_Y2,            /* mixer output, fp32 [M][...]                                            */
    MKS_P_CONV_W,        /* fp32 [conv_dim][4]                                                     */
    MKS_P_A_LOG, MKS_P_DT_BIAS, MKS_P_GDN_NORM,
    MKS_P_CONV_STATE,    /* fp32 [M][conv_dim][4] ring by position & 3                             */
    MKS_P_SSM_STATE,     /* fp32 [M][value heads][128 v][128 k]                                    */

    /* ATTN */
    MKS_P_A_Y = 0, MKS_P_A_Y2, MKS_P_Q_NORM, MKS_P_K_NORM,
    MKS_P_K_CACHE, MKS_P_V_CACHE,   /* [pages][kv heads][64][head dim]                             */
    MKS_P_BLOCK_TABLE,   /* int32 [M][max pages]                                                   */
    MKS_P_ROPE_COS, MKS_P_ROPE_SIN, /* fp32 [max_seq][pairs]                                       */
    MKS_P_A_PART,        /* fp32 split partials [M][kv heads][max chunks][q per kv * (head dim + 2), rounded up to 4], then
                            per-CTA scratch [grid][16][q per kv][128]                               */
    MKS_P_A_CNT,         /* u32 [M][kv heads]                                                      */

    /* ROUTE */
    MKS_P_LOGITS = 0, MKS_P_EXPERT_SCALE,
    MKS_P_ROUTE_OUT,     /* optional i32 [M][top k]: the chosen expert ids in rank order (for tests and traces;
                            the reference's debug_route, gemma4-26b-a4b-gfx942/tests/test_decode.py)  */

    /* VEC */
    MKS_P_VEC_BASE = 0,  /* fp32 [M][n] added unchanged, or 0                                        */
    MKS_P_VEC_A,         /* fp32 [M][n]: first normed term                                           */
    MKS_P_VEC_A_SSQ,     /* its sums of squares per 16 elements [M][n / 16] (an E_STORE / E_RESID output) */
    MKS_P_VEC_A_W,       /* its norm weight [n]                                                      */
    MKS_P_VEC_B, MKS_P_VEC_B_SSQ, MKS_P_VEC_B_W,   /* optional second normed term (VEC_B = 0: none)   */
    MKS_P_VEC_OUT,       /* fp32 [M][n] (may be VEC_BASE: in place)                                  */
    MKS_P_VEC_OUT_SSQ,   /* sums of squares of the result per 16 elements, or 0                      */

    MKS_P_COUNT = 16
};

typedef struct mk_stage_desc {
    int32_t op;
    int32_t flags;
    int32_t i[MKS_I_COUNT];
    float f[MKS_F_COUNT];
    uint64_t p[MKS_P_COUNT];
} mk_stage_desc;   /* 288 bytes */

#define MKS_MAX_BATCH 8
#define MKS_MAX_RANKS 8

/* Per-launch arguments.  Replaces the reference's `glob` table (kernel.py:66-90) and the host-side
 * step bookkeeping of Engine.step (runner.py:202-213). */
typedef struct mk_stage_args {
    uint64_t program;        /* mk_stage_desc[n_stages] in device memory                           */
    int32_t n_stages;
    int32_t batch;           /* M, 1..8                                                            */
    int32_t n_steps;         /* decode steps of this launch; each later step feeds the arg-max of the one before */
    int32_t device;
    uint64_t tok;            /* int32[M]: tokens of the first step; holds the next tokens afterwards */
    uint64_t pos;            /* int32[M]: positions of the first step; advanced by n_steps afterwards */
    uint64_t tokens_out;     /* optional int32[n_steps][M]: the greedy choice after every step     */
    uint64_t barrier;        /* u64[1] grid-barrier counter (zero at reset)                        */
    uint64_t barrier_base;   /* value of the counter when the launch starts; the host carries it   */
    uint64_t status;         /* int32[4]: first wait that ran out: code, site, CTA, thread         */
    int64_t spin_limit_ns;   /* bound on every device-side wait; 0 = 2 s                           */
    uint64_t prof;           /* optional u64[n_stages][8]: GPU ns of CTA `prof_cta` in the last step, per stage:
                                entered, input staged, work done, barrier passed                  */
    /* tensor parallelism: every rank runs the same program on its shard; row-parallel GEMVs with
     * ALLREDUCE push their partial tiles into every rank's mailbox with plain peer stores and poll
     * their own (qwen3.8-27b-gfx942/mk/stages.py:180-267, mk/sync.py:69-163) */
    int32_t tp;              /* ranks, 1..8                                                        */
    int32_t rank;
    uint64_t mailbox[MKS_MAX_RANKS];   /* every rank's mailbox as this device addresses it         */
    uint64_t ar_base;        /* all-reduce sequence number before this launch (the host carries it)*/
    int32_t grid;            /* CTAs, 0 = one per SM                                               */
    int32_t prof_cta;        /* the CTA whose timestamps go to `prof`; -1: every CTA, prof is u64[grid][n_stages][8] */
    uint64_t tokens_in;      /* optional i32[n_tokens_in][batch]: the inputs of the first n_tokens_in steps (a prompt);
                                step s < n_tokens_in feeds tokens_in[s] instead of `tok` / the previous choice    */
    int32_t xs_bytes;        /* shared staging area the program needs (mk_stage_scratch_bytes; 0: the maximum);
                                what it leaves of the SM's shared memory becomes ring slots (2..4 per warp) */
    int32_t n_tokens_in;
    uint64_t row_valid;      /* optional i32[batch]: 0 marks a padding row for this launch.  Its recurrent state, conv
                                history, KV cache and position stay as they are and it selects no routed expert;
                                what the launch writes to its activations, logits and token is undefined (the
                                reference's `valid` / slot < 0 rows: qwen3.6-35b-a3b-gfx942/mk/runner.py:187-192,
                                qwen3.8-27b-gfx942/mk/kernel.py:25-27)                                           */
} mk_stage_args;

/* Launch.  Asynchronous on `stream`. */
int mk_stage_launch(const mk_stage_args* args, void* stream);

/* Checks a host copy of a program against the kernel's structural limits (ring slot, input staging
 * area, MMA columns, mailbox size) before it is uploaded; MK_ERR_BADARG names the stage. */
int mk_stage_validate(const mk_stage_desc* program, int n_stages, int batch);

/* Bytes of shared staging area `program` needs at `batch` sequences (for mk_stage_args.xs_bytes). */
int64_t mk_stage_scratch_bytes(const mk_stage_desc* program, int n_stages, int batch);

/* Barriers and all-reduces one step of `program` (host copy) performs: what the caller adds to
 * barrier_base / ar_base per step. */
int mk_stage_count(const mk_stage_desc* program, int n_stages, int64_t* barriers, int64_t* allreduces);

enum { MKS_Q_SMEM_BYTES = 0, MKS_Q_N_THREADS, MKS_Q_SLOT_BYTES, MKS_Q_XS_BYTES, MKS_Q_DESC_BYTES, MKS_Q_MAX_GROUPS,
       MKS_Q_MAILBOX_BYTES, MKS_Q_ATTN_MAX_CHUNK };
int64_t mk_stage_query(int what);

/* What a stage boundary costs on this GPU apart from any work.  mode 0: the kernel's grid barrier (one CTA per SM;
 * `stores` global stores per thread before each barrier), mode 1: a flag round trip between two CTAs.  Runs
 * `iters` iterations on the default stream, synchronously; *ns_per_iter receives the average.  The counterpart of
 * the reference's barrier microbenchmark (qwen3.5-0.8b/bench/barrier.cu:27-59). */
int mk_sync_probe(int device, int mode, int iters, int stores, int64_t* ns_per_iter);

/* Peer-visible device memory for the tensor-parallel mailboxes: allocate on this process's device,
 * export a handle (64 bytes) another process on the same node opens.  The counterpart of the
 * reference's hipIpc peer buffer (qwen3.8-27b-gfx942/mk/peer.py:26-126). */
int mk_peer_alloc(int device, int64_t bytes, uint64_t* ptr, uint8_t handle[64]);
int mk_peer_open(int device, const uint8_t handle[64], uint64_t* ptr);
int mk_peer_close(uint64_t ptr);
int mk_peer_free(uint64_t ptr);

#ifdef __cplusplus
}
#endif
#endif
