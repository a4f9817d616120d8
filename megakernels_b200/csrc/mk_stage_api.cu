// C ABI of the stage-machine megakernel (declarations and reference citations: include/mk_stage.h).
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/mk_b200.h"
#include "mk_stage_ops.cuh"

using namespace mks;

// defined in mk_api.cu: stores the text behind mk_last_error() for the calling thread
int mk_set_error(int code, const char* text);

static int sfail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    return mk_set_error(code, buf);
}
#define MKS_CUDA(call)                                                                      \
    do {                                                                                    \
        cudaError_t err__ = (call);                                                         \
        if (err__ != cudaSuccess)                                                           \
            return sfail(MK_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(err__));   \
    } while (0)

static int steps_k(int fmt) { return fmt == MKS_FMT_MXFP4 ? 64 : (fmt == MKS_FMT_BF16 ? 16 : 32); }

// Structural limits of one program (a host copy): what the kernel's shared-memory staging and ring can hold.
extern "C" int mk_stage_validate(const mk_stage_desc* prog, int n_stages, int batch) {
    if (!prog || n_stages < 1) return sfail(MK_ERR_BADARG, "mk_stage_validate: empty program");
    if (batch < 1 || batch > MKS_MAX_BATCH) return sfail(MK_ERR_BADARG, "mk_stage_validate: batch %d out of [1, %d]", batch, MKS_MAX_BATCH);
    if (prog[0].op != MKS_OP_EMBED) return sfail(MK_ERR_BADARG, "mk_stage_validate: the first stage must be the embedding");
    for (int s = 0; s < n_stages; s++) {
        const mk_stage_desc& d = prog[s];
        if (d.op == MKS_OP_GEMV) {
            const int fmt = d.i[MKS_I_FMT], kc = d.i[MKS_I_KC], pieces = d.i[MKS_I_PIECES];
            if (fmt < MKS_FMT_BF16 || fmt > MKS_FMT_INT8) return sfail(MK_ERR_BADARG, "stage %d: weight format %d", s, fmt);
            if (pieces != 1 && pieces != 2) return sfail(MK_ERR_BADARG, "stage %d: pieces %d", s, pieces);
            if (pieces * batch > 8) return sfail(MK_ERR_BADARG, "stage %d: %d input pieces x %d sequences exceed the 8 MMA columns", s, pieces, batch);
            if (kc < 128) return sfail(MK_ERR_BADARG, "stage %d: fewer than 128 columns per split", s);
            if (pieces == 2 && (long long)kc * batch > 8192) return sfail(MK_ERR_BADARG, "stage %d: two-piece inputs hold at most 8192 values per panel", s);
            if (kc < 1 || kc % steps_k(fmt)) return sfail(MK_ERR_BADARG, "stage %d: %d columns per split are not whole tile steps", s, kc);
            if (d.i[MKS_I_UNIT_STEPS] * steps_k(fmt) != kc) return sfail(MK_ERR_BADARG, "stage %d: unit steps %d x %d != kc %d", s, d.i[MKS_I_UNIT_STEPS], steps_k(fmt), kc);
            if (d.i[MKS_I_CHUNK_STEPS] < 1 || d.i[MKS_I_UNIT_STEPS] % d.i[MKS_I_CHUNK_STEPS])
                return sfail(MK_ERR_BADARG, "stage %d: chunk steps %d do not divide unit steps %d", s, d.i[MKS_I_CHUNK_STEPS], d.i[MKS_I_UNIT_STEPS]);
            if (d.i[MKS_I_CHUNK_BYTES] > mks::SLOT_BYTES || d.i[MKS_I_CHUNK_BYTES] % 16 || d.i[MKS_I_CHUNK_BYTES] < d.i[MKS_I_CHUNK_STEPS] * 512)
                return sfail(MK_ERR_BADARG, "stage %d: chunk of %d bytes (slot: %d)", s, d.i[MKS_I_CHUNK_BYTES], mks::SLOT_BYTES);
            if (fmt == MKS_FMT_FP8 && d.i[MKS_I_BLOCK_SCALES] && d.i[MKS_I_CHUNK_STEPS] % 4)
                return sfail(MK_ERR_BADARG, "stage %d: block-scaled chunks must hold whole 128-column blocks", s);
            const int stride = ((kc * 2 + 127) / 128) * 128 + 32;
            if ((long long)stride * 8 > XS_BYTES) return sfail(MK_ERR_BADARG, "stage %d: %d columns per split do not fit the input staging area", s, kc);
            if (d.i[MKS_I_TILES] < 1 || d.i[MKS_I_SPLITS] < 1) return sfail(MK_ERR_BADARG, "stage %d: tiles / splits", s);
            if ((long long)d.i[MKS_I_TILES] * d.i[MKS_I_SPLITS] * (d.i[MKS_I_GROUPS] > 0 ? d.i[MKS_I_GROUPS] : MAX_GROUPS) >= (1 << 24))
                return sfail(MK_ERR_BADARG, "stage %d: more than 2^24 units", s);
            if (d.i[MKS_I_GROUPS] > MAX_GROUPS || d.i[MKS_I_GROUPS] == 0) return sfail(MK_ERR_BADARG, "stage %d: groups %d", s, d.i[MKS_I_GROUPS]);
            const bool reduce = d.i[MKS_I_REDUCE_GROUPS] != 0;
            if ((d.i[MKS_I_SPLITS] > 1 || reduce) && (!d.p[MKS_P_CNT] || !d.p[MKS_P_PART]))
                return sfail(MK_ERR_BADARG, "stage %d: split or reduced units need counters and a partial buffer", s);
            if (d.i[MKS_I_ALLREDUCE] && d.i[MKS_I_TILES] > MAILBOX_TILES) return sfail(MK_ERR_BADARG, "stage %d: %d tiles exceed the mailbox", s, d.i[MKS_I_TILES]);
            if (!d.p[MKS_P_W] || (d.p[MKS_P_W] & 15) || !d.p[MKS_P_X] || !d.p[MKS_P_OUT]) return sfail(MK_ERR_BADARG, "stage %d: weights / input / output missing or misaligned", s);
            if (d.i[MKS_I_PROLOGUE] == MKS_P_NORM && (!d.p[MKS_P_X_SSQ] || !d.p[MKS_P_NORM_W])) return sfail(MK_ERR_BADARG, "stage %d: norm prologue without sums of squares / weights", s);
            if (d.i[MKS_I_EPILOGUE] == MKS_E_LOGITS && !d.p[MKS_P_KEYS]) return sfail(MK_ERR_BADARG, "stage %d: logits without a key buffer", s);
        } else if (d.op == MKS_OP_ATTN) {
            const int QPK = d.i[MKS_I_NKV] > 0 ? d.i[MKS_I_NQ] / d.i[MKS_I_NKV] : 0, HD = d.i[MKS_I_HD], CP = d.i[MKS_I_CHUNK_POS];
            if (QPK < 1 || QPK > 8 || QPK + 2 > NCW) return sfail(MK_ERR_BADARG, "stage %d: %d query heads per KV head", s, QPK);
            if (HD != 256 && HD != 512) return sfail(MK_ERR_BADARG, "stage %d: head dim %d", s, HD);
            if (CP < 16 || CP > ATTN_MAX_CHUNK) return sfail(MK_ERR_BADARG, "stage %d: %d positions per task", s, CP);
            if ((long long)(QPK * HD + 2 * HD + QPK * CP + QPK * ATTN_MAX_CHUNKS + 2 * QPK + CP + 4) * 4 > XS_BYTES) return sfail(MK_ERR_BADARG, "stage %d: attention scratch does not fit", s);
            if (d.i[MKS_I_KV_BLOCK] < 0 || (d.i[MKS_I_KV_BLOCK] & (d.i[MKS_I_KV_BLOCK] - 1))) return sfail(MK_ERR_BADARG, "stage %d: %d positions per cache page (a power of two)", s, d.i[MKS_I_KV_BLOCK]);
            if (d.i[MKS_I_KV_S_PAGE] && (d.i[MKS_I_KV_S_POS] < HD || d.i[MKS_I_KV_S_HEAD] < 1 || d.i[MKS_I_KV_S_POS] % 8)) return sfail(MK_ERR_BADARG, "stage %d: cache strides", s);
            if (d.i[MKS_I_MAX_CHUNKS] < 1 || d.i[MKS_I_MAX_CHUNKS] > ATTN_MAX_CHUNKS) return sfail(MK_ERR_BADARG, "stage %d: %d split records per head (at most %d)", s, d.i[MKS_I_MAX_CHUNKS], ATTN_MAX_CHUNKS);
        } else if (d.op == MKS_OP_GDN) {
            if (d.i[MKS_I_NKH] < 1 || d.i[MKS_I_NVH] % d.i[MKS_I_NKH]) return sfail(MK_ERR_BADARG, "stage %d: DeltaNet heads", s);
        } else if (d.op == MKS_OP_ROUTE) {
            if ((d.i[MKS_I_EXPERTS] != 128 && d.i[MKS_I_EXPERTS] != 256) || d.i[MKS_I_TOPK] < 1 || d.i[MKS_I_TOPK] > 8)
                return sfail(MK_ERR_BADARG, "stage %d: %d experts, top %d", s, d.i[MKS_I_EXPERTS], d.i[MKS_I_TOPK]);
            if (batch * d.i[MKS_I_TOPK] + 1 > MAX_GROUPS) return sfail(MK_ERR_BADARG, "stage %d: too many routed groups", s);
        } else if (d.op == MKS_OP_VEC) {
            if (d.i[MKS_I_VEC_N] == 0) continue;              // an empty stage: its barrier only
            if (d.i[MKS_I_VEC_N] < 16 || d.i[MKS_I_VEC_N] % 16) return sfail(MK_ERR_BADARG, "stage %d: vector of %d elements", s, d.i[MKS_I_VEC_N]);
            if (!d.p[MKS_P_VEC_A] || !d.p[MKS_P_VEC_A_SSQ] || !d.p[MKS_P_VEC_A_W] || !d.p[MKS_P_VEC_OUT])
                return sfail(MK_ERR_BADARG, "stage %d: vector step without its term, sums of squares, weight or output", s);
            if (d.p[MKS_P_VEC_B] && (!d.p[MKS_P_VEC_B_SSQ] || !d.p[MKS_P_VEC_B_W])) return sfail(MK_ERR_BADARG, "stage %d: second term without sums of squares / weight", s);
        } else if (d.op != MKS_OP_EMBED) {
            return sfail(MK_ERR_BADARG, "stage %d: unknown op %d", s, d.op);
        }
    }
    return MK_OK;
}

// Bytes of the shared staging area a program needs at `batch` sequences: the widest staged GEMV input or
// the largest mixer scratch.  What is left of the SM's shared memory becomes ring slots.
static int64_t scratch_bytes(const mk_stage_desc* prog, int n_stages, int batch) {
    int64_t need = 4096;
    for (int s = 0; s < n_stages; s++) {
        const mk_stage_desc& d = prog[s];
        int64_t b = 0;
        if (d.op == MKS_OP_GEMV) {
            const int stride = ((d.i[MKS_I_KC] * 2 + 127) / 128) * 128 + 32;
            b = (int64_t)stride * batch * d.i[MKS_I_PIECES];
        } else if (d.op == MKS_OP_ATTN) {
            const int QPK = d.i[MKS_I_NQ] / d.i[MKS_I_NKV], HD = d.i[MKS_I_HD], CP = d.i[MKS_I_CHUNK_POS];
            b = (int64_t)(QPK * HD + 2 * HD + QPK * CP + QPK * ATTN_MAX_CHUNKS + 2 * QPK + CP + 4) * 4;
        }
        need = b > need ? b : need;
    }
    return (need + 127) / 128 * 128;
}
extern "C" int64_t mk_stage_scratch_bytes(const mk_stage_desc* prog, int n_stages, int batch) {
    if (!prog || n_stages < 1 || batch < 1 || batch > MKS_MAX_BATCH) return -1;
    return scratch_bytes(prog, n_stages, batch);
}

extern "C" int mk_stage_count(const mk_stage_desc* prog, int n_stages, int64_t* barriers, int64_t* allreduces) {
    if (!prog || n_stages < 1) return sfail(MK_ERR_BADARG, "mk_stage_count: empty program");
    int64_t b = 0, a = 0;
    for (int s = 0; s < n_stages; s++) {
        if (!(prog[s].flags & MKS_FLAG_NO_BARRIER)) b++;
        if (prog[s].op == MKS_OP_GEMV && prog[s].i[MKS_I_ALLREDUCE]) a++;
    }
    if (barriers) *barriers = b;
    if (allreduces) *allreduces = a;
    return MK_OK;
}

extern "C" int64_t mk_stage_query(int what) {
    switch (what) {
        case MKS_Q_SMEM_BYTES: return SMEM_TOTAL;
        case MKS_Q_N_THREADS: return mks::NTHREADS;
        case MKS_Q_SLOT_BYTES: return mks::SLOT_BYTES;
        case MKS_Q_XS_BYTES: return XS_BYTES;
        case MKS_Q_DESC_BYTES: return sizeof(mk_stage_desc);
        case MKS_Q_MAX_GROUPS: return MAX_GROUPS;
        case MKS_Q_MAILBOX_BYTES: return MAILBOX_BYTES;
        case MKS_Q_ATTN_MAX_CHUNK: return ATTN_MAX_CHUNK;
        default: return -1;
    }
}
static_assert(sizeof(mk_stage_desc) == 288, "descriptor layout");

extern "C" int mk_stage_launch(const mk_stage_args* a, void* stream) {
    if (!a) return sfail(MK_ERR_BADARG, "mk_stage_launch: null argument");
    if (!a->program || a->n_stages < 1) return sfail(MK_ERR_BADARG, "mk_stage_launch: no program");
    if (a->batch < 1 || a->batch > MKS_MAX_BATCH) return sfail(MK_ERR_BADARG, "mk_stage_launch: batch %d out of [1, %d]", a->batch, MKS_MAX_BATCH);
    if (a->n_steps < 1) return sfail(MK_ERR_BADARG, "mk_stage_launch: n_steps %d", a->n_steps);
    if (!a->tok || !a->pos || !a->barrier || !a->status) return sfail(MK_ERR_BADARG, "mk_stage_launch: tok / pos / barrier / status missing");
    if (a->n_tokens_in < 0 || (a->n_tokens_in > 0 && !a->tokens_in)) return sfail(MK_ERR_BADARG, "mk_stage_launch: n_tokens_in %d without tokens_in", a->n_tokens_in);
    if (a->barrier & 7) return sfail(MK_ERR_BADARG, "mk_stage_launch: barrier counter not 8-byte aligned");
    if (a->tp < 1 || a->tp > MKS_MAX_RANKS || a->rank < 0 || a->rank >= a->tp) return sfail(MK_ERR_BADARG, "mk_stage_launch: rank %d of %d", a->rank, a->tp);
    if (a->tp > 1)
        for (int r = 0; r < a->tp; r++)
            if (!a->mailbox[r] || (a->mailbox[r] & 15)) return sfail(MK_ERR_BADARG, "mk_stage_launch: mailbox of rank %d missing", r);
    int n_sm = 0;
    MKS_CUDA(cudaSetDevice(a->device));
    MKS_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, a->device));
    const int grid = a->grid > 0 ? a->grid : n_sm;
    if (grid > n_sm) return sfail(MK_ERR_BADARG, "mk_stage_launch: grid %d exceeds the %d SMs (every CTA must be resident)", grid, n_sm);
    if (a->barrier_base % (uint64_t)grid) return sfail(MK_ERR_BADARG, "mk_stage_launch: barrier_base is not a multiple of the grid");

    mks::Args A;
    memset(&A, 0, sizeof A);
    A.prog = reinterpret_cast<const mk_stage_desc*>(a->program);
    A.n_stages = a->n_stages;
    A.M = a->batch;
    A.n_steps = a->n_steps;
    A.tok = reinterpret_cast<int*>(a->tok);
    A.pos = reinterpret_cast<int*>(a->pos);
    A.tokens_out = reinterpret_cast<int*>(a->tokens_out);
    A.bar = reinterpret_cast<unsigned long long*>(a->barrier);
    A.bar_base = a->barrier_base;
    A.status = reinterpret_cast<int*>(a->status);
    A.spin_limit_ns = a->spin_limit_ns > 0 ? a->spin_limit_ns : 2000000000ll;
    A.prof = reinterpret_cast<unsigned long long*>(a->prof);
    A.tp = a->tp;
    A.rank = a->rank;
    for (int r = 0; r < MKS_MAX_RANKS; r++) A.mailbox[r] = reinterpret_cast<unsigned long long*>(a->mailbox[r]);
    A.ar_base = a->ar_base;
    A.tokens_in = reinterpret_cast<const int*>(a->tokens_in);
    A.n_tokens_in = a->tokens_in ? a->n_tokens_in : 0;
    A.row_valid = reinterpret_cast<const int*>(a->row_valid);
    A.prof_cta = a->prof_cta;
    // shared memory: the staging area the program needs (the caller computes it with mk_stage_scratch_bytes), the rest ring slots
    const int xs = a->xs_bytes > 0 ? (a->xs_bytes + 127) / 128 * 128 : XS_BYTES;
    if (xs > XS_BYTES) return sfail(MK_ERR_BADARG, "mk_stage_launch: staging area of %d bytes exceeds %d", xs, XS_BYTES);
    int depth = (SMEM_TOTAL - MISC_BYTES - xs) / (16 * mks::SLOT_BYTES);
    depth = depth > MAX_RING_DEPTH ? MAX_RING_DEPTH : depth;
    if (depth < 2) return sfail(MK_ERR_BADARG, "mk_stage_launch: no room for two ring slots per warp");
    A.xs_bytes = xs;
    A.ring_depth = depth;

    const int smem = MISC_BYTES + xs + 16 * depth * mks::SLOT_BYTES;
    MKS_CUDA(cudaFuncSetAttribute(stage_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    void* kargs[] = {&A};
    MKS_CUDA(cudaLaunchCooperativeKernel((const void*)stage_kernel, dim3(grid), dim3(mks::NTHREADS), kargs, smem, static_cast<cudaStream_t>(stream)));
    return MK_OK;
}


// ---- synchronisation probes ------------------------------------------------------------------------------------
// What a stage boundary costs on this GPU, apart from any work: (0) the grid barrier protocol of stage_kernel
// (512 consumer threads meet, one thread adds to a global counter with release semantics and polls it with acquire
// loads, they meet again) over one CTA per SM, with `stores` global stores per thread in front of it; (1) a flag
// hand-off between two CTAs: CTA 0 publishes k, CTA 1 answers k, per round trip.  Both spin with a bound.
namespace mks {
__device__ __forceinline__ unsigned long long probe_clock() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__global__ void __launch_bounds__(NTHREADS, 1) sync_probe_kernel(unsigned long long* words, float* data, long long* out, int iters, int mode, int stores) {
    const int tid = (int)threadIdx.x;
    if (tid >= NCT) return;
    const unsigned long long t0 = probe_clock();
    bool ok = true;
    if (mode == 0) {
        for (int k = 1; k <= iters && ok; k++) {
            for (int s = 0; s < stores; s++) __stcg(data + ((size_t)blockIdx.x * NCT + tid) * 4 + (s & 3), (float)k);
            consumer_sync();
            if (tid == 0) {
                asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(words), "l"(1ull) : "memory");
                const unsigned long long target = (unsigned long long)k * gridDim.x;
                unsigned long long v = 0;
                int spins = 0;
                do {
                    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(words) : "memory");
                } while (v < target && ++spins < 4000000);
                if (v < target) out[1] = k;                      // gave up: the host reports it
            }
            consumer_sync();
        }
    } else if (blockIdx.x < 2 && tid == 0) {
        unsigned long long* mine = words + 16 * blockIdx.x;      // separate 128-byte lines
        unsigned long long* theirs = words + 16 * (1 - blockIdx.x);
        for (unsigned long long k = 1; k <= (unsigned long long)iters && ok; k++) {
            if (blockIdx.x == 0) asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(theirs), "l"(k) : "memory");
            unsigned long long v = 0;
            int spins = 0;
            do {
                asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
            } while (v < k && ++spins < 4000000);
            if (v < k) {
                out[1] = (long long)k;
                ok = false;
            }
            if (blockIdx.x == 1) asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(theirs), "l"(k) : "memory");
        }
    }
    if (blockIdx.x == 0 && tid == 0) out[0] = (long long)(probe_clock() - t0);
}
}  // namespace mks

extern "C" int mk_sync_probe(int device, int mode, int iters, int stores, int64_t* ns_per_iter) {
    if (!ns_per_iter || iters < 1 || iters > 1000000 || mode < 0 || mode > 1 || stores < 0 || stores > 64)
        return sfail(MK_ERR_BADARG, "mk_sync_probe: bad argument");
    MKS_CUDA(cudaSetDevice(device));
    int n_sm = 0;
    MKS_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    unsigned long long* words = nullptr;
    float* data = nullptr;
    long long* out = nullptr;
    MKS_CUDA(cudaMalloc(&words, 512));
    MKS_CUDA(cudaMalloc(&data, (size_t)n_sm * NCT * 16));
    MKS_CUDA(cudaMalloc(&out, 64));
    cudaMemset(words, 0, 512);
    cudaMemset(out, 0, 64);
    const int grid = mode == 0 ? n_sm : 2;
    void* kargs[] = {&words, &data, &out, &iters, &mode, &stores};
    cudaError_t err = cudaLaunchCooperativeKernel((const void*)mks::sync_probe_kernel, dim3(grid), dim3(mks::NTHREADS), kargs, 0, nullptr);
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    long long host[2] = {0, 0};
    if (err == cudaSuccess) err = cudaMemcpy(host, out, 16, cudaMemcpyDeviceToHost);
    cudaFree(words);
    cudaFree(data);
    cudaFree(out);
    if (err != cudaSuccess) return sfail(MK_ERR_CUDA, "mk_sync_probe: %s", cudaGetErrorString(err));
    if (host[1] != 0) return sfail(MK_ERR_TIMEOUT, "mk_sync_probe: a wait ran out at iteration %lld", host[1]);
    *ns_per_iter = host[0] / iters;
    return MK_OK;
}

// ---- peer-visible memory ---------------------------------------------------------------------------------------
extern "C" int mk_peer_alloc(int device, int64_t bytes, uint64_t* ptr, uint8_t handle[64]) {
    if (!ptr || !handle || bytes < 1) return sfail(MK_ERR_BADARG, "mk_peer_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    MKS_CUDA(cudaSetDevice(device));
    void* p = nullptr;
    MKS_CUDA(cudaMalloc(&p, (size_t)bytes));
    MKS_CUDA(cudaMemset(p, 0, (size_t)bytes));
    cudaIpcMemHandle_t h;
    MKS_CUDA(cudaIpcGetMemHandle(&h, p));
    memcpy(handle, &h, 64);
    *ptr = reinterpret_cast<uint64_t>(p);
    return MK_OK;
}
extern "C" int mk_peer_open(int device, const uint8_t handle[64], uint64_t* ptr) {
    if (!ptr || !handle) return sfail(MK_ERR_BADARG, "mk_peer_open: bad argument");
    MKS_CUDA(cudaSetDevice(device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void* p = nullptr;
    MKS_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = reinterpret_cast<uint64_t>(p);
    return MK_OK;
}
extern "C" int mk_peer_close(uint64_t ptr) {
    if (ptr) MKS_CUDA(cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)));
    return MK_OK;
}
extern "C" int mk_peer_free(uint64_t ptr) {
    if (ptr) MKS_CUDA(cudaFree(reinterpret_cast<void*>(ptr)));
    return MK_OK;
}
