// Block-scaled tcgen05 GEMV for MXFP4 weights (declarations and the packed layout: include/mk_umma.h).
//
// One persistent CTA per SM, 16 warps.  All of them stage the input digit planes; then
//   warp 4, 8 lanes:  producers.  They stream this CTA's chunks (8704 bytes: 128 rows x 128 columns of e2m1 pairs and
//                     their scale atom) into a shared-memory ring with cp.async.bulk.
//   warp 5, one lane: issuer.  Per chunk: tcgen05.cp of the scale atom into tensor memory, two tcgen05.mma
//                     (kind::mxf4, block scaled, M = 128, N = pieces x sequences rounded up to 8, K = 64), tcgen05.commit onto the
//                     slot's `empty` barrier; after the last chunk of a row block a commit onto `d_full`.
//   warps 0-3:        epilogue.  tcgen05.ld of the 128 x N accumulators (lane = row), sum over the digit
//                     planes, then either the final store or a partial tile plus a counter; the CTA that
//                     arrives last adds the partial tiles in a fixed order.
// The chunks of one K slice are dealt to the slice's CTAs as equal contiguous ranges, so a row block can be
// shared by two or three CTAs; which ones, and in which order their partial tiles are added, follows from the
// shape alone.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/mk_b200.h"
#include "../../include/mk_umma.h"

int mk_set_error(int code, const char* text);

namespace mku {

constexpr int NT = 512;
constexpr int CHUNK_DATA = 8192;
constexpr int D_COLS = 64;                  // columns of one accumulator buffer (N <= 64)
constexpr int T_D = 0, T_SFA = 128, T_SFB = 256;
constexpr int N_PRODUCERS = 8;
constexpr int MAX_DEPTH = 24;               // ring slots (SFA columns: 4 per slot, T_SFA + 96 <= T_SFB)
constexpr unsigned W_FULL = 201, W_EMPTY = 202, W_DFULL = 203, W_DEMPTY = 204, W_DRAIN = 205;

struct Args {
    const uint8_t* w;
    const float* x;
    float* out;
    float* part;
    unsigned* cnt;
    unsigned* status;
    unsigned long long* prof;
    long long spin_limit_ns;
    int rows, k, batch, pieces, splits, round_bf16;
    int row_blocks, cps, ks, n, depth, amax, mp;       // mp: rows of the B operand per digit plane (1, 2, 4, 8 >= batch)
};

struct Bars {
    unsigned long long full[MAX_DEPTH], empty[MAX_DEPTH], d_full[2], d_empty[2];
    uint32_t tmem;
    int dead;
    int last;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(unsigned long long* b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ bool mbar_try(unsigned long long* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
// Every wait ends: by the barrier, by another role's failure, or by the clock (the code then lands in status).
__device__ __noinline__ bool mbar_wait(Bars& B, const Args& A, unsigned long long* b, uint32_t parity, unsigned code) {
    unsigned long long t0 = 0;
    for (unsigned it = 0;; it++) {
        if (mbar_try(b, parity)) return true;
        if ((it & 255u) == 255u) {
            if (*(volatile int*)&B.dead) return false;
            const unsigned long long now = gtime();
            if (!t0) t0 = now;
            if (now - t0 > (unsigned long long)A.spin_limit_ns) {
                *(volatile int*)&B.dead = 1;
                if (atomicCAS(A.status, 0u, code) == 0u) {
                    A.status[1] = blockIdx.x;
                    A.status[2] = parity;
                }
                return false;
            }
        }
    }
}
// shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices, `lbo` bytes between
// neighbours along K, `sbo` bytes between neighbours along the rows
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}

// This CTA's slice and chunk range.  CTAs c with c % splits == s work on slice s; the j-th of the G of them
// takes chunks [j T / G, (j + 1) T / G) of the slice's T = row_blocks * cps chunks (row-block major).
struct Share {
    int s, j, G;
    long long T, lo, hi;
};
// members of slice s's group that get work: never more than there are chunks, so every member's range is non-empty
__host__ __device__ inline int group_size(int grid, int splits, int s, long long T) {
    const long long g = (grid - s + splits - 1) / splits;
    return (int)(g < T ? g : T);
}
__host__ __device__ inline Share share_of(int cta, int grid, int splits, int row_blocks, int cps) {
    Share h;
    h.s = cta % splits;
    h.j = cta / splits;
    h.T = (long long)row_blocks * cps;
    h.G = group_size(grid, splits, h.s, h.T);
    h.lo = h.j < h.G ? h.j * h.T / h.G : 0;
    h.hi = h.j < h.G ? (h.j + 1) * h.T / h.G : 0;
    return h;
}
// the member of a slice's group that owns chunk q
__host__ __device__ inline int owner(long long q, int G, long long T) { return (int)(((q + 1) * G - 1) / T); }
// arrivals at row block rb, and the arrival slot of (slice s, member j)
__host__ __device__ inline int arrivals(int rb, int grid, int splits, int cps, long long T, int s, int j, int* slot) {
    int total = 0;
    for (int t = 0; t < splits; t++) {
        const int G = group_size(grid, splits, t, T);
        const int jl = owner((long long)rb * cps, G, T), jh = owner((long long)(rb + 1) * cps - 1, G, T);
        if (t == s && slot) *slot = total + (j - jl);
        total += jh - jl + 1;
    }
    return total;
}

// ---- input digit planes ------------------------------------------------------------------------------------------
// Four neighbouring lanes take one sequence's 32-column block, eight values each: q = round(|x| 2^(2P - 1 - e)) with
// e the exponent of the block's largest value, digit p = (q >> 2p) & 3 stored as the e2m1 code of digit / 2 (codes
// 0..3 are 0, 0.5, 1, 1.5) with block scale 2^(e + 2 - 2P + 2p).  Plane p of sequence m is row p * mp + m of the B operand.
__device__ void stage_planes(const Args& A, uint8_t* xs, uint8_t* sfb, int slice) {
    const int P = A.pieces, nblk = A.ks / 32;
    for (int i = threadIdx.x * 16; i < A.n * A.ks / 2; i += NT * 16) *reinterpret_cast<uint4*>(xs + i) = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x * 16; i < A.cps * 512; i += NT * 16) *reinterpret_cast<uint4*>(sfb + i) = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
    __syncthreads();
    const int items = A.batch * nblk * 4;                          // a multiple of 4: the four lanes of a block stay together
    for (int it0 = 0; it0 < items; it0 += NT) {
        const int it = it0 + (int)threadIdx.x;
        const bool live = it < items;
        const int b = live ? it >> 2 : 0, quarter = it & 3;
        const int m = b / nblk, kb = b % nblk;
        float v[8];
        if (live) {
            const float4* src = reinterpret_cast<const float4*>(A.x + (size_t)m * A.k + (size_t)slice * A.ks + (size_t)kb * 32 + quarter * 8);
            const float4 f0 = __ldg(src), f1 = __ldg(src + 1);
            v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w; v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = 0.f;
        }
        float mx = 0.f;
        uint32_t sign = 0;                                         // bit 3 of every nibble of a negative value
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (A.round_bf16) v[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
            sign |= (v[i] < 0.f ? 8u : 0u) << (4 * i);
            v[i] = fabsf(v[i]);
            mx = fmaxf(mx, v[i]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const int e = (int)(__float_as_uint(mx) >> 23) - 127;
        if (!live || !(mx > 0.f) || e < -100 || e > 100) continue;  // a zero block stays zero (no shuffle follows)
        const float up = __uint_as_float((uint32_t)(127 + 2 * P - 1 - e) << 23);
        const uint32_t qmax = (1u << (2 * P)) - 1u;
        // word i: the eight values' digit p in nibble p (two-bit digits spread to nibbles), the sign in every nibble
        uint32_t y[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t x = min(__float2uint_rn(v[i] * up), qmax);
            x = (x | (x << 8)) & 0x00FF00FFu;
            x = (x | (x << 4)) & 0x0F0F0F0Fu;
            x = (x | (x << 2)) & 0x33333333u;
            y[i] = x | ((sign >> (4 * i + 3)) & 1u ? 0x88888888u : 0u);
        }
        // 8 x 8 nibble transpose: afterwards word p holds plane p's eight nibbles, value i in nibble i
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t lo = __byte_perm(y[i], y[i + 4], 0x5410), hi = __byte_perm(y[i], y[i + 4], 0x7632);
            y[i] = lo;
            y[i + 4] = hi;
        }
#pragma unroll
        for (int i = 0; i < 8; i += 4)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const uint32_t lo = __byte_perm(y[i + j], y[i + j + 2], 0x6240), hi = __byte_perm(y[i + j], y[i + j + 2], 0x7351);
                y[i + j] = lo;
                y[i + j + 2] = hi;
            }
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const uint32_t lo = (y[i] & 0x0F0F0F0Fu) | ((y[i + 1] & 0x0F0F0F0Fu) << 4);
            const uint32_t hi = ((y[i] >> 4) & 0x0F0F0F0Fu) | (y[i + 1] & 0xF0F0F0F0u);
            y[i] = lo;
            y[i + 1] = hi;
        }
#pragma unroll
        for (int p = 0; p < 8; p++)
            if (p < P) {
                const int n = p * A.mp + m;
                *reinterpret_cast<uint32_t*>(xs + ((size_t)(n >> 3) * nblk + kb) * 128 + (n & 7) * 16 + quarter * 4) = y[p];
                if (quarter == 0) sfb[(kb >> 2) * 512 + (n & 31) * 16 + (n >> 5) * 4 + (kb & 3)] = (uint8_t)(127 + e + 2 - 2 * P + 2 * p);
            }
    }
}

__global__ void __launch_bounds__(NT, 1) gemv_kernel(const Args A) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int xbytes = A.n * A.ks / 2;
    uint8_t* xs = smem;
    uint8_t* sfb = xs + xbytes;
    uint8_t* ring = sfb + A.cps * 512;
    Bars& B = *reinterpret_cast<Bars*>(ring + (size_t)A.depth * MKU_CHUNK_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Share sh = share_of(blockIdx.x, gridDim.x, A.splits, A.row_blocks, A.cps);
    unsigned long long* prof = A.prof ? A.prof + (size_t)blockIdx.x * 8 : nullptr;
    if (prof && threadIdx.x == 0) prof[0] = gtime();

    if (threadIdx.x == 0) {
        for (int i = 0; i < A.depth; i++) {
            mbar_init(&B.full[i], 1);
            mbar_init(&B.empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&B.d_full[i], 1);
            mbar_init(&B.d_empty[i], 4);
        }
        B.dead = 0;
        B.last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&B.tmem)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    stage_planes(A, xs, sfb, sh.s);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tbase = B.tmem;
    const int nchunks = (int)(sh.hi - sh.lo);
    if (prof && threadIdx.x == 0) prof[1] = gtime();

    if (warp == 4 && lane < min(N_PRODUCERS, A.depth)) {
        // ---- producers: lane l of np brings chunks l, l + np, ...  (32-bit counters that step: a 64-bit division per
        // chunk in a lone thread costs more than the chunk's copy).  np <= depth: a lane that has passed the wait for
        // chunk i - np knows that chunk i - np - depth >= i - 2 depth is consumed, so the parity it waits for next
        // cannot be mistaken for the one two uses of the slot back. ----
        const int np = min(N_PRODUCERS, A.depth);
        const uint8_t* src = A.w + ((size_t)sh.s * sh.T + (size_t)sh.lo) * MKU_CHUNK_BYTES;
        unsigned long long policy;                                   // every weight byte is read once per launch
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
        int i = lane, slot = lane;
        uint32_t phase = 0;
        for (; i < nchunks; i += np) {
            if (!mbar_try(&B.empty[slot], phase ^ 1u) && !mbar_wait(B, A, &B.empty[slot], phase ^ 1u, W_EMPTY)) break;
            const uint32_t bar = smem_u32(&B.full[slot]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(MKU_CHUNK_BYTES) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                         ::"r"(smem_u32(ring + (size_t)slot * MKU_CHUNK_BYTES)), "l"(src + (size_t)i * MKU_CHUNK_BYTES), "r"(MKU_CHUNK_BYTES), "r"(bar), "l"(policy) : "memory");
            slot += np;
            while (slot >= A.depth) {
                slot -= A.depth;
                phase ^= 1u;
            }
        }
        if (*(volatile int*)&B.dead) {
            // a role gave up: this lane's copies still in flight must land before the CTA leaves
            for (int c = i - np, n = 0; c >= 0 && n < A.depth; c -= np, n++) {
                const unsigned long long t0 = gtime();
                while (!mbar_try(&B.full[c % A.depth], (uint32_t)((c / A.depth) & 1)) && gtime() - t0 < 1000000ull) {}
            }
        }
    } else if (warp == 5 && lane == 0) {
        // ---- issuer ----
        // the input planes' scales: one atom per 128 columns of the slice, kept in tensor memory for the whole launch
        for (int i = 0; i < A.cps; i++) {
            const uint64_t d = smem_desc(smem_u32(sfb + i * 512), 128, 128);
            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tbase + T_SFB + 4 * i), "l"(d) : "memory");
        }
        // e2m1 x e2m1, e8m0 scales, M = 128, N = A.n
        const uint32_t idesc0 = (1u << 7) | (1u << 10) | ((uint32_t)(A.n >> 3) << 17) | (1u << 23) | (8u << 24);
        const uint32_t xsbo = (uint32_t)(A.ks / 32) * 128;
        const uint64_t xdesc0 = smem_desc(smem_u32(xs), 128, xsbo);
        // The loop below is this thread's whole budget: the tensor pipe takes one 128 x 64 tile of weights per ~130
        // cycles whatever N is, and everything else this thread does per chunk adds to that.  So: loop state in
        // registers, stepping counters, and the barrier's fast path inline.
        const int depth = A.depth, cps = A.cps;
        const uint32_t ring0 = smem_u32(ring), tsfa0 = tbase + T_SFA, tsfb0 = tbase + T_SFB;
        int unit = 0, slot = 0, kc = (int)(sh.lo % A.cps);
        uint32_t phase = 0, sbase = ring0;
        uint64_t db = xdesc0 + (uint64_t)(kc * 32);                // 4 core matrices x 128 bytes per chunk, in 16-byte units
        bool alive = true;
        for (int i = 0; i < nchunks && alive; unit++) {
            const int buf = unit & 1;
            if (!mbar_wait(B, A, &B.d_empty[buf], (uint32_t)((unit >> 1) & 1) ^ 1u, W_DEMPTY)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t td = tbase + T_D + buf * D_COLS;
            uint32_t accumulate = 0;
            // the chunks of this row block that are ours: up to the block's last column chunk or the end of the range
            for (; i < nchunks;) {
                if (!mbar_try(&B.full[slot], phase) && !mbar_wait(B, A, &B.full[slot], phase, W_FULL)) {
                    alive = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (prof && i == 0) prof[2] = gtime();
                const uint32_t tsfa = tsfa0 + 4 * slot, tsfb = tsfb0 + 4 * kc;
                asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tsfa), "l"(smem_desc(sbase + CHUNK_DATA, 128, 128)));
                const uint64_t da = smem_desc(sbase, 128, 512);
                // two MMAs of K = 64: 256 bytes further along K in both operands, scale bytes 0-1 then 2-3
                asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                             " tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
                             ::"r"(td), "l"(da), "l"(db), "r"(idesc0), "r"(accumulate), "r"(tsfa), "r"(tsfb));
                asm volatile("tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], 1;\n"
                             ::"r"(td), "l"(da + 16), "l"(db + 16), "r"(idesc0 | (2u << 4) | (2u << 29)), "r"(tsfa), "r"(tsfb));
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&B.empty[slot])) : "memory");
                accumulate = 1;
                i++;
                sbase += MKU_CHUNK_BYTES;
                if (++slot == depth) {
                    slot = 0;
                    phase ^= 1u;
                    sbase = ring0;
                }
                db += 32;
                if (++kc == cps) {
                    kc = 0;
                    db = xdesc0;
                    break;
                }
            }
            if (!alive) break;
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&B.d_full[buf])) : "memory");
        }
        if (prof) prof[3] = gtime();
    } else if (warp < 4) {
        // ---- epilogue: thread = row of the block ----
        const int row = warp * 32 + lane;
        int unit = 0;
        for (long long q = sh.lo; q < sh.hi; unit++) {
            const int rb = (int)(q / A.cps);
            const long long qend = min(sh.hi, (long long)(rb + 1) * A.cps);
            const int buf = unit & 1;
            // the four warps leave together: a wait that ran out marks the CTA dead, and everybody reads the mark
            // behind a barrier that all of them reach
            mbar_wait(B, A, &B.d_full[buf], (uint32_t)((unit >> 1) & 1), W_DFULL);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*(volatile int*)&B.dead) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (prof && threadIdx.x == 0 && qend == sh.hi) prof[4] = gtime();
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const uint32_t td = tbase + T_D + buf * D_COLS + ((uint32_t)(warp * 32) << 16);
            // column n = plane * mp + sequence; the planes are added least significant first
            for (int c = 0; c < A.n; c += 8) {
                uint32_t r[8];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(td + c));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (A.mp == 8) {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] += __uint_as_float(r[j]);
                } else if (A.mp == 4) {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j & 3] += __uint_as_float(r[j]);
                } else if (A.mp == 2) {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j & 1] += __uint_as_float(r[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[0] += __uint_as_float(r[j]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&B.d_empty[buf]);
            int slot = 0;
            const int total = arrivals(rb, gridDim.x, A.splits, A.cps, sh.T, sh.s, sh.j, &slot);
            const int grow = rb * MKU_ROWS + row;
            if (total == 1) {
                if (grow < A.rows)
                    for (int m = 0; m < A.batch; m++) A.out[(size_t)m * A.rows + grow] = v[m];
            } else {
                float* mine = A.part + (((size_t)rb * A.amax + slot) * 8) * MKU_ROWS + row;
#pragma unroll
                for (int m = 0; m < 8; m++) __stcg(mine + m * MKU_ROWS, v[m]);
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 0) {
                    const unsigned old = atomicAdd(A.cnt + rb, 1u);
                    const int last = old + 1u == (unsigned)total;
                    if (last) A.cnt[rb] = 0u;
                    B.last = last;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int last = *(volatile int*)&B.last;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (last) {
                    __threadfence();
                    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    for (int a = 0; a < total; a++) {
                        const float* src = A.part + (((size_t)rb * A.amax + a) * 8) * MKU_ROWS + row;
#pragma unroll
                        for (int m = 0; m < 8; m++) s[m] += __ldcg(src + m * MKU_ROWS);
                    }
                    if (grow < A.rows)
                        for (int m = 0; m < A.batch; m++) A.out[(size_t)m * A.rows + grow] = s[m];
                }
            }
            q = qend;
        }
    }
    if (prof && threadIdx.x == 0) prof[5] = gtime();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(512));
}

static int ufail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    return mk_set_error(code, buf);
}

static int resolve_grid(int device, int grid, int* out) {
    if (grid > 0) {
        *out = grid;
        return MK_OK;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 1)
        return ufail(MK_ERR_CUDA, "mk_umma: cannot read the SM count of device %d", device);
    *out = sms;
    return MK_OK;
}

static int max_arrivals(int row_blocks, int cps, int splits, int grid) {
    int amax = 1;
    const long long T = (long long)row_blocks * cps;
    for (int rb = 0; rb < row_blocks; rb++) {
        const int a = arrivals(rb, grid, splits, cps, T, 0, 0, nullptr);
        amax = a > amax ? a : amax;
    }
    return amax;
}

static int check_shape(int rows, int k, int batch, int splits) {
    if (rows < 1 || k < 1) return ufail(MK_ERR_BADARG, "mk_umma: rows %d, k %d", rows, k);
    if (batch < 1 || batch > 8) return ufail(MK_ERR_BADARG, "mk_umma: batch %d out of [1, 8]", batch);
    if (splits < 1 || splits > MKU_MAX_SPLITS || k % splits) return ufail(MK_ERR_BADARG, "mk_umma: %d splits of k = %d", splits, k);
    const int ks = k / splits;
    if (ks % MKU_CHUNK_K || ks > MKU_MAX_SLICE_K)
        return ufail(MK_ERR_BADARG, "mk_umma: %d columns per split (a multiple of %d, at most %d)", ks, MKU_CHUNK_K, MKU_MAX_SLICE_K);
    if ((long long)((rows + MKU_ROWS - 1) / MKU_ROWS) * (ks / MKU_CHUNK_K) >= (1ll << 30))
        return ufail(MK_ERR_BADARG, "mk_umma: more than 2^30 chunks per split");
    return MK_OK;
}

}  // namespace mku

extern "C" int64_t mk_umma_scratch_bytes(int rows, int k, int batch, int splits, int device, int grid) {
    if (mku::check_shape(rows, k, batch, splits) != MK_OK) return MK_ERR_BADARG;
    int g = 0;
    if (mku::resolve_grid(device, grid, &g) != MK_OK) return MK_ERR_CUDA;
    if (g < splits) return mku::ufail(MK_ERR_BADARG, "mk_umma: %d CTAs for %d splits", g, splits);
    const int rbs = (rows + MKU_ROWS - 1) / MKU_ROWS;
    return (int64_t)rbs * mku::max_arrivals(rbs, k / splits / MKU_CHUNK_K, splits, g) * 8 * MKU_ROWS * 4;
}

extern "C" int mk_umma_gemv(const mk_umma_args* a) {
    using namespace mku;
    if (!a) return ufail(MK_ERR_BADARG, "mk_umma_gemv: null arguments");
    const int rc = check_shape(a->rows, a->k, a->batch, a->splits);
    if (rc != MK_OK) return rc;
    if (a->pieces < 4 || a->pieces > 8) return ufail(MK_ERR_BADARG, "mk_umma_gemv: %d digit planes (4..8)", a->pieces);
    if (!a->w || !a->x || !a->out || !a->cnt || !a->status) return ufail(MK_ERR_BADARG, "mk_umma_gemv: a buffer is missing");
    if ((a->w | a->x | a->out) & 15) return ufail(MK_ERR_BADARG, "mk_umma_gemv: w, x and out must be 16-byte aligned");
    if (a->k % 4) return ufail(MK_ERR_BADARG, "mk_umma_gemv: k must be a multiple of 4");
    int grid = 0;
    if (resolve_grid(a->device, a->grid, &grid) != MK_OK) return MK_ERR_CUDA;
    if (grid < a->splits) return ufail(MK_ERR_BADARG, "mk_umma_gemv: %d CTAs for %d splits", grid, a->splits);
    Args A;
    A.w = reinterpret_cast<const uint8_t*>(a->w);
    A.x = reinterpret_cast<const float*>(a->x);
    A.out = reinterpret_cast<float*>(a->out);
    A.part = reinterpret_cast<float*>(a->part);
    A.cnt = reinterpret_cast<unsigned*>(a->cnt);
    A.status = reinterpret_cast<unsigned*>(a->status);
    A.prof = reinterpret_cast<unsigned long long*>(a->prof);
    A.spin_limit_ns = a->spin_limit_ns > 0 ? a->spin_limit_ns : 2000000000ll;
    A.rows = a->rows; A.k = a->k; A.batch = a->batch; A.pieces = a->pieces; A.splits = a->splits;
    A.round_bf16 = a->round_bf16;
    A.row_blocks = (a->rows + MKU_ROWS - 1) / MKU_ROWS;
    A.ks = a->k / a->splits;
    A.cps = A.ks / MKU_CHUNK_K;
    A.mp = a->batch > 4 ? 8 : (a->batch > 2 ? 4 : a->batch);
    A.n = (a->pieces * A.mp + 7) / 8 * 8;
    A.amax = max_arrivals(A.row_blocks, A.cps, a->splits, grid);
    if (A.amax > 1 && !a->part) return ufail(MK_ERR_BADARG, "mk_umma_gemv: row blocks are shared by up to %d CTAs and there is no scratch", A.amax);
    if (cudaSetDevice(a->device) != cudaSuccess) return ufail(MK_ERR_CUDA, "mk_umma_gemv: cudaSetDevice(%d) failed", a->device);
    int smem_max = 0;
    cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, a->device);
    const int fixed = A.n * A.ks / 2 + A.cps * 512 + (int)sizeof(Bars) + 128;
    int depth = (smem_max - fixed) / MKU_CHUNK_BYTES;
    depth = depth > MAX_DEPTH ? MAX_DEPTH : depth;
    if (depth < 2) return ufail(MK_ERR_BADARG, "mk_umma_gemv: %d planes x %d columns leave no room for the weight ring", A.n, A.ks);
    A.depth = depth;
    const int smem = fixed + depth * MKU_CHUNK_BYTES;
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return ufail(MK_ERR_CUDA, "mk_umma_gemv: %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    gemv_kernel<<<grid, NT, smem, reinterpret_cast<cudaStream_t>(a->stream)>>>(A);
    e = cudaGetLastError();
    if (e != cudaSuccess) return ufail(MK_ERR_CUDA, "mk_umma_gemv: launch failed: %s", cudaGetErrorString(e));
    return MK_OK;
}
