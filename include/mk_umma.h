/* mk_umma.h -- C ABI of the block-scaled tcgen05 GEMV for MXFP4 weights on B200 (sm_100a).
 *
 * out[m][r] = sum_k W[r][k] * x[m][k] for m < batch <= 8 sequences, W in MXFP4 (e2m1 values, one e8m0 scale per
 * 32 columns of a row: the format of the reference's 27B engine, qwen3.8-27b-gfx942/mk/reference.py:40-83
 * `dequant_mxfp4`, consumed there by the scalar GEMV of common/mkcore/gemv.py:48-52).  Here the weights are the
 * 128-row A operand of `tcgen05.mma.kind::mxf4.block_scale`: they go from HBM to shared memory by bulk copies and
 * from there into the tensor core without passing through registers; the accumulators live in tensor memory.
 * The inputs are the B operand: every sequence's x (rounded to bf16 as the reference decoders do) is split into
 * `pieces` base-4 digits relative to the largest value of its 32-column block, each digit plane an e2m1 row with
 * its own e8m0 block scale, so the products are exact and the sum over the planes restores x to 2 * pieces bits
 * below the block's largest value.
 *
 * Conventions as in mk_b200.h: the caller owns every device buffer and passes raw addresses, every function
 * returns MK_OK or a negative MK_ERR_*, mk_last_error() has the text, every device-side wait is bounded.
 */
#ifndef MK_UMMA_H
#define MK_UMMA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    MKU_ROWS = 128,            /* rows of one weight block (the M of the MMA)                                  */
    MKU_CHUNK_K = 128,         /* columns of one streamed chunk (two MMAs of K = 64)                           */
    MKU_CHUNK_BYTES = 8704,    /* 8192 bytes of e2m1 pairs + one 512-byte scale atom                           */
    MKU_MAX_SLICE_K = 5120,    /* columns one CTA keeps staged (k / splits)                                    */
    MKU_MAX_SPLITS = 8
};

/* Packed weights: [splits][row_blocks][chunks_per_split] chunks of MKU_CHUNK_BYTES, row_blocks = ceil(rows / 128),
 * chunks_per_split = k / splits / 128.  One chunk = 128 rows x 128 columns:
 *   bytes [0, 8192): [row / 8][column / 32][row % 8][16 bytes = 32 e2m1 values, even column in the low nibble]
 *                    (the canonical K-major shared-memory layout of the MMA, no swizzle);
 *   bytes [8192, 8704): e8m0 scales, byte (row % 32) * 16 + (row / 32) * 4 + (column / 32).
 * Rows beyond `rows` are zero. */
typedef struct {
    uint64_t w;            /* packed weights (16-byte aligned)                                                 */
    uint64_t x;            /* fp32 [batch][k]                                                                  */
    uint64_t out;          /* fp32 [batch][rows]                                                               */
    uint64_t part;         /* fp32 scratch, mk_umma_scratch_bytes() bytes (unused when no row block is shared) */
    uint64_t cnt;          /* uint32 [row_blocks], zero before the first call (the kernel leaves it zero)      */
    uint64_t status;       /* uint32 [4]: [0] = 0 or a wait code, [1] = CTA, [2] = detail                      */
    uint64_t stream;       /* cudaStream_t or 0                                                                */
    uint64_t prof;         /* 0, or uint64 [grid][8] globaltimer stamps: start, planes staged, first chunk landed,
                              last MMA issued, last accumulator complete, epilogue done                        */
    int64_t spin_limit_ns; /* bound of every device-side wait; 0 = 2 s                                         */
    int32_t rows, k, batch, pieces;   /* pieces: 4..8 digit planes per input value                             */
    int32_t splits, device, round_bf16, grid;   /* grid: CTAs (0 = one per SM)                                 */
} mk_umma_args;

/* Bytes of `part` that mk_umma_gemv needs for this shape on `grid` CTAs (0 = one per SM of `device`). */
int64_t mk_umma_scratch_bytes(int rows, int k, int batch, int splits, int device, int grid);

/* One launch.  MK_ERR_BADARG for shapes the kernel cannot hold (k / splits not a multiple of 128 or above
 * MKU_MAX_SLICE_K, batch outside 1..8, pieces outside 4..8), MK_ERR_CUDA for launch failures.  The call returns
 * after the launch; status is read by the caller after synchronising (nonzero [0]: a wait ran out). */
int mk_umma_gemv(const mk_umma_args* args);

#ifdef __cplusplus
}
#endif
#endif
