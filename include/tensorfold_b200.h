/* tensorfold_b200 — C ABI of the B200 (sm_100a) lane-verify kernels.
 *
 * Every entry point takes raw device pointers, plain sizes and the CUDA stream to launch on
 * (passed as void*; NULL is the legacy default stream). Nothing here allocates device memory: the
 * caller owns inputs, outputs and scratch. A call returns TF_OK after the launch was queued, or a
 * negative TF_E* code when an argument is unsupported (nothing was launched). A bounded
 * device-side wait that ran out is reported through the optional `status` word (int32 in device
 * memory, zero-initialised by the caller): the kernel writes TF_ESTALL there and still terminates.
 *
 * Each declaration names the function of the TensorFold reference (path inside that project) whose
 * job it takes over. Layout conventions: activations are row-major bf16, "rows" are the packed
 * (sequence, draft row) pairs of one verify window, and a row's result never depends on the other
 * rows of the call.
 */
#ifndef TENSORFOLD_B200_H
#define TENSORFOLD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TF_OK 0
#define TF_EINVAL (-1)   /* unsupported shape, size or flag */
#define TF_EALIGN (-2)   /* a pointer or stride is not aligned as required */
#define TF_ESCRATCH (-3) /* scratch buffer missing or too small */
#define TF_ECUDA (-4)    /* the CUDA runtime refused the launch */
#define TF_ESTALL (-5)   /* written to `status` by a kernel whose bounded wait ran out */

#define TF_QMM_MAX_ROWS 128
#define TF_QMM_F32_OUT 1 /* flags: write unrounded fp32 sums (a tensor-parallel rank's partial) */

/* Library/ABI version: major * 1000 + minor. */
int tf_version(void);

/* Number of persistent workers (CTAs) the matmul schedule is cut for. A compile-time constant of
 * the library (148 = B200 SM count), NOT queried from the device: the schedule fixes the order in
 * which K segments are summed, so it must not vary between machines or calls. */
int tf_qmm_workers(void);

/* ---- 4-bit group-affine lane matmul ---------------------------------------------------------
 * Replaces: families/qwen3_5/cuda/qmm.py:117-144 (lane_matmul), qmm_fast.py:115-140
 * (lane_matmul_tiled), families/qwen4_exp/cuda/qmm.py:246-285 (group-32 matmul), and the Metal
 * kernels/qwen/dense/v1/lane_qmm.py:284-335.
 *
 *   y[m, n] = round_bf16( sum over groups g in order of  s[n,g] * (x[m, g-block] . q[n, g-block])
 *                                                       + b[n,g] * xs[m,g] )
 *
 * x_packed: the M input rows (1..128) in packed form — per 64-input k tile, Mp = M rounded up to 4
 *          rows of 128 bytes, then the tile's group sums [64/group][Mp] fp32; tf_packed_bytes bytes,
 *          16-byte aligned. tf_pack_rows builds it from row-major bf16; the glue kernels below
 *          write it directly.
 * w_tiled: weights in this library's tile layout (tf_qmm_tiled_bytes / tf_qmm_tile below).
 * y  [M, N] bf16 (fp32 with TF_QMM_F32_OUT).  group is 64 or 32.  K a multiple of 64.
 * scratch: tf_qmm_scratch_bytes() bytes, 256-byte aligned; its first TF_QMM_COUNTER_BYTES bytes
 *          must be zero before the first call and are left zero by every call (the rest needs no
 *          initialisation). Calls that overlap on the GPU must not share scratch.
 */
#define TF_QMM_COUNTER_BYTES 16384
size_t tf_qmm_scratch_bytes(void);
size_t tf_packed_bytes(int M, int K, int group);
int tf_qmm(const void* x_packed, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M, int N,
           int K, int group, int flags, int* status, void* stream);

/* Row-major bf16 rows x [M, K] -> packed rows with their group sums; when xs is not NULL the sums
 * are also written as [M, K/group] fp32. A group's sum is formed in eights: eight (group 64) or four
 * (group 32) sequential 8-element sums combined by a pairwise tree.
 * Replaces: families/qwen3_5/cuda/qmm.py:49-59,106-114 (group_sums); lane_qmm.py:50-58 (xsum). */
int tf_pack_rows(const void* x, void* x_packed, void* xs, int M, int K, int group, void* stream);

/* Size in bytes of the tiled form of an [N, K] 4-bit weight with the given group size. */
size_t tf_qmm_tiled_bytes(int N, int K, int group);

/* Relayout (device to device, one launch): MLX-stored words [N, K/8] uint32 (element i of a row at
 * bits 4*(i%8) of word i/8) plus bf16 scales and biases [N, K/group] -> tiled buffer, and back.
 * Replaces: families/qwen3_5/cuda/qmm_fast.py:80-93 (tile_weight, group_major) and :149-156
 * (untile); kernels/qwen/dense/v1/lane_qmm.py:254-271 (pack_scales, tile_weight, untile_weight).
 * Same bits, different order; columns beyond N inside the last 16-column tile are zero. */
int tf_qmm_tile(const void* words, const void* scales, const void* biases, void* w_tiled, int N, int K, int group,
                void* stream);
int tf_qmm_untile(const void* w_tiled, void* words, void* scales, void* biases, int N, int K, int group,
                  void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TENSORFOLD_B200_H */
