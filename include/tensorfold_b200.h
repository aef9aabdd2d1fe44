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
 * x_packed: the M input rows (1..128) in packed form: per 64-input k tile, Mp rows of 128 bytes (Mp = M
 *          rounded up to its bucket 8, 16, 32, 64 or 128; rows past M zero; 16-byte chunk c of row r
 *          stored at chunk c ^ 4*(r&1)), then the tile's group sums [64/group][Mp] fp32;
 *          tf_packed_bytes bytes, 16-byte aligned. tf_pack_rows builds it from row-major bf16; the glue
 *          kernels below write it directly.
 * w_tiled: weights in this library's tile layout (tf_qmm_tiled_bytes / tf_qmm_tile below).
 * y  [M, N] bf16 (fp32 with TF_QMM_F32_OUT).  group is 64 or 32.  K a multiple of 64.
 * scratch: tf_qmm_scratch_bytes() bytes, 256-byte aligned, all zero before the first call; afterwards
 *          it belongs to the library (it holds parked K segments, their ready tags and a launch number
 *          per worker that every call advances). Calls that overlap on the GPU must not share scratch;
 *          calls on one stream, programmatic dependent launches included, may.
 */
#define TF_QMM_COUNTER_BYTES 16384
size_t tf_qmm_scratch_bytes(void);
size_t tf_packed_bytes(int M, int K, int group);
int tf_qmm(const void* x_packed, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M, int N,
           int K, int group, int flags, int* status, void* stream);

/* tf_qmm with a hint: next_w_tiled (may be NULL) is the tiled weight [next_N, next_K] of the matmul that the
 * caller launches next on this stream. Once a worker has issued all of its own copies it asks L2 for the
 * first bytes the same worker of that launch will stream, so the next matmul starts from L2 while this
 * one finishes and the kernels between them run. Only a hint: results never depend on it. */
int tf_qmm_next(const void* x_packed, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M, int N,
                int K, int group, int flags, const void* next_w_tiled, int next_N, int next_K, int next_group, int* status,
                void* stream);

/* Profiling aid, no counterpart in the reference: with `stamps` not NULL (zeroed device memory of
 * (148 + 512 * 148 * 16) uint64: a launch counter per worker, then a ring of the last 512 launches) every
 * later tf_qmm / tf_qmm_grouped launch on the current device writes %globaltimer values per worker CTA:
 * slot 0 kernel entry, 1 first weight copy issued, 2 predecessor's memory visible, 3 first stage ready,
 * 4 main loop done, 5 first segment parked, 6 later segments added, 7 last copy issued, 9 last output
 * written; NULL switches it off. */
int tf_qmm_set_trace(void* stamps);

/* Grouped form for mixture-of-experts layers: up to max_probs independent problems of 8 rows each in
 * one launch. Problem p multiplies its packed rows (x_packed + p * tf_packed_bytes(8, K, group)) with
 * weight slot prob_expert[p] (w_tiled + slot * tf_qmm_tiled_bytes(N, K, group): the experts' tiled
 * weights stacked) into y + p * 8 * N elements. The number of live problems is read on the device from
 * prob_count[0] (clamped to max_probs), so a captured step serves any routing. With prob_sel not NULL
 * the launch covers problems prob_sel[0 .. prob_count[0]) only (an expert-parallel rank's own
 * experts), still addressed by their own index p. A row's result is that of tf_qmm on the same row and
 * weight: the arithmetic is the 8-row bucket's always.
 * Replaces: families/qwen4_exp/cuda/qmm.py:421-602 (Experts, Group, moe_gateup, moe_down). */
int tf_qmm_grouped(const void* x_packed, const void* w_tiled, const int* prob_expert, const int* prob_count,
                   const int* prob_sel, int max_probs, void* y, void* scratch, size_t scratch_bytes, int N, int K, int group,
                   int flags, int* status, void* stream);

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


/* ---- wide-row 4-bit matmul on tcgen05 tensor cores -------------------------------------------
 * No counterpart in the reference: its prompt prefill and its many-row verify windows go through the
 * same lane kernels in chains of up to 128 rows (families/qwen3_5/cuda/decode.py:34-60,
 * qmm_fast.py:108-140). This kernel is this library's own wide-row path: 32..128 rows per launch on
 * tcgen05.mma with the accumulators in tensor memory.
 *
 * Same formula as tf_qmm, different arithmetic, hence different bits: the 4-bit codes are dequantised
 * to bf16 weights bf16(s * q + b) (one fused multiply-add, one rounding) and multiplied with the bf16
 * activations by tcgen05.mma kind::f16 into fp32 accumulators (M = 128 output columns, N = the row
 * bucket 32/64/128, K = 16); K segments are added in k order and rounded once. Results are within the
 * bf16 bound of tf_qmm's and do not depend on the number of rows in the call; an engine must run all
 * its steps (serial and windowed) through one of the two kernels, never a mixture.
 *
 * x_packed: tf_packed_tc_bytes bytes from tf_pack_rows_tc (row-major bf16 rows; xs is ignored and may
 * be NULL) or from tf_repack_tc (the lane kernel's packed rows, as every glue kernel writes them);
 * w_tiled: tf_qmm_tc_tiled_bytes bytes from tf_qmm_tc_tile (a different order from tf_qmm_tile's).
 * scratch as for tf_qmm. M is 1..128 per launch. */
size_t tf_packed_tc_bytes(int M, int K, int group);
size_t tf_qmm_tc_tiled_bytes(int N, int K, int group);
int tf_qmm_tc(const void* x_packed, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M, int N,
              int K, int group, int flags, int* status, void* stream);
int tf_pack_rows_tc(const void* x, void* x_packed, void* xs, int M, int K, int group, void* stream);
int tf_repack_tc(const void* lane_packed, void* x_packed, int M, int K, int group, void* stream);
/* Profiling hook (no reference counterpart): with a device buffer of 148 * 16 64-bit words set, the latest
 * tf_qmm_tc launch writes 16 globaltimer stamps (ns) per worker (roles' milestones); NULL switches it off. */
int tf_qmm_tc_set_trace(void* stamps);
int tf_qmm_tc_tile(const void* words, const void* scales, const void* biases, void* w_tiled, int N, int K, int group,
                   void* stream);
int tf_qmm_tc_untile(const void* w_tiled, void* words, void* scales, void* biases, int N, int K, int group,
                     void* stream);


/* ---- glue: the steps between two matmuls ----------------------------------------------------
 * Each writes the next matmul's input in packed form (group sums included) when given a packed
 * output, and/or plain row-major bf16. M is 1..128 rows. Strides are in elements. */

/* h = bf16(x + r) where r is a bf16 row set (`residual`) or the rank-ordered sum, rounded once to
 * bf16, of `nparts` fp32 partial row sets `partials + p * part_stride` (a row-parallel projection's
 * per-rank outputs); y = bf16(h * rsqrt(mean(h^2) + eps) * weight). h_out receives h when a residual
 * is given; y goes to y_rows [M, D] and/or y_packed. D a multiple of 256 up to 8192.
 * Replaces: families/qwen3_5/cuda/glue.py:15-45 (add_rmsnorm), kernels/qwen/dense/v1/lane_glue.py:237-268
 * (norm_xs), families/qwen3_5/cuda/distributed.py:267-289 (rank-ordered partial sum). */
int tf_norm_xs(const void* x, const void* residual, const void* partials, int nparts, size_t part_stride,
               const void* weight, void* h_out, void* y_rows, void* y_packed, int M, int D, int group, float eps,
               void* stream);

/* out = bf16(silu(gate) * up); gate and up are [M, I] views with row stride in_stride.
 * Replaces: families/qwen3_5/cuda/glue.py:133-154 (swiglu), lane_glue.py:307-317 (mlp_act). */
int tf_swiglu(const void* gate, const void* up, size_t in_stride, void* out_packed, void* out_rows, int M, int I,
              int group, void* stream);
/* The same for a [gate; up] stack whose output columns are interleaved by 16-column tile (tile 2a = gate columns
 * 16a..16a+15, tile 2a+1 = up columns 16a..16a+15): gate_up [M, >= 2 I] with row stride in_stride. This is the
 * order tf_qmm_act wants the stacked weight in; both give the same bits. No reference counterpart for the order. */
int tf_swiglu_tiled(const void* gate_up, size_t in_stride, void* out_packed, void* out_rows, int M, int I, int group,
                    void* stream);

/* out = bf16(silu(z) * (y * rsqrt(mean_head(y^2) + eps) * weight)) per value head; y [M, v_heads, dv]
 * contiguous, z a [M, v_heads*dv] view with row stride z_stride, dv = 128.
 * Replaces: families/qwen3_5/cuda/glue.py:108-130 (gated_norm), lane_glue.py:294-304 (gdn_post). */
int tf_gated_norm(const void* y, const void* z, size_t z_stride, const void* weight, void* out_packed, void* out_rows,
                  int M, int v_heads, int dv, int group, float eps, void* stream);

/* out = bf16(o * sigmoid(gate)); o [M, heads, D] contiguous, gate = second half of each head's
 * [q | gate] block in the rows `qg` (row stride qg_stride). D = 128 or 256.
 * Replaces: families/qwen3_5/cuda/glue.py:206-226 (gate_mul), families/qwen4_exp/cuda/glue.py:369-387. */
int tf_gate_mul(const void* o, const void* qg, size_t qg_stride, void* out_packed, void* out_rows, int M, int heads,
                int head_dim, int group, void* stream);

/* Per head: bf16(weight * x * rsqrt(mean(x^2) + eps)), then rotate-half RoPE at row_pos[row] over the
 * first 2*rope_half dims with inv_freq[rope_half]; queries from the [q_h | gate_h] rows `qg`, keys from
 * `k`; values are copied. Outputs contiguous q [M, heads, D], k and v [M, kv_heads, D].
 * Replaces: families/qwen3_5/cuda/glue.py:157-203 (attn_prep), families/qwen4_exp/cuda/glue.py:298-366. */
int tf_attn_prep(const void* qg, size_t qg_stride, const void* k, size_t k_stride, const void* v, size_t v_stride,
                 const void* q_norm, const void* k_norm, const int* row_pos, const float* inv_freq, int rope_half,
                 void* q_out, void* k_out, void* v_out, int M, int heads, int kv_heads, int head_dim, float eps,
                 void* stream);

/* Depthwise causal conv (4 taps) over each row's own chain [conv_state of its sequence (3 rows);
 * the sequence's earlier window rows; the row], SiLU (rounded to bf16), split into q, k, v heads
 * of 128; q and k RMS-normalised (eps 1e-6) and scaled by 1/dk and dk^-1/2; g = exp(-exp(a_log) *
 * softplus(a + dt_bias)), beta = sigmoid(b). row_seq / row_idx give each packed row's sequence and
 * its place in that sequence's window (a sequence's rows are consecutive, in chain order).
 * conv_state [n_seqs, 3, C], conv_w [C, 4], C = (2*k_heads + v_heads) * 128.
 * Replaces: families/qwen3_5/cuda/glue.py:48-105 (gdn_pre), lane_glue.py:271-291,
 * families/qwen4_exp/cuda/gdn.cu:74-106 (conv + gates inside the chain kernel). */
int tf_gdn_pre(const void* qkv, size_t qkv_stride, const void* conv_state, const void* conv_w, const int* row_seq,
               const int* row_idx, const void* a, const void* b, size_t ab_stride, const float* a_log,
               const float* dt_bias, void* q_out, void* k_out, void* v_out, float* g_out, float* beta_out, int M,
               int k_heads, int v_heads, int dk, int dv, int taps, void* stream);

/* x[row] = bf16(q * s + b) of embedding row ids[row]; table in the stored MLX layout
 * (words [vocab, D/8], scales/biases [vocab, D/group]).
 * Replaces: families/qwen3_5/cuda/glue.py:229-246 (embed), families/qwen4_exp/cuda/glue.py:34-59. */
int tf_embed(const int* ids, const void* words, const void* scales, const void* biases, void* out, int M, int D,
             int group, int vocab, void* stream);

/* ---- gated-DeltaNet recurrence ---------------------------------------------------------------
 * For each sequence (rows seq_start[s] .. seq_start[s+1]-1, in chain order), value head and value
 * row:  S <- S*g;  mem = S.k;  delta = (v - mem)*beta;  S <- S + k*delta;  y = S.q  (fp32).
 * state [n_seqs, v_heads, dv, 128] fp32 is only read; state_out (optional, same shape) receives
 * the state after the window's last row. q, k [R, k_heads, 128], v, y [R, v_heads, dv] bf16;
 * g, beta [R, v_heads] fp32. dk = 128, dv a multiple of 32.
 * Replaces: families/qwen3_5/cuda/gdn_tree.cu:46-87 (tree_kernel, chain form),
 * families/qwen4_exp/cuda/gdn.cu:49-152 (chain_kernel), kernels/qwen/dense/v1/lane_tree.py:132-182. */
int tf_gdn_chain(const void* q, const void* k, const void* v, const float* g, const float* beta, const float* state,
                 float* state_out, void* y, const int* seq_start, int n_seqs, int k_heads, int v_heads, int dk, int dv,
                 void* stream);

/* Commit: advance `state` in place over the first keep[s] rows of each sequence's window with the
 * same statements as tf_gdn_chain, for `layers` layers in one launch (records and states of
 * successive layers `*_stride` elements apart).
 * Replaces: families/qwen3_5/cuda/gdn_tree.cu:89-154 (replay_kernel, replay_many_kernel),
 * families/qwen4_exp/cuda/gdn.cu:154-181. */
int tf_gdn_replay(const void* k, const void* v, const float* g, const float* beta, float* state, const int* seq_start,
                  const int* keep, int n_seqs, int layers, long long rec_k_stride, long long rec_v_stride,
                  long long rec_g_stride, long long state_stride, int k_heads, int v_heads, int dk, int dv,
                  void* stream);

/* The whole GDN mixer between its two projections in ONE launch: causal conv + SiLU + q/k RMS scale +
 * g/beta (tf_gdn_pre), the recurrence over each sequence's window rows (tf_gdn_chain) and the gated
 * RMSNorm with SiLU(z) written as the output projection's packed input (tf_gated_norm). q, k, v, g, beta
 * and y stay on chip; k, v, g, beta are also written to the record the commit replays. Every statement is
 * the separate kernels', so the results have their bits. qkv [rows, 2*k_heads*128 + v_heads*128] conv
 * input rows (qkv_stride elements a row), z [rows, v_heads*128], a, b [rows, v_heads] (ab_stride),
 * conv_state [n_seqs, 3, C], conv_w [C, 4], norm_w [128], state [n_seqs, v_heads, 128, 128] fp32 (read
 * only). out_packed: tf_packed_bytes(rows, v_heads*128, group) and/or out_rows [rows, v_heads*128] bf16.
 * One CTA per (value head, sequence). rows <= 128.
 * Replaces: families/qwen4_exp/cuda/gdn.cu:49-152 (the fused chain kernel) and, for the dense family,
 * glue.py:48-130 + gdn_tree.cu:46-87 run back to back. */
int tf_gdn_fused(const void* qkv, size_t qkv_stride, const void* z, size_t z_stride, const void* a, const void* b,
                 size_t ab_stride, const void* conv_state, const void* conv_w, const float* a_log, const float* dt_bias,
                 const void* norm_w, const float* state, void* k_out, void* v_out, float* g_out, float* beta_out,
                 void* out_packed, void* out_rows, const int* seq_start, int rows, int n_seqs, int k_heads, int v_heads,
                 int dk, int dv, int taps, int group, float eps, void* stream);

/* Commit: conv_state[s] <- last 3 rows of [conv_state[s]; first keep[s] window rows of qkv].
 * Replaces: families/qwen3_5/cuda/forward.py:226-236 (conv rows in commit). */
int tf_conv_commit(const void* qkv, size_t qkv_stride, long long rec_qkv_stride, void* conv_state,
                   long long state_stride, const int* seq_start, const int* keep, int n_seqs, int layers,
                   int channels, void* stream);

/* ---- lane attention over a paged KV cache ------------------------------------------------------
 * Causal GQA for every window row of every sequence: row t of sequence s attends to the committed
 * tokens 0..seq_lens[s]-1 (pages: k_pages / v_pages [page, kv_head, 16, D] bf16 through
 * page_table [n_seqs, max_pages]) and to window rows 0..t of s (k_new / v_new [rows, kv_heads, D]).
 * Keys are cut by absolute position into chunks of 64-key tiles (128 keys a chunk below position 8192,
 * 512 up to 65536, 2048 beyond; tf_attention_chunks(n) = chunks holding keys 0..n-1); per-chunk
 * (m, l, O) partials go to `scratch` (tf_attention_scratch_bytes) and are merged per row: four quarters
 * of the row's chunks in order, then the quarters in order.
 * row_nkeys[row] = seq_lens[s] + t + 1. max_window = longest window, max_chunks >= tf_attention_chunks(
 * max over s of seq_lens[s] + window); a row that would need more chunks than max_chunks is merged
 * over the first max_chunks only and TF_EINVAL is written to `status` (gated form), scratch is never
 * read past its end. q, out [rows, heads, D]; D = 128 or 256; heads/kv_heads <= 16.
 * Replaces: families/qwen3_5/cuda/attention.py:152-201 (attention), families/qwen4_exp/cuda/attention.py:126-140,
 * kernels/qwen/dense/v1/lane_attention.py:430-518 (lane_sdpa, lane_tree_sdpa; chains only). */
size_t tf_attention_scratch_bytes(int rows, int heads, int head_dim, int max_chunks);
int tf_attention_chunks(int n_keys);
int tf_lane_attention_paged(const void* q, const void* k_new, const void* v_new, const void* k_pages,
                            const void* v_pages, const int* page_table, int max_pages, const int* seq_lens,
                            const int* seq_start, const int* row_nkeys, void* out, void* scratch, size_t scratch_bytes,
                            int rows, int n_seqs, int max_window, int max_chunks, int heads, int kv_heads, int head_dim,
                            float scale, void* stream);

/* The same attention with the layer's output gate and the next matmul's input fused into the merge:
 * with qg not NULL (the q projection's output rows, per head [q_h ; gate_h], qg_stride elements a row)
 * the result is bf16(o * sigmoid(gate)); with out_packed not NULL it is also written as the packed input
 * of the output projection (tf_packed_bytes(rows, heads * D, group)) with its group sums; `out` may then
 * be NULL. Replaces: families/qwen3_5/cuda/glue.py:206-226 (gate_mul) after the attention above. */
int tf_lane_attention_paged_gated(const void* q, const void* k_new, const void* v_new, const void* k_pages,
                                  const void* v_pages, const int* page_table, int max_pages, const int* seq_lens,
                                  const int* seq_start, const int* row_nkeys, void* out, const void* qg, size_t qg_stride,
                                  void* out_packed, int group, void* scratch, size_t scratch_bytes, int rows, int n_seqs,
                                  int max_window, int max_chunks, int heads, int kv_heads, int head_dim, float scale,
                                  int* status, void* stream);

/* The same attention for callers that cannot allocate or pass scratch: a server whose device memory
 * was handed out once at start-up, a plugin inside a runtime that forbids allocation on the serving
 * path, code for which every buffer address must be fixed in advance. This entry point has no
 * counterpart in the TensorFold reference. The chunk partials live in a fixed array inside the
 * loaded library (TF_ATTN_STATIC_SCRATCH_BYTES on every GPU that loads it, until the process exits);
 * the call allocates nothing. Limits: tf_attention_scratch_bytes(rows, heads, head_dim, max_chunks)
 * must not exceed TF_ATTN_STATIC_SCRATCH_BYTES, else TF_ESCRATCH and nothing runs. The first call on
 * each device looks up the array's device address; make that call before any stream capture. All
 * calls share the array: calls that overlap on one GPU race and must be serialised by the caller;
 * stale contents from earlier calls are never read, so nothing needs clearing. Results are
 * bit-identical to tf_lane_attention_paged. */
#define TF_ATTN_STATIC_SCRATCH_BYTES (8u << 20)
int tf_lane_attention_paged_static(const void* q, const void* k_new, const void* v_new, const void* k_pages,
                                   const void* v_pages, const int* page_table, int max_pages, const int* seq_lens,
                                   const int* seq_start, const int* row_nkeys, void* out, int rows, int n_seqs,
                                   int max_window, int max_chunks, int heads, int kv_heads, int head_dim, float scale,
                                   void* stream);

/* Commit: copy the first keep[s] window rows of each sequence into its pages at positions
 * seq_lens[s].., for `layers` layers in one launch.
 * Replaces: families/qwen3_5/cuda/forward.py:237-251 (key/value rows in commit). */
int tf_kv_commit(const void* k_new, const void* v_new, long long rec_stride, void* k_pages, void* v_pages,
                 long long pages_stride, const int* page_table, int max_pages, const int* seq_lens, const int* seq_start,
                 const int* keep, int n_seqs, int layers, int kv_heads, int head_dim, void* stream);

/* ---- mixture-of-experts block -------------------------------------------------------------------
 * Replaces: families/qwen4_exp/cuda/moe.py:42-163 (router, select, MoEBuffers, moe) and the combine of
 * families/qwen4_exp/cuda/glue.py:85-91. The expert projections run through tf_qmm_grouped.
 *
 * tf_moe_router: logits[r, e] = fp32 x[r] . router[e] for e < experts_total (the routed experts' rows,
 *   then optionally the shared expert's gate row); bf16 inputs, D a multiple of 256, one fixed
 *   summation order per D.
 * tf_moe_select: per row the top_k routed experts by (logit descending, id ascending) with weights
 *   bf16(exp(l_k - l_0) / sum) and, when experts_total = experts + 1, the shared expert (id `experts`)
 *   as the last slot with weight bf16(sigmoid(bf16(gate logit))). pick int32, wts fp32 [rows, slots].
 * tf_moe_group: the window's problem list for tf_qmm_grouped: distinct experts in ascending id, each
 *   cut into problems of up to 8 members in row order. prob_expert [max_probs], prob_count [1],
 *   prob_rows [max_probs, 8] (row * 32 + slot, or -1), pair_loc [rows, slots] = problem * 8 + place.
 *   max_probs from tf_moe_max_problems. rows <= 128.
 * tf_moe_pack: problem p's member rows of x [rows, K], packed for the matmul (absent members zero).
 * tf_moe_act: compact gate/up results [problem, 8, 2 I] bf16 -> bf16(silu(gate) * up), packed for the
 *   down projection of the same problems.
 * tf_moe_combine: out[r] = bf16(sum over slots, in slot order, of wts[r, k] * y[pair_loc[r, k]]) with
 *   y the compact fp32 down results [problem * 8 + place, D]; fma, one rounding.
 * Expert parallelism (world > 1; no counterpart in the reference, which shards expert width instead):
 *   every rank routes all rows and builds the same list; routed expert e belongs to rank
 *   e / (experts / world) as local weight slot e % (experts / world), the shared expert is replicated
 *   as local slot experts / world with its problems dealt round-robin. tf_moe_group then also writes
 *   prob_sel (this rank's problems, ascending) and sel_count, and prob_expert holds local slots: pass
 *   prob_sel / sel_count to tf_qmm_grouped. tf_moe_push stores the rank's results as 16-byte packets
 *   {value, n, value, n} into EVERY rank's buffer (peer_bufs as for tf_peer_exchange) at the problem's
 *   own index, and - also when the rank owns no problem - one presence cell {n, n, n, n} for `rank` at the
 *   head of every rank's slot. A buffer is two slots of slot_bytes >= tf_moe_slot_bytes(max_probs, D)
 *   (1024 bytes of presence cells, then max_probs * 8 * D * 8 bytes of packets), zero before first use;
 *   the slot of exchange n is n & 1, chosen on the device. tf_moe_combine_peer polls the packets its
 *   pairs need in this rank's own buffer (bounded, TF_ESTALL) and combines as tf_moe_combine does - the
 *   result has the bits of the one-GPU block - and advances the exchange number only after all `world`
 *   presence cells carry n, so a slot is never overwritten while a slower rank still reads it. seq and
 *   tickets as for tf_peer_exchange; every rank issues one push and one combine per exchange. */
size_t tf_moe_slot_bytes(int max_probs, int D);
int tf_moe_max_problems(int rows, int slots, int experts_total);
int tf_moe_router(const void* x, size_t x_stride, const void* router, float* logits, int rows, int D, int experts_total,
                  void* stream);
int tf_moe_select(const float* logits, int rows, int experts_total, int experts, int top_k, int* pick, float* wts, void* stream);
int tf_moe_group(const int* pick, int rows, int slots, int experts_total, int max_probs, int* prob_expert, int* prob_count,
                 int* prob_rows, int* pair_loc, int experts, int rank, int world, int* prob_sel, int* sel_count, void* stream);
int tf_moe_pack(const void* x, size_t x_stride, const int* prob_rows, const int* prob_count, int max_probs, void* x_packed, int K,
                int group, void* stream);
int tf_moe_act(const void* gate_up, const int* prob_count, int max_probs, void* act_packed, int I, int group, void* stream);
int tf_moe_combine(const float* y, const int* pair_loc, const float* wts, int slots, void* out, int rows, int D, void* stream);
int tf_moe_push(const float* y, const int* prob_sel, const int* sel_count, int max_probs, int D, void* const* peer_bufs,
                size_t slot_bytes, int rank, int world, const void* seq, void* stream);
int tf_moe_combine_peer(const void* my_buf, size_t slot_bytes, const int* pair_loc, const float* wts, int slots, void* out, int rows,
                        int D, int world, void* seq, void* tickets, int* status, void* stream);

/* ---- tensor-parallel exchange over peer memory ---------------------------------------------------
 * Replaces: families/qwen3_5/cuda/distributed.py:267-289 (gather_rank_partials over NCCL) and the
 * hand-bound collective of families/qwen4_exp/cuda/comm.py:41-85.
 * One call per rank and exchange: the rank's fp32 partial local [rows, D] is turned into 16-byte
 * packets {value, n, value, n} (n = the exchange number, a device counter every rank advances alike)
 * and stored into block `rank` of the slot at slot_off of EVERY rank's buffer (peer_bufs: device array
 * of the world's buffer base addresses, the same symmetric allocation on every rank, zero before the
 * first exchange); each rank then polls its own slot until every packet carries n and writes the
 * payload to `gathered` [world, rows, D] fp32 (local memory). A slot is at least tf_peer_slot_bytes bytes.
 * seq and tickets: one zero-initialised 32-bit word each in local device memory, private to this rank
 * group. Consecutive exchanges must alternate between two slots; all ranks must issue the same
 * exchanges in the same order; the slot of an exchange is chosen on the device (n & 1), the buffer is
 * 2 * slot_bytes. The polling is bounded and reports TF_ESTALL through `status`. */
size_t tf_peer_slot_bytes(int rows, int D, int world);
int tf_peer_exchange(const float* local, int rows, int D, void* const* peer_bufs, size_t slot_bytes, float* gathered, int rank,
                     int world, void* seq, void* tickets, int* status, void* stream);

/* The same exchange fused into its neighbours (no kernel of its own, no staging pass): tf_qmm_peer is the
 * row-parallel matmul whose epilogue stores the rank's fp32 partial as packets {row 2i, n, row 2i+1, n}
 * straight into block `rank` of slot n & 1 (n = *seq + 1) of EVERY rank's buffer (peer_bufs, plain peer
 * stores, no multicast); tf_norm_xs_peer is tf_norm_xs whose residual addend is the sum, in rank order with
 * one rounding, of the `world` partials it finds in this rank's own buffer (my_buf) once their packets
 * carry n (bounded wait, TF_ESTALL through `status`); its last CTA advances *seq. Every rank must issue the
 * same sequence of (tf_qmm_peer, tf_norm_xs_peer) pairs; buffers are 2 * slot_bytes, slot_bytes >=
 * tf_peer_slot_bytes(rows, D, world), zero before first use; seq and tickets: one zeroed 32-bit word each.
 * Replaces: families/qwen3_5/cuda/distributed.py:267-289 (row_partial + gather_rank_partials +
 * sum_rank_partials) around the two row-parallel projections of a layer. */
/* tf_qmm_next for the stacked [gate; up] projection (columns interleaved by 16-column tile, see tf_swiglu_tiled) with
 * the SwiGLU fused into the epilogue: no y; the owner of each column block writes bf16(silu(bf16 gate) * bf16 up) and
 * its group sums as the packed input (N / 2 inputs, group `group`) of the down projection - the bits tf_swiglu_tiled
 * writes from the same projection's output. M is 1..8 (the bucket whose warps own a gate tile and its up tile).
 * Replaces: glue.swiglu after the gate and up matmuls (families/qwen3_5/cuda/forward.py:186-189). */
int tf_qmm_act(const void* x_packed, const void* w_tiled, void* act_packed, void* scratch, size_t scratch_bytes, int M, int N,
               int K, int group, const void* next_w_tiled, int next_N, int next_K, int next_group, int* status, void* stream);
int tf_qmm_peer(const void* x_packed, const void* w_tiled, void* scratch, size_t scratch_bytes, int M, int N, int K, int group,
                void* const* peer_bufs, size_t slot_bytes, const void* seq, int rank, int world, const void* next_w_tiled,
                int next_N, int next_K, int next_group, int* status, void* stream);
int tf_norm_xs_peer(const void* x, const void* residual, const void* partials, int nparts, size_t part_stride,
                    const void* weight, void* h_out, void* y_rows, void* y_packed, int M, int D, int group, float eps,
                    const void* my_buf, size_t slot_bytes, void* seq, void* tickets, int world, int* status, void* stream);

/* Polls of one location another rank writes before a kernel gives up and writes TF_ESTALL (default 2^22,
 * seconds; 0 restores it). Applies to later launches of this process. The reference has no counterpart:
 * its collectives time out on the host (families/qwen4_exp/cuda/comm.py:41-85). */
void tf_set_poll_limit(unsigned polls);

/* ---- exact top-k and keyed sampling --------------------------------------------------------------
 * Each row's k largest bf16 logits (k <= 64), ordered by value descending then id ascending; ties at
 * the cut go to the smallest ids. idx int32 [rows, k], val fp32 [rows, k]. scratch: the slices'
 * candidates, tf_topk_scratch_bytes bytes, 8-byte aligned, no initialisation; two launches.
 * Replaces: engine/topk.py:20-146 (radix_topk, topk_rows). */
size_t tf_topk_scratch_bytes(int rows, int vocab, int k);
int tf_topk_rows(const void* x, size_t row_stride, int rows, int vocab, int k, int* idx, float* val, void* scratch,
                 size_t scratch_bytes, void* stream);

/* token = argmax over the kept candidates of val/temperature + Gumbel(splitmix64(seed, position, id));
 * candidates (already ordered as tf_topk_rows writes them) are cut to top_k, then to the smallest
 * prefix whose tempered probability reaches top_p. fp64 arithmetic.
 * Replaces: engine/exact_sampling.py:57-109 (uniform_rows, choose_rows), engine/gpu_sampling.py:298-363. */
int tf_sample_rows(const int* idx, const float* val, int width, const long long* positions, unsigned long long seed,
                   double temperature, int top_k, double top_p, int* tokens, int rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TENSORFOLD_B200_H */
