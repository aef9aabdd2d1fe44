// Gated-DeltaNet recurrence over the rows of each sequence's verify window, and the commit replay.
//
// Per (sequence, value head, value row) the fp32 state row S[0..127] (key dimension) stays in
// registers across the window's rows, split over 4 lanes of 32 values each:
//     S    <- S * g
//     mem   = S . k                      (fp32: per lane four 8-term fma chains combined pairwise, then a 4-lane xor tree)
//     delta = (v - mem) * beta
//     S    <- S + k * delta              (fma)
//     y     = S . q
// rows in chain order. The committed state is only read; `tf_gdn_replay` later advances it over the
// accepted rows with the same statements in the same order, so a replayed state has the bits a
// serial one-row step would have produced, and row t of a window equals the t-th serial step.
//
// q and k of the rows being processed are staged as fp32 in shared memory, 8 rows at a time, and
// shared by the 32 value rows a CTA owns.

#include "common.cuh"

namespace tf {
namespace {

constexpr int kDk = 128;            // key head dim (state row length)
constexpr int kRowsPerCta = 32;     // value rows per CTA: 4 lanes each -> 128 threads
constexpr int kTile = 8;            // window rows staged per pass

// One window row applied to the 32 state values a lane holds (key elements 16*i + 4*j + e of one value row),
// the same statements in the chain, replay and fused kernels: four partial dot products per lane (one per
// element of the float4s, eight terms each, so the fma chains are short), combined pairwise, then the
// 4-lane xor tree.
template <bool OUT>
__device__ __forceinline__ float gdn_row_step(float4 (&s)[8], const float* krow, const float* qrow, int j, float decay, float vval,
                                              float beta) {
    float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 kv = *reinterpret_cast<const float4*>(krow + i * 16 + j * 4);
        s[i].x *= decay; s[i].y *= decay; s[i].z *= decay; s[i].w *= decay;
        m0 = __fmaf_rn(s[i].x, kv.x, m0);
        m1 = __fmaf_rn(s[i].y, kv.y, m1);
        m2 = __fmaf_rn(s[i].z, kv.z, m2);
        m3 = __fmaf_rn(s[i].w, kv.w, m3);
    }
    float mem = (m0 + m1) + (m2 + m3);
    mem += __shfl_xor_sync(0xffffffffu, mem, 1);
    mem += __shfl_xor_sync(0xffffffffu, mem, 2);
    const float delta = (vval - mem) * beta;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 kv = *reinterpret_cast<const float4*>(krow + i * 16 + j * 4);
        s[i].x = __fmaf_rn(kv.x, delta, s[i].x);
        s[i].y = __fmaf_rn(kv.y, delta, s[i].y);
        s[i].z = __fmaf_rn(kv.z, delta, s[i].z);
        s[i].w = __fmaf_rn(kv.w, delta, s[i].w);
        if (OUT) {
            const float4 qv = *reinterpret_cast<const float4*>(qrow + i * 16 + j * 4);
            o0 = __fmaf_rn(s[i].x, qv.x, o0);
            o1 = __fmaf_rn(s[i].y, qv.y, o1);
            o2 = __fmaf_rn(s[i].z, qv.z, o2);
            o3 = __fmaf_rn(s[i].w, qv.w, o3);
        }
    }
    float out = 0.f;
    if (OUT) {
        out = (o0 + o1) + (o2 + o3);
        out += __shfl_xor_sync(0xffffffffu, out, 1);
        out += __shfl_xor_sync(0xffffffffu, out, 2);
    }
    return out;
}

struct GdnArgs {
    const __nv_bfloat16* q;         // [R, KH, 128]   (unused by replay)
    const __nv_bfloat16* k;         // [R, KH, 128]
    const __nv_bfloat16* v;         // [R, VH, DV]
    const float* g;                 // [R, VH]
    const float* beta;              // [R, VH]
    const float* state_in;          // [S, VH, DV, 128]
    float* state_out;               // same shape, or null
    __nv_bfloat16* y;               // [R, VH, DV], or null
    const int* seq_start;           // [S + 1] first packed row of each sequence
    const int* keep;                // [S] rows to apply (null: all rows of the window)
    int KH, VH, DV;
    // several layers in one launch (commit): element strides between layers, 0 for one layer
    long long rec_q, rec_v, rec_g, rec_state;
    int S;
};

template <bool OUT>
__global__ void __launch_bounds__(kRowsPerCta * 4) gdn_kernel(const GdnArgs a) {
    __shared__ float ks[kTile][kDk];
    __shared__ float qs[OUT ? kTile : 1][kDk];
    __shared__ float vs[kTile][kRowsPerCta];
    __shared__ float gs[kTile], bs[kTile];
    pdl_launch_dependents();
    pdl_wait();
    const int layer = blockIdx.z / a.S, seq = blockIdx.z % a.S, head = blockIdx.y;
    const int tid = threadIdx.x, j = tid & 3, lr = tid >> 2;
    const int dvrow = blockIdx.x * kRowsPerCta + lr;
    const int kh = head / (a.VH / a.KH);
    const int r0 = a.seq_start[seq];
    int n = a.seq_start[seq + 1] - r0;
    if (a.keep != nullptr) n = min(n, a.keep[seq]);
    const __nv_bfloat16* qp = a.q + layer * a.rec_q;
    const __nv_bfloat16* kp = a.k + layer * a.rec_q;
    const __nv_bfloat16* vp = a.v + layer * a.rec_v;
    const float* gp = a.g + layer * a.rec_g;
    const float* bp = a.beta + layer * a.rec_g;
    const size_t srow = (size_t)layer * a.rec_state + (((size_t)seq * a.VH + head) * a.DV + dvrow) * kDk;

    // lane j of a value row holds key elements 16*i + 4*j + e (i = 0..7, e = 0..3): float4 loads that coalesce
    float4 s[8];
    const bool live = dvrow < a.DV;
    if (live) {
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = reinterpret_cast<const float4*>(a.state_in + srow)[i * 4 + j];
    }

    for (int t0 = 0; t0 < n; t0 += kTile) {
        const int rows = min(kTile, n - t0);
        __syncthreads();
        // 16-byte loads: 8 bf16 values of a key/query row, or of a row's 32 values, per thread
        for (int e = tid; e < rows * (kDk / 8); e += kRowsPerCta * 4) {
            const int r = e / (kDk / 8), d = (e % (kDk / 8)) * 8;
            const size_t at = ((size_t)(r0 + t0 + r) * a.KH + kh) * kDk + d;
            float f[8];
            unpack8(*reinterpret_cast<const uint4*>(kp + at), f);
#pragma unroll
            for (int i = 0; i < 8; ++i) ks[r][d + i] = f[i];
            if (OUT) {
                unpack8(*reinterpret_cast<const uint4*>(qp + at), f);
#pragma unroll
                for (int i = 0; i < 8; ++i) qs[r][d + i] = f[i];
            }
        }
        if ((a.DV & 7) == 0) {
            for (int e = tid; e < rows * (kRowsPerCta / 8); e += kRowsPerCta * 4) {
                const int r = e / (kRowsPerCta / 8), c = (e % (kRowsPerCta / 8)) * 8;
                const int dr = blockIdx.x * kRowsPerCta + c;
                float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (dr < a.DV) unpack8(*reinterpret_cast<const uint4*>(vp + ((size_t)(r0 + t0 + r) * a.VH + head) * a.DV + dr), f);
#pragma unroll
                for (int i = 0; i < 8; ++i) vs[r][c + i] = f[i];
            }
        } else {
            for (int e = tid; e < rows * kRowsPerCta; e += kRowsPerCta * 4) {
                const int r = e / kRowsPerCta, c = e % kRowsPerCta;
                const int dr = blockIdx.x * kRowsPerCta + c;
                vs[r][c] = dr < a.DV ? bf2f(vp[((size_t)(r0 + t0 + r) * a.VH + head) * a.DV + dr]) : 0.f;
            }
        }
        if (tid < rows) {
            gs[tid] = gp[(size_t)(r0 + t0 + tid) * a.VH + head];
            bs[tid] = bp[(size_t)(r0 + t0 + tid) * a.VH + head];
        }
        __syncthreads();
        if (!live) continue;
        for (int r = 0; r < rows; ++r) {
            const float out = gdn_row_step<OUT>(s, ks[r], qs[OUT ? r : 0], j, gs[r], vs[r][lr], bs[r]);
            if (OUT && j == 0) a.y[((size_t)(r0 + t0 + r) * a.VH + head) * a.DV + dvrow] = f2bf(out);
        }
    }
    if (live && a.state_out != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(a.state_out + srow)[i * 4 + j] = s[i];
    }
}

// ---- the whole GDN mixer between its two projections, one launch ----------------------------------------
// One CTA of 512 threads per (value head, sequence) does, for the sequence's window rows in passes of 8:
//   1. the causal 4-tap conv + SiLU on the head's q, k and v channels, the RMS scale of q and k, the decay
//      g and the write strength beta (one warp per (row, q | k | v), a lane's 4 channels: the statements of
//      gdn_pre_kernel), into shared memory; k, v, g, beta also go to the record the commit replays;
//   2. the delta-rule recurrence over the pass's rows with the fp32 state row in registers (4 lanes x 32
//      values per value row: the statements of gdn_kernel), y rounded to bf16 into shared memory;
//   3. the gated RMSNorm of y with SiLU(z) (16 lanes per row: the statements of gated_norm_kernel) written
//      as the output projection's packed input with its group sums.
// q, k, v, g, beta, y never travel through HBM between the steps and the three launches become one; every
// statement is the unfused kernel's, so the results carry the same bits.
struct GdnFusedArgs {
    const __nv_bfloat16* qkv; size_t qkv_stride;      // [R, 2*KH*128 + VH*128] conv input rows
    const __nv_bfloat16* z; size_t z_stride;          // [R, VH*128]
    const __nv_bfloat16* a_in; const __nv_bfloat16* b_in; size_t ab_stride;   // [R, VH]
    const __nv_bfloat16* conv_state;                  // [S, 3, C]
    const __nv_bfloat16* conv_w;                      // [C, 4]
    const float* a_log; const float* dt_bias;         // [VH]
    const __nv_bfloat16* norm_w;                      // [128]
    const float* state_in;                            // [S, VH, 128, 128]
    __nv_bfloat16* k_out; __nv_bfloat16* v_out; float* g_out; float* beta_out;   // the record
    uint8_t* out_packed; __nv_bfloat16* out_rows;     // [R, VH*128] packed (and optionally plain rows)
    const int* seq_start;
    int KH, VH, S, R, group;
    float eps;
};

template <int G>
__global__ void __launch_bounds__(512) gdn_fused_kernel(const GdnFusedArgs a) {
    __shared__ float ks[kTile][kDk], qs[kTile][kDk], vs[kTile][kDk], ys[kTile][kDk];
    __shared__ float gs[kTile], bs[kTile];
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, seq = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int j = tid & 3, dvrow = tid >> 2;                       // recurrence roles: value row, quarter of the key axis
    const int kh = head / (a.VH / a.KH);
    const int C = (2 * a.KH + a.VH) * 128;
    const int r0 = a.seq_start[seq], n = a.seq_start[seq + 1] - r0;
    const int Mp = tf_padded_rows(a.R), total = a.VH * 16;         // chunks of 8 in an output row
    // the last sequence's CTAs also zero the packed buffer's padding rows for their head
    if (seq == a.S - 1 && a.out_packed != nullptr) {
        for (int e = tid; e < (Mp - a.R) * 16; e += 512)
            packed_store<G>(a.out_packed, Mp, a.R + e / 16, head * 16 + (e & 15), make_uint4(0, 0, 0, 0), 0.f);
    }
    if (n <= 0) return;
    const size_t srow = (((size_t)seq * a.VH + head) * kDk + dvrow) * kDk;
    float4 s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = reinterpret_cast<const float4*>(a.state_in + srow)[i * 4 + j];

    for (int t0 = 0; t0 < n; t0 += kTile) {
        const int rows = min(kTile, n - t0);
        __syncthreads();
        // ---- 1. conv + gates: warps 0..7 take q and k of row `warp`, warps 8..15 v and the gates of row
        //         `warp - 8`; a warp's loads are all issued before the first use, so the pass costs one trip ----
        {
            const int r = warp & 7;
            if (r < rows) {
                const int row = r0 + t0 + r, idx = t0 + r;         // idx: the row's place in its sequence's chain
                constexpr int NP = 2;
                const int nparts = warp < 8 ? 2 : 1;
                uint4 wq[NP][2];
                uint2 xv[NP][4];
#pragma unroll
                for (int pi = 0; pi < NP; ++pi) {
                    if (pi < nparts) {
                        const int part = warp < 8 ? pi : 2;
                        const int chead = part == 0 ? kh : part == 1 ? a.KH + kh : 2 * a.KH + head;
                        const int ch0 = chead * 128 + lane * 4;
                        const uint4* wp = reinterpret_cast<const uint4*>(a.conv_w + (size_t)ch0 * 4);
                        wq[pi][0] = wp[0]; wq[pi][1] = wp[1];
#pragma unroll
                        for (int tap = 0; tap < 4; ++tap) {
                            const int src = idx + tap;             // index into [conv_state (3 rows); window rows]
                            const __nv_bfloat16* p = src < 3 ? a.conv_state + ((size_t)seq * 3 + src) * C + ch0
                                                             : a.qkv + (size_t)(row - idx + src - 3) * a.qkv_stride + ch0;
                            xv[pi][tap] = *reinterpret_cast<const uint2*>(p);
                        }
                    }
                }
                float av = 0.f, bv = 0.f;
                if (warp >= 8 && lane == 0) {
                    av = bf2f(a.a_in[(size_t)row * a.ab_stride + head]);
                    bv = bf2f(a.b_in[(size_t)row * a.ab_stride + head]);
                }
#pragma unroll
                for (int pi = 0; pi < NP; ++pi) {
                    if (pi < nparts) {
                        const int part = warp < 8 ? pi : 2;
                        float wt[16];
                        {
                            float lo[8], hi[8];
                            unpack8(wq[pi][0], lo);
                            unpack8(wq[pi][1], hi);
#pragma unroll
                            for (int i = 0; i < 8; ++i) { wt[i] = lo[i]; wt[8 + i] = hi[i]; }
                        }
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int tap = 0; tap < 4; ++tap) {
                            const float xf[4] = {bf16_lo(xv[pi][tap].x), bf16_hi(xv[pi][tap].x), bf16_lo(xv[pi][tap].y), bf16_hi(xv[pi][tap].y)};
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[i] = __fmaf_rn(xf[i], wt[i * 4 + tap], acc[i]);
                        }
                        float c[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) c[i] = round_bf16(acc[i] * sigmoidf_(acc[i]));
                        if (part < 2) {
                            float ss = 0.f;
#pragma unroll
                            for (int i = 0; i < 4; ++i) ss += c[i] * c[i];
                            const float inv = 1.0f / sqrtf(warp_sum(ss) / 128.0f + 1e-6f);
                            const float scale = part == 0 ? 1.0f / 128.0f : 0.08838834764831845f;   // 1/dk, dk^-1/2
                            const uint2 packed = make_uint2(pack_bf16(c[0] * inv * scale, c[1] * inv * scale),
                                                            pack_bf16(c[2] * inv * scale, c[3] * inv * scale));
                            float* dst = (part == 0 ? qs[r] : ks[r]) + lane * 4;
                            dst[0] = bf16_lo(packed.x); dst[1] = bf16_hi(packed.x); dst[2] = bf16_lo(packed.y); dst[3] = bf16_hi(packed.y);
                            // one of the value heads that share this key head keeps k for the commit
                            if (part == 1 && head % (a.VH / a.KH) == 0)
                                *reinterpret_cast<uint2*>(a.k_out + ((size_t)row * a.KH + kh) * 128 + lane * 4) = packed;
                        } else {
                            const uint2 packed = make_uint2(pack_bf16(c[0], c[1]), pack_bf16(c[2], c[3]));
                            float* dst = vs[r] + lane * 4;
                            dst[0] = c[0]; dst[1] = c[1]; dst[2] = c[2]; dst[3] = c[3];
                            *reinterpret_cast<uint2*>(a.v_out + ((size_t)row * a.VH + head) * 128 + lane * 4) = packed;
                            if (lane == 0) {
                                const float ag = av + a.dt_bias[head];
                                const float sp = ag > 20.0f ? ag : logf(1.0f + expf(ag));
                                const float gv = expf(-expf(a.a_log[head]) * sp);
                                const float bvv = sigmoidf_(bv);
                                gs[r] = gv; bs[r] = bvv;
                                a.g_out[(size_t)row * a.VH + head] = gv;
                                a.beta_out[(size_t)row * a.VH + head] = bvv;
                            }
                        }
                    }
                }
            }
        }
        // the gated norm's z and weight, fetched now so that the trip hides behind the recurrence
        uint4 z_pre = make_uint4(0, 0, 0, 0), w_pre = make_uint4(0, 0, 0, 0);
        if (warp * 2 + (lane >> 4) < rows) {
            const int row = r0 + t0 + warp * 2 + (lane >> 4), l16 = lane & 15;
            // two 8-byte loads: a row stride that is only a multiple of four values (narrow tensor-parallel shards)
            const uint2* zp = reinterpret_cast<const uint2*>(a.z + (size_t)row * a.z_stride + head * 128 + 8 * l16);
            const uint2 z0 = zp[0], z1 = zp[1];
            z_pre = make_uint4(z0.x, z0.y, z1.x, z1.y);
            w_pre = reinterpret_cast<const uint4*>(a.norm_w)[l16];
        }
        __syncthreads();
        // ---- 2. recurrence over the pass's rows ----
        for (int r = 0; r < rows; ++r) {
            const float out = gdn_row_step<true>(s, ks[r], qs[r], j, gs[r], vs[r][dvrow], bs[r]);
            if (j == 0) ys[r][dvrow] = round_bf16(out);
        }
        __syncthreads();
        // ---- 3. gated norm + packing: 16 lanes per row, 8 values a lane ----
        if (warp * 2 < rows) {
            const int r = warp * 2 + (lane >> 4), l16 = lane & 15;
            const bool live = r < rows;
            const int row = r0 + t0 + (live ? r : 0);
            float yv[8], zv[8], wv[8], o[8];
            float ss = 0.f;
            uint4 ov = make_uint4(0, 0, 0, 0);
            if (live) {
#pragma unroll
                for (int i = 0; i < 8; ++i) yv[i] = ys[r][l16 * 8 + i];
                unpack8(z_pre, zv);
                unpack8(w_pre, wv);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += yv[i] * yv[i];
            }
#pragma unroll
            for (int o2 = 1; o2 < 16; o2 <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
            if (live) {
                const float inv = 1.0f / sqrtf(ss / 128.0f + a.eps);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = zv[i] * sigmoidf_(zv[i]) * (yv[i] * inv * wv[i]);
                ov = pack8(o);
            }
            const float gsum = group_sum8<G>(ov);
            if (live) {
                const int c = head * 16 + l16;
                if (a.out_rows != nullptr) reinterpret_cast<uint4*>(a.out_rows)[(size_t)row * total + c] = ov;
                if (a.out_packed != nullptr) packed_store<G>(a.out_packed, Mp, row, c, ov, gsum);
            }
        }
    }
}

// Conv tail after a commit: the last 3 rows of [old tail (3 rows); the sequence's kept window rows].
__global__ void conv_commit_kernel(const __nv_bfloat16* qkv, size_t qkv_stride, long long rec_qkv, __nv_bfloat16* conv_state,
                                   long long rec_state, const int* seq_start, const int* keep, int C, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const int layer = blockIdx.z / S, seq = blockIdx.z % S;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int r0 = seq_start[seq];
    const int n = min(keep[seq], seq_start[seq + 1] - r0);
    __nv_bfloat16* st = conv_state + layer * rec_state + (size_t)seq * 3 * C + c;
    const __nv_bfloat16* rows = qkv + layer * rec_qkv + c;
    uint4 out[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const int src = n + i;                    // index into [old tail; kept rows]
        out[i] = src < 3 ? *reinterpret_cast<const uint4*>(st + (size_t)src * C)
                         : *reinterpret_cast<const uint4*>(rows + (size_t)(r0 + src - 3) * qkv_stride);
    }
#pragma unroll
    for (int i = 0; i < 3; ++i) *reinterpret_cast<uint4*>(st + (size_t)i * C) = out[i];
}

int check(int S, int layers, int KH, int VH, int DK, int DV) {
    if (S < 1 || layers < 1 || KH < 1 || VH < 1 || VH % KH || DK != kDk || DV < 1 || DV % kRowsPerCta) return TF_EINVAL;
    if ((long long)S * layers > 65535) return TF_EINVAL;
    return TF_OK;
}

}  // namespace
}  // namespace tf

extern "C" {

int tf_gdn_chain(const void* q, const void* k, const void* v, const float* g, const float* beta, const float* state,
                 float* state_out, void* y, const int* seq_start, int n_seqs, int k_heads, int v_heads, int dk, int dv,
                 void* stream) {
    if (tf::check(n_seqs, 1, k_heads, v_heads, dk, dv) != TF_OK) return TF_EINVAL;
    if (!q || !k || !v || !g || !beta || !state || !y || !seq_start) return TF_EINVAL;
    if (((uintptr_t)state | (uintptr_t)state_out | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) return TF_EALIGN;
    tf::GdnArgs a = {};
    a.q = static_cast<const __nv_bfloat16*>(q); a.k = static_cast<const __nv_bfloat16*>(k);
    a.v = static_cast<const __nv_bfloat16*>(v); a.g = g; a.beta = beta;
    a.state_in = state; a.state_out = state_out; a.y = static_cast<__nv_bfloat16*>(y);
    a.seq_start = seq_start; a.keep = nullptr;
    a.KH = k_heads; a.VH = v_heads; a.DV = dv; a.S = n_seqs;
    void* args[] = {&a};
    dim3 grid((dv + tf::kRowsPerCta - 1) / tf::kRowsPerCta, v_heads, n_seqs);
    cudaError_t e = tf::launch_pdl((const void*)tf::gdn_kernel<true>, grid, dim3(tf::kRowsPerCta * 4), 0,
                                   static_cast<cudaStream_t>(stream), args);
    if (e != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

int tf_gdn_fused(const void* qkv, size_t qkv_stride, const void* z, size_t z_stride, const void* a, const void* b, size_t ab_stride,
                 const void* conv_state, const void* conv_w, const float* a_log, const float* dt_bias, const void* norm_w,
                 const float* state, void* k_out, void* v_out, float* g_out, float* beta_out, void* out_packed, void* out_rows,
                 const int* seq_start, int rows, int n_seqs, int k_heads, int v_heads, int dk, int dv, int taps, int group, float eps,
                 void* stream) {
    if (rows < 1 || rows > TF_QMM_MAX_ROWS || n_seqs < 1 || n_seqs > 65535 || k_heads < 1 || v_heads < 1 || v_heads % k_heads) return TF_EINVAL;
    if (dk != 128 || dv != 128 || taps != 4 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!qkv || !z || !a || !b || !conv_state || !conv_w || !a_log || !dt_bias || !norm_w || !state || !seq_start) return TF_EINVAL;
    if (!k_out || !v_out || !g_out || !beta_out || (!out_packed && !out_rows) || qkv_stride % 4 || z_stride % 4) return TF_EINVAL;
    if (((uintptr_t)qkv | (uintptr_t)conv_state | (uintptr_t)k_out | (uintptr_t)v_out) & 7) return TF_EALIGN;
    if (((uintptr_t)z) & 7) return TF_EALIGN;
    if (((uintptr_t)conv_w | (uintptr_t)norm_w | (uintptr_t)state | (uintptr_t)out_packed | (uintptr_t)out_rows) & 15) return TF_EALIGN;
    tf::GdnFusedArgs g = {};
    g.qkv = static_cast<const __nv_bfloat16*>(qkv); g.qkv_stride = qkv_stride;
    g.z = static_cast<const __nv_bfloat16*>(z); g.z_stride = z_stride;
    g.a_in = static_cast<const __nv_bfloat16*>(a); g.b_in = static_cast<const __nv_bfloat16*>(b); g.ab_stride = ab_stride;
    g.conv_state = static_cast<const __nv_bfloat16*>(conv_state); g.conv_w = static_cast<const __nv_bfloat16*>(conv_w);
    g.a_log = a_log; g.dt_bias = dt_bias; g.norm_w = static_cast<const __nv_bfloat16*>(norm_w); g.state_in = state;
    g.k_out = static_cast<__nv_bfloat16*>(k_out); g.v_out = static_cast<__nv_bfloat16*>(v_out); g.g_out = g_out; g.beta_out = beta_out;
    g.out_packed = static_cast<uint8_t*>(out_packed); g.out_rows = static_cast<__nv_bfloat16*>(out_rows);
    g.seq_start = seq_start; g.KH = k_heads; g.VH = v_heads; g.S = n_seqs; g.R = rows; g.group = group; g.eps = eps;
    void* args[] = {&g};
    const void* fn = group == 64 ? (const void*)tf::gdn_fused_kernel<64> : (const void*)tf::gdn_fused_kernel<32>;
    cudaError_t e = tf::launch_pdl(fn, dim3(v_heads, n_seqs), dim3(512), 0, static_cast<cudaStream_t>(stream), args);
    if (e != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

int tf_gdn_replay(const void* k, const void* v, const float* g, const float* beta, float* state, const int* seq_start,
                  const int* keep, int n_seqs, int layers, long long rec_k_stride, long long rec_v_stride,
                  long long rec_g_stride, long long state_stride, int k_heads, int v_heads, int dk, int dv, void* stream) {
    if (tf::check(n_seqs, layers, k_heads, v_heads, dk, dv) != TF_OK) return TF_EINVAL;
    if (!k || !v || !g || !beta || !state || !seq_start || !keep) return TF_EINVAL;
    if ((uintptr_t)state & 15 || state_stride % 4 || (((uintptr_t)k | (uintptr_t)v) & 15) || rec_k_stride % 8 || rec_v_stride % 8) return TF_EALIGN;
    tf::GdnArgs a = {};
    a.q = nullptr; a.k = static_cast<const __nv_bfloat16*>(k);
    a.v = static_cast<const __nv_bfloat16*>(v); a.g = g; a.beta = beta;
    a.state_in = state; a.state_out = state; a.y = nullptr;          // each thread rewrites only what it read
    a.seq_start = seq_start; a.keep = keep;
    a.KH = k_heads; a.VH = v_heads; a.DV = dv; a.S = n_seqs;
    a.rec_q = rec_k_stride; a.rec_v = rec_v_stride; a.rec_g = rec_g_stride; a.rec_state = state_stride;
    void* args[] = {&a};
    dim3 grid((dv + tf::kRowsPerCta - 1) / tf::kRowsPerCta, v_heads, n_seqs * layers);
    cudaError_t e = tf::launch_pdl((const void*)tf::gdn_kernel<false>, grid, dim3(tf::kRowsPerCta * 4), 0,
                                   static_cast<cudaStream_t>(stream), args);
    if (e != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

int tf_conv_commit(const void* qkv, size_t qkv_stride, long long rec_qkv_stride, void* conv_state, long long state_stride,
                   const int* seq_start, const int* keep, int n_seqs, int layers, int channels, void* stream) {
    if (n_seqs < 1 || layers < 1 || channels < 8 || channels % 8 || qkv_stride % 8) return TF_EINVAL;
    if (!qkv || !conv_state || !seq_start || !keep || (long long)n_seqs * layers > 65535) return TF_EINVAL;
    if (((uintptr_t)qkv | (uintptr_t)conv_state) & 15 || rec_qkv_stride % 8 || state_stride % 8) return TF_EALIGN;
    void* args[] = {&qkv, &qkv_stride, &rec_qkv_stride, &conv_state, &state_stride, &seq_start, &keep, &channels, &n_seqs};
    dim3 grid((channels / 8 + 127) / 128, 1, n_seqs * layers);
    cudaError_t e = tf::launch_pdl((const void*)tf::conv_commit_kernel, grid, dim3(128), 0, static_cast<cudaStream_t>(stream), args);
    if (e != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

}  // extern "C"
