// Gated-DeltaNet recurrence over the rows of each sequence's verify window, and the commit replay.
//
// Per (sequence, value head, value row) the fp32 state row S[0..127] (key dimension) stays in
// registers across the window's rows, split over 4 lanes of 32 values each:
//     S    <- S * g
//     mem   = S . k                      (fp32, 32 sequential fma per lane, then a 4-lane xor tree)
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
            const float decay = gs[r];
            float mem = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 kv = *reinterpret_cast<const float4*>(&ks[r][i * 16 + j * 4]);
                s[i].x *= decay; s[i].y *= decay; s[i].z *= decay; s[i].w *= decay;
                mem = __fmaf_rn(s[i].x, kv.x, mem);
                mem = __fmaf_rn(s[i].y, kv.y, mem);
                mem = __fmaf_rn(s[i].z, kv.z, mem);
                mem = __fmaf_rn(s[i].w, kv.w, mem);
            }
            mem += __shfl_xor_sync(0xffffffffu, mem, 1);
            mem += __shfl_xor_sync(0xffffffffu, mem, 2);
            const float delta = (vs[r][lr] - mem) * bs[r];
            float out = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 kv = *reinterpret_cast<const float4*>(&ks[r][i * 16 + j * 4]);
                s[i].x = __fmaf_rn(kv.x, delta, s[i].x);
                s[i].y = __fmaf_rn(kv.y, delta, s[i].y);
                s[i].z = __fmaf_rn(kv.z, delta, s[i].z);
                s[i].w = __fmaf_rn(kv.w, delta, s[i].w);
                if (OUT) {
                    const float4 qv = *reinterpret_cast<const float4*>(&qs[r][i * 16 + j * 4]);
                    out = __fmaf_rn(s[i].x, qv.x, out);
                    out = __fmaf_rn(s[i].y, qv.y, out);
                    out = __fmaf_rn(s[i].z, qv.z, out);
                    out = __fmaf_rn(s[i].w, qv.w, out);
                }
            }
            if (OUT) {
                out += __shfl_xor_sync(0xffffffffu, out, 1);
                out += __shfl_xor_sync(0xffffffffu, out, 2);
                if (j == 0) a.y[((size_t)(r0 + t0 + r) * a.VH + head) * a.DV + dvrow] = f2bf(out);
            }
        }
    }
    if (live && a.state_out != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(a.state_out + srow)[i * 4 + j] = s[i];
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
