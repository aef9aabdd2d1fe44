// The small kernels between the matmuls of a verify forward, each one step between two matmuls:
//   norm_xs     residual add (bf16, or fp32 per-rank partials summed in rank order) + RMSNorm
//   gdn_pre     causal depthwise conv over each row's own path + SiLU + q/k RMS scale + g, beta
//   gated_norm  per-head RMSNorm(y) * w * silu(z)
//   swiglu      silu(gate) * up
//   attn_prep   per-head RMSNorm + partial rotate-half RoPE at the row's own position
//   gate_mul    attention output * sigmoid(gate)
//   embed       dequantise one 4-bit embedding row per token
// Every value is a function of its own row only (each row is handled by its own CTA or warp, and
// every reduction has a fixed shape), so a row's bits never depend on the window it rides in.
// Kernels that feed a matmul write its input in packed form with the group sums (common.cuh).
// Math is fp32 with bf16 storage where the model stores bf16, unfused (--fmad=false) unless an
// fma is written out.

#include "common.cuh"

namespace tf {
namespace {

__device__ __forceinline__ float inv_rms(float sumsq, int n, float eps) { return 1.0f / sqrtf(sumsq / (float)n + eps); }

// Sum over the whole CTA in a fixed order: xor-tree inside each warp, then the warp totals in warp
// order. Every thread gets the result. `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nw; ++i) total += scratch[i];
    __syncthreads();
    return total;
}

// ---- norm_xs ------------------------------------------------------------------------------------
// One CTA per row, D/8 threads, 8 elements a thread.
// Tensor-parallel form: the residual's addend arrives as self-signalling packets in this rank's exchange
// buffer, written by every rank's row-parallel matmul (tf_qmm_peer): block p of slot n & 1 holds rank p's
// fp32 partial as {row 2i, n, row 2i+1, n}. The kernel waits (bounded) for the exchange number n = *seq + 1 in
// every packet it needs, adds the ranks in order and rounds once; the last CTA to finish advances *seq.
struct PeerIn {
    const uint8_t* mine;        // this rank's buffer (null: not the peer form)
    size_t slot_bytes;
    uint32_t* seq;
    int* tickets;
    int* status;
    int world;
    unsigned spin_limit;
};

__device__ __forceinline__ uint4 ld_volatile16(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <int G>
__global__ void norm_xs_kernel(const __nv_bfloat16* x, const __nv_bfloat16* r, const float* parts, int nparts,
                               size_t part_stride, const __nv_bfloat16* w, __nv_bfloat16* h_out,
                               __nv_bfloat16* y_rows, uint8_t* y_packed, int M, int D, float eps, const PeerIn peer) {
    __shared__ float scratch[32];
    __shared__ int is_last;
    pdl_launch_dependents();
    // In the peer form the kernel does NOT wait for its predecessor (the row-parallel matmul) to complete: its
    // other inputs are older than that, and the matmul's output arrives as packets that announce themselves,
    // so the wait below is on the data, not on the grid. This hides the completion of the matmul's remote
    // stores (an NVLink round trip). Whoever runs after this kernel still waits for it, and it ends only
    // after every rank's packets of this exchange have arrived.
    if (peer.mine == nullptr) pdl_wait();
    const int row = blockIdx.x, c = threadIdx.x;           // chunk c = elements 8c..8c+7
    if (row >= M) {                                        // padding rows of the packed buffer are zero
        if (y_packed != nullptr) packed_store<G>(y_packed, tf_padded_rows(M), row, c, make_uint4(0, 0, 0, 0), 0.f);
        return;
    }
    const size_t at = (size_t)row * (D >> 3) + c;
    float h[8];
    unpack8(reinterpret_cast<const uint4*>(x)[at], h);
    if (r != nullptr || nparts > 0 || peer.mine != nullptr) {
        float add[8];
        if (peer.mine != nullptr) {
            const uint32_t want = *reinterpret_cast<volatile uint32_t*>(peer.seq) + 1u;
            const uint4* slot = reinterpret_cast<const uint4*>(peer.mine + (want & 1u) * peer.slot_bytes);
            const size_t per_rank = (size_t)((M + 1) / 2) * D;
            // once a wait has run out anywhere in this process the exchange is lost: do not wait again
            bool stalled = peer.status != nullptr && *reinterpret_cast<volatile int*>(peer.status) != 0;
            for (int p = 0; p < peer.world; ++p) {
                const uint4* src = slot + p * per_rank + (size_t)(row >> 1) * D + 8 * c;
                uint4 pk[8];
                bool ready = false;
                for (unsigned spins = 0; !ready; ++spins) {
                    ready = true;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        pk[i] = ld_volatile16(src + i);
                        ready = ready && pk[i].y == want && pk[i].w == want;
                    }
                    if (stalled || spins >= peer.spin_limit) { stalled = stalled || !ready; break; }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float v = __uint_as_float((row & 1) ? pk[i].z : pk[i].x);
                    add[i] = p == 0 ? v : add[i] + v;
                }
            }
            if (stalled) report(peer.status, TF_ESTALL);
#pragma unroll
            for (int i = 0; i < 8; ++i) add[i] = round_bf16(add[i]);
        } else if (nparts > 0) {
            // a row-parallel projection's per-rank fp32 partials: rank order, one rounding
#pragma unroll
            for (int i = 0; i < 8; ++i) add[i] = 0.f;
            for (int p = 0; p < nparts; ++p) {
                const float4* src = reinterpret_cast<const float4*>(parts + p * part_stride + (size_t)row * D + 8 * c);
                const float4 a = src[0], b = src[1];
                const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) add[i] = p == 0 ? v[i] : add[i] + v[i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) add[i] = round_bf16(add[i]);
        } else {
            unpack8(reinterpret_cast<const uint4*>(r)[at], add);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = round_bf16(h[i] + add[i]);
        reinterpret_cast<uint4*>(h_out)[at] = pack8(h);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += h[i] * h[i];
    const float inv = inv_rms(block_sum(ss, scratch), D, eps);
    float wv[8], y[8];
    unpack8(reinterpret_cast<const uint4*>(w)[c], wv);
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = h[i] * inv * wv[i];
    const uint4 yv = pack8(y);
    if (y_rows != nullptr) reinterpret_cast<uint4*>(y_rows)[at] = yv;
    const float gs = group_sum8<G>(yv);
    if (y_packed != nullptr) packed_store<G>(y_packed, tf_padded_rows(M), row, c, yv, gs);
    if (peer.mine != nullptr) {
        // every live row's CTA has read the exchange number by now; the last one to get here advances it
        __syncthreads();
        if (threadIdx.x == 0) is_last = atomicAdd(peer.tickets, 1) == M - 1;
        __syncthreads();
        if (is_last && threadIdx.x == 0) {
            *peer.tickets = 0;
            *reinterpret_cast<volatile uint32_t*>(peer.seq) = *reinterpret_cast<volatile uint32_t*>(peer.seq) + 1u;
        }
    }
}

// ---- swiglu: rows x (I/8) threads -----------------------------------------------------------------
// `tiled`: gate and up come interleaved by 16-column tile in one row ([gate 16a..16a+15 | up 16a..16a+15] for
// activation tile a), the order in which the lane matmul's SwiGLU epilogue wants the stacked weight; `gate` is then
// the row's start and `up` is unused.
template <int G>
__global__ void swiglu_kernel(const __nv_bfloat16* gate, const __nv_bfloat16* up, size_t in_stride, uint8_t* out_packed,
                              __nv_bfloat16* out_rows, int M, int I, int tiled) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    uint4 ov = make_uint4(0, 0, 0, 0);
    const bool live = c < (I >> 3) && row < M;
    if (live) {
        float g[8], u[8], o[8];
        const size_t goff = tiled ? (size_t)(c >> 1) * 32 + (c & 1) * 8 : (size_t)8 * c;
        const __nv_bfloat16* urow = tiled ? gate + 16 : up;
        unpack8(*reinterpret_cast<const uint4*>(gate + (size_t)row * in_stride + goff), g);
        unpack8(*reinterpret_cast<const uint4*>(urow + (size_t)row * in_stride + goff), u);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = g[i] * sigmoidf_(g[i]) * u[i];
        ov = pack8(o);
    }
    const float gs = group_sum8<G>(ov);
    if (c >= (I >> 3)) return;
    if (live && out_rows != nullptr) reinterpret_cast<uint4*>(out_rows)[(size_t)row * (I >> 3) + c] = ov;
    packed_store<G>(out_packed, tf_padded_rows(M), row, c, ov, gs);
}

// ---- gated_norm: 16 lanes per (row, head) of 128 values --------------------------------------------
template <int G>
__global__ void gated_norm_kernel(const __nv_bfloat16* y, const __nv_bfloat16* z, size_t z_stride, const __nv_bfloat16* w,
                                  uint8_t* out_packed, __nv_bfloat16* out_rows, int M, int VH, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;   // chunk of 8 inside the row: head = c / 16
    const int total = VH * 16;
    uint4 ov = make_uint4(0, 0, 0, 0);
    const bool live = c < total && row < M;
    float yv[8], zv[8], wv[8], o[8];
    float ss = 0.f;
    if (live) {
        unpack8(reinterpret_cast<const uint4*>(y)[(size_t)row * total + c], yv);
        unpack8(*reinterpret_cast<const uint4*>(z + (size_t)row * z_stride + 8 * c), zv);
        unpack8(reinterpret_cast<const uint4*>(w)[c & 15], wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += yv[i] * yv[i];
    }
#pragma unroll
    for (int o2 = 1; o2 < 16; o2 <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
    if (live) {
        const float inv = inv_rms(ss, 128, eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = zv[i] * sigmoidf_(zv[i]) * (yv[i] * inv * wv[i]);
        ov = pack8(o);
    }
    const float gs = group_sum8<G>(ov);
    if (c >= total) return;
    if (live && out_rows != nullptr) reinterpret_cast<uint4*>(out_rows)[(size_t)row * total + c] = ov;
    packed_store<G>(out_packed, tf_padded_rows(M), row, c, ov, gs);
}

// ---- gate_mul: one warp per (row, head), D/32 values a lane (D = 128 or 256) -----------------------
template <int G>
__global__ void gate_mul_kernel(const __nv_bfloat16* o, const __nv_bfloat16* qg, size_t qg_stride, uint8_t* out_packed,
                                __nv_bfloat16* out_rows, int M, int H, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;   // chunk of 8 in the row's H*D values
    const int per_head = D >> 3, total = H * per_head;
    uint4 ov = make_uint4(0, 0, 0, 0);
    const bool live = c < total && row < M;
    if (live) {
        const int head = c / per_head, cc = c - head * per_head;
        float a[8], g[8], r[8];
        unpack8(reinterpret_cast<const uint4*>(o)[(size_t)row * total + c], a);
        unpack8(*reinterpret_cast<const uint4*>(qg + (size_t)row * qg_stride + (size_t)head * 2 * D + D + 8 * cc), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = a[i] * sigmoidf_(g[i]);
        ov = pack8(r);
    }
    const float gs = group_sum8<G>(ov);
    if (c >= total) return;
    if (live && out_rows != nullptr) reinterpret_cast<uint4*>(out_rows)[(size_t)row * total + c] = ov;
    packed_store<G>(out_packed, tf_padded_rows(M), row, c, ov, gs);
}

// ---- attn_prep: one warp per (row, head); heads 0..H-1 queries, H..H+HK-1 keys, then HK value copies ---
__global__ void attn_prep_kernel(const __nv_bfloat16* qg, size_t qg_stride, const __nv_bfloat16* kin, size_t k_stride,
                                 const __nv_bfloat16* vin, size_t v_stride, const __nv_bfloat16* q_norm,
                                 const __nv_bfloat16* k_norm, const int* row_pos, const float* inv_freq, int half,
                                 __nv_bfloat16* q_out, __nv_bfloat16* k_out, __nv_bfloat16* v_out, int H, int HK, int D,
                                 float eps) {
    extern __shared__ float xn_s[];                        // [warps][D] normalised bf16 values as fp32
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int head = blockIdx.x * (blockDim.x >> 5) + wib;
    if (head >= H + 2 * HK) return;
    const int per = D >> 5;                                // values per lane
    if (head >= H + HK) {                                  // value rows: plain copy into the contiguous record
        const int hv = head - H - HK;
        const __nv_bfloat16* vs = vin + (size_t)row * v_stride + (size_t)hv * D + lane * per;
        __nv_bfloat16* vd = v_out + ((size_t)row * HK + hv) * D + lane * per;
        if (per == 8) *reinterpret_cast<uint4*>(vd) = *reinterpret_cast<const uint4*>(vs);      // head_dim 256: one 16-byte copy
        else if (per == 4) *reinterpret_cast<uint2*>(vd) = *reinterpret_cast<const uint2*>(vs);
        else for (int i = 0; i < per; ++i) vd[i] = vs[i];
        return;
    }
    const bool is_q = head < H;
    const __nv_bfloat16* src = is_q ? qg + (size_t)row * qg_stride + (size_t)head * 2 * D
                                    : kin + (size_t)row * k_stride + (size_t)(head - H) * D;
    const __nv_bfloat16* wn = is_q ? q_norm : k_norm;
    float* xn = xn_s + wib * D;
    float v[8];
    float ss = 0.f;
    if (per == 8) unpack8(*reinterpret_cast<const uint4*>(src + lane * 8), v);                    // same values, one 16-byte load
    else for (int i = 0; i < per; ++i) v[i] = bf2f(src[lane * per + i]);
    for (int i = 0; i < per; ++i) ss += v[i] * v[i];
    const float inv = inv_rms(warp_sum(ss), D, eps);
    for (int i = 0; i < per; ++i) xn[lane * per + i] = round_bf16(v[i] * inv * bf2f(wn[lane * per + i]));
    __syncwarp();
    const float pos = (float)row_pos[row];
    __nv_bfloat16* dst = is_q ? q_out + ((size_t)row * H + head) * D : k_out + ((size_t)row * HK + head - H) * D;
    for (int i = 0; i < per; ++i) {
        const int d = lane * per + i;
        float out = xn[d];
        if (d < 2 * half) {
            const int f = d < half ? d : d - half;
            const float ang = pos * inv_freq[f];
            const float cs = cosf(ang), sn = sinf(ang);
            out = d < half ? xn[d] * cs - xn[d + half] * sn : xn[d] * cs + xn[d - half] * sn;
        }
        dst[d] = f2bf(out);
    }
}

// ---- gdn_pre: one warp per (row, head of [q heads | k heads | v heads]); head size 128 -----------------
__global__ void gdn_pre_kernel(const __nv_bfloat16* qkv, size_t qkv_stride, const __nv_bfloat16* conv_state,
                               const __nv_bfloat16* conv_w, const int* row_seq, const int* row_idx,
                               const __nv_bfloat16* a_in, const __nv_bfloat16* b_in, size_t ab_stride, const float* a_log,
                               const float* dt_bias, __nv_bfloat16* q_out, __nv_bfloat16* k_out, __nv_bfloat16* v_out,
                               float* g_out, float* beta_out, int KH, int VH) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, lane = threadIdx.x & 31;
    const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (head >= 2 * KH + VH) return;
    const int C = (2 * KH + VH) * 128;
    const int seq = row_seq[row], idx = row_idx[row];      // idx: the row's place in its sequence's chain
    const int ch0 = head * 128 + lane * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // the 4 taps of this lane's 4 channels are 16 consecutive bf16 values: two 16-byte loads
    float wt[16];
    {
        const uint4* wp = reinterpret_cast<const uint4*>(conv_w + (size_t)ch0 * 4);
        float lo[8], hi[8];
        unpack8(wp[0], lo);
        unpack8(wp[1], hi);
#pragma unroll
        for (int i = 0; i < 8; ++i) { wt[i] = lo[i]; wt[8 + i] = hi[i]; }
    }
    // taps 0..3 read rows idx-3..idx of [conv_state (3 rows); this sequence's window rows]
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int src = idx + j;                           // index into the concatenation
        const __nv_bfloat16* p = src < 3 ? conv_state + ((size_t)seq * 3 + src) * C + ch0
                                         : qkv + (size_t)(row - idx + src - 3) * qkv_stride + ch0;
        const uint2 xv = *reinterpret_cast<const uint2*>(p);
        const float xf[4] = {bf16_lo(xv.x), bf16_hi(xv.x), bf16_lo(xv.y), bf16_hi(xv.y)};
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = __fmaf_rn(xf[i], wt[i * 4 + j], acc[i]);
    }
    float c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = round_bf16(acc[i] * sigmoidf_(acc[i]));
    if (head < 2 * KH) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) ss += c[i] * c[i];
        const float inv = inv_rms(warp_sum(ss), 128, 1e-6f);
        const bool is_q = head < KH;
        const float scale = is_q ? 1.0f / 128.0f : 0.08838834764831845f;   // 1/dk, dk^-1/2
        __nv_bfloat16* dst = (is_q ? q_out + ((size_t)row * KH + head) * 128 : k_out + ((size_t)row * KH + head - KH) * 128) + lane * 4;
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(c[0] * inv * scale, c[1] * inv * scale),
                                                    pack_bf16(c[2] * inv * scale, c[3] * inv * scale));
    } else {
        const int hv = head - 2 * KH;
        *reinterpret_cast<uint2*>(v_out + ((size_t)row * VH + hv) * 128 + lane * 4) =
            make_uint2(pack_bf16(c[0], c[1]), pack_bf16(c[2], c[3]));
        if (lane == 0) {
            const float a = bf2f(a_in[(size_t)row * ab_stride + hv]) + dt_bias[hv];
            const float sp = a > 20.0f ? a : logf(1.0f + expf(a));
            g_out[(size_t)row * VH + hv] = expf(-expf(a_log[hv]) * sp);
            beta_out[(size_t)row * VH + hv] = sigmoidf_(bf2f(b_in[(size_t)row * ab_stride + hv]));
        }
    }
}

// ---- embed: one thread per packed word (8 values) of the output row ---------------------------------
__global__ void embed_kernel(const int* ids, const uint32_t* words, const __nv_bfloat16* scales,
                             const __nv_bfloat16* biases, __nv_bfloat16* out, int D, int G, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= (D >> 3)) return;
    int tok = ids[row];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const uint32_t w = words[(size_t)tok * (D >> 3) + c];
    const float s = bf2f(scales[(size_t)tok * (D / G) + (8 * c) / G]);
    const float b = bf2f(biases[(size_t)tok * (D / G) + (8 * c) / G]);
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (float)((w >> (4 * i)) & 0xFu) * s + b;
    reinterpret_cast<uint4*>(out)[(size_t)row * (D >> 3) + c] = pack8(v);
}

inline int finish(cudaError_t e) {
    if (e != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

}  // namespace
}  // namespace tf

extern "C" {

int tf_norm_xs(const void* x, const void* residual, const void* partials, int nparts, size_t part_stride, const void* weight,
               void* h_out, void* y_rows, void* y_packed, int M, int D, int group, float eps, void* stream) {
    return tf_norm_xs_peer(x, residual, partials, nparts, part_stride, weight, h_out, y_rows, y_packed, M, D, group, eps, nullptr, 0,
                           nullptr, nullptr, 0, nullptr, stream);
}

int tf_norm_xs_peer(const void* x, const void* residual, const void* partials, int nparts, size_t part_stride, const void* weight,
                    void* h_out, void* y_rows, void* y_packed, int M, int D, int group, float eps, const void* my_buf,
                    size_t slot_bytes, void* seq, void* tickets, int world, int* status, void* stream) {
    if (my_buf && (residual || nparts > 0 || !seq || !tickets || world < 2 || world > 64 || ((uintptr_t)my_buf & 15) || (slot_bytes & 15)))
        return TF_EINVAL;
    if (my_buf && slot_bytes < tf_peer_slot_bytes(M, D, world)) return TF_EINVAL;
    if (M < 1 || M > TF_QMM_MAX_ROWS || D < 256 || D % 256 || D > 8192 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!x || !weight || nparts < 0 || (nparts > 0 && !partials) || (residual && nparts > 0)) return TF_EINVAL;
    if ((residual || nparts > 0 || my_buf) && !h_out) return TF_EINVAL;
    if (((uintptr_t)x | (uintptr_t)residual | (uintptr_t)partials | (uintptr_t)weight | (uintptr_t)h_out |
         (uintptr_t)y_rows | (uintptr_t)y_packed) & 15) return TF_EALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    tf::PeerIn peer = {static_cast<const uint8_t*>(my_buf), slot_bytes, static_cast<uint32_t*>(seq), static_cast<int*>(tickets),
                       status, world, tf::poll_limit_ref()};
    void* args[] = {&x, &residual, &partials, &nparts, &part_stride, &weight, &h_out, &y_rows, &y_packed, &M, &D, &eps, &peer};
    const void* fn = group == 64 ? (const void*)tf::norm_xs_kernel<64> : (const void*)tf::norm_xs_kernel<32>;
    return tf::finish(tf::launch_pdl(fn, dim3(y_packed ? tf::tf_padded_rows(M) : M), dim3(D / 8), 0, st, args, 2));
}

int tf_swiglu(const void* gate, const void* up, size_t in_stride, void* out_packed, void* out_rows, int M, int I,
              int group, void* stream) {
    if (M < 1 || M > TF_QMM_MAX_ROWS || I < 64 || I % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!gate || !up || !out_packed || in_stride % 8) return TF_EINVAL;
    if (((uintptr_t)gate | (uintptr_t)up | (uintptr_t)out_packed | (uintptr_t)out_rows) & 15) return TF_EALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int tiled = 0;
    void* args[] = {&gate, &up, &in_stride, &out_packed, &out_rows, &M, &I, &tiled};
    const void* fn = group == 64 ? (const void*)tf::swiglu_kernel<64> : (const void*)tf::swiglu_kernel<32>;
    return tf::finish(tf::launch_pdl(fn, dim3((I / 8 + 255) / 256, tf::tf_padded_rows(M)), dim3(256), 0, st, args, 3));
}

int tf_swiglu_tiled(const void* gate_up, size_t in_stride, void* out_packed, void* out_rows, int M, int I, int group, void* stream) {
    if (M < 1 || M > TF_QMM_MAX_ROWS || I < 64 || I % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!gate_up || !out_packed || in_stride % 8 || in_stride < (size_t)2 * I) return TF_EINVAL;
    if (((uintptr_t)gate_up | (uintptr_t)out_packed | (uintptr_t)out_rows) & 15) return TF_EALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int tiled = 1;
    const void* up = nullptr;
    void* args[] = {&gate_up, &up, &in_stride, &out_packed, &out_rows, &M, &I, &tiled};
    const void* fn = group == 64 ? (const void*)tf::swiglu_kernel<64> : (const void*)tf::swiglu_kernel<32>;
    return tf::finish(tf::launch_pdl(fn, dim3((I / 8 + 255) / 256, tf::tf_padded_rows(M)), dim3(256), 0, st, args, 3));
}

int tf_gated_norm(const void* y, const void* z, size_t z_stride, const void* weight, void* out_packed, void* out_rows,
                  int M, int v_heads, int dv, int group, float eps, void* stream) {
    if (M < 1 || M > TF_QMM_MAX_ROWS || v_heads < 1 || dv != 128 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!y || !z || !weight || !out_packed || z_stride % 8 || (v_heads * dv) % 64) return TF_EINVAL;
    if (((uintptr_t)y | (uintptr_t)z | (uintptr_t)weight | (uintptr_t)out_packed | (uintptr_t)out_rows) & 15) return TF_EALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* args[] = {&y, &z, &z_stride, &weight, &out_packed, &out_rows, &M, &v_heads, &eps};
    const void* fn = group == 64 ? (const void*)tf::gated_norm_kernel<64> : (const void*)tf::gated_norm_kernel<32>;
    return tf::finish(tf::launch_pdl(fn, dim3((v_heads * 16 + 255) / 256, tf::tf_padded_rows(M)), dim3(256), 0, st, args, 3));
}

int tf_gate_mul(const void* o, const void* qg, size_t qg_stride, void* out_packed, void* out_rows, int M, int heads,
                int head_dim, int group, void* stream) {
    if (M < 1 || M > TF_QMM_MAX_ROWS || heads < 1 || (head_dim != 128 && head_dim != 256)) return TF_EINVAL;
    if ((group != 64 && group != 32) || !o || !qg || !out_packed || qg_stride % 8) return TF_EINVAL;
    if (((uintptr_t)o | (uintptr_t)qg | (uintptr_t)out_packed | (uintptr_t)out_rows) & 15) return TF_EALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* args[] = {&o, &qg, &qg_stride, &out_packed, &out_rows, &M, &heads, &head_dim};
    const void* fn = group == 64 ? (const void*)tf::gate_mul_kernel<64> : (const void*)tf::gate_mul_kernel<32>;
    return tf::finish(tf::launch_pdl(fn, dim3((heads * head_dim / 8 + 255) / 256, tf::tf_padded_rows(M)), dim3(256), 0, st, args, 3));
}

int tf_attn_prep(const void* qg, size_t qg_stride, const void* k, size_t k_stride, const void* v, size_t v_stride,
                 const void* q_norm, const void* k_norm, const int* row_pos, const float* inv_freq, int rope_half,
                 void* q_out, void* k_out, void* v_out, int M, int heads, int kv_heads, int head_dim, float eps,
                 void* stream) {
    if (M < 1 || heads < 1 || kv_heads < 1 || (head_dim != 128 && head_dim != 256)) return TF_EINVAL;
    if (rope_half < 0 || 2 * rope_half > head_dim) return TF_EINVAL;
    if (!qg || !k || !v || !q_norm || !k_norm || !row_pos || !inv_freq || !q_out || !k_out || !v_out) return TF_EINVAL;
    if ((((uintptr_t)qg | (uintptr_t)k | (uintptr_t)v | (uintptr_t)v_out) & 15) || (qg_stride | k_stride | v_stride) % 8) return TF_EALIGN;
    const int warps = 4, total = heads + 2 * kv_heads;
    void* args[] = {&qg, &qg_stride, &k, &k_stride, &v, &v_stride, &q_norm, &k_norm, &row_pos, &inv_freq, &rope_half,
                    &q_out, &k_out, &v_out, &heads, &kv_heads, &head_dim, &eps};
    return tf::finish(tf::launch_pdl((const void*)tf::attn_prep_kernel, dim3((total + warps - 1) / warps, M),
                                     dim3(warps * 32), warps * head_dim * sizeof(float), static_cast<cudaStream_t>(stream), args, 3));
}

int tf_gdn_pre(const void* qkv, size_t qkv_stride, const void* conv_state, const void* conv_w, const int* row_seq,
               const int* row_idx, const void* a, const void* b, size_t ab_stride, const float* a_log, const float* dt_bias,
               void* q_out, void* k_out, void* v_out, float* g_out, float* beta_out, int M, int k_heads, int v_heads, int dk,
               int dv, int taps, void* stream) {
    if (M < 1 || k_heads < 1 || v_heads < 1 || dk != 128 || dv != 128 || taps != 4) return TF_EINVAL;
    if (!qkv || !conv_state || !conv_w || !row_seq || !row_idx || !a || !b || !a_log || !dt_bias) return TF_EINVAL;
    if (!q_out || !k_out || !v_out || !g_out || !beta_out || qkv_stride % 4) return TF_EINVAL;
    if (((uintptr_t)qkv | (uintptr_t)conv_state | (uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)v_out) & 7) return TF_EALIGN;
    if ((uintptr_t)conv_w & 15) return TF_EALIGN;
    const int warps = 4, total = 2 * k_heads + v_heads;
    void* args[] = {&qkv, &qkv_stride, &conv_state, &conv_w, &row_seq, &row_idx, &a, &b, &ab_stride, &a_log, &dt_bias,
                    &q_out, &k_out, &v_out, &g_out, &beta_out, &k_heads, &v_heads};
    return tf::finish(tf::launch_pdl((const void*)tf::gdn_pre_kernel, dim3((total + warps - 1) / warps, M), dim3(warps * 32),
                                     0, static_cast<cudaStream_t>(stream), args, 3));
}

int tf_embed(const int* ids, const void* words, const void* scales, const void* biases, void* out, int M, int D, int group,
             int vocab, void* stream) {
    if (M < 1 || D < 64 || D % 64 || (group != 64 && group != 32) || vocab < 1) return TF_EINVAL;
    if (!ids || !words || !scales || !biases || !out) return TF_EINVAL;
    if ((uintptr_t)out & 15) return TF_EALIGN;
    void* args[] = {&ids, &words, &scales, &biases, &out, &D, &group, &vocab};
    return tf::finish(tf::launch_pdl((const void*)tf::embed_kernel, dim3((D / 8 + 127) / 128, M), dim3(128), 0,
                                     static_cast<cudaStream_t>(stream), args));
}

}  // extern "C"
