// 4-bit group-affine lane matmul for sm_100a: weights stream once from HBM through a bulk-copy
// (TMA) pipeline into shared memory, are expanded to bf16 in registers and multiplied on the
// tensor cores; the scale/bias epilogue and the K-segment sums run in fp32.
//
// Arithmetic, per output element (row m, column n):
//   for each weight group g of the segment, in order:
//       P   = tensor-core chain over the group's 16-wide k-steps of  x[m,k] * (q[n,k] + 128),
//             started from  -128 * xs[m,g]            (so P = x . q up to fp32 rounding)
//       acc = fma(b[n,g], xs[m,g], fma(s[n,g], P, acc))
//   segments of K (fixed by N, K, group and the worker count only) are added in k order,
//   then one rounding to bf16.
// The chain never looks at the row count, so row m of an M-row call has the bits of a 1-row call.
//
// Tile layout of a weight (built by tf_qmm_tile): records indexed [column tile of 16][k tile of 64],
// each record = 512 bytes of nibbles + 64*(64/group) bytes of (scale, bias) pairs.
//   nibbles: lane (g = lane/4, t = lane%4) owns 16 bytes = 4 words; word s (k-step s) holds, at
//            nibble j, column 16c + g + 8*(j&1) and k = 64kt + 16t + 4s + {0,2,1,3}[j>>1 & 3]... see
//            nibble_k() below. (w >> 4i) & 0x000F000F is then register i of the mma A fragment.
//   pairs  : for each half-tile h (one per group inside the k tile) and g in 0..7:
//            bf16 s[16c+g], b[16c+g], s[16c+g+8], b[16c+g+8]   (8 bytes, one load per lane)
// The B operand (activations) uses the matching k order: lane (g, t) reads x[row g][64kt + 16t ..+16],
// 32 contiguous bytes, and feeds k-step s with elements 4s..4s+3 of them.

#include "common.cuh"

namespace tf {
namespace {

constexpr int kWorkers = 148;
constexpr int kItemTiles = 4;   // k tiles per schedule item: the same for every row bucket, so that the
                                // K segments (hence the bits) do not depend on the row count

__host__ __device__ constexpr int rec_bytes(int group) { return 512 + (64 / group) * 64; }

// position inside the 4-element k quad that nibble j of a word carries
__host__ __device__ constexpr int nibble_quad(int j) { return ((j >> 1) & 1) * 2 + ((j >> 2) & 1); }

template <int G, int MB, int WARPS, int KTS, int STAGES>
struct Cfg {
    static constexpr int REC = rec_bytes(G);
    static constexpr int GPT = 64 / G;                 // groups per k tile
    static constexpr int ROWS = MB * 8;
    static constexpr int XROW = KTS * 128 + 16;        // bytes per staged activation row (+16: bank spread)
    static constexpr int W_BYTES = WARPS * KTS * REC;
    static constexpr int X_BYTES = ROWS * XROW;
    static constexpr int XS_BYTES = ROWS * KTS * GPT * 4;
    static constexpr int STAGE_BYTES = ((W_BYTES + X_BYTES + XS_BYTES + 127) / 128) * 128;
    static constexpr int COLS = WARPS * 16;            // columns per column block
    static constexpr int THREADS = (WARPS + 1) * 32;   // consumers + one producer warp
    static constexpr int SMEM = STAGES * STAGE_BYTES + 2 * STAGES * 8 + 128;
};

struct Args {
    const __nv_bfloat16* x;
    const float* xs;
    const uint8_t* w;
    void* y;
    int* counters;
    float* slots;
    int* status;
    int M, N, K;
    int f32_out;
};

// The CTA that owns flattened work item `w` (items split evenly over kWorkers CTAs).
__host__ __device__ inline int owner_of(long long w, long long total) {
    return (int)(((w + 1) * kWorkers - 1) / total);
}
__host__ __device__ inline long long range_begin(int cta, long long total) { return (long long)cta * total / kWorkers; }

template <int G, int MB, int WARPS, int KTS, int STAGES>
__global__ void __launch_bounds__((WARPS + 1) * 32, 1) qmm_kernel(const Args a) {
    using C = Cfg<G, MB, WARPS, KTS, STAGES>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = a.K >> 6;                        // k tiles
    const int KG = a.K / G;                         // groups per row
    const int NT = (a.N + 15) >> 4;                 // column tiles
    const int CB = (NT + WARPS - 1) / WARPS;        // column blocks
    static_assert(kItemTiles % KTS == 0, "a schedule item is a whole number of pipeline stages");
    const int SPB = (KT + kItemTiles - 1) / kItemTiles;   // schedule items per column block
    const long long total = (long long)CB * SPB;
    const long long begin = range_begin(blockIdx.x, total), end = range_begin(blockIdx.x + 1, total);

    uint8_t* stage0 = smem;
    const uint32_t bars = smem_u32(smem + STAGES * C::STAGE_BYTES);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 33);             // producer lane 0 (with tx bytes) + 32 async xs arrivals
            mbar_init(empty_bar(s), WARPS);
        }
        mbar_fence_init();
    }
    // rows beyond M are never copied: keep them zero so the unused accumulator rows stay finite
    for (int s = 0; s < STAGES; ++s) {
        uint8_t* xb = stage0 + s * C::STAGE_BYTES + C::W_BYTES;
        for (int i = threadIdx.x; i < (C::X_BYTES + C::XS_BYTES) / 16; i += C::THREADS)
            reinterpret_cast<uint4*>(xb)[i] = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async();
    __syncthreads();
    pdl_wait();                                     // activations come from the previous kernel

    if (warp == WARPS) {
        // ------------------------------- producer warp ----------------------------------------
        int cnt = 0;
        for (long long it = begin; it < end; ++it)
        for (int sub = 0; sub < kItemTiles; sub += KTS) {
            const int cb = (int)(it / SPB), st = (int)(it % SPB);
            const int kt0 = st * kItemTiles + sub, nkt = min(KTS, KT - kt0);
            if (nkt <= 0) break;
            const int s = cnt % STAGES;
            const uint32_t parity = ((cnt / STAGES) & 1) ^ 1;
            mbar_wait(empty_bar(s), parity, a.status);
            uint8_t* sb = stage0 + s * C::STAGE_BYTES;
            const int tiles = min(WARPS, NT - cb * WARPS);
            if (lane == 0) mbar_arrive_expect_tx(full_bar(s), (uint32_t)(tiles * nkt * C::REC + a.M * nkt * 128));
            __syncwarp();
            for (int w = lane; w < tiles; w += 32) {
                const long long ct = (long long)cb * WARPS + w;
                bulk_g2s(smem_u32(sb + w * KTS * C::REC), a.w + (ct * KT + kt0) * C::REC, (uint32_t)(nkt * C::REC),
                         full_bar(s));
            }
            for (int r = lane; r < a.M; r += 32)
                bulk_g2s(smem_u32(sb + C::W_BYTES + r * C::XROW), a.x + (size_t)r * a.K + (size_t)kt0 * 64,
                         (uint32_t)(nkt * 128), full_bar(s));
            const int ng = nkt * C::GPT;
            for (int i = lane; i < a.M * ng; i += 32) {
                const int r = i / ng, j = i - r * ng;
                cp_async4(smem_u32(sb + C::W_BYTES + C::X_BYTES + (r * KTS * C::GPT + j) * 4),
                          a.xs + (size_t)r * KG + (size_t)kt0 * C::GPT + j);
            }
            cp_async_mbar_arrive_noinc(full_bar(s));
            ++cnt;
        }
        // drain: nothing may still be landing in shared memory when the CTA retires
        cp_async_wait<0>();
        return;
    }

    // ----------------------------------- consumer warps ---------------------------------------
    const int g = lane >> 2, t = lane & 3;
    float acc[MB][4];
    int cnt = 0;
    long long it = begin;
    while (it < end) {
        const int cb = (int)(it / SPB);
        const long long cb_begin = (long long)cb * SPB, cb_end = cb_begin + SPB;
        const long long seg_end = cb_end < end ? cb_end : end;
        const int ct = cb * WARPS + warp;
        const bool live = ct < NT;
#pragma unroll
        for (int rb = 0; rb < MB; ++rb) acc[rb][0] = acc[rb][1] = acc[rb][2] = acc[rb][3] = 0.f;

        for (; it < seg_end; ++it)
        for (int sub = 0; sub < kItemTiles; sub += KTS) {
            const int st = (int)(it - cb_begin);
            const int nkt = min(KTS, KT - (st * kItemTiles + sub));
            if (nkt <= 0) break;
            const int s = cnt % STAGES;
            mbar_wait(full_bar(s), (cnt / STAGES) & 1, a.status);
            if (live) {
                const uint8_t* sb = stage0 + s * C::STAGE_BYTES;
                const uint8_t* wrec = sb + warp * KTS * C::REC;
                const uint8_t* xrow = sb + C::W_BYTES;
                const float* xsst = reinterpret_cast<const float*>(sb + C::W_BYTES + C::X_BYTES);
                for (int kt = 0; kt < nkt; ++kt) {
                    const uint4 wq = *reinterpret_cast<const uint4*>(wrec + kt * C::REC + lane * 16);
                    const uint32_t wv[4] = {wq.x, wq.y, wq.z, wq.w};
                    uint32_t af[4][4];
#pragma unroll
                    for (int s4 = 0; s4 < 4; ++s4)
#pragma unroll
                        for (int i = 0; i < 4; ++i) af[s4][i] = ((wv[s4] >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
                    float sc[C::GPT][2], bi[C::GPT][2];
#pragma unroll
                    for (int h = 0; h < C::GPT; ++h) {
                        const uint2 p = *reinterpret_cast<const uint2*>(wrec + kt * C::REC + 512 + h * 64 + g * 8);
                        sc[h][0] = bf16_lo(p.x); bi[h][0] = bf16_hi(p.x);
                        sc[h][1] = bf16_lo(p.y); bi[h][1] = bf16_hi(p.y);
                    }
#pragma unroll
                    for (int rb = 0; rb < MB; ++rb) {
                        const uint8_t* xp = xrow + (rb * 8 + g) * C::XROW + kt * 128 + t * 32;
                        const uint4 x0 = *reinterpret_cast<const uint4*>(xp);
                        const uint4 x1 = *reinterpret_cast<const uint4*>(xp + 16);
                        const uint32_t xb[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                        for (int h = 0; h < C::GPT; ++h) {
                            const float xs0 = xsst[(rb * 8 + 2 * t) * KTS * C::GPT + kt * C::GPT + h];
                            const float xs1 = xsst[(rb * 8 + 2 * t + 1) * KTS * C::GPT + kt * C::GPT + h];
                            float p[4] = {-128.f * xs0, -128.f * xs1, -128.f * xs0, -128.f * xs1};
                            constexpr int SPG = 4 / C::GPT;   // k-steps per group
#pragma unroll
                            for (int s4 = h * SPG; s4 < (h + 1) * SPG; ++s4)
                                mma_bf16_16816(p, af[s4], xb[2 * s4], xb[2 * s4 + 1], p);
                            acc[rb][0] = __fmaf_rn(bi[h][0], xs0, __fmaf_rn(sc[h][0], p[0], acc[rb][0]));
                            acc[rb][1] = __fmaf_rn(bi[h][0], xs1, __fmaf_rn(sc[h][0], p[1], acc[rb][1]));
                            acc[rb][2] = __fmaf_rn(bi[h][1], xs0, __fmaf_rn(sc[h][1], p[2], acc[rb][2]));
                            acc[rb][3] = __fmaf_rn(bi[h][1], xs1, __fmaf_rn(sc[h][1], p[3], acc[rb][3]));
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));
            ++cnt;
        }

        // ---- segment done: whole column block -> write; part of one -> park it, last one sums ----
        const long long seg_begin = (cb_begin > begin) ? cb_begin : begin;
        const bool whole = (seg_begin == cb_begin) && (seg_end == cb_end);
        const int col0 = ct * 16 + g;
        if (whole) {
            if (live) {
#pragma unroll
                for (int rb = 0; rb < MB; ++rb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = rb * 8 + 2 * t + (i & 1), col = col0 + (i >> 1) * 8;
                        if (row < a.M && col < a.N) {
                            if (a.f32_out) reinterpret_cast<float*>(a.y)[(size_t)row * a.N + col] = acc[rb][i];
                            else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)row * a.N + col] = f2bf(acc[rb][i]);
                        }
                    }
            }
        } else {
            // slot 2*cta + 1 when this CTA entered the column block from an earlier one, else 2*cta
            float* slot = a.slots + (size_t)(2 * blockIdx.x + (begin < cb_begin ? 1 : 0)) * (TF_QMM_MAX_ROWS * C::COLS);
            if (live) {
#pragma unroll
                for (int rb = 0; rb < MB; ++rb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = rb * 8 + 2 * t + (i & 1);
                        if (row < a.M) __stcg(slot + row * C::COLS + warp * 16 + g + (i >> 1) * 8, acc[rb][i]);
                    }
            }
            __threadfence();
            named_bar_sync(1, WARPS * 32);
            __shared__ int ticket_s;
            const int first = owner_of(cb_begin, total), last = owner_of(cb_end - 1, total);
            if (threadIdx.x == 0) ticket_s = atomicAdd(a.counters + cb, 1);
            named_bar_sync(1, WARPS * 32);
            const bool reducer = ticket_s == last - first;
            named_bar_sync(1, WARPS * 32);       // everyone has read the ticket before it can be rewritten
            if (reducer) {
                __threadfence();
                const int ncol = min(C::COLS, a.N - cb * C::COLS);
                for (int idx = threadIdx.x; idx < a.M * C::COLS; idx += WARPS * 32) {
                    const int row = idx / C::COLS, col = idx - row * C::COLS;
                    if (col >= ncol) continue;
                    float sum = 0.f;
                    for (int o = first; o <= last; ++o) {
                        const int which = range_begin(o, total) < cb_begin ? 1 : 0;
                        const float v = __ldcg(a.slots + (size_t)(2 * o + which) * (TF_QMM_MAX_ROWS * C::COLS) +
                                               row * C::COLS + col);
                        sum = (o == first) ? v : sum + v;
                    }
                    const size_t at = (size_t)row * a.N + cb * C::COLS + col;
                    if (a.f32_out) reinterpret_cast<float*>(a.y)[at] = sum;
                    else reinterpret_cast<__nv_bfloat16*>(a.y)[at] = f2bf(sum);
                }
                if (threadIdx.x == 0) a.counters[cb] = 0;     // leave the counters zero for the next call
            }
        }
    }
    pdl_launch_dependents();
}

template <int G, int MB, int WARPS, int KTS, int STAGES>
int launch(const Args& a, cudaStream_t stream) {
    using C = Cfg<G, MB, WARPS, KTS, STAGES>;
    static_assert(C::SMEM <= 227 * 1024, "stage ring does not fit shared memory");
    auto kern = qmm_kernel<G, MB, WARPS, KTS, STAGES>;
    static bool configured = false;   // per instantiation; the attribute is per function and idempotent
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
            return TF_ECUDA;
        configured = true;
    }
    const int NT = (a.N + 15) / 16, CB = (NT + WARPS - 1) / WARPS;
    if (CB * 4 > TF_QMM_COUNTER_BYTES) return TF_EINVAL;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kWorkers);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, a) != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

constexpr int kWarps = 8;   // consumer warps = 128 columns per column block, for every row bucket

template <int G>
int dispatch(const Args& a, cudaStream_t stream) {
    if (a.M <= 8) return launch<G, 1, kWarps, 4, 8>(a, stream);
    if (a.M <= 16) return launch<G, 2, kWarps, 4, 6>(a, stream);
    if (a.M <= 32) return launch<G, 4, kWarps, 4, 5>(a, stream);
    if (a.M <= 64) return launch<G, 8, kWarps, 2, 5>(a, stream);
    return launch<G, 16, kWarps, 2, 4>(a, stream);
}

// ---- relayout kernels: one thread per output word / pair -----------------------------------------
__global__ void tile_kernel(const uint32_t* words, const uint16_t* scales, const uint16_t* biases, uint8_t* out,
                            int N, int K, int G) {
    const int KT = K >> 6, NT = (N + 15) >> 4, REC = rec_bytes(G), GPT = 64 / G;
    const long long recs = (long long)NT * KT;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per = 128 + 16 * GPT;                 // threads per record: 128 words + 16*GPT (s,b) pairs
    if (id >= recs * per) return;
    const long long rec = id / per;
    const int e = (int)(id % per);
    const int c = (int)(rec / KT), kt = (int)(rec % KT);
    uint8_t* r = out + rec * REC;
    if (e < 128) {
        const int lane = e >> 2, s = e & 3, g = lane >> 2, t = lane & 3;
        uint32_t w = 0;
        for (int j = 0; j < 8; ++j) {
            const int col = 16 * c + g + 8 * (j & 1);
            const int k = 64 * kt + 16 * t + 4 * s + nibble_quad(j);
            uint32_t q = 0;
            if (col < N) q = (words[(size_t)col * (K >> 3) + (k >> 3)] >> (4 * (k & 7))) & 0xFu;
            w |= q << (4 * j);
        }
        reinterpret_cast<uint32_t*>(r)[e] = w;
    } else {
        const int p = e - 128, h = p >> 4, q = p & 15, g = q >> 1, hi = q & 1;
        const int col = 16 * c + g + 8 * hi, grp = kt * GPT + h;
        uint16_t s = 0, b = 0;
        if (col < N) { s = scales[(size_t)col * (K / G) + grp]; b = biases[(size_t)col * (K / G) + grp]; }
        uint16_t* dst = reinterpret_cast<uint16_t*>(r + 512 + h * 64 + g * 8 + hi * 4);
        dst[0] = s; dst[1] = b;
    }
}

__global__ void untile_kernel(const uint8_t* in, uint32_t* words, uint16_t* scales, uint16_t* biases, int N, int K,
                              int G) {
    const int KT = K >> 6, REC = rec_bytes(G), GPT = 64 / G;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nwords = (long long)N * (K >> 3), npairs = (long long)N * (K / G);
    if (id < nwords) {
        const int col = (int)(id / (K >> 3)), wi = (int)(id % (K >> 3));
        uint32_t w = 0;
        for (int i = 0; i < 8; ++i) {
            const int k = wi * 8 + i, kt = k >> 6, kin = k & 63, t = kin >> 4, s = (kin >> 2) & 3, quad = kin & 3;
            const int c = col >> 4, cin = col & 15, g = cin & 7, hi = cin >> 3;
            // inverse of nibble_quad: quad {0,1,2,3} sits at (j>>1) = {0,2,1,3}
            const int j = hi + 2 * (((quad & 1) << 1) | (quad >> 1));
            const uint32_t v = reinterpret_cast<const uint32_t*>(in + ((long long)c * KT + kt) * REC)[(g * 4 + t) * 4 + s];
            w |= ((v >> (4 * j)) & 0xFu) << (4 * i);
        }
        words[id] = w;
    } else if (id < nwords + npairs) {
        const long long p = id - nwords;
        const int col = (int)(p / (K / G)), grp = (int)(p % (K / G));
        const int kt = grp / GPT, h = grp % GPT, c = col >> 4, cin = col & 15, g = cin & 7, hi = cin >> 3;
        const uint16_t* src =
            reinterpret_cast<const uint16_t*>(in + ((long long)c * KT + kt) * REC + 512 + h * 64 + g * 8 + hi * 4);
        scales[p] = src[0];
        biases[p] = src[1];
    }
}

template <int G>
__global__ void group_sums_kernel(const __nv_bfloat16* x, float* xs, int M, int K) {
    // one lane per 8 contiguous inputs: sequential sum of 8, then a pairwise tree across G/8 lanes
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long chunks = (long long)M * (K >> 3);
    float s = 0.f;
    if (id < chunks) {
        const uint4 v = reinterpret_cast<const uint4*>(x)[id];
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { s += bf16_lo(u[i]); s += bf16_hi(u[i]); }
    }
#pragma unroll
    for (int o = 1; o < G / 8; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (id < chunks && (id & (G / 8 - 1)) == 0) xs[id / (G / 8)] = s;
}

}  // namespace
}  // namespace tf

extern "C" {

int tf_version(void) { return 1000; }
int tf_qmm_workers(void) { return tf::kWorkers; }

size_t tf_qmm_tiled_bytes(int N, int K, int group) {
    if (N <= 0 || K <= 0 || K % 64 || (group != 64 && group != 32)) return 0;
    return (size_t)((N + 15) / 16) * (K / 64) * tf::rec_bytes(group);
}

size_t tf_qmm_scratch_bytes(int M, int N, int K, int group) {
    (void)M; (void)N; (void)K; (void)group;
    // counters + two parked partial blocks (128 rows x 128 columns fp32) per worker
    return TF_QMM_COUNTER_BYTES + (size_t)2 * tf::kWorkers * TF_QMM_MAX_ROWS * (tf::kWarps * 16) * sizeof(float);
}

int tf_qmm(const void* x, const void* xs, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M,
           int N, int K, int group, int flags, int* status, void* stream) {
    if (M < 1 || M > TF_QMM_MAX_ROWS || N < 1 || K < 64 || K % 64) return TF_EINVAL;
    if (group != 64 && group != 32) return TF_EINVAL;
    if (flags & ~TF_QMM_F32_OUT) return TF_EINVAL;
    if (!x || !xs || !w_tiled || !y) return TF_EINVAL;
    if (((uintptr_t)x | (uintptr_t)w_tiled) & 15) return TF_EALIGN;
    if (((uintptr_t)xs | (uintptr_t)y) & 3) return TF_EALIGN;
    if (!scratch || ((uintptr_t)scratch & 255)) return TF_ESCRATCH;
    if (scratch_bytes < tf_qmm_scratch_bytes(M, N, K, group)) return TF_ESCRATCH;
    tf::Args a;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.xs = static_cast<const float*>(xs);
    a.w = static_cast<const uint8_t*>(w_tiled);
    a.y = y;
    a.counters = static_cast<int*>(scratch);
    a.slots = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + TF_QMM_COUNTER_BYTES);
    a.status = status;
    a.M = M; a.N = N; a.K = K;
    a.f32_out = (flags & TF_QMM_F32_OUT) ? 1 : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return group == 64 ? tf::dispatch<64>(a, st) : tf::dispatch<32>(a, st);
}

int tf_qmm_tile(const void* words, const void* scales, const void* biases, void* w_tiled, int N, int K, int group,
                void* stream) {
    if (N < 1 || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!words || !scales || !biases || !w_tiled) return TF_EINVAL;
    const long long recs = (long long)((N + 15) / 16) * (K / 64);
    const long long threads = recs * (128 + 16 * (64 / group));
    tf::tile_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint32_t*>(words), static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases),
        static_cast<uint8_t*>(w_tiled), N, K, group);
    return cudaGetLastError() == cudaSuccess ? TF_OK : TF_ECUDA;
}

int tf_qmm_untile(const void* w_tiled, void* words, void* scales, void* biases, int N, int K, int group,
                  void* stream) {
    if (N < 1 || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!words || !scales || !biases || !w_tiled) return TF_EINVAL;
    const long long threads = (long long)N * (K / 8) + (long long)N * (K / group);
    tf::untile_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(w_tiled), static_cast<uint32_t*>(words), static_cast<uint16_t*>(scales),
        static_cast<uint16_t*>(biases), N, K, group);
    return cudaGetLastError() == cudaSuccess ? TF_OK : TF_ECUDA;
}

int tf_group_sums(const void* x, void* xs, int M, int K, int group, void* stream) {
    if (M < 1 || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!x || !xs) return TF_EINVAL;
    if ((uintptr_t)x & 15) return TF_EALIGN;
    const long long chunks = (long long)M * (K / 8);
    const unsigned blocks = (unsigned)((chunks + 255) / 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (group == 64) tf::group_sums_kernel<64><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<float*>(xs), M, K);
    else tf::group_sums_kernel<32><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<float*>(xs), M, K);
    return cudaGetLastError() == cudaSuccess ? TF_OK : TF_ECUDA;
}

}  // extern "C"
