// 4-bit group-affine lane matmul for sm_100a: weights stream once from HBM through a bulk-copy
// (TMA) pipeline into shared memory, are expanded to bf16 in registers and multiplied on the
// tensor cores; the scale/bias epilogue and the K-segment sums run in fp32.
//
// Arithmetic, per output element (row m, column n):
//   for each weight group g of the segment, in order:
//       P   = tensor-core chain over the group's 16-wide k-steps of  x[m,k] * (q[n,k] + 128),
//             started from  -128 * xs[m,g]            (so P = x . q up to fp32 rounding)
//       acc = fma(b[n,g], xs[m,g], fma(s[n,g], P, acc))
//   segments of K (fixed by N, K and the worker count only) are added in k order,
//   then one rounding to bf16.
// The chain never looks at the row count, so row m of an M-row call has the bits of a 1-row call.
//
// Weight tile layout (built by tf_qmm_tile): records indexed [column block of 256][k tile of 64]
// [column tile of 16 inside the block]; a pipeline stage (all 16 column tiles of a block, a few k
// tiles) is therefore ONE contiguous range and arrives with a single bulk copy. Each record is
// 512 bytes of nibbles + 64*(64/group) bytes of (scale, bias) pairs.
//   nibbles: lane (g = lane/4, t = lane%4) owns 16 bytes = 4 words; word s (k-step s) holds, at
//            nibble j, column 16c + g + 8*(j&1) and input tile_k(t, s, nibble_quad(j)) of the k tile,
//            so that (w >> 4i) & 0x000F000F is register i of the mma A fragment. K-steps 0,1 cover
//            inputs 0..31 of the tile and k-steps 2,3 inputs 32..63: a group of 32 is two whole k-steps.
//   pairs  : for each half-tile h (one per group inside the k tile) and g in 0..7:
//            bf16 s[16c+g], b[16c+g], s[16c+g+8], b[16c+g+8]   (8 bytes, one load per lane)
//
// Activations arrive "packed" (tf_pack_rows, or written directly by the glue kernels): per k tile,
// Mp rows (M rounded up to its bucket 8/16/32/64/128, extra rows zero) of 128 bytes (the tile's 64
// bf16 inputs, with the two 64-byte halves swapped on odd rows so that shared-memory reads spread
// over all banks), then the tile's group sums as [groups in tile][Mp] fp32. A stage's activations
// are again one contiguous range.
//
// Warp roles in a CTA: 16 consumer warps (one 16-column tile each), one producer thread (bulk
// copies), one finisher warp that sums parked K segments so the consumers never wait on a fence.

#include "common.cuh"

namespace tf {
namespace {

constexpr int kWorkers = 148;
constexpr int kItemTiles = 4;   // k tiles per schedule item: the same for every row bucket, so that the
                                // K segments (hence the bits) do not depend on the row count
constexpr int kWarps = 16;      // consumer warps = column tiles per column block (baked into the layout)
constexpr int kCols = kWarps * 16;

__host__ __device__ constexpr int rec_bytes(int group) { return 512 + (64 / group) * 64; }

// position inside the 4-element k quad that nibble j of a word carries
__host__ __device__ constexpr int nibble_quad(int j) { return ((j >> 1) & 1) * 2 + ((j >> 2) & 1); }
// input (0..63) of a k tile that lane t feeds to k-step s at quad position `quad`
__host__ __device__ constexpr int tile_k(int t, int s, int quad) { return 32 * (s >> 1) + 8 * t + 4 * (s & 1) + quad; }

template <int G, int MB, int KTS, int STAGES>
struct Cfg {
    static constexpr int REC = rec_bytes(G);
    static constexpr int GPT = 64 / G;                 // groups per k tile
    static constexpr int ROWS = MB * 8;                // = tf_padded_rows(M) for every M of the bucket
    static constexpr int XTILE = ROWS * (128 + 4 * GPT);   // packed activation bytes per k tile
    static constexpr int W_BYTES = kWarps * KTS * REC;
    static constexpr int X_BYTES = KTS * XTILE;
    static constexpr int STAGE_BYTES = ((W_BYTES + X_BYTES + 127) / 128) * 128;
    static constexpr int THREADS = (kWarps + 2) * 32;   // consumers + producer warp + finisher warp
    static constexpr int SMEM = STAGES * STAGE_BYTES + 2 * STAGES * 8 + 128;
};

struct Args {
    const uint8_t* xp;
    const uint8_t* w;
    void* y;
    int* counters;
    float* slots;
    int* status;
    int M, N, K;
    int f32_out;
    // grouped form (MoE experts): `max_probs` problems of 8 rows each, problem p multiplying its own
    // packed rows (xp + p * xp_stride) with the weight of expert prob_expert[p] (w + e * w_stride)
    // into y + p * y_stride elements; the live count is read on the device. nullptr: one problem.
    // With prob_sel, the launch covers the problems prob_sel[0 .. count) only (an expert-parallel rank's
    // own experts); addresses are still formed from the selected problem's index.
    const int* prob_expert;
    const int* prob_count;
    const int* prob_sel;
    int max_probs;
    long long w_stride, xp_stride, y_stride;
};

// Work items (column block, group of kItemTiles k tiles) are split evenly over kWorkers CTAs.
__host__ __device__ inline int range_begin(int cta, int total) { return (int)((long long)cta * total / kWorkers); }
__host__ __device__ inline int owner_of(int w, int total) { return (int)((((long long)w + 1) * kWorkers - 1) / total); }

constexpr size_t kSlotFloats = (size_t)TF_QMM_MAX_ROWS * kCols;

// A parked K segment of column block `cb` is complete in global memory: take a ticket; the last of
// the block's segments to arrive adds them all in k order and writes the output. Run by NT threads:
// the finisher warp (NT = 32) for a segment at the start of a CTA's range, while the consumers go on,
// or all consumer warps together for the segment that ends the range, when they have nothing left
// to do and the sum is on the kernel's critical path.
template <int NT>
__device__ __forceinline__ void group_sync() {
    if (NT == 32) __syncwarp();
    else named_bar_sync(1, NT);
}

template <int NT, bool MULTI>
__device__ void finish_segment(const Args& a, int gb, int CB, int SPB, int total, int tid, int* list) {
    __threadfence();
    group_sync<NT>();
    const int cb_begin = gb * SPB;
    const int q = MULTI ? gb / CB : 0, cb = gb - q * CB;
    const int prob = (MULTI && a.prob_sel) ? a.prob_sel[q] : q;
    if (tid == 0) {
        const int first = owner_of(cb_begin, total), last = owner_of(cb_begin + SPB - 1, total);
        int nseg = 0;
        for (int o = first; o <= last; ++o) {
            const int ob = range_begin(o, total);
            if (ob == range_begin(o + 1, total)) continue;       // a worker without work
            list[nseg++] = 2 * o + (ob < cb_begin ? 1 : 0);      // its slot, in k order
        }
        list[kWorkers] = nseg;
        list[kWorkers + 1] = atomicAdd(a.counters + gb, 1);
    }
    group_sync<NT>();
    const int nseg = list[kWorkers];
    if (list[kWorkers + 1] != nseg - 1) return;
    __threadfence();
    const int ncol4 = (min(kCols, a.N - cb * kCols) + 3) >> 2;
    const int n4 = a.M * (kCols / 4);
    constexpr int U = 4;          // elements in flight per thread and segment
    for (int base = tid; base < n4; base += NT * U) {
        float4 sum[U];
#pragma unroll
        for (int u = 0; u < U; ++u) sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < nseg; j += 2) {
            float4 v[2][U];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int idx = base + NT * u;
                    v[jj][u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (j + jj < nseg && idx < n4)
                        v[jj][u] = __ldcg(reinterpret_cast<const float4*>(a.slots + (size_t)list[j + jj] * kSlotFloats) + idx);
                }
#pragma unroll
            for (int jj = 0; jj < 2; ++jj)
                if (j + jj < nseg) {
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (j + jj == 0) sum[u] = v[jj][u];
                        else { sum[u].x += v[jj][u].x; sum[u].y += v[jj][u].y; sum[u].z += v[jj][u].z; sum[u].w += v[jj][u].w; }
                    }
                }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = base + NT * u;
            if (idx >= n4) continue;
            const int row = idx / (kCols / 4), c4 = idx - row * (kCols / 4);
            if (c4 >= ncol4) continue;
            const float e[4] = {sum[u].x, sum[u].y, sum[u].z, sum[u].w};
            const int col = cb * kCols + c4 * 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (col + i >= a.N) break;
                const size_t at = (size_t)prob * a.y_stride + (size_t)row * a.N + col + i;
                if (a.f32_out) reinterpret_cast<float*>(a.y)[at] = e[i];
                else reinterpret_cast<__nv_bfloat16*>(a.y)[at] = f2bf(e[i]);
            }
        }
    }
    if (tid == 0) a.counters[gb] = 0;      // leave the counters zero for the next call (every reader is past its ticket)
}

template <int G, int MB, int KTS, int STAGES, bool MULTI>
__global__ void __launch_bounds__((kWarps + 2) * 32, 1) qmm_kernel(const Args a) {
    using C = Cfg<G, MB, KTS, STAGES>;
    static_assert(kItemTiles % KTS == 0, "a schedule item is a whole number of pipeline stages");
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int seg_list[2][kWorkers + 2];   // [0] finisher warp, [1] consumers
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = a.K >> 6;                              // k tiles
    const int CB = (a.N + kCols - 1) / kCols;             // column blocks
    constexpr bool multi = MULTI;      // the grouped form is its own instantiation: the plain one pays nothing for it
    // Grouped launches never cut a column block along K: where the cut falls would depend on how many
    // problems the launch holds, that is on the other rows' routing. One item = a whole (problem, block).
    const int item_tiles = multi ? ((KT + KTS - 1) / KTS) * KTS : kItemTiles;   // a constant in the plain form
    const int SPB = (KT + item_tiles - 1) / item_tiles;   // schedule items per column block
    if (multi) pdl_wait();                                // the problem list is the previous kernel's output
    const int probs = multi ? min(*a.prob_count, a.max_probs) : 1;
    const int total = probs * CB * SPB;                   // "column block" below: (problem, column block) pairs
    const int begin = range_begin(blockIdx.x, total), end = range_begin(blockIdx.x + 1, total);

    uint8_t* stage0 = smem;
    const uint32_t bars = smem_u32(smem + STAGES * C::STAGE_BYTES);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), kWarps);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();     // the next kernel may be scheduled; it still waits for this one's memory

    // the first and the last segment of this CTA's range may be parts of a column block
    const int cb_first = begin < end ? begin / SPB : 0, cb_last = begin < end ? (end - 1) / SPB : 0;
    // a partial segment that ends the range is summed by the consumers themselves; one that starts a
    // longer range goes to the finisher warp
    const bool part_first = cb_last != cb_first && begin > cb_first * SPB;

    if (warp == kWarps) {
        // ------------------------------- producer: one thread ----------------------------------
        // Weights never change during a forward, so the first ring of weight copies is issued before
        // waiting for the previous kernel; the activations (its output) follow after the wait.
        if (lane == 0 && begin < end) {
            int s = 0, issued = 0;
            uint32_t phase = 1;
            int gb = cb_first, st = begin - gb * SPB;
            int prob = MULTI ? gb / CB : 0, cb = gb - prob * CB;
            auto picked = [&](int q) { return (MULTI && a.prob_sel) ? a.prob_sel[q] : q; };
            const uint8_t* wbase = a.w + (multi ? (size_t)a.prob_expert[picked(prob)] * a.w_stride : 0);
            const uint8_t* xbase = a.xp + (size_t)picked(prob) * a.xp_stride;
            int early_kt0[STAGES], early_nkt[STAGES];
            bool waited = multi;
            for (int it = begin; it < end; ++it) {
                for (int sub = 0; sub < item_tiles; sub += KTS) {
                    const int kt0 = st * item_tiles + sub, nkt = min(KTS, KT - kt0);
                    if (nkt <= 0) break;
                    if (issued == STAGES && !waited) {
                        pdl_wait();
                        for (int e = 0; e < STAGES; ++e)
                            bulk_g2s(smem_u32(stage0 + e * C::STAGE_BYTES + C::W_BYTES),
                                     a.xp + (size_t)early_kt0[e] * C::XTILE, (uint32_t)(early_nkt[e] * C::XTILE), full_bar(e));
                        waited = true;
                    }
                    mbar_wait(empty_bar(s), phase, a.status);
                    uint8_t* sb = stage0 + s * C::STAGE_BYTES;
                    const uint32_t wbytes = (uint32_t)(nkt * kWarps * C::REC), xbytes = (uint32_t)(nkt * C::XTILE);
                    mbar_arrive_expect_tx(full_bar(s), wbytes + xbytes);
                    bulk_g2s(smem_u32(sb), wbase + ((size_t)cb * KT + kt0) * (kWarps * C::REC), wbytes, full_bar(s));
                    if (waited) bulk_g2s(smem_u32(sb + C::W_BYTES), xbase + (size_t)kt0 * C::XTILE, xbytes, full_bar(s));
                    else { early_kt0[issued] = kt0; early_nkt[issued] = nkt; }
                    ++issued;
                    if (++s == STAGES) { s = 0; phase ^= 1; }
                }
                if (++st == SPB) {
                    st = 0;
                    ++gb;
                    if (++cb == CB) {
                        cb = 0;
                        ++prob;
                        if (multi && it + 1 < end) {
                            wbase = a.w + (size_t)a.prob_expert[picked(prob)] * a.w_stride;
                            xbase = a.xp + (size_t)picked(prob) * a.xp_stride;
                        }
                    }
                }
            }
            if (!waited) {
                pdl_wait();
                for (int e = 0; e < issued; ++e)
                    bulk_g2s(smem_u32(stage0 + e * C::STAGE_BYTES + C::W_BYTES), a.xp + (size_t)early_kt0[e] * C::XTILE,
                             (uint32_t)(early_nkt[e] * C::XTILE), full_bar(e));
            }
        }
        return;
    }
    pdl_wait();                  // everything below reads or writes what other kernels produce or read
    if (begin >= end) return;
    if (warp == kWarps + 1) {
        // ------------------- finisher: sums parked segments while the consumers go on -----------
        if (part_first) {
            named_bar_sync(2, (kWarps + 1) * 32);
            finish_segment<32, MULTI>(a, cb_first, CB, SPB, total, lane, seg_list[0]);
        }
        return;
    }

    // ----------------------------------- consumer warps ---------------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int xlane = g * 128 + ((t * 16) ^ ((g & 1) << 6));   // this lane's B-operand bytes inside a row block
    float acc[MB][4];
    int s = 0;
    uint32_t phase = 0;
    int it = begin;
    while (it < end) {
        const int gb = it / SPB, pq = MULTI ? gb / CB : 0, cb = gb - pq * CB;
        const int prob = (MULTI && a.prob_sel) ? a.prob_sel[pq] : pq;
        const int cb_begin = gb * SPB, cb_end = cb_begin + SPB;
        const int seg_begin = it, seg_end = cb_end < end ? cb_end : end;
#pragma unroll
        for (int rb = 0; rb < MB; ++rb) acc[rb][0] = acc[rb][1] = acc[rb][2] = acc[rb][3] = 0.f;

        for (; it < seg_end; ++it)
        for (int sub = 0; sub < item_tiles; sub += KTS) {
            const int nkt = min(KTS, KT - ((it - cb_begin) * item_tiles + sub));
            if (nkt <= 0) break;
            mbar_wait(full_bar(s), phase, a.status);
            const uint8_t* sb = stage0 + s * C::STAGE_BYTES;
            const uint8_t* wrec = sb + warp * C::REC;
            const uint8_t* xst = sb + C::W_BYTES;
#pragma unroll
            for (int kt = 0; kt < KTS; ++kt) {
                if (kt < nkt) {
                    const uint8_t* rec = wrec + kt * (kWarps * C::REC);
                    const uint4 wq = *reinterpret_cast<const uint4*>(rec + lane * 16);
                    const uint32_t wv[4] = {wq.x, wq.y, wq.z, wq.w};
                    uint32_t af[4][4];
#pragma unroll
                    for (int s4 = 0; s4 < 4; ++s4)
#pragma unroll
                        for (int i = 0; i < 4; ++i) af[s4][i] = ((wv[s4] >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
                    float sc[C::GPT][2], bi[C::GPT][2];
#pragma unroll
                    for (int h = 0; h < C::GPT; ++h) {
                        const uint2 p = *reinterpret_cast<const uint2*>(rec + 512 + h * 64 + g * 8);
                        sc[h][0] = bf16_lo(p.x); bi[h][0] = bf16_hi(p.x);
                        sc[h][1] = bf16_lo(p.y); bi[h][1] = bf16_hi(p.y);
                    }
                    const uint8_t* xt = xst + kt * C::XTILE;
                    const float* xsums = reinterpret_cast<const float*>(xt + C::ROWS * 128) + 2 * t;
#pragma unroll
                    for (int rb = 0; rb < MB; ++rb) {
                        const uint4 x0 = *reinterpret_cast<const uint4*>(xt + rb * 1024 + xlane);
                        const uint4 x1 = *reinterpret_cast<const uint4*>(xt + rb * 1024 + (xlane ^ 64));
                        const uint32_t xb[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                        constexpr int SPG = 4 / C::GPT;   // k-steps per group
#pragma unroll
                        for (int h = 0; h < C::GPT; ++h) {
                            const float2 xs = *reinterpret_cast<const float2*>(xsums + h * C::ROWS + rb * 8);
                            float p[4] = {-128.f * xs.x, -128.f * xs.y, -128.f * xs.x, -128.f * xs.y};
#pragma unroll
                            for (int s4 = h * SPG; s4 < (h + 1) * SPG; ++s4)
                                mma_bf16_16816(p, af[s4], xb[2 * s4], xb[2 * s4 + 1], p);
                            acc[rb][0] = __fmaf_rn(bi[h][0], xs.x, __fmaf_rn(sc[h][0], p[0], acc[rb][0]));
                            acc[rb][1] = __fmaf_rn(bi[h][0], xs.y, __fmaf_rn(sc[h][0], p[1], acc[rb][1]));
                            acc[rb][2] = __fmaf_rn(bi[h][1], xs.x, __fmaf_rn(sc[h][1], p[2], acc[rb][2]));
                            acc[rb][3] = __fmaf_rn(bi[h][1], xs.y, __fmaf_rn(sc[h][1], p[3], acc[rb][3]));
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));
            if (++s == STAGES) { s = 0; phase ^= 1; }
        }

        // ---- segment done: whole column block -> write; part of one -> park it for the finisher ----
        const bool whole = (seg_begin == cb_begin) && (seg_end == cb_end);
        const int col0 = cb * kCols + warp * 16 + g;
        if (whole) {
#pragma unroll
            for (int rb = 0; rb < MB; ++rb)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = rb * 8 + 2 * t + (i & 1), col = col0 + (i >> 1) * 8;
                    if (row < a.M && col < a.N) {
                        const size_t at = (size_t)prob * a.y_stride + (size_t)row * a.N + col;
                        if (a.f32_out) reinterpret_cast<float*>(a.y)[at] = acc[rb][i];
                        else reinterpret_cast<__nv_bfloat16*>(a.y)[at] = f2bf(acc[rb][i]);
                    }
                }
        } else {
            // slot 2*cta + 1 when this CTA entered the column block from an earlier one, else 2*cta
            const int later = begin < cb_begin ? 1 : 0;
            float* slot = a.slots + (size_t)(2 * blockIdx.x + later) * kSlotFloats;
#pragma unroll
            for (int rb = 0; rb < MB; ++rb)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = rb * 8 + 2 * t + (i & 1);
                    if (row < a.M) __stcg(slot + row * kCols + warp * 16 + g + (i >> 1) * 8, acc[rb][i]);
                }
            if (seg_end == end) finish_segment<kWarps * 32, MULTI>(a, gb, CB, SPB, total, threadIdx.x, seg_list[1]);
            else asm volatile("bar.arrive 2, %0;" ::"r"((kWarps + 1) * 32) : "memory");   // the finisher takes it; go on
        }
    }
}

template <int G, int MB, int KTS, int STAGES, bool MULTI = false>
int launch(const Args& a, cudaStream_t stream) {
    using C = Cfg<G, MB, KTS, STAGES>;
    static_assert(C::SMEM <= 227 * 1024, "stage ring does not fit shared memory");
    auto kern = qmm_kernel<G, MB, KTS, STAGES, MULTI>;
    static bool configured = false;   // per instantiation; the attribute is per function and idempotent
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
            return TF_ECUDA;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kWorkers);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(1) ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, a) != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

template <int G, int MB, int KTS>
constexpr int stages_for() {
    constexpr int budget = 224 * 1024;
    constexpr int stage = ((kWarps * KTS * rec_bytes(G) + KTS * MB * 8 * (128 + 4 * (64 / G)) + 127) / 128) * 128 + 16;
    return budget / stage > 8 ? 8 : budget / stage;
}

template <int G>
int dispatch(const Args& a, cudaStream_t stream) {
    // one CTA per SM; the stage ring takes nearly all of shared memory (about 30 MB in flight chip-wide)
    if (a.M <= 8) return launch<G, 1, 4, stages_for<G, 1, 4>()>(a, stream);
    if (a.M <= 16) return launch<G, 2, 4, stages_for<G, 2, 4>()>(a, stream);
    if (a.M <= 32) return launch<G, 4, 4, stages_for<G, 4, 4>()>(a, stream);
    if (a.M <= 64) return launch<G, 8, 2, stages_for<G, 8, 2>()>(a, stream);
    return launch<G, 16, 2, stages_for<G, 16, 2>()>(a, stream);
}

// ---- relayout kernels: one thread per output word / pair -----------------------------------------
__device__ __forceinline__ size_t record_offset(int col_tile, int kt, int KT, int REC) {
    return (((size_t)(col_tile / kWarps) * KT + kt) * kWarps + (col_tile % kWarps)) * REC;
}

__global__ void tile_kernel(const uint32_t* words, const uint16_t* scales, const uint16_t* biases, uint8_t* out,
                            int N, int K, int G) {
    const int KT = K >> 6, CB = (N + kCols - 1) / kCols, REC = rec_bytes(G), GPT = 64 / G;
    const long long recs = (long long)CB * kWarps * KT;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per = 128 + 16 * GPT;                 // threads per record: 128 words + 16*GPT (s,b) pairs
    if (id >= recs * per) return;
    const long long rec = id / per;
    const int e = (int)(id % per);
    const int c = (int)(rec / KT), kt = (int)(rec % KT);
    uint8_t* r = out + record_offset(c, kt, KT, REC);
    if (e < 128) {
        const int lane = e >> 2, s = e & 3, g = lane >> 2, t = lane & 3;
        uint32_t w = 0;
        for (int j = 0; j < 8; ++j) {
            const int col = 16 * c + g + 8 * (j & 1);
            const int k = 64 * kt + tile_k(t, s, nibble_quad(j));
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
            const int k = wi * 8 + i, kt = k >> 6, kin = k & 63, t = (kin >> 3) & 3, s = 2 * (kin >> 5) + ((kin >> 2) & 1),
                      quad = kin & 3;
            const int c = col >> 4, cin = col & 15, g = cin & 7, hi = cin >> 3;
            // inverse of nibble_quad: quad {0,1,2,3} sits at (j>>1) = {0,2,1,3}
            const int j = hi + 2 * (((quad & 1) << 1) | (quad >> 1));
            const uint32_t v = reinterpret_cast<const uint32_t*>(in + record_offset(c, kt, KT, REC))[(g * 4 + t) * 4 + s];
            w |= ((v >> (4 * j)) & 0xFu) << (4 * i);
        }
        words[id] = w;
    } else if (id < nwords + npairs) {
        const long long p = id - nwords;
        const int col = (int)(p / (K / G)), grp = (int)(p % (K / G));
        const int kt = grp / GPT, h = grp % GPT, c = col >> 4, cin = col & 15, g = cin & 7, hi = cin >> 3;
        const uint16_t* src =
            reinterpret_cast<const uint16_t*>(in + record_offset(c, kt, KT, REC) + 512 + h * 64 + g * 8 + hi * 4);
        scales[p] = src[0];
        biases[p] = src[1];
    }
}

// Row-major bf16 rows -> packed activations (+ group sums). One lane per 8 contiguous inputs:
// sequential sum of 8, then a pairwise tree across the G/8 lanes of a group.
template <int G>
__global__ void pack_rows_kernel(const __nv_bfloat16* x, uint8_t* xp, float* xs_out, int M, int K) {
    const int Mp = tf_padded_rows(M);
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long chunks = (long long)Mp * (K >> 3);
    const int row = (int)(id / (K >> 3)), c = (int)(id % (K >> 3));       // chunk c = inputs 8c..8c+7
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id < chunks && row < M) v = reinterpret_cast<const uint4*>(x)[(size_t)row * (K >> 3) + c];
    const float s = group_sum8<G>(v);
    if (id >= chunks) return;
    packed_store<G>(xp, Mp, row, c, v, s);
    if ((c & (G / 8 - 1)) == 0 && xs_out != nullptr && row < M) xs_out[(size_t)row * (K / G) + c / (G / 8)] = s;
}

}  // namespace
}  // namespace tf

extern "C" {

int tf_version(void) { return 1000; }
int tf_qmm_workers(void) { return tf::kWorkers; }

size_t tf_qmm_tiled_bytes(int N, int K, int group) {
    if (N <= 0 || K <= 0 || K % 64 || (group != 64 && group != 32)) return 0;
    return (size_t)((N + tf::kCols - 1) / tf::kCols) * tf::kWarps * (K / 64) * tf::rec_bytes(group);
}

size_t tf_packed_bytes(int M, int K, int group) {
    if (M <= 0 || K <= 0 || K % 64 || (group != 64 && group != 32)) return 0;
    return (size_t)(K / 64) * tf::tf_padded_rows(M) * (128 + 4 * (64 / group));
}

size_t tf_qmm_scratch_bytes(void) {
    // counters + two parked partial blocks (128 rows x 256 columns fp32) per worker
    return TF_QMM_COUNTER_BYTES + (size_t)2 * tf::kWorkers * TF_QMM_MAX_ROWS * tf::kCols * sizeof(float);
}

int tf_qmm(const void* x_packed, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M, int N, int K,
           int group, int flags, int* status, void* stream) {
    if (M < 1 || M > TF_QMM_MAX_ROWS || N < 1 || K < 64 || K % 64) return TF_EINVAL;
    if (group != 64 && group != 32) return TF_EINVAL;
    if (flags & ~TF_QMM_F32_OUT) return TF_EINVAL;
    if (!x_packed || !w_tiled || !y) return TF_EINVAL;
    const long long CB = (N + tf::kCols - 1) / tf::kCols, SPB = (K / 64 + tf::kItemTiles - 1) / tf::kItemTiles;
    if (CB * 4 > TF_QMM_COUNTER_BYTES || CB * SPB > (1 << 30) / tf::kWorkers) return TF_EINVAL;
    if (((uintptr_t)x_packed | (uintptr_t)w_tiled) & 15) return TF_EALIGN;
    if ((uintptr_t)y & 3) return TF_EALIGN;
    if (!scratch || ((uintptr_t)scratch & 255)) return TF_ESCRATCH;
    if (scratch_bytes < tf_qmm_scratch_bytes()) return TF_ESCRATCH;
    tf::Args a;
    a.xp = static_cast<const uint8_t*>(x_packed);
    a.w = static_cast<const uint8_t*>(w_tiled);
    a.y = y;
    a.counters = static_cast<int*>(scratch);
    a.slots = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + TF_QMM_COUNTER_BYTES);
    a.status = status;
    a.M = M; a.N = N; a.K = K;
    a.f32_out = (flags & TF_QMM_F32_OUT) ? 1 : 0;
    a.prob_expert = nullptr; a.prob_count = nullptr; a.prob_sel = nullptr; a.max_probs = 1;
    a.w_stride = a.xp_stride = a.y_stride = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return group == 64 ? tf::dispatch<64>(a, st) : tf::dispatch<32>(a, st);
}

int tf_qmm_grouped(const void* x_packed, const void* w_tiled, const int* prob_expert, const int* prob_count,
                   const int* prob_sel, int max_probs, void* y, void* scratch, size_t scratch_bytes, int N, int K, int group, int flags, int* status,
                   void* stream) {
    if (max_probs < 1 || N < 1 || K < 64 || K % 64) return TF_EINVAL;
    if (group != 64 && group != 32) return TF_EINVAL;
    if (flags & ~TF_QMM_F32_OUT) return TF_EINVAL;
    if (!x_packed || !w_tiled || !y || !prob_expert || !prob_count) return TF_EINVAL;
    const long long CB = (N + tf::kCols - 1) / tf::kCols;     // one schedule item per (problem, column block)
    if (CB * max_probs * 4 > TF_QMM_COUNTER_BYTES || CB * max_probs > (1 << 30) / tf::kWorkers) return TF_EINVAL;
    if (((uintptr_t)x_packed | (uintptr_t)w_tiled) & 15) return TF_EALIGN;
    if ((uintptr_t)y & 3) return TF_EALIGN;
    if (!scratch || ((uintptr_t)scratch & 255)) return TF_ESCRATCH;
    if (scratch_bytes < tf_qmm_scratch_bytes()) return TF_ESCRATCH;
    tf::Args a;
    a.xp = static_cast<const uint8_t*>(x_packed);
    a.w = static_cast<const uint8_t*>(w_tiled);
    a.y = y;
    a.counters = static_cast<int*>(scratch);
    a.slots = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + TF_QMM_COUNTER_BYTES);
    a.status = status;
    a.M = 8; a.N = N; a.K = K;
    a.f32_out = (flags & TF_QMM_F32_OUT) ? 1 : 0;
    a.prob_expert = prob_expert; a.prob_count = prob_count; a.prob_sel = prob_sel; a.max_probs = max_probs;
    a.w_stride = (long long)tf_qmm_tiled_bytes(N, K, group);
    a.xp_stride = (long long)tf_packed_bytes(8, K, group);
    a.y_stride = 8ll * N;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return group == 64 ? tf::launch<64, 1, 4, tf::stages_for<64, 1, 4>(), true>(a, st)
                       : tf::launch<32, 1, 4, tf::stages_for<32, 1, 4>(), true>(a, st);
}

int tf_qmm_tile(const void* words, const void* scales, const void* biases, void* w_tiled, int N, int K, int group,
                void* stream) {
    if (N < 1 || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!words || !scales || !biases || !w_tiled) return TF_EINVAL;
    const long long recs = (long long)((N + tf::kCols - 1) / tf::kCols) * tf::kWarps * (K / 64);
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

int tf_pack_rows(const void* x, void* x_packed, void* xs, int M, int K, int group, void* stream) {
    if (M < 1 || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!x || !x_packed) return TF_EINVAL;
    if (((uintptr_t)x | (uintptr_t)x_packed) & 15) return TF_EALIGN;
    const long long chunks = (long long)tf::tf_padded_rows(M) * (K / 8);
    const unsigned blocks = (unsigned)((chunks + 255) / 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto* xi = static_cast<const __nv_bfloat16*>(x);
    if (group == 64) tf::pack_rows_kernel<64><<<blocks, 256, 0, st>>>(xi, static_cast<uint8_t*>(x_packed), static_cast<float*>(xs), M, K);
    else tf::pack_rows_kernel<32><<<blocks, 256, 0, st>>>(xi, static_cast<uint8_t*>(x_packed), static_cast<float*>(xs), M, K);
    return cudaGetLastError() == cudaSuccess ? TF_OK : TF_ECUDA;
}

}  // extern "C"
