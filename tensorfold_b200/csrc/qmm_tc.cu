// Wide-row 4-bit group-affine matmul for sm_100a on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// This is the kernel for many rows per launch (32..128: prompt prefill in chunks, or a verify step over many
// concurrent sequences), where one tcgen05.mma covers 128 output columns x up to 128 rows x 16 inputs. It has its
// own arithmetic (weights dequantised to bf16 before the product), hence its own bits; an engine runs either this
// kernel or the lane kernel (qmm.cu) for ALL its steps, serial and windowed, so a row in a window keeps the bits
// of the same row alone. Its weights use their own tile layout.
//
// Weights stream once from HBM through a bulk-copy (TMA) ring into shared memory. Eight "dequantiser" warps turn
// the 4-bit codes into bf16 weights w = bf16(s * q + b) (one fused multiply-add per pair of codes, one rounding)
// and store them with tcgen05.st into tensor memory, where they are the A operand (128 output columns x 16 inputs
// per step) - the tensor core then reads only the activations from shared memory. The activations arrive packed
// as bf16 in the tensor core's K-major core-matrix form and are the B operand. One elected thread issues
// tcgen05.mma (kind::f16, bf16 x bf16 -> fp32, M = 128, N = row bucket, K = 16); a column block's accumulator
// lives in TMEM for its whole K segment and four epilogue warps read it back once with tcgen05.ld.
//
// Arithmetic, per output element (row m, column n):
//   acc = tensor-core chain over the segment's inputs in k order of bf16(s[n,g] * q[n,k] + b[n,g]) * x[m,k], fp32;
//   segments of K (fixed by N, K and the worker count only) are added in k order, then one rounding to bf16.
// The chain never looks at the row count, so row m of an M-row call has the bits of a 1-row call.
//
// Weight tile layout (built by tf_qmm_tc_tile): records indexed [column block of 128][k tile of 64], so a
// pipeline stage (a few k tiles of one block) is ONE contiguous range = one bulk copy. A record is
//   4096 bytes of nibbles: [quarter q 0..3][half hf 0..1][lane L 0..31][16 bytes] for column 32q + L;
//       word j = 4*hf + j' of the column's eight words holds, in byte b, input 8j + b of the k tile in
//       the low nibble and input 8j + 4 + b in the high nibble, so that `(w >> 4i) & 0x000F000F` is a pair of
//       codes: inputs 8j + {0,2}, {4,6}, {1,3}, {5,7} for i = 0..3 - the order in which a packed activation
//       chunk stores its eight values;
//   128 * (64/group) * 4 bytes of bf16 (scale, bias) pairs: [group in tile][column].
//
// Warp roles: 0-15 dequantise (TMEM lane quarter = warp % 4, k-step of a k tile = warp / 4), 16 TMA producer (one
// thread), 17 MMA issuer (one thread) and TMEM owner, 18-21 epilogue (TMEM lane quarter = warp % 4; and the
// sum of a column block's parked K segments, by whichever CTA parks the last one). Every wait is bounded (common.cuh): a wait that runs out writes TF_ESTALL and the
// kernel goes on to its end, where the TMEM it holds is freed.

#include <cuda_bf16.h>

#include "common.cuh"

namespace tf {
namespace {

// ---- packed activations of the wide-row kernel ------------------------------------------------------
// Per k tile (64 inputs), for Mp = M rounded up to its bucket 32/64/128 (rows past M are zero): Mp rows of 128
// bytes in the tensor core's K-major 128-byte-swizzle operand form (16-byte chunk c of row r at chunk c ^ (r % 8)
// of the row; 8 rows = one 1024-byte swizzle atom). The eight bf16 values of a 16-byte chunk are stored in the
// order 0,2,4,6,1,3,5,7 - the order the dequantisers produce weight pairs in.
__host__ __device__ constexpr int tc_padded_rows(int m) { return m <= 32 ? 32 : m <= 64 ? 64 : 128; }
__host__ __device__ constexpr int tc_packed_tile_bytes(int mp) { return mp * 128; }

// Store chunk c (inputs 8c..8c+7, natural order in v) of `row`.
__device__ __forceinline__ void tc_packed_store(uint8_t* xp, int Mp, int row, int c, uint4 v) {
    uint8_t* tile = xp + (size_t)(c >> 3) * tc_packed_tile_bytes(Mp);
    const int off = row * 128 + (((c & 7) ^ (row & 7)) << 4);
    uint4 o;
    o.x = __byte_perm(v.x, v.y, 0x5410);       // values 0, 2
    o.y = __byte_perm(v.z, v.w, 0x5410);       // values 4, 6
    o.z = __byte_perm(v.x, v.y, 0x7632);       // values 1, 3
    o.w = __byte_perm(v.z, v.w, 0x7632);       // values 5, 7
    *reinterpret_cast<uint4*>(tile + off) = o;
}


constexpr int kWorkers = 148;
constexpr int kItemTiles = 4;   // k tiles per schedule item: the same for every row bucket, so that the
                                // K segments (hence the bits) do not depend on the row count
constexpr int kCols = 128;      // columns per column block = TMEM lanes = tensor-core M
constexpr int kDequant = 16;         // dequantiser warps: four per TMEM lane quarter, one k-step (16 inputs) of a k tile each
constexpr int kThreads = (kDequant + 7) * 32;   // dequantisers, weight producer, MMA issuer, 4 epilogue, activation producer

__host__ __device__ constexpr int rec_bytes(int group) { return 4096 + 512 * (64 / group); }
__host__ __device__ constexpr int pow2_cols(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

// A pipeline stage is KTS k tiles of one column block. Their weight records and their activation tiles travel in
// two rings of their own: the small weight ring (WS stages) lets the dequantisers run ahead of the tensor core,
// the activation ring (XS stages of KTS * NB * 128 bytes) only has to cover the copy behind the running products.
// The A operand ring holds AU stages of dequantised tiles (32 tensor-memory columns a tile: 64 inputs as bf16
// pairs), the accumulator ring DU column-block accumulators of NB columns.
template <int G, int NB, int KTS, int XS>
struct Cfg {
    static constexpr int REC = rec_bytes(G);
    static constexpr int GPT = 64 / G;                     // groups per k tile
    static constexpr int XTILE = NB * 128;                 // packed activation bytes per k tile
    static constexpr int W_BYTES = ((KTS * REC + 127) / 128) * 128;
    static constexpr int X_BYTES = KTS * XTILE;            // swizzle atoms want 1024-byte alignment: activations first
    static constexpr int WS = 4;
    static constexpr int DU = 2;
    static constexpr int AU_FIT = (512 - DU * NB) / (KTS * 32);
    static constexpr int AU = AU_FIT > 4 ? 4 : AU_FIT;   // as deep as tensor memory allows
    static constexpr int NBARS = 2 * XS + 2 * WS + 2 * AU + 2 * DU;
    static constexpr int SMEM = XS * X_BYTES + WS * W_BYTES + NBARS * 8 + 128 + 1024;
    static constexpr int A_COLS = AU * KTS * 32;
    static constexpr int D_COL0 = A_COLS;
    static constexpr int TMEM_COLS = pow2_cols(A_COLS + DU * NB);
    static_assert(A_COLS + DU * NB <= 512, "rings do not fit tensor memory");
    static_assert(AU >= 2, "the dequantisers need a slot to run ahead into");
};

// Optional per-CTA timeline for profiling (tf_qmm_tc_set_trace): the latest launch writes 16 globaltimer stamps (ns)
// per CTA: 0 entry, 1 tensor memory allocated, 2 activation producer past griddepcontrol.wait, 3 dequantisers past
// their first full barrier, 4 first stage dequantised, 5 first tensor-core step issued, 6 last stage dequantised,
// 7 last step issued, 8 epilogue past its first accumulator barrier, 9 epilogue done, 10 past the closing barrier
// (the stamp may be read early by the compiler), 11 weight producer's last copy issued, 12/13 first stage's
// tensor-memory stores issued / complete, 14 first accumulator batch loaded, 15 first segment stored.
__device__ long long* g_tc_trace = nullptr;
__device__ __forceinline__ void tc_stamp(long long* tr, int slot) {
    if (tr != nullptr) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        tr[blockIdx.x * 16 + slot] = (long long)t;
    }
}

struct Args {
    const uint8_t* xp;
    const uint8_t* w;
    void* y;
    int* counters;
    float* slots;
    int* status;
    int M, N, K;
    int f32_out;
};

// Work items (column block, group of kItemTiles k tiles) are split evenly over kWorkers CTAs.
__host__ __device__ inline int range_begin(int cta, int total) { return (int)((long long)cta * total / kWorkers); }
__host__ __device__ inline int owner_of(int w, int total) { return (int)((((long long)w + 1) * kWorkers - 1) / total); }

// When the column blocks fill the workers' rounds to 85 % or more, a worker takes whole column blocks and nothing
// is parked; otherwise the (block, k item) stream is cut evenly and a block's K segments are summed by the CTA that
// parks the last one. The choice depends on N and K only.
__host__ __device__ inline bool whole_blocks(int CB) {
    const int rounds = (CB + kWorkers - 1) / kWorkers;
    return CB * 100 >= rounds * kWorkers * 85;
}
__host__ __device__ inline int worker_begin(int cta, int CB, int SPB) {
    return whole_blocks(CB) ? range_begin(cta, CB) * SPB : range_begin(cta, CB * SPB);
}

constexpr size_t kSlotFloats = (size_t)TF_QMM_MAX_ROWS * kCols;

// ---- tcgen05 wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor], bf16 x bf16 -> fp32, M = 128, K = 16
__device__ __forceinline__ void tc_mma_ts(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d), "r"(a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                   "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
                   "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
                   "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]),
                   "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]),
                   "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand in shared memory with the 128-byte swizzle: rows of 128 bytes, 8-row atoms 1024 bytes apart
// (stride offset); a k-step inside the row is reached by advancing the start address (the atom base stays
// 1024-byte aligned, so the base-offset field is zero).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

struct Ring {          // position in a ring of mbarrier-guarded slots
    int i, n;
    uint32_t phase;
    __device__ Ring(int n_, uint32_t first_phase) : i(0), n(n_), phase(first_phase) {}
    __device__ void next() { if (++i == n) { i = 0; phase ^= 1; } }
};
// A parked K segment of column block `cb` is complete in global memory: take a ticket; the last of the block's
// segments to arrive adds them all in k order and writes the output. Called by the four epilogue warps together
// (128 threads, named barrier 2).
__device__ void finish_segment(const Args& a, int cb, int SPB, int total, int t, int* list) {
    __threadfence();
    const int cb_begin = cb * SPB;
    asm volatile("bar.sync 2, 128;" ::: "memory");
    if (t == 0) {
        const int first = owner_of(cb_begin, total), last = owner_of(cb_begin + SPB - 1, total);
        int nseg = 0;
        for (int o = first; o <= last; ++o) {
            const int ob = range_begin(o, total);
            if (ob == range_begin(o + 1, total)) continue;       // a worker without work
            list[nseg++] = 2 * o + (ob < cb_begin ? 1 : 0);      // its slot, in k order
        }
        list[kWorkers] = nseg;
        list[kWorkers + 1] = atomicAdd(a.counters + cb, 1);
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
    const int nseg = list[kWorkers];
    if (list[kWorkers + 1] != nseg - 1) return;
    __threadfence();
    const int M = a.M, N = a.N;
    const bool f32_out = a.f32_out != 0;
    float* const y32 = reinterpret_cast<float*>(a.y);
    __nv_bfloat16* const y16 = reinterpret_cast<__nv_bfloat16*>(a.y);
    const float* const slots = a.slots;
    int seg[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) seg[j] = j < nseg ? list[j] : 0;
    // thread t: columns 4 * (t % 32) .. + 3 of rows t / 32 + 4 i
    const int c4 = (t & 31) * 4, col = cb * kCols + c4;
    constexpr int U = 4;          // rows in flight per thread and segment
    for (int r0 = t >> 5; r0 < M; r0 += 4 * U) {
        float4 sum[U];
        for (int j = 0; j < nseg; ++j) {
            const float* slot = slots + (size_t)(j < 8 ? seg[j] : list[j]) * kSlotFloats + c4;
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                v[u] = r0 + 4 * u < M ? __ldcg(reinterpret_cast<const float4*>(slot + (r0 + 4 * u) * kCols)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (j == 0) sum[u] = v[u];
                else { sum[u].x += v[u].x; sum[u].y += v[u].y; sum[u].z += v[u].z; sum[u].w += v[u].w; }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int row = r0 + 4 * u;
            if (row >= M) continue;
            const float e[4] = {sum[u].x, sum[u].y, sum[u].z, sum[u].w};
            const size_t at = (size_t)row * N + col;
            if (col + 3 < N && (N & 3) == 0) {
                if (f32_out) *reinterpret_cast<float4*>(y32 + at) = sum[u];
                else *reinterpret_cast<uint2*>(y16 + at) = make_uint2(pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]));
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (col + i < N) {
                        if (f32_out) y32[at + i] = e[i];
                        else y16[at + i] = f2bf(e[i]);
                    }
            }
        }
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
    if (t == 0) a.counters[cb] = 0;     // leave the counters zero for the next call
}

// Walks a CTA's stream of pipeline stages: schedule items (column block, 4 k tiles) cut into stages of KTS tiles.
template <int KTS>
struct StageWalk {
    int it, end, SPB, KT, sub, cb, st;
    __device__ StageWalk(int begin, int end_, int SPB_, int KT_) : it(begin), end(end_), SPB(SPB_), KT(KT_), sub(0) {
        cb = begin / SPB;
        st = begin - cb * SPB;
    }
    __device__ bool valid() const { return it < end; }
    __device__ int kt0() const { return st * kItemTiles + sub; }
    __device__ int nkt() const { return min(KTS, KT - kt0()); }
    __device__ void advance() {
        sub += KTS;
        if (sub >= kItemTiles || st * kItemTiles + sub >= KT) {
            sub = 0;
            ++it;
            if (++st == SPB) { st = 0; ++cb; }
        }
    }
};

template <int G, int NB, int KTS, int XS>
__global__ void __launch_bounds__(kThreads, 1) qmm_kernel(const __grid_constant__ Args a) {
    using C = Cfg<G, NB, KTS, XS>;
    constexpr int WS = C::WS;
    static_assert(kItemTiles % KTS == 0, "a schedule item is a whole number of pipeline stages");
    constexpr int AU = C::AU, DU = C::DU;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int seg_list[kWorkers + 2];
    __shared__ uint32_t tmem_base_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long* tr = g_tc_trace;
    if (threadIdx.x == 0) tc_stamp(tr, 0);
    const int KT = a.K >> 6;                              // k tiles
    const int CB = (a.N + kCols - 1) / kCols;             // column blocks
    const int SPB = (KT + kItemTiles - 1) / kItemTiles;   // schedule items per column block
    const int total = CB * SPB;
    const int begin = worker_begin(blockIdx.x, CB, SPB), end = worker_begin(blockIdx.x + 1, CB, SPB);
    if (begin >= end) return;                             // a worker without work (whole CTA leaves together)

    uint8_t* xring = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
    uint8_t* wring = xring + XS * C::X_BYTES;
    const uint32_t bars = smem_u32(wring + WS * C::W_BYTES);
    auto x_full = [&](int s) { return bars + 8u * s; };
    auto x_empty = [&](int s) { return bars + 8u * (XS + s); };
    auto w_full = [&](int s) { return bars + 8u * (2 * XS + s); };
    auto w_empty = [&](int s) { return bars + 8u * (2 * XS + WS + s); };
    auto a_full = [&](int s) { return bars + 8u * (2 * XS + 2 * WS + s); };
    auto a_empty = [&](int s) { return bars + 8u * (2 * XS + 2 * WS + AU + s); };
    auto d_full = [&](int s) { return bars + 8u * (2 * XS + 2 * WS + 2 * AU + s); };
    auto d_empty = [&](int s) { return bars + 8u * (2 * XS + 2 * WS + 2 * AU + DU + s); };

    if (threadIdx.x == 0) {
        // a weight stage is free when the dequantiser warps have read it, an activation stage when the tensor core has
        for (int s = 0; s < XS; ++s) { mbar_init(x_full(s), 1); mbar_init(x_empty(s), 1); }
        for (int s = 0; s < WS; ++s) { mbar_init(w_full(s), 1); mbar_init(w_empty(s), kDequant); }
        for (int s = 0; s < AU; ++s) { mbar_init(a_full(s), kDequant); mbar_init(a_empty(s), 1); }
        for (int s = 0; s < DU; ++s) { mbar_init(d_full(s), 1); mbar_init(d_empty(s), 4); }
        mbar_fence_init();
    }
    if (warp == kDequant + 1) {                            // this warp owns the tensor memory
        const uint32_t dst = smem_u32(&tmem_base_s), ncols = C::TMEM_COLS;
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    if (threadIdx.x == 0) tc_stamp(tr, 1);
    pdl_launch_dependents();     // the next kernel may be scheduled; it still waits for this one's memory

    // the first and the last segment of this CTA's range may be parts of a column block

    if (warp == kDequant) {
        // ------------------------------- weight producer: one thread ----------------------------------
        // Weights never change during a forward: their copies do not wait for the previous kernel.
        if (lane == 0) {
            Ring ring(WS, 1);
            for (StageWalk<KTS> wk(begin, end, SPB, KT); wk.valid(); wk.advance()) {
                const uint32_t wbytes = (uint32_t)(wk.nkt() * C::REC);
                mbar_wait_idle(w_empty(ring.i), ring.phase, a.status, 500);
                mbar_arrive_expect_tx(w_full(ring.i), wbytes);
                bulk_g2s(smem_u32(wring + ring.i * C::W_BYTES), a.w + ((size_t)wk.cb * KT + wk.kt0()) * C::REC, wbytes, w_full(ring.i));
                ring.next();
            }
            tc_stamp(tr, 11);
        }
        __syncwarp();            // the warp reaches the closing barrier together
    } else if (warp == kDequant + 6) {
        // ------------------------------- activation producer: one thread ------------------------------
        if (lane == 0) {
            pdl_wait();          // the activations are the previous kernel's output
            tc_stamp(tr, 2);
            Ring ring(XS, 1);
            for (StageWalk<KTS> wk(begin, end, SPB, KT); wk.valid(); wk.advance()) {
                const uint32_t xbytes = (uint32_t)(wk.nkt() * C::XTILE);
                mbar_wait_idle(x_empty(ring.i), ring.phase, a.status, 500);
                mbar_arrive_expect_tx(x_full(ring.i), xbytes);
                bulk_g2s(smem_u32(xring + ring.i * C::X_BYTES), a.xp + (size_t)wk.kt0() * C::XTILE, xbytes, x_full(ring.i));
                ring.next();
            }
        }
        __syncwarp();
    } else if (warp == kDequant + 1) {
        // ------------------------------- MMA issuer ------------------------------------------------
        // The whole warp walks the stages converged (so that addresses and descriptors live in uniform registers);
        // one elected lane issues the tensor-core instructions.
        {
            // fp32 D, bf16 x bf16, A from tensor memory, B K-major from shared memory, N = row bucket, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(kCols >> 4) << 24);
            Ring xr(XS, 0), ar(AU, 0), dr(DU, 1);
            int cur_cb = -1;
            uint32_t accumulate = 0;
            const bool leader = elect_one();
            for (StageWalk<KTS> wk(begin, end, SPB, KT); wk.valid();) {
                const int nkt = wk.nkt();
                if (wk.cb != cur_cb) {                    // a new column block: its accumulator must be drained
                    mbar_wait(d_empty(dr.i), dr.phase, a.status);
                    cur_cb = wk.cb;
                    accumulate = 0;
                }
                mbar_wait(x_full(xr.i), xr.phase, a.status);
                mbar_wait(a_full(ar.i), ar.phase, a.status);
                tc_fence_after();
                const uint32_t xbase = smem_u32(xring + xr.i * C::X_BYTES);
                const uint32_t abase = tmem + ar.i * (KTS * 32);
                const uint32_t d = tmem + C::D_COL0 + dr.i * NB;
                if (tr != nullptr && leader && wk.it == begin && wk.sub == 0) tc_stamp(tr, 5);
#pragma unroll
                for (int kt = 0; kt < KTS; ++kt) {
                    if (kt < nkt) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const uint64_t bdesc = smem_desc(xbase + kt * C::XTILE + ks * 32);
                            if (leader) tc_mma_ts(d, abase + kt * 32 + ks * 8, bdesc, idesc, accumulate);
                            accumulate = 1;
                        }
                    }
                }
                if (leader) {
                    tc_commit(x_empty(xr.i));             // arrive when the tensor core has read the stage's activations
                    tc_commit(a_empty(ar.i));             // ... and its dequantised weights
                    tc_stamp(tr, 7);
                }
                wk.advance();
                if (!wk.valid() || wk.cb != cur_cb) {     // the segment's last stage: its sums are complete after these
                    if (leader) tc_commit(d_full(dr.i));
                    dr.next();
                }
                ar.next();
                xr.next();
                __syncwarp();
            }
        }
    } else if (warp < kDequant) {
        // ------------------- dequantisers: 4-bit codes -> bf16(s * q + b) -> tensor memory (A operand) ---------
        const int q = warp & 3, part = warp >> 2;         // TMEM lane quarter; which k-step (16 inputs) of a k tile
        const int hf = part >> 1;
        Ring wr(WS, 0), ar(AU, 1);
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
        uint32_t nib_mask = 0x000F000Fu, magic = 0x43004300u;      // bf16 128 + code
        asm volatile("" : "+r"(nib_mask), "+r"(magic));
        const __nv_bfloat162 c128 = __floats2bfloat162_rn(128.f, 128.f);
        for (StageWalk<KTS> wk(begin, end, SPB, KT); wk.valid(); wk.advance()) {
            const int nkt = wk.nkt();
            mbar_wait(w_full(wr.i), wr.phase, a.status);
            if (tr != nullptr && threadIdx.x == 0 && wk.it == begin && wk.sub == 0) tc_stamp(tr, 3);
            const uint8_t* wst = wring + wr.i * C::W_BYTES;
            uint2 u[KTS];
            uint32_t sbw[KTS];
            // the group of this k-step's inputs: the tile's only one, or (32-input groups) group hf
            const int grp = C::GPT == 1 ? 0 : hf;
#pragma unroll
            for (int kt = 0; kt < KTS; ++kt) {
                if (kt < nkt) {
                    const uint8_t* rec = wst + kt * C::REC;
                    u[kt] = *reinterpret_cast<const uint2*>(rec + ((q * 2 + hf) * 32 + lane) * 16 + (part & 1) * 8);
                    sbw[kt] = *reinterpret_cast<const uint32_t*>(rec + 4096 + (grp * kCols + q * 32 + lane) * 4);
                }
            }
            // all tiles of the stage go to tensor memory before one wait: the store latency is paid once
            mbar_wait(a_empty(ar.i), ar.phase, a.status);
            tc_fence_after();
#pragma unroll
            for (int kt = 0; kt < KTS; ++kt) {
                if (kt < nkt) {
                    const uint32_t w2[2] = {u[kt].x, u[kt].y};
                    uint32_t cells[8];
                    __nv_bfloat162 s2, b2;
                    *reinterpret_cast<uint32_t*>(&s2) = __byte_perm(sbw[kt], sbw[kt], 0x1010);
                    *reinterpret_cast<uint32_t*>(&b2) = __byte_perm(sbw[kt], sbw[kt], 0x3232);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t t = and_or(i ? w2[j] >> (4 * i) : w2[j], nib_mask, magic);
                            const __nv_bfloat162 code = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&t), c128);
                            const __nv_bfloat162 wv = __hfma2(code, s2, b2);
                            cells[4 * j + i] = *reinterpret_cast<const uint32_t*>(&wv);
                        }
                    }
                    tc_st8(lane_base + (ar.i * KTS + kt) * 32 + part * 8, cells);
                }
            }
            if (tr != nullptr && threadIdx.x == 0 && wk.it == begin && wk.sub == 0) tc_stamp(tr, 12);
            tc_wait_st();
            if (tr != nullptr && threadIdx.x == 0 && wk.it == begin && wk.sub == 0) tc_stamp(tr, 13);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(a_full(ar.i)); mbar_arrive(w_empty(wr.i)); }
            if (tr != nullptr && threadIdx.x == 0) { if (wk.it == begin && wk.sub == 0) tc_stamp(tr, 4); tc_stamp(tr, 6); }
            ar.next();
            wr.next();
        }
    } else {
        // ------------------- epilogue warps: a column block's sums from tensor memory -> output ----------
        // A warp reads the 32 tensor-memory lanes (output columns) of its quadrant q = warp % 4.
        pdl_wait();
        const int q = warp & 3, col_local = q * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16) + C::D_COL0;
        // scalars in registers: a store through y cannot be taken to change them (the argument block may live in memory)
        const int M = a.M, N = a.N;
        const bool f32_out = a.f32_out != 0;
        float* const y32 = reinterpret_cast<float*>(a.y);
        __nv_bfloat16* const y16 = reinterpret_cast<__nv_bfloat16*>(a.y);
        float* const slots = a.slots;
        Ring dr(DU, 0);
        StageWalk<KTS> wk(begin, end, SPB, KT);
        while (wk.valid()) {
            const int cb = wk.cb, seg_begin = wk.it;
            while (wk.valid() && wk.cb == cb) wk.advance();
            const int cb_begin = cb * SPB;
            const bool whole = seg_begin == cb_begin && wk.it >= cb_begin + SPB;
            const int col = cb * kCols + col_local;
            // slot 2*cta + 1 when this CTA entered the column block from an earlier one, else 2*cta
            float* slot = slots + (size_t)(2 * blockIdx.x + (begin < cb_begin ? 1 : 0)) * kSlotFloats;
            mbar_wait_idle(d_full(dr.i), dr.phase, a.status);
            if (tr != nullptr && warp == kDequant + 2 && lane == 0 && seg_begin == begin) tc_stamp(tr, 8);
            tc_fence_after();
#pragma unroll 1
            for (int r0 = 0; r0 < NB; r0 += 32) {
                float v[32];
                tc_ld32(lane_base + dr.i * NB + r0, v);
                tc_wait_ld();
                if (tr != nullptr && warp == kDequant + 2 && lane == 0 && seg_begin == begin && r0 == 0) tc_stamp(tr, 14);
                if (r0 + 32 >= NB) {                       // drained: the next column block may overwrite it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(d_empty(dr.i));
                }
                // one compact store loop per output form: the unrolled body stays small
                const int live = M - r0;                   // rows of this batch that exist
                if (!whole) {
                    float* p = slot + r0 * kCols + col_local;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (i < live) __stcg(p + i * kCols, v[i]);
                } else if (col < N) {
                    if (f32_out) {
                        float* p = y32 + (size_t)r0 * N + col;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (i < live) *p = v[i];
                            p += N;
                        }
                    } else {
                        __nv_bfloat16* p = y16 + (size_t)r0 * N + col;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (i < live) *p = f2bf(v[i]);
                            p += N;
                        }
                    }
                }
            }
            if (tr != nullptr && warp == kDequant + 2 && lane == 0 && seg_begin == begin) tc_stamp(tr, 15);
            dr.next();
            if (!whole) finish_segment(a, cb, SPB, total, col_local, seg_list);
            if (warp == kDequant + 2 && lane == 0) tc_stamp(tr, 9);
        }
    }

    // ---- everyone is done with the tensor memory: give it back ----
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) tc_stamp(tr, 10);
    if (warp == kDequant + 1) {
        tc_fence_after();
        const uint32_t ncols = C::TMEM_COLS;
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
    }
}

template <int G, int NB, int KTS, int XS>
int launch(const Args& a, cudaStream_t stream) {
    using C = Cfg<G, NB, KTS, XS>;
    static_assert(C::SMEM <= 227 * 1024, "the rings do not fit shared memory");
    auto kern = qmm_kernel<G, NB, KTS, XS>;
    // the opt-in is per device: keep one flag per device ordinal
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return TF_ECUDA; }
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
            return TF_ECUDA;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kWorkers);
    cfg.blockDim = dim3(kThreads);
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

template <int G>
int dispatch(const Args& a, cudaStream_t stream) {
    // <group, row bucket, k tiles per stage, activation stages>: 64 KB of activations a stage at 128 rows
    if (a.M <= 32) return launch<G, 32, 4, 4>(a, stream);
    if (a.M <= 64) return launch<G, 64, 4, 4>(a, stream);
    return launch<G, 128, 4, 2>(a, stream);
}

// ---- relayout kernels: one thread per output word / pair -----------------------------------------
// word (q, hf, L, j') of a record: column 32q + L, word j = 4*hf + j' of that column
__global__ void tile_kernel(const uint32_t* words, const uint16_t* scales, const uint16_t* biases, uint8_t* out,
                            int N, int K, int G) {
    const int KT = K >> 6, CB = (N + kCols - 1) / kCols, REC = rec_bytes(G), GPT = 64 / G;
    const long long recs = (long long)CB * KT;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per = 1024 + 128 * GPT;               // threads per record: 1024 words + 128*GPT (s,b) pairs
    if (id >= recs * per) return;
    const long long rec = id / per;
    const int e = (int)(id % per);
    const int cb = (int)(rec / KT), kt = (int)(rec % KT);
    uint8_t* r = out + rec * REC;
    if (e < 1024) {
        const int q = e >> 8, hf = (e >> 7) & 1, L = (e >> 2) & 31, j = 4 * hf + (e & 3);
        const int col = cb * kCols + 32 * q + L;
        uint32_t w = 0;
        if (col < N) {
            // stored word j of the tile holds inputs 8j..8j+7 at nibbles 0..7
            const uint32_t src = words[(size_t)col * (K >> 3) + kt * 8 + j];
            for (int b = 0; b < 4; ++b) {
                w |= ((src >> (4 * b)) & 0xFu) << (8 * b);              // input 8j + b     -> low nibble of byte b
                w |= ((src >> (4 * (b + 4))) & 0xFu) << (8 * b + 4);    // input 8j + 4 + b -> high nibble of byte b
            }
        }
        reinterpret_cast<uint32_t*>(r)[e] = w;
    } else {
        const int p = e - 1024, h = p >> 7, cl = p & 127;
        const int col = cb * kCols + cl, grp = kt * GPT + h;
        uint16_t s = 0, b = 0;
        if (col < N) { s = scales[(size_t)col * (K / G) + grp]; b = biases[(size_t)col * (K / G) + grp]; }
        uint16_t* dst = reinterpret_cast<uint16_t*>(r + 4096 + (h * kCols + cl) * 4);
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
        const int kt = wi >> 3, j = wi & 7, cb = col / kCols, cl = col % kCols, q = cl >> 5, L = cl & 31;
        const uint8_t* r = in + ((long long)cb * KT + kt) * REC;
        const uint32_t v = reinterpret_cast<const uint32_t*>(r)[((q * 2 + (j >> 2)) * 32 + L) * 4 + (j & 3)];
        uint32_t w = 0;
        for (int b = 0; b < 4; ++b) {
            w |= ((v >> (8 * b)) & 0xFu) << (4 * b);
            w |= ((v >> (8 * b + 4)) & 0xFu) << (4 * (b + 4));
        }
        words[id] = w;
    } else if (id < nwords + npairs) {
        const long long p = id - nwords;
        const int col = (int)(p / (K / G)), grp = (int)(p % (K / G));
        const int kt = grp / GPT, h = grp % GPT, cb = col / kCols, cl = col % kCols;
        const uint16_t* src = reinterpret_cast<const uint16_t*>(in + ((long long)cb * KT + kt) * REC + 4096 + (h * kCols + cl) * 4);
        scales[p] = src[0];
        biases[p] = src[1];
    }
}

// Row-major bf16 rows -> packed activations. One lane per 8 contiguous inputs.
__global__ void pack_rows_kernel(const __nv_bfloat16* x, uint8_t* xp, int M, int K) {
    const int Mp = tc_padded_rows(M);
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long chunks = (long long)Mp * (K >> 3);
    if (id >= chunks) return;
    const int row = (int)(id / (K >> 3)), c = (int)(id % (K >> 3));       // chunk c = inputs 8c..8c+7
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < M) v = reinterpret_cast<const uint4*>(x)[(size_t)row * (K >> 3) + c];
    tc_packed_store(xp, Mp, row, c, v);
}

// The lane kernel's packed rows (common.cuh) -> this kernel's: the same values, regrouped; the sums are dropped.
__global__ void repack_kernel(const uint8_t* lane_packed, uint8_t* xp, int M, int K, int GPT) {
    pdl_launch_dependents();
    pdl_wait();
    const int Mp = tc_padded_rows(M), MpL = tf_padded_rows(M);
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long chunks = (long long)Mp * (K >> 3);
    if (id >= chunks) return;
    const int c = (int)(id / Mp), row = (int)(id % Mp);                   // a warp: 32 rows of one chunk
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < MpL) {
        const uint8_t* tile = lane_packed + (size_t)(c >> 3) * MpL * (128 + 4 * GPT);
        v = *reinterpret_cast<const uint4*>(tile + row * 128 + (((c & 7) * 16) ^ ((row & 1) << 6)));
    }
    tc_packed_store(xp, Mp, row, c, v);
}

}  // namespace
}  // namespace tf

extern "C" {


int tf_qmm_tc_set_trace(void* stamps) {
    long long* p = static_cast<long long*>(stamps);
    return cudaMemcpyToSymbol(tf::g_tc_trace, &p, sizeof(p)) == cudaSuccess ? TF_OK : TF_ECUDA;
}

size_t tf_qmm_tc_tiled_bytes(int N, int K, int group) {
    if (N <= 0 || K <= 0 || K % 64 || (group != 64 && group != 32)) return 0;
    return (size_t)((N + tf::kCols - 1) / tf::kCols) * (K / 64) * tf::rec_bytes(group);
}

size_t tf_packed_tc_bytes(int M, int K, int group) {
    if (M <= 0 || K <= 0 || K % 64 || (group != 64 && group != 32)) return 0;
    return (size_t)(K / 64) * tf::tc_packed_tile_bytes(tf::tc_padded_rows(M));
}

int tf_qmm_tc(const void* x_packed, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M, int N, int K,
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
    if (scratch_bytes < TF_QMM_COUNTER_BYTES + (size_t)2 * tf::kWorkers * TF_QMM_MAX_ROWS * tf::kCols * sizeof(float)) return TF_ESCRATCH;
    tf::Args a;
    a.xp = static_cast<const uint8_t*>(x_packed);
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

int tf_qmm_tc_tile(const void* words, const void* scales, const void* biases, void* w_tiled, int N, int K, int group,
                void* stream) {
    if (N < 1 || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!words || !scales || !biases || !w_tiled) return TF_EINVAL;
    const long long recs = (long long)((N + tf::kCols - 1) / tf::kCols) * (K / 64);
    const long long threads = recs * (1024 + 128 * (64 / group));
    tf::tile_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint32_t*>(words), static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases),
        static_cast<uint8_t*>(w_tiled), N, K, group);
    return cudaGetLastError() == cudaSuccess ? TF_OK : TF_ECUDA;
}

int tf_qmm_tc_untile(const void* w_tiled, void* words, void* scales, void* biases, int N, int K, int group,
                  void* stream) {
    if (N < 1 || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!words || !scales || !biases || !w_tiled) return TF_EINVAL;
    const long long threads = (long long)N * (K / 8) + (long long)N * (K / group);
    tf::untile_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(w_tiled), static_cast<uint32_t*>(words), static_cast<uint16_t*>(scales),
        static_cast<uint16_t*>(biases), N, K, group);
    return cudaGetLastError() == cudaSuccess ? TF_OK : TF_ECUDA;
}

int tf_pack_rows_tc(const void* x, void* x_packed, void* xs, int M, int K, int group, void* stream) {
    (void)xs;
    if (M < 1 || M > TF_QMM_MAX_ROWS || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!x || !x_packed) return TF_EINVAL;
    if (((uintptr_t)x | (uintptr_t)x_packed) & 15) return TF_EALIGN;
    const long long chunks = (long long)tf::tc_padded_rows(M) * (K / 8);
    const unsigned blocks = (unsigned)((chunks + 255) / 256);
    tf::pack_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                                                 static_cast<uint8_t*>(x_packed), M, K);
    return cudaGetLastError() == cudaSuccess ? TF_OK : TF_ECUDA;
}

int tf_repack_tc(const void* lane_packed, void* x_packed, int M, int K, int group, void* stream) {
    if (M < 1 || M > TF_QMM_MAX_ROWS || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!lane_packed || !x_packed) return TF_EINVAL;
    if (((uintptr_t)lane_packed | (uintptr_t)x_packed) & 15) return TF_EALIGN;
    const long long chunks = (long long)tf::tc_padded_rows(M) * (K / 8);
    const unsigned blocks = (unsigned)((chunks + 255) / 256);
    const uint8_t* src = static_cast<const uint8_t*>(lane_packed);
    uint8_t* dst = static_cast<uint8_t*>(x_packed);
    int gpt = 64 / group;
    void* args[] = {&src, &dst, &M, &K, &gpt};
    return tf::launch_pdl((const void*)tf::repack_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), args) ==
                   cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

}  // extern "C"
