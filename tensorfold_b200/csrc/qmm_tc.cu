// Prefill-width 4-bit group-affine matmul for sm_100a on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// This is the kernel for a PHASE, not for a row count: prompt prefill (hundreds of rows per launch in
// chunks of up to 128), where the tensor core's ~200-cycle occupancy per instruction is amortised over
// wide tiles. It has its own arithmetic (activations as two e4m3 planes), hence its own bits; the
// serial/verify regime always runs the lane kernel (qmm.cu). Its weights use their own tile layout.
//
// Weights stream once from HBM through a bulk-copy (TMA) ring into shared memory. A 4-bit code q in a
// byte 0x0q IS the e4m3 number q * 2^-9, so four "dequantiser" warps only mask nibbles apart and
// store them with tcgen05.st into tensor memory, where they are the A operand (128 output columns x
// 32 inputs per step). The activations arrive packed as two e4m3 planes per value plus group sums
// and unscale factors (common.cuh) and are the B operand, read by the tensor core straight from
// shared memory, hi and lo planes side by side along N (one step multiplies both). One elected thread
// issues tcgen05.mma (kind::f8f6f4, M = 128, N = 2 x rows, K = 32); accumulators live in TMEM and
// four epilogue warps read them back with tcgen05.ld for the fp32 scale/bias step.
//
// Arithmetic, per output element (row m, column n):
//   for each weight group g of the segment, in order:
//       Phi, Plo = tensor-core chains from zero over the group's 32-wide k-steps, one per activation plane
//       acc = fma(b[n,g], xs[m,g], fma(s[n,g], (Phi + Plo) * unscale[m,g], acc))
//   segments of K (fixed by N, K and the worker count only) are added in k order,
//   then one rounding to bf16.
// The chain never looks at the row count, so row m of an M-row call has the bits of a 1-row call.
//
// Weight tile layout (built by tf_qmm_tile): records indexed [column block of 128][k tile of 64], so a
// pipeline stage (a few k tiles of one block) is ONE contiguous range = one bulk copy. A record is
//   4096 bytes of nibbles: [quarter q 0..3][half hf 0..1][lane L 0..31][16 bytes] for column 32q + L;
//       word j = 4*hf + j' of the column's eight words holds, in byte b, input 8j + b of the k tile in
//       the low nibble and input 8j + 4 + b in the high nibble: `w & 0x0F0F0F0F` and
//       `(w >> 4) & 0x0F0F0F0F` are then TMEM cells 2j and 2j+1 (4 consecutive inputs each);
//   128 * (64/group) * 4 bytes of bf16 (scale, bias) pairs: [group in tile][column].
//
// Warp roles: 0-3 dequantise (TMEM lane quarter = warp), 4-7 epilogue (same quarters), 8 TMA producer
// (one thread), 9 MMA issuer (one thread) and TMEM owner, 10 finisher (sums parked K segments).
// Every wait is bounded (common.cuh): a wait that runs out writes TF_ESTALL and the kernel goes on
// to its end, where the TMEM it holds is freed.

#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace tf {
namespace {

// ---- packed activations of the prefill-width kernel ------------------------------------------------
// The lane matmul multiplies on the FP8 tensor-core path: a 4-bit code q stored in a byte as 0x0q IS
// the e4m3 number q * 2^-9 (subnormals and the first binade share one step), so weights need no
// conversion at all. Activations (bf16, 8 significant bits) are split into two e4m3 planes, hi + lo,
// after scaling each (row, weight group) by a power of two that puts the group's largest magnitude
// in [128, 256): hi = nearest e4m3 of the scaled value, lo = nearest e4m3 of the remainder. The sum
// hi + lo reproduces the value exactly unless it is more than ~2^9 below the group's maximum (then
// to within 2^-9 of the scaled unit). Products and the fp32 accumulation are exact tensor-core steps.
//
// Packed layout, per k tile (64 inputs), for Mp = M rounded up to its bucket 16/32/64/128 (rows past M
// are zero), RB = min(Mp, 64): for each 32-input k-step, for each chunk of RB rows, an RB x 32-byte hi
// block followed by an RB x 32-byte lo block, each in the tensor core's K-major no-swizzle operand form
// (8-row x 16-byte core matrices: byte (row r, k byte b) at (r/8)*256 + (b/16)*128 + (r%8)*16 + b%16), so
// that [hi; lo] of a chunk is ONE operand tile of 2*RB rows; then [groups in tile][Mp] fp32 group sums
// of the bf16 values; then [groups in tile][Mp] fp32 "unscale" factors 2^(9 - E) that turn the fp8 dot
// product back. Every kernel that produces matmul input writes this form with the helpers below, so
// sums, scales and planes are formed the same way everywhere.
__host__ __device__ constexpr int tc_padded_rows(int m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }
__host__ __device__ constexpr int tc_packed_tile_bytes(int mp, int group) { return mp * (128 + 8 * (64 / group)); }

struct GroupStats { float sum, amax; };

// Sum and largest magnitude of a G-input group: each lane takes its 8 contiguous bf16 values in
// order, then the G/8 lanes holding the group combine in a pairwise tree. Call with whole warps;
// every lane of the group gets the result.
template <int G>
__device__ __forceinline__ GroupStats tc_group_stats8(uint4 v) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    GroupStats r = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = bf16_lo(u[i]), b = bf16_hi(u[i]);
        r.sum += a; r.sum += b;
        r.amax = fmaxf(r.amax, fmaxf(fabsf(a), fabsf(b)));
    }
#pragma unroll
    for (int o = 1; o < G / 8; o <<= 1) {
        r.sum += __shfl_xor_sync(0xffffffffu, r.sum, o);
        r.amax = fmaxf(r.amax, __shfl_xor_sync(0xffffffffu, r.amax, o));
    }
    return r;
}

__device__ __forceinline__ float fp8_e4m3_value(uint8_t b) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3)));
}

// Store chunk c (inputs 8c..8c+7) of `row` as hi/lo planes and, from the group's first lane, the
// group's sum and unscale factor. No shuffles: lanes may call it independently.
template <int G>
__device__ __forceinline__ void tc_packed_store(uint8_t* xp, int Mp, int row, int c, uint4 v, GroupStats st) {
    constexpr int GPT = 64 / G;
    uint8_t* tile = xp + (size_t)(c >> 3) * tc_packed_tile_bytes(Mp, G);
    int E = 0;
    if (st.amax > 0.f) E = 7 - (int)((__float_as_uint(st.amax) >> 23) & 0xffu) + 127;
    E = max(-100, min(100, E));
    const float scale = __uint_as_float((uint32_t)(E + 127) << 23);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    uint32_t hi[2] = {0, 0}, lo[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float x = ((i & 1) ? bf16_hi(u[i >> 1]) : bf16_lo(u[i >> 1])) * scale;
        const uint8_t h = (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
        const uint8_t l = (uint8_t)__nv_cvt_float_to_fp8(x - fp8_e4m3_value(h), __NV_SATFINITE, __NV_E4M3);
        hi[i >> 2] |= (uint32_t)h << (8 * (i & 3));
        lo[i >> 2] |= (uint32_t)l << (8 * (i & 3));
    }
    const int ck = c & 7;                      // inputs 8ck..8ck+7 of the tile: k-step ck/4, bytes 8*(ck%4)..+7 of it
    const int RB = Mp < 64 ? Mp : 64, nr = row % RB;
    const int off = (ck >> 2) * (Mp * 64) + (row / RB) * (RB * 64) + (nr >> 3) * 256 + ((ck & 3) >> 1) * 128 + (nr & 7) * 16 + (ck & 1) * 8;
    *reinterpret_cast<uint2*>(tile + off) = make_uint2(hi[0], hi[1]);
    *reinterpret_cast<uint2*>(tile + RB * 32 + off) = make_uint2(lo[0], lo[1]);
    if ((c & (G / 8 - 1)) == 0) {
        float* f = reinterpret_cast<float*>(tile + Mp * 128);
        const int slot = ((c / (G / 8)) % GPT) * Mp + row;
        f[slot] = st.sum;
        f[GPT * Mp + slot] = __uint_as_float((uint32_t)(9 - E + 127) << 23);
    }
}


constexpr int kWorkers = 148;
constexpr int kItemTiles = 4;   // k tiles per schedule item: the same for every row bucket, so that the
                                // K segments (hence the bits) do not depend on the row count
constexpr int kCols = 128;      // columns per column block = TMEM lanes = tensor-core M
constexpr int kThreads = 15 * 32;   // 4 dequantisers, 4 epilogue, producer, MMA issuer, finisher, 4 more epilogue (128-row bucket)

__host__ __device__ constexpr int rec_bytes(int group) { return 4096 + 512 * (64 / group); }
__host__ __device__ constexpr int pow2_cols(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

// The activation operand of one tensor-core step is [hi rows; lo rows] of a chunk of RB rows (N = 2*RB);
// an accumulator "unit" is USG (group, chunk) pairs, one mbarrier pair per unit, UPS units per stage,
// so the roles synchronise a few times per stage instead of once per tile. The A operand ring holds
// AU stages of dequantised tiles (16 tensor-memory columns a tile).
template <int G, int NB, int KTS, int STAGES, int UPS>
struct Cfg {
    static constexpr int REC = rec_bytes(G);
    static constexpr int GPT = 64 / G;                     // groups per k tile
    static constexpr int XTILE = NB * (128 + 8 * GPT);     // packed activation bytes per k tile
    static constexpr int W_BYTES = KTS * REC;
    static constexpr int STAGE_BYTES = ((W_BYTES + KTS * XTILE + 127) / 128) * 128;
    static constexpr int RB = NB < 64 ? NB : 64;           // rows per chunk
    static constexpr int NC = NB / RB;                     // chunks
    static constexpr int NMMA = 2 * RB;                    // tensor-core N
    static constexpr int SSG = KTS * GPT * NC;             // (group, chunk) pairs per stage
    static constexpr int USG = SSG / UPS;                  // pairs per unit
    static constexpr int AU = 2, DU = 2;
    static constexpr int ESETS = NC;                       // epilogue warp sets: one per row chunk (two in the 128-row bucket)
    static_assert(ESETS == 1 || (USG == 1 && UPS % 2 == 0), "with two epilogue sets, units alternate between the row chunks");
    static constexpr int NBARS = 2 * STAGES + 2 * AU + 2 * DU;
    static constexpr int SMEM = STAGES * STAGE_BYTES + NBARS * 8 + 128;
    static constexpr int A_COLS = AU * KTS * 16;
    static constexpr int D_COL0 = A_COLS;
    static constexpr int TMEM_COLS = pow2_cols(A_COLS + DU * USG * NMMA);
    static_assert(SSG % UPS == 0 && USG >= 1, "a stage is a whole number of accumulator units");
    static_assert(A_COLS + DU * USG * NMMA <= 512, "rings do not fit tensor memory");
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
};

// Work items (column block, group of kItemTiles k tiles) are split evenly over kWorkers CTAs.
__host__ __device__ inline int range_begin(int cta, int total) { return (int)((long long)cta * total / kWorkers); }
__host__ __device__ inline int owner_of(int w, int total) { return (int)((((long long)w + 1) * kWorkers - 1) / total); }

constexpr size_t kSlotFloats = (size_t)TF_QMM_MAX_ROWS * kCols;

// ---- tcgen05 wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor], e4m3 x e4m3 -> fp32, M = 128, K = 32
__device__ __forceinline__ void tc_mma_ts(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d), "r"(a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                   "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
                   "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, no-swizzle operand in shared memory: 8-row x 16-byte core matrices, the two 16-byte K halves
// 128 bytes apart (leading offset), 8-row groups 256 bytes apart (stride offset).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(256 >> 4) << 32) | (1ull << 46);
}

struct Ring {          // position in a ring of mbarrier-guarded slots
    int i, n;
    uint32_t phase;
    __device__ Ring(int n_, uint32_t first_phase) : i(0), n(n_), phase(first_phase) {}
    __device__ void next() { if (++i == n) { i = 0; phase ^= 1; } }
};
// A parked K segment of column block `cb` is complete in global memory: take a ticket; the last of
// the block's segments to arrive adds them all in k order and writes the output. One warp.
__device__ void finish_segment(const Args& a, int cb, int SPB, int total, int lane, int* list) {
    __threadfence();
    const int cb_begin = cb * SPB;
    const int first = owner_of(cb_begin, total), last = owner_of(cb_begin + SPB - 1, total);
    int nseg = 0;
    if (lane == 0) {
        for (int o = first; o <= last; ++o) {
            const int ob = range_begin(o, total);
            if (ob == range_begin(o + 1, total)) continue;       // a worker without work
            list[nseg++] = 2 * o + (ob < cb_begin ? 1 : 0);      // its slot, in k order
        }
        list[kWorkers] = nseg;
        list[kWorkers + 1] = atomicAdd(a.counters + cb, 1);
    }
    __syncwarp();
    nseg = list[kWorkers];
    if (list[kWorkers + 1] != nseg - 1) return;
    __threadfence();
    const int ncol4 = (min(kCols, a.N - cb * kCols) + 3) >> 2;
    const int n4 = a.M * (kCols / 4);
    constexpr int U = 4;          // elements in flight per lane
    for (int base = lane; base < n4; base += 32 * U) {
        float4 sum[U];
#pragma unroll
        for (int u = 0; u < U; ++u) sum[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < nseg; j += 2) {
            float4 v[2][U];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int idx = base + 32 * u;
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
            const int idx = base + 32 * u;
            if (idx >= n4) continue;
            const int row = idx / (kCols / 4), c4 = idx - row * (kCols / 4);
            if (c4 >= ncol4) continue;
            const float e[4] = {sum[u].x, sum[u].y, sum[u].z, sum[u].w};
            const int col = cb * kCols + c4 * 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (col + i >= a.N) break;
                const size_t at = (size_t)row * a.N + col + i;
                if (a.f32_out) reinterpret_cast<float*>(a.y)[at] = e[i];
                else reinterpret_cast<__nv_bfloat16*>(a.y)[at] = f2bf(e[i]);
            }
        }
    }
    __syncwarp();
    if (lane == 0) a.counters[cb] = 0;     // leave the counters zero for the next call
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

template <int G, int NB, int KTS, int STAGES, int UPS>
__global__ void __launch_bounds__(kThreads, 1) qmm_kernel(const Args a) {
    using C = Cfg<G, NB, KTS, STAGES, UPS>;
    static_assert(kItemTiles % KTS == 0, "a schedule item is a whole number of pipeline stages");
    constexpr int AU = C::AU, DU = C::DU;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int seg_list[kWorkers + 2];
    __shared__ uint32_t tmem_base_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = a.K >> 6;                              // k tiles
    const int CB = (a.N + kCols - 1) / kCols;             // column blocks
    const int SPB = (KT + kItemTiles - 1) / kItemTiles;   // schedule items per column block
    const int total = CB * SPB;
    const int begin = range_begin(blockIdx.x, total), end = range_begin(blockIdx.x + 1, total);
    if (begin >= end) return;                             // a worker without work (whole CTA leaves together)

    uint8_t* stage0 = smem;
    const uint32_t bars = smem_u32(smem + STAGES * C::STAGE_BYTES);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto a_full = [&](int s) { return bars + 8u * (2 * STAGES + s); };
    auto a_empty = [&](int s) { return bars + 8u * (2 * STAGES + AU + s); };
    auto d_full = [&](int s) { return bars + 8u * (2 * STAGES + 2 * AU + s); };
    auto d_empty = [&](int s) { return bars + 8u * (2 * STAGES + 2 * AU + DU + s); };

    if (threadIdx.x == 0) {
        // a stage is free when the 4 dequantiser warps and the 4 epilogue warps are done with it; the epilogue
        // warps arrive only after the tensor core's last unit of the stage completed, so its reads are over too
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 4 + 4 * C::ESETS); }
        for (int s = 0; s < AU; ++s) { mbar_init(a_full(s), 4); mbar_init(a_empty(s), 4); }
        for (int s = 0; s < DU; ++s) { mbar_init(d_full(s), 1); mbar_init(d_empty(s), 4); }
        mbar_fence_init();
    }
    if (warp == 9) {                                      // this warp owns the tensor memory
        const uint32_t dst = smem_u32(&tmem_base_s), ncols = C::TMEM_COLS;
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    pdl_launch_dependents();     // the next kernel may be scheduled; it still waits for this one's memory

    // the first and the last segment of this CTA's range may be parts of a column block
    const int cb_first = begin / SPB, cb_last = (end - 1) / SPB;
    const bool part_first = begin > cb_first * SPB || end < (cb_first + 1) * SPB;
    const bool part_last = cb_last != cb_first && end < (cb_last + 1) * SPB;

    if (warp == 8) {
        // ------------------------------- producer: one thread ----------------------------------
        // Weights never change during a forward, so the first ring of weight copies is issued before
        // waiting for the previous kernel; the activations (its output) follow after the wait.
        if (lane == 0) {
            Ring ring(STAGES, 1);
            int issued = 0;
            int early_kt0[STAGES], early_nkt[STAGES];
            bool waited = false;
            for (StageWalk<KTS> wk(begin, end, SPB, KT); wk.valid(); wk.advance()) {
                const int kt0 = wk.kt0(), nkt = wk.nkt();
                if (issued == STAGES && !waited) {
                    pdl_wait();
                    for (int e = 0; e < STAGES; ++e)
                        bulk_g2s(smem_u32(stage0 + e * C::STAGE_BYTES + C::W_BYTES), a.xp + (size_t)early_kt0[e] * C::XTILE,
                                 (uint32_t)(early_nkt[e] * C::XTILE), full_bar(e));
                    waited = true;
                }
                mbar_wait(empty_bar(ring.i), ring.phase, a.status);
                uint8_t* sb = stage0 + ring.i * C::STAGE_BYTES;
                const uint32_t wbytes = (uint32_t)(nkt * C::REC), xbytes = (uint32_t)(nkt * C::XTILE);
                mbar_arrive_expect_tx(full_bar(ring.i), wbytes + xbytes);
                bulk_g2s(smem_u32(sb), a.w + ((size_t)wk.cb * KT + kt0) * C::REC, wbytes, full_bar(ring.i));
                if (waited) bulk_g2s(smem_u32(sb + C::W_BYTES), a.xp + (size_t)kt0 * C::XTILE, xbytes, full_bar(ring.i));
                else { early_kt0[issued] = kt0; early_nkt[issued] = nkt; }
                ++issued;
                ring.next();
            }
            if (!waited) {
                pdl_wait();
                for (int e = 0; e < issued; ++e)
                    bulk_g2s(smem_u32(stage0 + e * C::STAGE_BYTES + C::W_BYTES), a.xp + (size_t)early_kt0[e] * C::XTILE,
                             (uint32_t)(early_nkt[e] * C::XTILE), full_bar(e));
            }
        }
    } else if (warp == 9) {
        // ------------------------------- MMA issuer: one thread ---------------------------------
        if (lane == 0) {
            // fp32 D, e4m3 x e4m3, both K-major, N = hi rows + lo rows of one chunk, M = 128
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(C::NMMA >> 3) << 17) | ((uint32_t)(kCols >> 4) << 24);
            constexpr int SPG = 2 / C::GPT;               // k-steps per group
            Ring stage(STAGES, 0), ar(AU, 0), dr(DU, 1);
            for (StageWalk<KTS> wk(begin, end, SPB, KT); wk.valid(); wk.advance()) {
                const int ngroups = wk.nkt() * C::GPT;
                mbar_wait(full_bar(stage.i), stage.phase, a.status);
                mbar_wait(a_full(ar.i), ar.phase, a.status);
                const uint32_t xbase = smem_u32(stage0 + stage.i * C::STAGE_BYTES + C::W_BYTES);
                const uint32_t abase = tmem + ar.i * (KTS * 16);
#pragma unroll
                for (int u = 0; u < UPS; ++u) {
                    mbar_wait(d_empty(dr.i), dr.phase, a.status);
                    tc_fence_after();
#pragma unroll
                    for (int e = 0; e < C::USG; ++e) {
                        const int sg = u * C::USG + e, grp = sg / C::NC, chunk = sg % C::NC;
                        if (grp < ngroups) {
                            const int kt = grp / C::GPT, h = grp % C::GPT;
                            const uint32_t d = tmem + C::D_COL0 + (dr.i * C::USG + e) * C::NMMA;
#pragma unroll
                            for (int i = 0; i < SPG; ++i) {
                                const int ks = h * SPG + i;
                                tc_mma_ts(d, abase + kt * 16 + ks * 8,
                                          smem_desc(xbase + kt * C::XTILE + ks * (NB * 64) + chunk * (C::RB * 64)), idesc, i > 0 ? 1u : 0u);
                            }
                        }
                    }
                    tc_commit(d_full(dr.i));              // arrives when the unit's products are in tensor memory
                    dr.next();
                }
                ar.next();
                stage.next();
            }
        }
    } else if (warp == 10) {
        // ------------------- finisher: sums parked segments while the others go on ----------------
        pdl_wait();
        if (part_first) {
            named_bar_sync(2, (4 * C::ESETS + 1) * 32);
            finish_segment(a, cb_first, SPB, total, lane, seg_list);
        }
        if (part_last) {
            named_bar_sync(3, (4 * C::ESETS + 1) * 32);
            finish_segment(a, cb_last, SPB, total, lane, seg_list);
        }
    } else if (warp < 4) {
        // ------------------- dequantisers: nibbles -> e4m3 bytes -> tensor memory (A operand) ---------
        Ring stage(STAGES, 0), ar(AU, 1);
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        for (StageWalk<KTS> wk(begin, end, SPB, KT); wk.valid(); wk.advance()) {
            const int nkt = wk.nkt();
            mbar_wait(full_bar(stage.i), stage.phase, a.status);
            const uint8_t* wst = stage0 + stage.i * C::STAGE_BYTES;
            // all tiles of the stage go to tensor memory before one wait: the store latency is paid once
            mbar_wait(a_empty(ar.i), ar.phase, a.status);
            tc_fence_after();
#pragma unroll
            for (int kt = 0; kt < KTS; ++kt) {
                if (kt < nkt) {
                    const uint8_t* rec = wst + kt * C::REC + (warp * 64 + lane) * 16;
                    const uint4 u0 = *reinterpret_cast<const uint4*>(rec);
                    const uint4 u1 = *reinterpret_cast<const uint4*>(rec + 512);
                    const uint32_t w8[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
                    uint32_t cells[16];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        cells[2 * j] = w8[j] & 0x0F0F0F0Fu;
                        cells[2 * j + 1] = (w8[j] >> 4) & 0x0F0F0F0Fu;
                    }
                    tc_st16(lane_base + (ar.i * KTS + kt) * 16, cells);
                }
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(a_full(ar.i)); mbar_arrive(empty_bar(stage.i)); }
            ar.next();
            stage.next();
        }
    } else if (warp < 8 || C::ESETS == 2) {
        // ------------------- epilogue warps: products from tensor memory -> fp32 scale/bias -> output ----------
        // A warp reads the 32 tensor-memory lanes (columns) of its quadrant q = warp % 4. In the 128-row
        // bucket there are two sets of four warps, one per 64-row chunk: units alternate between the chunks,
        // so set c always drains accumulator slot c, and each thread holds 64 sums, not 128.
        pdl_wait();
        constexpr bool SPLIT = C::ESETS == 2;
        constexpr int ACC = NB / C::ESETS;
        const int set = SPLIT ? (warp >= 11 ? 1 : 0) : 0, row0 = set * ACC;
        const int q = warp & 3, col_local = q * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16) + C::D_COL0;
        Ring stage(STAGES, 0), dr(DU, 0), ar(AU, 0);
        if (SPLIT) dr.i = set;
        float acc[ACC];
        StageWalk<KTS> wk(begin, end, SPB, KT);
        while (wk.valid()) {
            const int cb = wk.cb, seg_begin = wk.it;
#pragma unroll
            for (int n = 0; n < ACC; ++n) acc[n] = 0.f;
            while (wk.valid() && wk.cb == cb) {
                const int ngroups = wk.nkt() * C::GPT;
                mbar_wait(full_bar(stage.i), stage.phase, a.status);
                const uint8_t* wst = stage0 + stage.i * C::STAGE_BYTES;
#pragma unroll
                for (int u = 0; u < UPS; ++u) {
                    if (SPLIT && (u & 1) != set) continue;            // the other set's unit
                    mbar_wait(d_full(dr.i), dr.phase, a.status);
                    tc_fence_after();
                    if (u == UPS - 1) {                   // the stage's last unit is done: the tensor core has read all of its A operand
                        __syncwarp();
                        if (lane == 0) mbar_arrive(a_empty(ar.i));
                    }
                    // a unit = USG (group, row chunk) pairs of 2*RB columns; it is drained 32 rows (two 16-row pieces,
                    // hi and lo each) per wait
                    constexpr int PIECES = C::RB / 16, BATCH = (PIECES >= 2 && NB <= 64) ? 2 : 1;
#pragma unroll
                    for (int e = 0; e < C::USG; ++e) {
                        const int sg = u * C::USG + e, grp = sg / C::NC, chunk = sg % C::NC;
                        const int kt = grp / C::GPT, h = grp % C::GPT;
                        const uint32_t sbw = *reinterpret_cast<const uint32_t*>(wst + kt * C::REC + 4096 + (h * kCols + col_local) * 4);
                        const float sc = bf16_lo(sbw), bi = bf16_hi(sbw);
                        const float4* xs4 = reinterpret_cast<const float4*>(wst + C::W_BYTES + kt * C::XTILE + NB * 128) + h * (NB / 4);
                        const float4* un4 = xs4 + C::GPT * (NB / 4);
                        const uint32_t dcol = lane_base + (dr.i * C::USG + e) * C::NMMA;
#pragma unroll
                        for (int p0 = 0; p0 < PIECES; p0 += BATCH) {
                            float hi[BATCH][16], lo[BATCH][16];
#pragma unroll
                            for (int b = 0; b < BATCH; ++b) {
                                tc_ld16(dcol + (p0 + b) * 16, hi[b]);
                                tc_ld16(dcol + C::RB + (p0 + b) * 16, lo[b]);
                            }
                            tc_wait_ld();
                            if (e == C::USG - 1 && p0 + BATCH >= PIECES) {     // the unit is drained: the next one may overwrite it
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(d_empty(dr.i));
                            }
                            if (grp < ngroups) {
#pragma unroll
                                for (int b = 0; b < BATCH; ++b)
#pragma unroll
                                    for (int i4 = 0; i4 < 4; ++i4) {
                                        const int nn = chunk * C::RB + (p0 + b) * 16 + i4 * 4, n = nn - (SPLIT ? chunk * C::RB : 0);
                                        const float4 xs = xs4[nn / 4], un = un4[nn / 4];
                                        acc[n + 0] = __fmaf_rn(bi, xs.x, __fmaf_rn(sc, (hi[b][i4 * 4 + 0] + lo[b][i4 * 4 + 0]) * un.x, acc[n + 0]));
                                        acc[n + 1] = __fmaf_rn(bi, xs.y, __fmaf_rn(sc, (hi[b][i4 * 4 + 1] + lo[b][i4 * 4 + 1]) * un.y, acc[n + 1]));
                                        acc[n + 2] = __fmaf_rn(bi, xs.z, __fmaf_rn(sc, (hi[b][i4 * 4 + 2] + lo[b][i4 * 4 + 2]) * un.z, acc[n + 2]));
                                        acc[n + 3] = __fmaf_rn(bi, xs.w, __fmaf_rn(sc, (hi[b][i4 * 4 + 3] + lo[b][i4 * 4 + 3]) * un.w, acc[n + 3]));
                                    }
                            }
                        }
                    }
                    if (SPLIT) dr.phase ^= 1;             // this set's slot comes round again after the other set's unit
                    else dr.next();
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(stage.i));
                ar.next();
                stage.next();
                wk.advance();
            }
            // ---- segment done: whole column block -> write; part of one -> park it for the finisher ----
            const int cb_begin = cb * SPB;
            const bool whole = seg_begin == cb_begin && wk.it >= cb_begin + SPB;
            const int col = cb * kCols + col_local;
            if (whole) {
                if (col < a.N) {
#pragma unroll
                    for (int n = 0; n < ACC; ++n) {
                        if (row0 + n < a.M) {
                            if (a.f32_out) reinterpret_cast<float*>(a.y)[(size_t)(row0 + n) * a.N + col] = acc[n];
                            else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)(row0 + n) * a.N + col] = f2bf(acc[n]);
                        }
                    }
                }
            } else {
                // slot 2*cta + 1 when this CTA entered the column block from an earlier one, else 2*cta
                float* slot = a.slots + (size_t)(2 * blockIdx.x + (begin < cb_begin ? 1 : 0)) * kSlotFloats;
#pragma unroll
                for (int n = 0; n < ACC; ++n)
                    if (row0 + n < a.M) __stcg(slot + (row0 + n) * kCols + col_local, acc[n]);
                // hand over to the finisher warp without waiting for it
                if (cb == cb_first) asm volatile("bar.arrive 2, %0;" ::"r"((4 * C::ESETS + 1) * 32) : "memory");
                else asm volatile("bar.arrive 3, %0;" ::"r"((4 * C::ESETS + 1) * 32) : "memory");
            }
        }
    }

    // ---- everyone is done with the tensor memory: give it back ----
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        const uint32_t ncols = C::TMEM_COLS;
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(ncols) : "memory");
    }
}

template <int G, int NB, int KTS, int STAGES, int UPS>
int launch(const Args& a, cudaStream_t stream) {
    using C = Cfg<G, NB, KTS, STAGES, UPS>;
    static_assert(C::SMEM <= 227 * 1024, "stage ring does not fit shared memory");
    auto kern = qmm_kernel<G, NB, KTS, STAGES, UPS>;
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

// as many stages as fit ~220 KB of shared memory (at most 8): the ring has to cover the copy latency
// plus the stages the dequantisers, the tensor core and the epilogue hold at any moment
template <int G, int NB, int KTS>
constexpr int stages_for() {
    constexpr int stage = ((KTS * rec_bytes(G) + KTS * NB * (128 + 8 * (64 / G)) + 127) / 128) * 128;
    constexpr int n = (220 * 1024) / stage;
    return n > 8 ? 8 : n;
}

template <int G>
int dispatch(const Args& a, cudaStream_t stream) {
    // <group, row bucket, k tiles per stage, stages, accumulator units per stage>: a unit is at most 128
    // tensor-memory columns, two units are in flight
    constexpr bool g64 = G == 64;
    if (a.M <= 16) return launch<G, 16, 4, stages_for<G, 16, 4>(), 2>(a, stream);
    if (a.M <= 32) return launch<G, 32, g64 ? 4 : 2, stages_for<G, 32, g64 ? 4 : 2>(), 2>(a, stream);
    if (a.M <= 64) return launch<G, 64, g64 ? 2 : 1, stages_for<G, 64, g64 ? 2 : 1>(), 2>(a, stream);
    return launch<G, 128, 1, stages_for<G, 128, 1>(), g64 ? 2 : 4>(a, stream);
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

// Row-major bf16 rows -> packed activations (+ group sums). One lane per 8 contiguous inputs.
template <int G>
__global__ void pack_rows_kernel(const __nv_bfloat16* x, uint8_t* xp, float* xs_out, int M, int K) {
    const int Mp = tc_padded_rows(M);
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long chunks = (long long)Mp * (K >> 3);
    const int row = (int)(id / (K >> 3)), c = (int)(id % (K >> 3));       // chunk c = inputs 8c..8c+7
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id < chunks && row < M) v = reinterpret_cast<const uint4*>(x)[(size_t)row * (K >> 3) + c];
    const GroupStats st = tc_group_stats8<G>(v);
    if (id >= chunks) return;
    tc_packed_store<G>(xp, Mp, row, c, v, st);
    if ((c & (G / 8 - 1)) == 0 && xs_out != nullptr && row < M) xs_out[(size_t)row * (K / G) + c / (G / 8)] = st.sum;
}

}  // namespace
}  // namespace tf

extern "C" {


size_t tf_qmm_tc_tiled_bytes(int N, int K, int group) {
    if (N <= 0 || K <= 0 || K % 64 || (group != 64 && group != 32)) return 0;
    return (size_t)((N + tf::kCols - 1) / tf::kCols) * (K / 64) * tf::rec_bytes(group);
}

size_t tf_packed_tc_bytes(int M, int K, int group) {
    if (M <= 0 || K <= 0 || K % 64 || (group != 64 && group != 32)) return 0;
    return (size_t)(K / 64) * tf::tc_packed_tile_bytes(tf::tc_padded_rows(M), group);
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
    if (M < 1 || M > TF_QMM_MAX_ROWS || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!x || !x_packed) return TF_EINVAL;
    if (((uintptr_t)x | (uintptr_t)x_packed) & 15) return TF_EALIGN;
    const long long chunks = (long long)tf::tc_padded_rows(M) * (K / 8);
    const unsigned blocks = (unsigned)((chunks + 255) / 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto* xi = static_cast<const __nv_bfloat16*>(x);
    if (group == 64) tf::pack_rows_kernel<64><<<blocks, 256, 0, st>>>(xi, static_cast<uint8_t*>(x_packed), static_cast<float*>(xs), M, K);
    else tf::pack_rows_kernel<32><<<blocks, 256, 0, st>>>(xi, static_cast<uint8_t*>(x_packed), static_cast<float*>(xs), M, K);
    return cudaGetLastError() == cudaSuccess ? TF_OK : TF_ECUDA;
}

}  // extern "C"
