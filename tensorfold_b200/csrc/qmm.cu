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
// Warp roles in a CTA: consumer warps (each one or two 16-column tiles of the block) and one producer
// thread (bulk copies).
//
// What bounds the loop once the bytes arrive is the integer pipe (16 lanes a cycle per sub-partition):
// a 16 x 64 record costs 12 shifts + 16 and-or operations there, so each of the 16 is one lop3.

#include "common.cuh"

namespace tf {
namespace {

constexpr int kWorkers = 148;
// k tiles per schedule item: a function of the weight's shape only, the same for every row bucket, so that
// the K segments (hence the bits) do not depend on the row count. One tile keeps the workers' shares within
// a tile of each other; a narrow weight (fewer than 18 column blocks) would then be cut into dozens of
// segments a block, so its blocks are cut into eight items instead.
constexpr int kMaxCutsNarrow = 8;
__host__ __device__ inline int item_tiles_for(int CB, int KT) {
    return CB * kMaxCutsNarrow < kWorkers ? (KT + kMaxCutsNarrow - 1) / kMaxCutsNarrow : 1;
}
constexpr int kWarps = 16;      // column tiles per column block (baked into the layout)
constexpr int kCols = kWarps * 16;

__host__ __device__ constexpr int rec_bytes(int group) { return 512 + (64 / group) * 64; }

// position inside the 4-element k quad that nibble j of a word carries
__host__ __device__ constexpr int nibble_quad(int j) { return ((j >> 1) & 1) * 2 + ((j >> 2) & 1); }
// input (0..63) of a k tile that lane t feeds to k-step s at quad position `quad`
__host__ __device__ constexpr int tile_k(int t, int s, int quad) { return 32 * (s >> 1) + 8 * t + 4 * (s & 1) + quad; }

// One instantiation per row bucket: MB blocks of 8 rows, KTS k tiles a pipeline stage, T column tiles per
// consumer warp (they share the activation loads), CTAS CTAs of the kernel that fit one SM.
template <int G_, int MB_, int KTS_, int T_, int CTAS_>
struct Cfg {
    static constexpr int G = G_, MB = MB_, KTS = KTS_, T = T_, CTAS = CTAS_;
    static constexpr int REC = rec_bytes(G);
    static constexpr int GPT = 64 / G;                 // groups per k tile
    static constexpr int ROWS = MB * 8;                // = tf_padded_rows(M) for every M of the bucket
    static constexpr int XTILE = ROWS * (128 + 4 * GPT);   // packed activation bytes per k tile
    static constexpr int W_BYTES = kWarps * KTS * REC;
    static constexpr int X_BYTES = KTS * XTILE;
    static constexpr int STAGE_BYTES = ((W_BYTES + X_BYTES + 127) / 128) * 128;
    static constexpr int CW = kWarps / T;               // consumer warps
    static constexpr int THREADS = (CW + 1) * 32;       // consumers + producer warp
    // the ring takes the SM's shared memory (1 KB a CTA belongs to the system), split between CTAS CTAs
    static constexpr int BUDGET = (CTAS == 2 ? 113 : 226) * 1024 - 512;
    static constexpr int STAGES = BUDGET / (STAGE_BYTES + 16) > 12 ? 12 : BUDGET / (STAGE_BYTES + 16);
    static constexpr int SMEM = STAGES * STAGE_BYTES + 2 * STAGES * 8 + 128;
    static_assert(STAGES >= 2, "the ring needs at least two stages");
};

// Optional per-CTA timeline for profiling: when set (tf_qmm_set_trace), each launch writes eight
// globaltimer stamps per CTA: 0 kernel entry, 1 first weight copy issued, 2 predecessor's memory visible
// (griddepcontrol.wait passed), 3 consumers past their first full barrier, 4 main loop done, 5 last
// segment parked or written, 6 ordered sum done, 7 producer's last copy issued.
__device__ unsigned long long* g_trace = nullptr;
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
constexpr int kTraceLaunches = 512, kTraceSlots = 16;
// layout: [148] per-CTA launch counters, then [launch % 512][cta][16] stamps
__device__ __forceinline__ void stamp(unsigned long long* tr, int slot) {
    if (tr != nullptr) tr[blockIdx.x * kTraceSlots + slot] = now_ns();
}

struct Args {
    const uint8_t* xp;
    const uint8_t* w;
    void* y;
    uint32_t* epochs;
    float* slots;
    int* status;
    int M, N, K;
    int f32_out;
    // grouped form (MoE experts): `max_probs` problems of 8 rows each, problem p multiplying its own
    // packed rows (xp + p * xp_stride) with the weight of expert prob_expert[p] (w + e * w_stride)
    // into y + p * y_stride elements; the live count is read on the device. nullptr: one problem.
    // With prob_sel, the launch covers the problems prob_sel[0 .. count) only (an expert-parallel rank's
    // own experts); addresses are still formed from the selected problem's index.
    // the matmul that runs next on this stream (may be null): once this kernel's own copies are all
    // issued, each worker asks L2 for the first bytes the SAME worker of that launch will stream
    const uint8_t* next_w;
    int next_N, next_K, next_group, prefetch_bytes;
    // tensor-parallel partial (may be null): instead of y, the fp32 sums go as 16-byte packets
    // {row 2i, n, row 2i+1, n} (n = exchange number = *peer_seq + 1) into block peer_rank of slot n & 1 of
    // EVERY rank's exchange buffer (plain peer stores); the consuming norm kernel waits for the number
    uint8_t* const* peer_bufs;
    const uint32_t* peer_seq;
    size_t peer_slot_bytes;
    int peer_rank, peer_world;
    // SwiGLU epilogue (may be null): the weight is a [gate; up] stack interleaved by column tile (tile 2a = gate
    // columns 16a..16a+15, tile 2a+1 = up columns 16a..16a+15), a consumer warp owns both tiles of an activation tile,
    // and instead of y the block's owner writes bf16(silu(bf16 gate) * bf16 up) with its group sums as the packed
    // input of the down projection (N / 2 inputs) - the bits the separate SwiGLU kernel would write
    uint8_t* act_packed;
    const int* prob_expert;
    const int* prob_count;
    const int* prob_sel;
    int max_probs;
    long long w_stride, xp_stride, y_stride;
};

// Work items (column block, group of item_tiles_for k tiles) are split evenly over kWorkers CTAs.
// cta * total stays below 2^31: the entry points refuse shapes with more than 2^30 / kWorkers items
__host__ __device__ inline int range_begin(int cta, int total) { return (int)((unsigned)cta * (unsigned)total / (unsigned)kWorkers); }

constexpr size_t kSlotFloats = (size_t)TF_QMM_MAX_ROWS * kCols;
// scratch: [ticket words of the prefill kernel][parked segments, one slot of 2 x 128 x 256 floats a worker]
//          [launch numbers, one a worker]
constexpr size_t kEpochOffset = TF_QMM_COUNTER_BYTES + 2 * kWorkers * kSlotFloats * sizeof(float);
constexpr size_t kScratchBytes = kEpochOffset + 1024;

// 16-byte load that is performed every time it is executed (a polled location)
__device__ __forceinline__ float4 ld_volatile16(const float4* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// How a column block cut along K is put together. The work items of a block are consecutive, so its
// segments belong to consecutive workers: the first segment (the block's first k items) ends one
// worker's range, every later segment starts the next worker's range. A worker therefore "parks" at
// most one segment, the first of its range, early in the kernel: each consumer thread stores its
// accumulators as 16-byte packets {value, value, launch number, launch number} (thread-major, so the
// stores coalesce; a packet is stored whole, so whoever reads this launch's number in it has the values).
// The worker that holds the block's FIRST segment is the one that finishes the block: at the end of its
// range it keeps that segment in registers, fetches the later segments' packets (again, bounded, while
// one still carries an older number), which were parked long before unless their worker started late,
// adds them in worker order, which is k order, and writes the output. No tickets, flags or fences, one
// round trip on the critical path, and nothing to reset. The launch number is the worker's own counter in scratch, advanced once
// per launch before dependents may start, so every worker of a launch holds the same number.
template <class C, bool MULTI>
__global__ void __launch_bounds__(C::THREADS, C::CTAS) qmm_kernel(const Args a) {
    constexpr int MB = C::MB, KTS = C::KTS, STAGES = C::STAGES, CW = C::CW, T = C::T, NC = CW * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint32_t epoch_s;
    // every thread derives the same per-launch trace base: the CTA's launch counter is bumped by thread 0
    // only after all threads have read it (the barrier below)
    unsigned long long* tr = g_trace;
    if (tr != nullptr) tr += kWorkers + (tr[blockIdx.x] % kTraceLaunches) * (kWorkers * kTraceSlots);
    if (threadIdx.x == 0) stamp(tr, 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = a.K >> 6;                              // k tiles
    const int CB = (a.N + kCols - 1) / kCols;             // column blocks
    constexpr bool multi = MULTI;      // the grouped form is its own instantiation: the plain one pays nothing for it
    // Grouped launches never cut a column block along K: where the cut falls would depend on how many
    // problems the launch holds, that is on the other rows' routing. One item = a whole (problem, block).
    const int item_tiles = multi ? ((KT + KTS - 1) / KTS) * KTS : item_tiles_for(CB, KT);
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
            mbar_init(empty_bar(s), CW);
        }
        mbar_fence_init();
        epoch_s = atomicAdd(a.epochs + blockIdx.x, 1u) + 1u;   // this launch's number: the same on every worker
        if (g_trace != nullptr) g_trace[blockIdx.x] += 1;
    }
    __syncthreads();
    pdl_launch_dependents();     // the next kernel may be scheduled; it still waits for this one's memory

    if (warp == CW) {
        // ------------------------------- producer: one thread ----------------------------------
        // Weights never change during a forward, so the first ring of weight copies is issued before
        // waiting for the previous kernel; the activations (its output) follow after the wait.
        if (lane == 0 && begin < end) {
            int s = 0, issued = 0;
            uint32_t phase = 1;
            auto picked = [&](int q) { return (MULTI && a.prob_sel) ? a.prob_sel[q] : q; };
            int early_kt0[STAGES], early_nkt[STAGES];
            bool waited = multi;
            int it = begin;
            while (it < end) {
                const int gb = it / SPB, pq = MULTI ? gb / CB : 0, cb = gb - pq * CB;
                const int cb_begin = gb * SPB, seg_end = min(cb_begin + SPB, end);
                const uint8_t* wbase = a.w + (multi ? (size_t)a.prob_expert[picked(pq)] * a.w_stride : 0) +
                                       (size_t)cb * KT * (kWarps * C::REC);
                const uint8_t* xbase = a.xp + (multi ? (size_t)picked(pq) * a.xp_stride : 0);
                const int kt_end = min(KT, (seg_end - cb_begin) * item_tiles);
                for (int kt0 = (it - cb_begin) * item_tiles; kt0 < kt_end; kt0 += KTS) {
                    const int nkt = min(KTS, kt_end - kt0);
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
                    bulk_g2s(smem_u32(sb), wbase + (size_t)kt0 * (kWarps * C::REC), wbytes, full_bar(s));
                    if (issued == 0) stamp(tr, 1);
                    if (waited) bulk_g2s(smem_u32(sb + C::W_BYTES), xbase + (size_t)kt0 * C::XTILE, xbytes, full_bar(s));
                    else { early_kt0[issued] = kt0; early_nkt[issued] = nkt; }
                    ++issued;
                    if (++s == STAGES) { s = 0; phase ^= 1; }
                }
                it = seg_end;
            }
            stamp(tr, 7);
            if (a.next_w != nullptr) {
                // where this worker's range of the next matmul starts (its items are cut like this one's)
                const int nKT = a.next_K >> 6, nCB = (a.next_N + kCols - 1) / kCols, nIT = item_tiles_for(nCB, nKT), nSPB = (nKT + nIT - 1) / nIT;
                const int ntotal = nCB * nSPB;
                const int nb = range_begin(blockIdx.x, ntotal), ne = range_begin(blockIdx.x + 1, ntotal);
                const size_t tile_bytes = (size_t)kWarps * rec_bytes(a.next_group);      // one k tile of a column block
                const size_t at = ((size_t)(nb / nSPB) * nKT + (size_t)(nb % nSPB) * nIT) * tile_bytes;
                const size_t whole = (size_t)nCB * nKT * tile_bytes;
                size_t len = (size_t)(ne - nb) * nIT * tile_bytes;
                if (len > (size_t)a.prefetch_bytes) len = (size_t)a.prefetch_bytes;
                if (at + len > whole) len = whole > at ? whole - at : 0;
                for (size_t off = 0; off < len; off += 32768) {
                    const uint32_t piece = (uint32_t)(len - off < 32768 ? len - off : 32768);
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.next_w + at + off), "r"(piece) : "memory");
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
    if (threadIdx.x == 0) stamp(tr, 2);
    if (begin >= end) return;

    // ----------------------------------- consumer warps ---------------------------------------
    const int g = lane >> 2, t = lane & 3;
    const int xlane = g * 128 + ((t * 16) ^ ((g & 1) << 6));   // this lane's B-operand bytes inside a row block
    // opaque to the compiler on purpose: as registers they let (w >> s) & mask | magic be one lop3
    uint32_t nib_mask = 0x000F000Fu, magic = 0x43004300u;
    asm volatile("" : "+r"(nib_mask), "+r"(magic));
    const uint32_t epoch = epoch_s;
    float acc[T][MB][4];
    int s = 0;
    uint32_t phase = 0;
    int it = begin;
    while (it < end) {
        const int gb = it / SPB, pq = MULTI ? gb / CB : 0, cb = gb - pq * CB;
        const int prob = (MULTI && a.prob_sel) ? a.prob_sel[pq] : pq;
        const int cb_begin = gb * SPB, cb_end = cb_begin + SPB;
        const int seg_begin = it, seg_end = cb_end < end ? cb_end : end;
#pragma unroll
        for (int ti = 0; ti < T; ++ti)
#pragma unroll
            for (int rb = 0; rb < MB; ++rb) acc[ti][rb][0] = acc[ti][rb][1] = acc[ti][rb][2] = acc[ti][rb][3] = 0.f;

        const int kt_end = min(KT, (seg_end - cb_begin) * item_tiles);
        for (int kt0 = (it - cb_begin) * item_tiles; kt0 < kt_end; kt0 += KTS) {
            const int nkt = min(KTS, kt_end - kt0);
            mbar_wait(full_bar(s), phase, a.status);
            if (tr != nullptr && threadIdx.x == 0 && it == begin && kt0 == (it - cb_begin) * item_tiles) stamp(tr, 3);
            const uint8_t* sb = stage0 + s * C::STAGE_BYTES;
            const uint8_t* wrec = sb + warp * T * C::REC;
            const uint8_t* xst = sb + C::W_BYTES;
#pragma unroll
            for (int kt = 0; kt < KTS; ++kt) {
                if (kt < nkt) {
                    const uint8_t* xt = xst + kt * C::XTILE;
                    const float* xsums = reinterpret_cast<const float*>(xt + C::ROWS * 128) + 2 * t;
                    uint32_t af[T][4][4];
                    float sc[T][C::GPT][2], bi[T][C::GPT][2];
#pragma unroll
                    for (int ti = 0; ti < T; ++ti) {
                        const uint8_t* rec = wrec + kt * (kWarps * C::REC) + ti * C::REC;
                        const uint4 wq = *reinterpret_cast<const uint4*>(rec + lane * 16);
                        const uint32_t wv[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
                        for (int s4 = 0; s4 < 4; ++s4)
#pragma unroll
                            for (int i = 0; i < 4; ++i) af[ti][s4][i] = and_or(i ? wv[s4] >> (4 * i) : wv[s4], nib_mask, magic);
#pragma unroll
                        for (int h = 0; h < C::GPT; ++h) {
                            const uint2 p = *reinterpret_cast<const uint2*>(rec + 512 + h * 64 + g * 8);
                            sc[ti][h][0] = bf16_lo(p.x); bi[ti][h][0] = bf16_hi(p.x);
                            sc[ti][h][1] = bf16_lo(p.y); bi[ti][h][1] = bf16_hi(p.y);
                        }
                    }
#pragma unroll
                    for (int rb = 0; rb < MB; ++rb) {
                        const uint4 x0 = *reinterpret_cast<const uint4*>(xt + rb * 1024 + xlane);
                        const uint4 x1 = *reinterpret_cast<const uint4*>(xt + rb * 1024 + (xlane ^ 64));
                        const uint32_t xb[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                        constexpr int SPG = 4 / C::GPT;   // k-steps per group
#pragma unroll
                        for (int h = 0; h < C::GPT; ++h) {
                            const float2 xs = *reinterpret_cast<const float2*>(xsums + h * C::ROWS + rb * 8);
                            const float i0 = -128.f * xs.x, i1 = -128.f * xs.y;
#pragma unroll
                            for (int ti = 0; ti < T; ++ti) {
                                float p[4] = {i0, i1, i0, i1};
#pragma unroll
                                for (int s4 = h * SPG; s4 < (h + 1) * SPG; ++s4)
                                    mma_bf16_16816(p, af[ti][s4], xb[2 * s4], xb[2 * s4 + 1], p);
                                float* ac = acc[ti][rb];
                                ac[0] = __fmaf_rn(bi[ti][h][0], xs.x, __fmaf_rn(sc[ti][h][0], p[0], ac[0]));
                                ac[1] = __fmaf_rn(bi[ti][h][0], xs.y, __fmaf_rn(sc[ti][h][0], p[1], ac[1]));
                                ac[2] = __fmaf_rn(bi[ti][h][1], xs.x, __fmaf_rn(sc[ti][h][1], p[2], ac[2]));
                                ac[3] = __fmaf_rn(bi[ti][h][1], xs.y, __fmaf_rn(sc[ti][h][1], p[3], ac[3]));
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));
            if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        it = seg_end;

        // ---- segment done ----
        if (tr != nullptr && threadIdx.x == 0 && seg_end == end) stamp(tr, 4);
        if (seg_begin > cb_begin) {
            // a later segment of a block some earlier worker finishes: park it (always the first of this range)
            // as 16-byte packets {value, value, launch number, launch number}: a packet is stored whole, so a
            // reader that sees this launch's number in it has the values too. No fence, no flag.
            float4* slot = reinterpret_cast<float4*>(a.slots + (size_t)blockIdx.x * (2 * kSlotFloats));
            const float tagf = __uint_as_float(epoch);
#pragma unroll
            for (int ti = 0; ti < T; ++ti)
#pragma unroll
                for (int rb = 0; rb < MB; ++rb) {
                    __stcg(slot + ((ti * MB + rb) * 2 + 0) * NC + threadIdx.x, make_float4(acc[ti][rb][0], acc[ti][rb][1], tagf, tagf));
                    __stcg(slot + ((ti * MB + rb) * 2 + 1) * NC + threadIdx.x, make_float4(acc[ti][rb][2], acc[ti][rb][3], tagf, tagf));
                }
            if (tr != nullptr && threadIdx.x == 0) stamp(tr, 5);
            continue;
        }
        if (seg_end < cb_end) {
            // the block's first segment: add the later ones, parked by the next workers, in worker order.
            // Up to four segments are waited for and fetched together (their latencies overlap) and then
            // added one by one, so the sum is the plain sequential one.
            int o = blockIdx.x + 1;
            bool more = true;
            while (more) {
                constexpr int SB = MB <= 2 ? 4 : 1;              // segments fetched together
                constexpr int UN = T * MB, UB = UN >= 4 ? 4 : UN;  // accumulator units (4 values each), units per fetch
                int who[SB], cnt = 0;
                for (; o < kWorkers && cnt < SB; ++o) {
                    const int ob = range_begin(o, total);
                    if (ob >= cb_end) { more = false; break; }
                    if (range_begin(o + 1, total) == ob) continue;       // a worker without work
                    who[cnt++] = o;
                }
                if (o >= kWorkers) more = false;
                if (cnt == 0) break;
#pragma unroll
                for (int u0 = 0; u0 < UN; u0 += UB) {
                    // fetch the packets of these units from every segment of the batch; a packet that does not
                    // carry this launch's number yet is fetched again (bounded)
                    float4 v[SB][UB][2];
                    bool ready = false;
                    for (int spin = 0; spin < (1 << 20) && !ready; ++spin) {
                        ready = true;
#pragma unroll
                        for (int j = 0; j < SB; ++j)
                            if (j < cnt) {
                                const float4* slot = reinterpret_cast<const float4*>(a.slots + (size_t)who[j] * (2 * kSlotFloats));
#pragma unroll
                                for (int u = 0; u < UB; ++u)
#pragma unroll
                                    for (int h = 0; h < 2; ++h) {
                                        const float4 pk = ld_volatile16(slot + ((u0 + u) * 2 + h) * NC + threadIdx.x);
                                        v[j][u][h] = pk;
                                        ready = ready && __float_as_uint(pk.z) == epoch && __float_as_uint(pk.w) == epoch;
                                    }
                            }
                    }
                    if (!ready) report(a.status, TF_ESTALL);
#pragma unroll
                    for (int j = 0; j < SB; ++j)
                        if (j < cnt) {
#pragma unroll
                            for (int u = 0; u < UB; ++u) {
                                float* ac = acc[(u0 + u) / MB][(u0 + u) % MB];
                                ac[0] += v[j][u][0].x; ac[1] += v[j][u][0].y;
                                ac[2] += v[j][u][1].x; ac[3] += v[j][u][1].y;
                            }
                        }
                }
            }
            if (tr != nullptr && threadIdx.x == 0) stamp(tr, 6);
        }
        // a whole block, or a finished one: write the output
        if constexpr (!MULTI && T == 2) {
            if (a.act_packed != nullptr) {
                __shared__ float act_part[kWarps / 2][C::ROWS];
                const int at = cb * (kWarps / 2) + warp;            // activation tile: 16 inputs of the down projection
                const int q4 = at & 3;                              // its place in the down projection's k tile
                uint8_t* tile = a.act_packed + (size_t)(at >> 2) * (C::ROWS * (128 + 4 * C::GPT));
                const bool in_range = at * 16 < (a.N >> 1);
#pragma unroll
                for (int rb = 0; rb < MB; ++rb)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int row = rb * 8 + 2 * t + j;
                        float pair = 0.f;
#pragma unroll
                        for (int hsel = 0; hsel < 2; ++hsel) {
                            const float gv = round_bf16(acc[0][rb][2 * hsel + j]), uv = round_bf16(acc[1][rb][2 * hsel + j]);
                            const float ov = round_bf16(gv * sigmoidf_(gv) * uv);
                            if (in_range)
                                *reinterpret_cast<__nv_bfloat16*>(tile + row * 128 + (((2 * q4 + hsel) * 16) ^ ((row & 1) << 6)) + g * 2) = f2bf(ov);
                            // the chunk's eight values added in column order (as the separate kernel's lane does), then the pair of chunks
                            float cs = 0.f;
#pragma unroll
                            for (int i = 0; i < 8; ++i) cs += __shfl_sync(0xffffffffu, ov, i * 4 + t);
                            pair = hsel == 0 ? cs : pair + cs;
                        }
                        if (g == 0) act_part[warp][row] = pair;
                    }
                named_bar_sync(4, NC);
                constexpr int WPG = 4 / C::GPT;                     // warps (activation tiles) per group
                if ((warp % WPG) == 0 && lane < C::ROWS && in_range) {
                    float sum = act_part[warp][lane] + act_part[warp + 1][lane];
                    if (WPG == 4) sum = sum + (act_part[warp + 2][lane] + act_part[warp + 3][lane]);
                    reinterpret_cast<float*>(tile + C::ROWS * 128)[(C::GPT == 1 ? 0 : (q4 >> 1)) * C::ROWS + lane] = sum;
                }
                named_bar_sync(4, NC);
                continue;
            }
        }
        if (!MULTI && a.peer_bufs != nullptr) {
            // a tensor-parallel rank's partial: straight into every rank's exchange buffer, self-signalling
            const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(a.peer_seq) + 1u;
            const size_t base = (want & 1u) * a.peer_slot_bytes + (size_t)a.peer_rank * ((a.M + 1) / 2) * a.N * 16;
#pragma unroll
            for (int ti = 0; ti < T; ++ti) {
                const int col0 = cb * kCols + (warp * T + ti) * 16 + g;
#pragma unroll
                for (int rb = 0; rb < MB; ++rb)
#pragma unroll
                    for (int hsel = 0; hsel < 2; ++hsel) {
                        const int row = rb * 8 + 2 * t, col = col0 + hsel * 8;
                        if (row < a.M && col < a.N) {
                            const uint4 pkt = make_uint4(__float_as_uint(acc[ti][rb][2 * hsel]), want,
                                                         __float_as_uint(acc[ti][rb][2 * hsel + 1]), want);
                            const size_t at = base + ((size_t)(row >> 1) * a.N + col) * 16;
                            for (int peer = 0; peer < a.peer_world; ++peer)
                                asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(a.peer_bufs[peer] + at), "r"(pkt.x),
                                             "r"(pkt.y), "r"(pkt.z), "r"(pkt.w) : "memory");
                        }
                    }
            }
            continue;
        }
#pragma unroll
        for (int ti = 0; ti < T; ++ti) {
            const int col0 = cb * kCols + (warp * T + ti) * 16 + g;
#pragma unroll
            for (int rb = 0; rb < MB; ++rb)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = rb * 8 + 2 * t + (i & 1), col = col0 + (i >> 1) * 8;
                    if (row < a.M && col < a.N) {
                        const size_t at = (size_t)prob * a.y_stride + (size_t)row * a.N + col;
                        if (a.f32_out) reinterpret_cast<float*>(a.y)[at] = acc[ti][rb][i];
                        else reinterpret_cast<__nv_bfloat16*>(a.y)[at] = f2bf(acc[ti][rb][i]);
                    }
                }
        }
    }
    if (threadIdx.x == 0) stamp(tr, 9);
}

template <class C, bool MULTI = false>
int launch(const Args& a, cudaStream_t stream) {
    static_assert(C::SMEM <= (C::CTAS == 2 ? 113 : 227) * 1024, "stage ring does not fit shared memory");
    auto kern = qmm_kernel<C, MULTI>;
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

// bytes of the next matmul's weight each worker asks L2 for (TF_QMM_PREFETCH_KB, default the ring's size)
// the peer destination of the launch being set up (tf_qmm_peer hands it to tf_qmm_next on the same thread)
struct PeerOut {
    uint8_t* const* bufs = nullptr;
    const uint32_t* seq = nullptr;
    size_t slot_bytes = 0;
    int rank = 0, world = 0;
};
thread_local PeerOut g_peer;
// the SwiGLU destination of the launch being set up (tf_qmm_act hands it to tf_qmm_next on the same thread)
thread_local uint8_t* g_act = nullptr;

inline int prefetch_bytes() {
    static const int v = [] { const char* e = std::getenv("TF_QMM_PREFETCH_KB"); return (e ? atoi(e) : 224) * 1024; }();
    return v;
}

template <int G>
int dispatch(const Args& a, cudaStream_t stream) {
    // up to 16 rows the kernel streams from HBM: a warp takes two column tiles, which share the activation
    // loads; the wider buckets are bound by the tensor pipe and keep one tile a warp (their accumulators
    // take the registers)
    if (a.M <= 8) return launch<Cfg<G, 1, 4, 2, 1>>(a, stream);
    if (a.M <= 16) return launch<Cfg<G, 2, 4, 2, 1>>(a, stream);
    if (a.M <= 32) return launch<Cfg<G, 4, 4, 1, 1>>(a, stream);
    if (a.M <= 64) return launch<Cfg<G, 8, 2, 1, 1>>(a, stream);
    return launch<Cfg<G, 16, 2, 1, 1>>(a, stream);
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

int tf_version(void) { return 1001; }

int tf_qmm_set_trace(void* stamps) {
    unsigned long long* p = static_cast<unsigned long long*>(stamps);
    return cudaMemcpyToSymbol(tf::g_trace, &p, sizeof(p)) == cudaSuccess ? TF_OK : TF_ECUDA;
}
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
    return tf::kScratchBytes;
}

int tf_qmm(const void* x_packed, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M, int N, int K,
           int group, int flags, int* status, void* stream) {
    return tf_qmm_next(x_packed, w_tiled, y, scratch, scratch_bytes, M, N, K, group, flags, nullptr, 0, 0, 0, status, stream);
}

int tf_qmm_next(const void* x_packed, const void* w_tiled, void* y, void* scratch, size_t scratch_bytes, int M, int N, int K,
                int group, int flags, const void* next_w_tiled, int next_N, int next_K, int next_group, int* status, void* stream) {
    if (next_w_tiled && (next_N < 1 || next_K < 64 || next_K % 64 || (next_group != 64 && next_group != 32) || ((uintptr_t)next_w_tiled & 15)))
        return TF_EINVAL;
    if (M < 1 || M > TF_QMM_MAX_ROWS || N < 1 || K < 64 || K % 64) return TF_EINVAL;
    if (group != 64 && group != 32) return TF_EINVAL;
    if (flags & ~TF_QMM_F32_OUT) return TF_EINVAL;
    if (!x_packed || !w_tiled || (!y && tf::g_peer.bufs == nullptr && tf::g_act == nullptr)) return TF_EINVAL;
    const long long CB = (N + tf::kCols - 1) / tf::kCols, IT = tf::item_tiles_for((int)CB, K / 64), SPB = (K / 64 + IT - 1) / IT;
    if (CB * SPB > (1 << 30) / tf::kWorkers) return TF_EINVAL;
    if (((uintptr_t)x_packed | (uintptr_t)w_tiled) & 15) return TF_EALIGN;
    if ((uintptr_t)y & 3) return TF_EALIGN;
    if (!scratch || ((uintptr_t)scratch & 255)) return TF_ESCRATCH;
    if (scratch_bytes < tf_qmm_scratch_bytes()) return TF_ESCRATCH;
    tf::Args a;
    a.xp = static_cast<const uint8_t*>(x_packed);
    a.w = static_cast<const uint8_t*>(w_tiled);
    a.y = y;
    a.epochs = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(scratch) + tf::kEpochOffset);
    a.slots = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + TF_QMM_COUNTER_BYTES);
    a.status = status;
    a.M = M; a.N = N; a.K = K;
    a.f32_out = (flags & TF_QMM_F32_OUT) ? 1 : 0;
    a.prob_expert = nullptr; a.prob_count = nullptr; a.prob_sel = nullptr; a.max_probs = 1;
    a.w_stride = a.xp_stride = a.y_stride = 0;
    a.next_w = static_cast<const uint8_t*>(next_w_tiled); a.next_N = next_N; a.next_K = next_K; a.next_group = next_group;
    a.prefetch_bytes = tf::prefetch_bytes();
    a.peer_bufs = tf::g_peer.bufs; a.peer_seq = tf::g_peer.seq; a.peer_slot_bytes = tf::g_peer.slot_bytes;
    a.peer_rank = tf::g_peer.rank; a.peer_world = tf::g_peer.world;
    tf::g_peer = tf::PeerOut();
    if (a.peer_bufs != nullptr) a.y = nullptr;
    a.act_packed = tf::g_act;
    tf::g_act = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return group == 64 ? tf::dispatch<64>(a, st) : tf::dispatch<32>(a, st);
}

int tf_qmm_act(const void* x_packed, const void* w_tiled, void* act_packed, void* scratch, size_t scratch_bytes, int M, int N, int K,
               int group, const void* next_w_tiled, int next_N, int next_K, int next_group, int* status, void* stream) {
    // the row bucket whose consumer warps own a gate tile and its up tile; whole activation tiles
    if (M < 1 || M > 8 || N < 32 || N % 32 || !act_packed || ((uintptr_t)act_packed & 15)) return TF_EINVAL;
    tf::g_act = static_cast<uint8_t*>(act_packed);
    const int rc = tf_qmm_next(x_packed, w_tiled, nullptr, scratch, scratch_bytes, M, N, K, group, 0, next_w_tiled, next_N, next_K,
                               next_group, status, stream);
    tf::g_act = nullptr;
    return rc;
}

int tf_qmm_peer(const void* x_packed, const void* w_tiled, void* scratch, size_t scratch_bytes, int M, int N, int K, int group,
                void* const* peer_bufs, size_t slot_bytes, const void* seq, int rank, int world, const void* next_w_tiled,
                int next_N, int next_K, int next_group, int* status, void* stream) {
    if (!peer_bufs || !seq || world < 2 || world > 64 || rank < 0 || rank >= world) return TF_EINVAL;
    if (slot_bytes < tf_peer_slot_bytes(M, N, world) || (slot_bytes & 15)) return TF_EINVAL;
    tf::g_peer.bufs = reinterpret_cast<uint8_t* const*>(peer_bufs);
    tf::g_peer.seq = static_cast<const uint32_t*>(seq);
    tf::g_peer.slot_bytes = slot_bytes; tf::g_peer.rank = rank; tf::g_peer.world = world;
    const int rc = tf_qmm_next(x_packed, w_tiled, nullptr, scratch, scratch_bytes, M, N, K, group, TF_QMM_F32_OUT, next_w_tiled, next_N,
                               next_K, next_group, status, stream);
    tf::g_peer = tf::PeerOut();
    return rc;
}

int tf_qmm_grouped(const void* x_packed, const void* w_tiled, const int* prob_expert, const int* prob_count,
                   const int* prob_sel, int max_probs, void* y, void* scratch, size_t scratch_bytes, int N, int K, int group, int flags, int* status,
                   void* stream) {
    if (max_probs < 1 || N < 1 || K < 64 || K % 64) return TF_EINVAL;
    if (group != 64 && group != 32) return TF_EINVAL;
    if (flags & ~TF_QMM_F32_OUT) return TF_EINVAL;
    if (!x_packed || !w_tiled || !y || !prob_expert || !prob_count) return TF_EINVAL;
    const long long CB = (N + tf::kCols - 1) / tf::kCols;     // one schedule item per (problem, column block)
    if (CB * max_probs > (1 << 30) / tf::kWorkers) return TF_EINVAL;
    if (((uintptr_t)x_packed | (uintptr_t)w_tiled) & 15) return TF_EALIGN;
    if ((uintptr_t)y & 3) return TF_EALIGN;
    if (!scratch || ((uintptr_t)scratch & 255)) return TF_ESCRATCH;
    if (scratch_bytes < tf_qmm_scratch_bytes()) return TF_ESCRATCH;
    tf::Args a;
    a.xp = static_cast<const uint8_t*>(x_packed);
    a.w = static_cast<const uint8_t*>(w_tiled);
    a.y = y;
    a.epochs = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(scratch) + tf::kEpochOffset);
    a.slots = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + TF_QMM_COUNTER_BYTES);
    a.status = status;
    a.M = 8; a.N = N; a.K = K;
    a.f32_out = (flags & TF_QMM_F32_OUT) ? 1 : 0;
    a.prob_expert = prob_expert; a.prob_count = prob_count; a.prob_sel = prob_sel; a.max_probs = max_probs;
    a.next_w = nullptr; a.next_N = a.next_K = a.next_group = a.prefetch_bytes = 0;
    a.peer_bufs = nullptr; a.peer_seq = nullptr; a.peer_slot_bytes = 0; a.peer_rank = a.peer_world = 0;
    a.act_packed = nullptr;
    a.w_stride = (long long)tf_qmm_tiled_bytes(N, K, group);
    a.xp_stride = (long long)tf_packed_bytes(8, K, group);
    a.y_stride = 8ll * N;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return group == 64 ? tf::launch<tf::Cfg<64, 1, 4, 2, 1>, true>(a, st) : tf::launch<tf::Cfg<32, 1, 4, 2, 1>, true>(a, st);
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
