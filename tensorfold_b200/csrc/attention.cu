// Lane GQA attention over a paged KV cache, for the ragged verify windows of many sequences.
//
// Keys of a sequence are its committed tokens (positions 0..L-1, read through the page table) followed
// by the window's own rows (positions L.., read from the forward's uncommitted K/V rows); window row t
// sees positions 0..L+t. The key axis is cut by ABSOLUTE position into chunks of 64-key tiles: 128 keys
// a chunk below position 8192, 512 up to 65536, 2048 beyond (short contexts still spread over the
// whole GPU, long ones do not drown in partials); one CTA handles (sequence, KV head, chunk) for all
// window rows and all query heads of that KV head at once (rows of 16 = one tensor-core tile a warp),
// with an fp32 online softmax per query row over the tiles in order, and writes per-chunk partials
// (m, l, O). A second kernel merges a row's partials: four warps take a quarter of the row's chunks
// each, in order, and their results are combined in warp order; the quarters depend on the row's key
// count only. It can also apply the layer's sigmoid output gate and write the output projection's
// packed input. Every step of a query row's arithmetic is fixed by that row's own
// (sequence, position): a row alone and the same row inside any window give the same bits, and a
// serial step after committing t rows reads the same keys at the same positions as window row t.
//
// Page layout (this library's): k_pages / v_pages [page][kv head][16 tokens][D] bf16, so one
// (page, head) is a contiguous 16 x D block. Masked-out keys never contribute: their scores are
// -inf and their V rows are loaded as zeros.

#include <mutex>

#include "common.cuh"

namespace tf {
namespace {

constexpr int kTileKeys = 64, kPage = 16, kQRows = 64, kAttnWarps = 4;
// chunk c covers keys [chunk_begin(c), chunk_begin(c + 1)): a function of the absolute position only
constexpr int kSmallKeys = 128, kSmallChunks = 64, kMidKeys = 512, kMidChunks = 112, kBigKeys = 2048;
constexpr int kSmallEnd = kSmallKeys * kSmallChunks, kMidEnd = kSmallEnd + kMidKeys * kMidChunks;   // 8192, 65536
__host__ __device__ inline int chunk_begin(int c) {
    if (c < kSmallChunks) return c * kSmallKeys;
    if (c < kSmallChunks + kMidChunks) return kSmallEnd + (c - kSmallChunks) * kMidKeys;
    return kMidEnd + (c - kSmallChunks - kMidChunks) * kBigKeys;
}
// number of chunks that hold keys 0..n-1
__host__ __device__ inline int chunks_for(int n) {
    if (n <= 0) return 0;
    if (n <= kSmallEnd) return (n + kSmallKeys - 1) / kSmallKeys;
    if (n <= kMidEnd) return kSmallChunks + (n - kSmallEnd + kMidKeys - 1) / kMidKeys;
    return kSmallChunks + kMidChunks + (n - kMidEnd + kBigKeys - 1) / kBigKeys;
}
constexpr float kLog2e = 1.4426950408889634f;

struct AttnArgs {
    const __nv_bfloat16* q;        // [R, H, D]
    const __nv_bfloat16* k_new;    // [R, HK, D] window rows (uncommitted)
    const __nv_bfloat16* v_new;
    const __nv_bfloat16* k_pages;  // [pages, HK, 16, D]
    const __nv_bfloat16* v_pages;
    const int* page_table;         // [S, max_pages]
    const int* seq_lens;           // [S] committed length L
    const int* seq_start;          // [S + 1] first packed row of each sequence
    float* part_o;                 // [chunks, R, H, D]
    float* part_m;                 // [chunks, R, H]   (log2 domain)
    float* part_l;
    int max_pages, H, HK, R, qgroups;
    float scale_log2;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

// byte offset of 16-byte chunk c of tile row r (rows of D bf16), xor-swizzled so ldmatrix is conflict free
template <int D>
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * (D * 2) + (((c & ~7) | ((c ^ r) & 7)) << 4)); }

template <int D>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_chunk_kernel(const AttnArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int ROWB = D * 2, TILEB = kTileKeys * ROWB, CPR = D / 8;       // chunks of 16 B per row
    uint8_t* q_s = smem;                       // [64][D]
    uint8_t* k_s = q_s + kQRows * ROWB;        // 2 x [64][D]
    uint8_t* v_s = k_s + 2 * TILEB;            // 2 x [64][D]
    pdl_launch_dependents();
    pdl_wait();
    const int chunk = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z / a.qgroups, qg = blockIdx.z % a.qgroups;
    const int G = a.H / a.HK;
    const int r0 = a.seq_start[seq], n = a.seq_start[seq + 1] - r0, L = a.seq_lens[seq];
    const int nq = n * G;                      // query rows of this (sequence, KV head): row = t * G + head-in-group
    const int q0 = qg * kQRows;
    if (q0 >= nq) return;
    const int key0 = chunk_begin(chunk), chunk_keys = chunk_begin(chunk + 1) - key0;
    if (key0 >= L + n) return;                 // nothing of this sequence in the chunk (partials are not read either)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    // ---- stage Q (rows past nq are zero) and the first K/V tile ----
    for (int e = tid; e < kQRows * CPR; e += kAttnWarps * 32) {
        const int r = e / CPR, c = e % CPR, qr = q0 + r;
        const bool ok = qr < nq;
        const int wr = ok ? qr / G : 0, hq = ok ? qr % G : 0;
        cp_async16_zfill(smem_u32(q_s + swz<D>(r, c)), a.q + ((size_t)(r0 + wr) * a.H + kvh * G + hq) * D + c * 8, ok);
    }
    const int* pt = a.page_table + (size_t)seq * a.max_pages;
    // A tile is four pages of 16 keys; warp w copies page w: the page number is looked up once, then
    // every lane streams its own 16-byte column of the page's rows (K and V), so the per-copy address
    // work is an add. Rows at or past the committed length come from the window's own K/V rows, rows
    // past the last key are zero-filled.
    auto load_tile = [&](int tile, int buf) {
        constexpr int RPI = 32 / CPR > 0 ? 32 / CPR : 1;      // rows a warp covers per step (1 for D = 256, 2 for D = 128)
        const int base = key0 + tile * kTileKeys + warp * kPage;
        const int c = lane % CPR, rsub = lane / CPR;
        const bool any_old = base < L;
        const size_t page_off = any_old ? ((size_t)pt[base / kPage] * a.HK + kvh) * kPage * D : 0;
#pragma unroll 4
        for (int rr = 0; rr < kPage; rr += RPI) {
            const int r = rr + rsub, p = base + r;
            const bool ok = p < L + n;
            size_t off = 0;
            const __nv_bfloat16 *ksrc = a.k_new, *vsrc = a.v_new;
            if (ok) {
                if (p < L) { off = page_off + (size_t)r * D + c * 8; ksrc = a.k_pages; vsrc = a.v_pages; }
                else off = ((size_t)(r0 + p - L) * a.HK + kvh) * D + c * 8;
            }
            const uint32_t dst = swz<D>(warp * kPage + r, c);
            cp_async16_zfill(smem_u32(k_s + buf * TILEB + dst), ksrc + off, ok);
            cp_async16_zfill(smem_u32(v_s + buf * TILEB + dst), vsrc + off, ok);
        }
    };
    const int ntiles = min(chunk_keys / kTileKeys, (L + n - key0 + kTileKeys - 1) / kTileKeys);
    load_tile(0, 0);
    cp_async_commit();

    // this warp's 16 query rows; lane holds rows g and g+8 of them
    const int qrow_lo = q0 + warp * 16 + g, qrow_hi = qrow_lo + 8;
    const bool warp_live = q0 + warp * 16 < nq;
    // last visible key position + 1 for the lane's two rows (0 for padding rows: everything masked)
    const int lim_lo = qrow_lo < nq ? L + qrow_lo / G + 1 : 0, lim_hi = qrow_hi < nq ? L + qrow_hi / G + 1 : 0;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (int tile = 0; tile < ntiles; ++tile) {
        const int buf = tile & 1;
        if (tile + 1 < ntiles) load_tile(tile + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (warp_live) {
            // ---- S = Q K^T for 16 rows x 64 keys ----
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            const uint32_t kb = smem_u32(k_s + buf * TILEB), qb = smem_u32(q_s);
#pragma unroll 4
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t af[4];
                ldsm_x4(af, qb + swz<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
                for (int np = 0; np < 4; ++np) {           // pairs of 8-key tiles
                    uint32_t bf[4];
                    ldsm_x4(bf, kb + swz<D>(np * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
                    mma_bf16_16816(s[2 * np], af, bf[0], bf[1], s[2 * np]);
                    mma_bf16_16816(s[2 * np + 1], af, bf[2], bf[3], s[2 * np + 1]);
                }
            }
            // ---- mask, online softmax (log2 domain) ----
            const int pbase = key0 + tile * kTileKeys + 2 * t;
            float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int p = pbase + i * 8;
                s[i][0] = p < lim_lo ? s[i][0] * a.scale_log2 : -INFINITY;
                s[i][1] = p + 1 < lim_lo ? s[i][1] * a.scale_log2 : -INFINITY;
                s[i][2] = p < lim_hi ? s[i][2] * a.scale_log2 : -INFINITY;
                s[i][3] = p + 1 < lim_hi ? s[i][3] * a.scale_log2 : -INFINITY;
                tmax_lo = fmaxf(tmax_lo, fmaxf(s[i][0], s[i][1]));
                tmax_hi = fmaxf(tmax_hi, fmaxf(s[i][2], s[i][3]));
            }
            tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
            tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
            tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
            tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
            const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
            const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
            const float al_lo = exp2f(m_lo - ms_lo), al_hi = exp2f(m_hi - ms_hi);
            float sum_lo = 0.f, sum_hi = 0.f;
            uint32_t pf[8][2];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float p0 = exp2f(s[i][0] - ms_lo), p1 = exp2f(s[i][1] - ms_lo);
                const float p2 = exp2f(s[i][2] - ms_hi), p3 = exp2f(s[i][3] - ms_hi);
                sum_lo += p0; sum_lo += p1; sum_hi += p2; sum_hi += p3;
                pf[i][0] = pack_bf16(p0, p1);
                pf[i][1] = pack_bf16(p2, p3);
            }
            sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
            sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
            sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
            sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
            l_lo = l_lo * al_lo + sum_lo; l_hi = l_hi * al_hi + sum_hi;
            m_lo = mn_lo; m_hi = mn_hi;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
            // ---- O += P V ----
            const uint32_t vb = smem_u32(v_s + buf * TILEB);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {               // 16 keys a step
                const uint32_t pa[4] = {pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1]};
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {      // pairs of 8-wide output tiles
                    uint32_t bf[4];
                    ldsm_x4_t(bf, vb + swz<D>(kk * 16 + (lane & 15), dp * 2 + (lane >> 4)));
                    mma_bf16_16816(o[2 * dp], pa, bf[0], bf[1], o[2 * dp]);
                    mma_bf16_16816(o[2 * dp + 1], pa, bf[2], bf[3], o[2 * dp + 1]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (!warp_live) return;
    // ---- write this chunk's partials ----
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int qr = half ? qrow_hi : qrow_lo;
        if (qr >= nq) continue;
        const int row = r0 + qr / G, head = kvh * G + qr % G;
        const size_t base = ((size_t)chunk * a.R + row) * a.H + head;
        if (t == 0) { a.part_m[base] = half ? m_hi : m_lo; a.part_l[base] = half ? l_hi : l_lo; }
        float* po = a.part_o + base * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
            *reinterpret_cast<float2*>(po + i * 8 + 2 * t) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
    }
}

// Merge the chunk partials of one (row, head): one CTA of four warps. Warp w merges chunks
// [w * q, (w + 1) * q) of the row's nch chunks in order (q = ceil(nch / 4): a function of the row's key
// count only), then the four results are combined in warp order. With `qg` the sigmoid output gate is
// applied (gate values interleaved per head in the q projection: [q_h ; gate_h]) and with `out_packed`
// the result is written as the output projection's packed input with its group sums.
struct MergeArgs {
    const float* part_o;
    const float* part_m;
    const float* part_l;
    const int* row_nkeys;
    __nv_bfloat16* out;            // [R, H, D] or null
    const __nv_bfloat16* qg;       // gate source or null
    size_t qg_stride;
    uint8_t* out_packed;           // or null
    int R, H, max_chunks, group;
    int* status;
};

template <int D>
__global__ void __launch_bounds__(128) attn_merge_kernel(const MergeArgs a) {
    constexpr int PER = D / 32, NW = 4;
    static_assert(PER % 4 == 0, "a lane's slice is whole 16-byte loads");
    __shared__ float sm_m[NW], sm_l[NW];
    __shared__ __align__(16) float sm_o[NW][D];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.y, head = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Mp = tf_padded_rows(a.R);
    if (row >= a.R) {                                     // padding rows of the packed buffer are zero
        if (a.out_packed != nullptr && warp == 0) {
            const int c = head * (D / 8) + lane;
            if (lane < D / 8) {
                if (a.group == 64) packed_store<64>(a.out_packed, Mp, row, c, make_uint4(0, 0, 0, 0), 0.f);
                else packed_store<32>(a.out_packed, Mp, row, c, make_uint4(0, 0, 0, 0), 0.f);
            }
        }
        return;
    }
    int nch = chunks_for(a.row_nkeys[row]);
    if (nch > a.max_chunks) {                             // the caller sized scratch for fewer chunks: never read past it
        if (threadIdx.x == 0) report(a.status, TF_EINVAL);
        nch = a.max_chunks;
    }
    const int quarter = (nch + NW - 1) / NW, c_lo = min(nch, warp * quarter), c_hi = min(nch, c_lo + quarter);
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    // chunks are read four at a time (independent loads in flight together) and applied one by one in
    // chunk order, so the arithmetic is that of the plain sequential merge of the warp's range
    constexpr int B = 4;
    for (int c0 = c_lo; c0 < c_hi; c0 += B) {
        float cm[B], cl[B];
        float4 po[B][PER / 4];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int c = min(c0 + j, c_hi - 1);
            const size_t base = ((size_t)c * a.R + row) * a.H + head;
            cm[j] = a.part_m[base];
            cl[j] = c0 + j < c_hi ? a.part_l[base] : 0.f;
            const float4* src = reinterpret_cast<const float4*>(a.part_o + base * D + lane * PER);
#pragma unroll
            for (int i = 0; i < PER / 4; ++i) po[j][i] = src[i];
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            if (!(cl[j] > 0.f)) continue;
            const float mn = fmaxf(m, cm[j]);
            const float sa = exp2f(m - mn), sb = exp2f(cm[j] - mn);       // m = -inf gives sa = 0
#pragma unroll
            for (int i = 0; i < PER / 4; ++i) {
                acc[4 * i + 0] = acc[4 * i + 0] * sa + po[j][i].x * sb;
                acc[4 * i + 1] = acc[4 * i + 1] * sa + po[j][i].y * sb;
                acc[4 * i + 2] = acc[4 * i + 2] * sa + po[j][i].z * sb;
                acc[4 * i + 3] = acc[4 * i + 3] * sa + po[j][i].w * sb;
            }
            l = l * sa + cl[j] * sb;
            m = mn;
        }
    }
    if (warp > 0) {
        if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
        for (int i = 0; i < PER; ++i) sm_o[warp][lane * PER + i] = acc[i];
    }
    __syncthreads();
    if (warp != 0) return;
    for (int w = 1; w < NW; ++w) {                        // the later quarters, in order
        const float cl = sm_l[w], cm = sm_m[w];
        if (!(cl > 0.f)) continue;
        const float mn = fmaxf(m, cm);
        const float sa = exp2f(m - mn), sb = exp2f(cm - mn);
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] = acc[i] * sa + sm_o[w][lane * PER + i] * sb;
        l = l * sa + cl * sb;
        m = mn;
    }
    float o[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) o[i] = round_bf16(acc[i] / l);
    if (a.qg != nullptr) {
        const __nv_bfloat16* gp = a.qg + (size_t)row * a.qg_stride + (size_t)head * 2 * D + D + lane * PER;
#pragma unroll
        for (int i = 0; i < PER; ++i) o[i] = round_bf16(o[i] * sigmoidf_(bf2f(gp[i])));
    }
    if (a.out != nullptr) {
        __nv_bfloat16* dst = a.out + ((size_t)row * a.H + head) * D + lane * PER;
#pragma unroll
        for (int i = 0; i < PER; ++i) dst[i] = f2bf(o[i]);
    }
    if (a.out_packed != nullptr) {
        // 8 values a chunk: D = 256 gives one chunk a lane; D = 128 (4 values a lane) pairs lanes up
        if (PER == 8) {
            const float o8[8] = {o[0], o[1], o[2], o[3], o[4 % PER], o[5 % PER], o[6 % PER], o[7 % PER]};
            const uint4 v = pack8(o8);
            const int c = head * (D / 8) + lane;
            if (a.group == 64) { const float gs = group_sum8<64>(v); packed_store<64>(a.out_packed, Mp, row, c, v, gs); }
            else { const float gs = group_sum8<32>(v); packed_store<32>(a.out_packed, Mp, row, c, v, gs); }
        } else {
            // lanes 2j and 2j+1 hold the two halves of chunk j: gather them in the even lane, then let lanes
            // 0..15 act as the chunk's owners (the odd lanes' data moves down so that owners are contiguous)
            float o8[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mine = o[i % PER];
                const float lo = __shfl_sync(0xffffffffu, mine, (2 * lane) & 31), hi = __shfl_sync(0xffffffffu, mine, (2 * lane + 1) & 31);
                o8[i] = lo; o8[4 + i] = hi;
            }
            const uint4 v = lane < 16 ? pack8(o8) : make_uint4(0, 0, 0, 0);
            const int c = head * (D / 8) + (lane & 15);
            if (a.group == 64) { const float gs = group_sum8<64>(v); if (lane < 16) packed_store<64>(a.out_packed, Mp, row, c, v, gs); }
            else { const float gs = group_sum8<32>(v); if (lane < 16) packed_store<32>(a.out_packed, Mp, row, c, v, gs); }
        }
    }
}

// Commit: copy each sequence's kept window rows into its pages at positions L.., for every layer.
__global__ void kv_commit_kernel(const __nv_bfloat16* k_new, const __nv_bfloat16* v_new, long long rec_stride,
                                 __nv_bfloat16* k_pages, __nv_bfloat16* v_pages, long long pages_stride, const int* page_table,
                                 int max_pages, const int* seq_lens, const int* seq_start, const int* keep, int HK, int D, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const int layer = blockIdx.z / S, seq = blockIdx.z % S;
    const int r0 = seq_start[seq], n = min(keep[seq], seq_start[seq + 1] - r0), L = seq_lens[seq];
    const int per_row = HK * D / 8;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < n * per_row; e += gridDim.x * blockDim.x) {
        const int r = e / per_row, c = e % per_row, hk = (c * 8) / D, d = (c * 8) % D;
        const int p = L + r;
        const size_t src = (size_t)layer * rec_stride + ((size_t)(r0 + r) * HK + hk) * D + d;
        const size_t dst = (size_t)layer * pages_stride +
                           (((size_t)page_table[(size_t)seq * max_pages + p / kPage] * HK + hk) * kPage + p % kPage) * D + d;
        *reinterpret_cast<uint4*>(k_pages + dst) = *reinterpret_cast<const uint4*>(k_new + src);
        *reinterpret_cast<uint4*>(v_pages + dst) = *reinterpret_cast<const uint4*>(v_new + src);
    }
}

struct GateArgs {
    const void* qg = nullptr;      // q projection output with the per-head gates, or null
    size_t qg_stride = 0;
    void* out_packed = nullptr;
    int group = 64;
    int* status = nullptr;
};

template <int D>
int run(const AttnArgs& a, int n_seqs, int max_chunks, const int* row_nkeys, void* out, cudaStream_t st, const GateArgs& ga = GateArgs()) {
    constexpr size_t smem = (size_t)(kQRows + 4 * kTileKeys) * D * 2;
    static bool configured[64] = {};       // the opt-in is per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return TF_ECUDA; }
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(attn_chunk_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return TF_ECUDA;
        configured[dev] = true;
    }
    AttnArgs args = a;
    void* p1[] = {&args};
    if (launch_pdl((const void*)attn_chunk_kernel<D>, dim3(max_chunks, a.HK, n_seqs * a.qgroups), dim3(kAttnWarps * 32), smem,
                   st, p1) != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    MergeArgs m;
    m.part_o = a.part_o; m.part_m = a.part_m; m.part_l = a.part_l; m.row_nkeys = row_nkeys;
    m.out = static_cast<__nv_bfloat16*>(out);
    m.qg = static_cast<const __nv_bfloat16*>(ga.qg); m.qg_stride = ga.qg_stride;
    m.out_packed = static_cast<uint8_t*>(ga.out_packed);
    m.R = a.R; m.H = a.H; m.max_chunks = max_chunks; m.group = ga.group; m.status = ga.status;
    void* p2[] = {&m};
    const int grid_rows = ga.out_packed ? tf_padded_rows(a.R) : a.R;
    if (launch_pdl((const void*)attn_merge_kernel<D>, dim3(a.H, grid_rows), dim3(128), 0, st, p2) != cudaSuccess) {
        cudaGetLastError(); return TF_ECUDA;
    }
    return TF_OK;
}

}  // namespace
}  // namespace tf

extern "C" {

size_t tf_attention_scratch_bytes(int rows, int heads, int head_dim, int max_chunks) {
    if (rows < 1 || heads < 1 || head_dim < 1 || max_chunks < 1) return 0;
    return (size_t)max_chunks * rows * heads * (head_dim + 2) * sizeof(float);
}

int tf_attention_chunks(int n_keys) { return tf::chunks_for(n_keys); }

int tf_lane_attention_paged(const void* q, const void* k_new, const void* v_new, const void* k_pages, const void* v_pages,
                            const int* page_table, int max_pages, const int* seq_lens, const int* seq_start,
                            const int* row_nkeys, void* out, void* scratch, size_t scratch_bytes, int rows, int n_seqs,
                            int max_window, int max_chunks, int heads, int kv_heads, int head_dim, float scale, void* stream) {
    return tf_lane_attention_paged_gated(q, k_new, v_new, k_pages, v_pages, page_table, max_pages, seq_lens, seq_start, row_nkeys,
                                         out, nullptr, 0, nullptr, 64, scratch, scratch_bytes, rows, n_seqs, max_window,
                                         max_chunks, heads, kv_heads, head_dim, scale, nullptr, stream);
}

int tf_lane_attention_paged_gated(const void* q, const void* k_new, const void* v_new, const void* k_pages, const void* v_pages,
                                  const int* page_table, int max_pages, const int* seq_lens, const int* seq_start,
                                  const int* row_nkeys, void* out, const void* qg, size_t qg_stride, void* out_packed, int group,
                                  void* scratch, size_t scratch_bytes, int rows, int n_seqs, int max_window, int max_chunks,
                                  int heads, int kv_heads, int head_dim, float scale, int* status, void* stream) {
    if (!out && !out_packed) return TF_EINVAL;
    if ((group != 64 && group != 32) || (qg && qg_stride % 8) || (out_packed && rows > TF_QMM_MAX_ROWS)) return TF_EINVAL;
    if (((uintptr_t)qg | (uintptr_t)out_packed | (uintptr_t)out) & 15) return TF_EALIGN;
    if (rows < 1 || n_seqs < 1 || max_window < 1 || max_chunks < 1 || heads < 1 || kv_heads < 1 || heads % kv_heads) return TF_EINVAL;
    if ((head_dim != 128 && head_dim != 256) || heads / kv_heads > 16 || !(scale > 0.f)) return TF_EINVAL;
    if (!q || !k_new || !v_new || !k_pages || !v_pages || !page_table || !seq_lens || !seq_start || !row_nkeys) return TF_EINVAL;
    if (((uintptr_t)q | (uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) return TF_EALIGN;
    if (!scratch || ((uintptr_t)scratch & 15) || scratch_bytes < tf_attention_scratch_bytes(rows, heads, head_dim, max_chunks))
        return TF_ESCRATCH;
    const int G = heads / kv_heads;
    tf::AttnArgs a;
    a.q = static_cast<const __nv_bfloat16*>(q);
    a.k_new = static_cast<const __nv_bfloat16*>(k_new); a.v_new = static_cast<const __nv_bfloat16*>(v_new);
    a.k_pages = static_cast<const __nv_bfloat16*>(k_pages); a.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
    a.page_table = page_table; a.seq_lens = seq_lens; a.seq_start = seq_start;
    float* sc = static_cast<float*>(scratch);
    const size_t nrh = (size_t)max_chunks * rows * heads;
    a.part_o = sc; a.part_m = sc + nrh * head_dim; a.part_l = a.part_m + nrh;
    a.max_pages = max_pages; a.H = heads; a.HK = kv_heads; a.R = rows;
    a.qgroups = (max_window * G + tf::kQRows - 1) / tf::kQRows;
    a.scale_log2 = scale * tf::kLog2e;
    if ((long long)n_seqs * a.qgroups > 65535) return TF_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    tf::GateArgs ga;
    ga.qg = qg; ga.qg_stride = qg_stride; ga.out_packed = out_packed; ga.group = group; ga.status = status;
    return head_dim == 256 ? tf::run<256>(a, n_seqs, max_chunks, row_nkeys, out, st, ga)
                           : tf::run<128>(a, n_seqs, max_chunks, row_nkeys, out, st, ga);
}

int tf_kv_commit(const void* k_new, const void* v_new, long long rec_stride, void* k_pages, void* v_pages,
                 long long pages_stride, const int* page_table, int max_pages, const int* seq_lens, const int* seq_start,
                 const int* keep, int n_seqs, int layers, int kv_heads, int head_dim, void* stream) {
    if (n_seqs < 1 || layers < 1 || kv_heads < 1 || head_dim % 8 || (long long)n_seqs * layers > 65535) return TF_EINVAL;
    if (!k_new || !v_new || !k_pages || !v_pages || !page_table || !seq_lens || !seq_start || !keep) return TF_EINVAL;
    if (((uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15 || rec_stride % 8 || pages_stride % 8)
        return TF_EALIGN;
    void* args[] = {&k_new, &v_new, &rec_stride, &k_pages, &v_pages, &pages_stride, &page_table, &max_pages, &seq_lens,
                    &seq_start, &keep, &kv_heads, &head_dim, &n_seqs};
    if (tf::launch_pdl((const void*)tf::kv_commit_kernel, dim3(4, 1, n_seqs * layers), dim3(256), 0,
                       static_cast<cudaStream_t>(stream), args) != cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

}  // extern "C"

// ---- the same attention for callers that may not allocate ------------------------------------------
// Some hosts of this library cannot hand it a scratch buffer: an inference server whose device memory
// is carved up once at start-up by its own pool and never grown, a plugin loaded into a runtime that
// forbids cudaMalloc on the serving path (an allocation synchronises the whole device and can fail when
// the pool already owns the memory), or code running inside a region where every buffer address must be
// known in advance. For them the chunk partials live in the fixed array below, which is part of the
// loaded module: every GPU that loads the library holds these bytes until the process exits.
//
// Rules that follow from one shared array: a call needs at most TF_ATTN_STATIC_SCRATCH_BYTES of
// partials (more is refused, nothing runs); the array keeps whatever the previous call left, which is
// harmless here because the merge kernel reads only entries the chunk kernel wrote in the same call, so
// nothing has to be cleared; and two calls that overlap on one GPU (different streams, or threads)
// would overwrite each other's partials — callers must serialise them.
static __device__ __align__(256) unsigned char g_static_partials[TF_ATTN_STATIC_SCRATCH_BYTES];

namespace tf {
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_lock;
void* g_static_addr[kMaxDevices];        // device address of g_static_partials, per device; null = not looked up yet

// The array's name is only a host-side handle here; kernels need its address on the device that is
// current, which the runtime resolves once per device.
int static_partials(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return TF_ECUDA; }
    std::lock_guard<std::mutex> hold(g_static_lock);
    if (g_static_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_partials) != cudaSuccess || p == nullptr) { cudaGetLastError(); return TF_ECUDA; }
        g_static_addr[dev] = p;
    }
    *out = g_static_addr[dev];
    return TF_OK;
}
}  // namespace
}  // namespace tf

extern "C" int tf_lane_attention_paged_static(const void* q, const void* k_new, const void* v_new, const void* k_pages,
                                              const void* v_pages, const int* page_table, int max_pages, const int* seq_lens,
                                              const int* seq_start, const int* row_nkeys, void* out, int rows, int n_seqs,
                                              int max_window, int max_chunks, int heads, int kv_heads, int head_dim, float scale,
                                              void* stream) {
    if (rows < 1 || n_seqs < 1 || max_window < 1 || max_chunks < 1 || heads < 1 || kv_heads < 1 || heads % kv_heads) return TF_EINVAL;
    if ((head_dim != 128 && head_dim != 256) || heads / kv_heads > 16 || !(scale > 0.f)) return TF_EINVAL;
    if (!q || !k_new || !v_new || !k_pages || !v_pages || !page_table || !seq_lens || !seq_start || !row_nkeys || !out) return TF_EINVAL;
    if (((uintptr_t)q | (uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) return TF_EALIGN;
    // too many rows x heads x chunks for the fixed array: refuse before anything is queued
    if (tf_attention_scratch_bytes(rows, heads, head_dim, max_chunks) > (size_t)TF_ATTN_STATIC_SCRATCH_BYTES) return TF_ESCRATCH;
    void* scratch = nullptr;
    const int rc = tf::static_partials(&scratch);
    if (rc != TF_OK) return rc;
    const int G = heads / kv_heads;
    tf::AttnArgs a;
    a.q = static_cast<const __nv_bfloat16*>(q);
    a.k_new = static_cast<const __nv_bfloat16*>(k_new); a.v_new = static_cast<const __nv_bfloat16*>(v_new);
    a.k_pages = static_cast<const __nv_bfloat16*>(k_pages); a.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
    a.page_table = page_table; a.seq_lens = seq_lens; a.seq_start = seq_start;
    float* sc = static_cast<float*>(scratch);
    const size_t nrh = (size_t)max_chunks * rows * heads;
    a.part_o = sc; a.part_m = sc + nrh * head_dim; a.part_l = a.part_m + nrh;
    a.max_pages = max_pages; a.H = heads; a.HK = kv_heads; a.R = rows;
    a.qgroups = (max_window * G + tf::kQRows - 1) / tf::kQRows;
    a.scale_log2 = scale * tf::kLog2e;
    if ((long long)n_seqs * a.qgroups > 65535) return TF_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return head_dim == 256 ? tf::run<256>(a, n_seqs, max_chunks, row_nkeys, out, st)
                           : tf::run<128>(a, n_seqs, max_chunks, row_nkeys, out, st);
}
