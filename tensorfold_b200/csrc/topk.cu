// Exact top-k over vocabulary rows and the keyed Gumbel-max draw.
//
// top-k: a bf16 logit is a 16-bit sortable key. A row is cut into contiguous slices of at most 16384
// entries, one CTA per (slice, row). The CTA stages its slice's keys in shared memory, finds the k-th
// largest key T with two 256-bin histograms (high byte, then low byte), and keeps everything above T
// plus the ties at T with the SMALLEST token ids: each thread scans a contiguous piece and a
// block-wide prefix sum places its finds, so no atomic decides which tie survives. A second kernel
// ranks the slices' candidates by (value descending, id ascending) and writes the first k. The row's
// k largest are among its slices' k largest, so the result is exact and a function of the row alone.
//
// draw: token = argmax over the kept candidates of logit/T + Gumbel(hash(seed, position, id)), the
// candidates being the top_k cut to the smallest prefix whose tempered probability reaches top_p.
// The hash (splitmix64) and the arithmetic (fp64) follow the host rule, so a row gets the same
// token whether it is drawn alone or inside a window.

#include "common.cuh"

namespace tf {
namespace {

constexpr int kMaxK = 64;
constexpr int kSliceThreads = 256, kSliceMax = 16384, kMaxSlices = 64, kMergeThreads = 1024;

__host__ __device__ inline int slice_len(int V) {
    const int slices = (V + kSliceMax - 1) / kSliceMax;
    return (((V + slices - 1) / slices) + 7) & ~7;          // a multiple of 8 entries: slices start 16-byte aligned
}
__host__ __device__ inline int slice_count(int V) { return (V + slice_len(V) - 1) / slice_len(V); }

__device__ __forceinline__ uint32_t sort_key(uint32_t b) { return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u); }
__device__ __forceinline__ uint32_t unsort_key(uint32_t k) { return (k & 0x8000u) ? (k & 0x7FFFu) : (~k & 0xFFFFu); }

// exclusive prefix sum of one int per thread over a CTA of NT threads, fixed order
template <int NT>
__device__ int block_scan(int v, int* warp_tot, int& total) {
    constexpr int NW = NT / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < NW ? warp_tot[lane] : 0, winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        if (lane < NW) warp_tot[lane] = winc - w;
        if (lane == 31) warp_tot[32] = winc;
    }
    __syncthreads();
    const int base = warp_tot[warp];
    total = warp_tot[32];
    __syncthreads();
    return base + inc - v;
}

// One histogram pass over the staged keys: bin = byte `shift` of the keys that pass `keep`; lanes of a
// warp that hit the same bin add once (logits crowd into a few exponents). Then the bin holding the
// K-th largest is found: found[0] = bin, found[1] = entries in higher bins.
template <class Keep>
__device__ void select_byte(const uint16_t* keys, int n, int shift, int K, int above0, unsigned* hist, int* warp_tot, int* found,
                            Keep keep) {
    const int tid = threadIdx.x;
    hist[tid] = 0;
    __syncthreads();
    const int padded = (n + kSliceThreads - 1) / kSliceThreads * kSliceThreads;
    for (int i = tid; i < padded; i += kSliceThreads) {
        const uint32_t key = i < n ? keys[i] : 0u;
        const int bin = (i < n && keep(key)) ? (int)((key >> shift) & 0xFFu) : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, bin);
        if (bin >= 0 && (tid & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], (unsigned)__popc(peers));
    }
    __syncthreads();
    // entries in bins above mine: an exclusive prefix sum over the bins in descending order
    const int mine = (int)hist[255 - tid];
    int total;
    const int above = above0 + block_scan<kSliceThreads>(mine, warp_tot, total);
    if (above < K && above + mine >= K) { found[0] = 255 - tid; found[1] = above; }
    __syncthreads();
}

__global__ void __launch_bounds__(kSliceThreads) topk_slice_kernel(const __nv_bfloat16* x, size_t row_stride, int V, int K, uint2* cand) {
    __shared__ __align__(16) uint16_t keys[kSliceMax];
    __shared__ unsigned hist[256];
    __shared__ int found[2];
    __shared__ int warp_tot[33];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, row = blockIdx.y, L = slice_len(V);
    const int v0 = blockIdx.x * L, n = min(L, V - v0);
    const uint16_t* xr = reinterpret_cast<const uint16_t*>(x) + (size_t)row * row_stride + v0;
    uint2* out = cand + ((size_t)row * gridDim.x + blockIdx.x) * K;
    const int kk = min(K, n);                                   // a short slice yields all it has
    for (int j = tid + kk; j < K; j += kSliceThreads) out[j] = make_uint2(0u, 0x7FFFFFFFu);   // ranks behind every real entry

    if ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) {
        for (int i = tid * 8; i < n; i += kSliceThreads * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (i + 2 * j < n) keys[i + 2 * j] = (uint16_t)sort_key(w[j] & 0xFFFFu);
                if (i + 2 * j + 1 < n) keys[i + 2 * j + 1] = (uint16_t)sort_key(w[j] >> 16);
            }
        }
    } else {
        for (int i = tid; i < n; i += kSliceThreads) keys[i] = (uint16_t)sort_key(xr[i]);
    }
    __syncthreads();

    select_byte(keys, n, 8, kk, 0, hist, warp_tot, found, [](uint32_t) { return true; });
    const uint32_t hb = (uint32_t)found[0];
    const int above_hb = found[1];
    __syncthreads();
    select_byte(keys, n, 0, kk, above_hb, hist, warp_tot, found, [hb](uint32_t key) { return (key >> 8) == hb; });
    const uint32_t T = (hb << 8) | (uint32_t)found[0];
    const int above = found[1], need = kk - above;              // entries strictly above T; ties still wanted

    // everything above T, then the first `need` ties, both in id order
    const int per = (n + kSliceThreads - 1) / kSliceThreads;
    const int lo = min(n, tid * per), hi = min(n, lo + per);
    int n_above = 0, n_tie = 0;
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = keys[i];
        n_above += key > T;
        n_tie += key == T;
    }
    int total;
    int at_above = block_scan<kSliceThreads>(n_above, warp_tot, total);
    int at_tie = block_scan<kSliceThreads>(n_tie, warp_tot, total);
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = keys[i];
        if (key > T) {
            out[at_above++] = make_uint2(key, (uint32_t)(v0 + i));
        } else if (key == T) {
            if (at_tie < need) out[above + at_tie] = make_uint2(key, (uint32_t)(v0 + i));
            ++at_tie;
        }
    }
}

// One CTA per row: rank the slices' candidates by (key descending, id ascending); ranks are distinct.
__global__ void __launch_bounds__(kMergeThreads) topk_merge_kernel(const uint2* cand, int n, int K, int* idx_out, float* val_out) {
    __shared__ uint2 c[kMaxSlices * kMaxK];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    for (int i = threadIdx.x; i < n; i += kMergeThreads) c[i] = cand[(size_t)row * n + i];
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kMergeThreads) {
        const uint2 me = c[i];
        if (me.y == 0x7FFFFFFFu) continue;
        int rank = 0;
        for (int j = 0; j < n; ++j) {
            const uint2 o = c[j];
            rank += (o.x > me.x) || (o.x == me.x && o.y < me.y);
        }
        if (rank < K) {
            idx_out[(size_t)row * K + rank] = (int)me.y;
            val_out[(size_t)row * K + rank] = __uint_as_float(unsort_key(me.x) << 16);
        }
    }
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// One thread per row: candidates are few (<= 64) and the rule is a chain of fp64 operations.
__global__ void sample_kernel(const int* idx, const float* val, int width, const long long* positions,
                              unsigned long long seed, double temperature, int top_k, double top_p, int* tokens, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const int* ids = idx + (size_t)row * width;
    const float* vals = val + (size_t)row * width;        // already ordered (value desc, id asc)
    const int k = max(1, min(top_k > 0 ? top_k : width, width));
    const double t = fmax(temperature, 1e-6);
    const double top = (double)vals[0] / t;
    int keep = k;
    if (top_p > 0.0 && top_p < 1.0) {
        double denom = 0.0;
        for (int j = 0; j < k; ++j) denom += exp((double)vals[j] / t - top);
        double cum = 0.0;
        int below = 0;
        for (int j = 0; j < k; ++j) {
            cum += exp((double)vals[j] / t - top) / denom;
            below += cum < top_p;
        }
        keep = min(k, below + 1);
    }
    const unsigned long long h0 = mix64(seed + 0x9E3779B97F4A7C15ull);
    const unsigned long long h1 = mix64(h0 ^ ((unsigned long long)positions[row] * 0xD1B54A32D192ED03ull));
    double best = -INFINITY;
    int pick = ids[0];
    for (int j = 0; j < keep; ++j) {
        const unsigned long long h = mix64(h1 ^ (unsigned long long)(long long)ids[j]);
        const double u = (double)(h >> 11) * 0x1.0p-53 + 0x1.0p-54;
        const double score = (double)vals[j] / t - log(-log(u));
        if (score > best) { best = score; pick = ids[j]; }
    }
    tokens[row] = pick;
}

}  // namespace
}  // namespace tf

extern "C" {

size_t tf_topk_scratch_bytes(int rows, int vocab, int k) {
    if (rows < 1 || vocab < 1 || k < 1 || k > tf::kMaxK) return 0;
    return (size_t)rows * tf::slice_count(vocab) * k * sizeof(uint2);
}

int tf_topk_rows(const void* x, size_t row_stride, int rows, int vocab, int k, int* idx, float* val, void* scratch,
                 size_t scratch_bytes, void* stream) {
    if (rows < 1 || rows > 65535 || vocab < 1 || k < 1 || k > tf::kMaxK || k > vocab || row_stride < (size_t)vocab) return TF_EINVAL;
    if (!x || !idx || !val) return TF_EINVAL;
    const int slices = tf::slice_count(vocab);
    if (slices > tf::kMaxSlices) return TF_EINVAL;
    if (!scratch || scratch_bytes < tf_topk_scratch_bytes(rows, vocab, k)) return TF_ESCRATCH;
    if (reinterpret_cast<uintptr_t>(scratch) & 7) return TF_EALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    void* a1[] = {&x, &row_stride, &vocab, &k, &scratch};
    if (tf::launch_pdl((const void*)tf::topk_slice_kernel, dim3(slices, rows), dim3(tf::kSliceThreads), 0, st, a1) != cudaSuccess) {
        cudaGetLastError();
        return TF_ECUDA;
    }
    int n = slices * k;
    void* a2[] = {&scratch, &n, &k, &idx, &val};
    if (tf::launch_pdl((const void*)tf::topk_merge_kernel, dim3(rows), dim3(tf::kMergeThreads), 0, st, a2) != cudaSuccess) {
        cudaGetLastError();
        return TF_ECUDA;
    }
    return TF_OK;
}

int tf_sample_rows(const int* idx, const float* val, int width, const long long* positions, unsigned long long seed,
                   double temperature, int top_k, double top_p, int* tokens, int rows, void* stream) {
    if (rows < 1 || width < 1 || width > tf::kMaxK || !idx || !val || !positions || !tokens) return TF_EINVAL;
    void* args[] = {&idx, &val, &width, &positions, &seed, &temperature, &top_k, &top_p, &tokens, &rows};
    if (tf::launch_pdl((const void*)tf::sample_kernel, dim3((rows + 63) / 64), dim3(64), 0, static_cast<cudaStream_t>(stream), args) !=
        cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

}  // extern "C"
