// Exact top-k over vocabulary rows and the keyed Gumbel-max draw.
//
// top-k: a bf16 logit is a 16-bit sortable key. Two 256-bin histogram passes find the k-th largest
// key T; a third pass collects everything above T plus the ties at T with the SMALLEST token ids;
// the k survivors are ordered by (value descending, id ascending). Each thread scans a contiguous
// slice of the row and a block-wide prefix sum places its finds, so the result is a function of the
// row alone: no atomics decide which tie survives. One CTA per row.
//
// draw: token = argmax over the kept candidates of logit/T + Gumbel(hash(seed, position, id)), the
// candidates being the top_k cut to the smallest prefix whose tempered probability reaches top_p.
// The hash (splitmix64) and the arithmetic (fp64) follow the host rule, so a row gets the same
// token whether it is drawn alone or inside a window.

#include "common.cuh"

namespace tf {
namespace {

constexpr int kThreads = 1024, kMaxK = 64;

__device__ __forceinline__ uint32_t sort_key(uint32_t b) { return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u); }

// exclusive prefix sum of one int per thread over the CTA (1024 threads), fixed order
__device__ int block_scan(int v, int* warp_tot, int& total) {
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
        int w = warp_tot[lane], winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        warp_tot[lane] = winc - w;
        if (lane == 31) warp_tot[32] = winc;
    }
    __syncthreads();
    const int base = warp_tot[warp];
    total = warp_tot[32];
    __syncthreads();
    return base + inc - v;
}

__global__ void __launch_bounds__(kThreads) topk_kernel(const __nv_bfloat16* x, size_t row_stride, int V, int K, int* idx_out,
                                                        float* val_out) {
    __shared__ unsigned hist[256];
    __shared__ int found[4];
    __shared__ int warp_tot[33];
    __shared__ uint32_t sel_key[kMaxK];
    __shared__ int sel_idx[kMaxK];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const uint16_t* xr = reinterpret_cast<const uint16_t*>(x) + (size_t)row * row_stride;
    const int per = (V + kThreads - 1) / kThreads;
    const int lo = min(V, tid * per), hi = min(V, lo + per);       // this thread's contiguous slice

    // pass 1: histogram of the key's high byte (counts do not depend on the order they are added in)
    for (int i = tid; i < 256; i += kThreads) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < V; i += kThreads) atomicAdd(&hist[sort_key(xr[i]) >> 8], 1u);
    __syncthreads();
    if (tid == 0) {
        unsigned above = 0;
        int b = 255;
        for (; b >= 0; --b) {
            if (above + hist[b] >= (unsigned)K) break;
            above += hist[b];
        }
        found[0] = max(b, 0);
        found[2] = (int)above;
    }
    __syncthreads();
    const uint32_t hb = (uint32_t)found[0];
    __syncthreads();
    // pass 2: histogram of the low byte inside that high byte
    for (int i = tid; i < 256; i += kThreads) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < V; i += kThreads) {
        const uint32_t key = sort_key(xr[i]);
        if ((key >> 8) == hb) atomicAdd(&hist[key & 0xFFu], 1u);
    }
    __syncthreads();
    if (tid == 0) {
        unsigned above = (unsigned)found[2];
        int b = 255;
        for (; b >= 0; --b) {
            if (above + hist[b] >= (unsigned)K) break;
            above += hist[b];
        }
        found[1] = (int)((hb << 8) | (uint32_t)max(b, 0));
        found[2] = (int)above;                 // elements strictly above the threshold key
    }
    __syncthreads();
    const uint32_t T = (uint32_t)found[1];
    const int above = found[2], need = K - above;
    // pass 3: everything above T (slot = rank in id order), then the first `need` ties in id order
    int n_above = 0, n_tie = 0;
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = sort_key(xr[i]);
        n_above += key > T;
        n_tie += key == T;
    }
    int total;
    int at_above = block_scan(n_above, warp_tot, total);
    int at_tie = block_scan(n_tie, warp_tot, total);
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = sort_key(xr[i]);
        if (key > T) {
            if (at_above < kMaxK) { sel_key[at_above] = key; sel_idx[at_above] = i; }
            ++at_above;
        } else if (key == T) {
            if (at_tie < need) { sel_key[above + at_tie] = key; sel_idx[above + at_tie] = i; }
            ++at_tie;
        }
    }
    __syncthreads();
    // order the K survivors: key descending, id ascending (rank by counting)
    if (tid < K) {
        const uint32_t kk = sel_key[tid];
        const int ii = sel_idx[tid];
        int rank = 0;
        for (int j = 0; j < K; ++j) rank += (sel_key[j] > kk) || (sel_key[j] == kk && sel_idx[j] < ii);
        idx_out[(size_t)row * K + rank] = ii;
        val_out[(size_t)row * K + rank] = __uint_as_float((uint32_t)xr[ii] << 16);
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

inline cudaError_t launch_pdl(const void* fn, dim3 grid, dim3 block, cudaStream_t st, void** args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelExC(&cfg, fn, args);
}

}  // namespace
}  // namespace tf

extern "C" {

int tf_topk_rows(const void* x, size_t row_stride, int rows, int vocab, int k, int* idx, float* val, void* stream) {
    if (rows < 1 || vocab < 1 || k < 1 || k > tf::kMaxK || k > vocab || row_stride < (size_t)vocab) return TF_EINVAL;
    if (!x || !idx || !val) return TF_EINVAL;
    void* args[] = {&x, &row_stride, &vocab, &k, &idx, &val};
    if (tf::launch_pdl((const void*)tf::topk_kernel, dim3(rows), dim3(tf::kThreads), static_cast<cudaStream_t>(stream), args) !=
        cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

int tf_sample_rows(const int* idx, const float* val, int width, const long long* positions, unsigned long long seed,
                   double temperature, int top_k, double top_p, int* tokens, int rows, void* stream) {
    if (rows < 1 || width < 1 || width > tf::kMaxK || !idx || !val || !positions || !tokens) return TF_EINVAL;
    void* args[] = {&idx, &val, &width, &positions, &seed, &temperature, &top_k, &top_p, &tokens, &rows};
    if (tf::launch_pdl((const void*)tf::sample_kernel, dim3((rows + 63) / 64), dim3(64), static_cast<cudaStream_t>(stream), args) !=
        cudaSuccess) { cudaGetLastError(); return TF_ECUDA; }
    return TF_OK;
}

}  // extern "C"
