// Mixture-of-experts block around the grouped lane matmul: router logits, per-row selection, the
// window's problem list, gather/pack of expert inputs, the expert activation, and the slot-ordered
// combine.
//
// Every step treats a row on its own: the router is one fixed-order fp32 dot per (row, expert), the
// selection looks at the row's logits only, an expert's rows are multiplied in 8-row problems whose
// arithmetic does not depend on the companions (tf_qmm_grouped), and the combine adds a row's slots in
// slot order. So a row of a window has the bits of the same row routed and computed alone.
//
// Problem list: the distinct experts of a window in ascending id, each cut into problems of up to 8
// members (a member = one (row, slot) pair, in row order). prob_expert[p] names the expert,
// prob_rows[p][j] the member (row * 32 + slot, or -1), pair_loc[row][slot] = p * 8 + j says where the
// pair's results live in the compact [problem][8][...] buffers. The shared expert is expert id E and
// rides as the last slot of every row.

#include "common.cuh"

namespace tf {
namespace {

constexpr int kMaxExperts = 1023;      // routed experts + the shared one fit one CTA of 1024 threads
constexpr int kMaxSlots = 32;          // member code = row * 32 + slot

// ---- router: logits[r, e] = fp32 x[r] . w[e] ------------------------------------------------------
// One warp per (expert, block of 8 rows). Lane l owns inputs 8l..8l+7 of every 256-input step and adds
// them in order with fma; the 32 lane sums combine in a pairwise tree. Fixed by D alone.
__global__ void __launch_bounds__(128) moe_router_kernel(const __nv_bfloat16* x, size_t x_stride, const __nv_bfloat16* w, float* out,
                                                         int R, int D, int NE) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 4 + warp, r0 = blockIdx.y * 8;
    if (e >= NE) return;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    const int rows = min(8, R - r0);
    for (int k = lane * 8; k < D; k += 256) {
        float wv[8];
        unpack8(*reinterpret_cast<const uint4*>(w + (size_t)e * D + k), wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < rows) {
                float xv[8];
                unpack8(*reinterpret_cast<const uint4*>(x + (size_t)(r0 + i) * x_stride + k), xv);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i] = __fmaf_rn(xv[j], wv[j], acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float v = acc[i];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && i < rows) out[(size_t)(r0 + i) * NE + e] = v;
    }
}

// ---- selection: one warp per row ------------------------------------------------------------------
// top_k experts by (logit descending, id ascending); weights bf16(exp(l_k - l_0) / sum), the sum in
// slot order; then the shared expert (id E) as slot top_k with weight bf16(sigmoid(bf16(its logit))).
__global__ void __launch_bounds__(32) moe_select_kernel(const float* logits, int NE, int E, int top_k, int* pick, float* wts) {
    __shared__ float v[kMaxExperts + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x, lane = threadIdx.x, slots = top_k + (NE > E ? 1 : 0);
    for (int i = lane; i < E; i += 32) v[i] = logits[(size_t)r * NE + i];
    __syncwarp();
    float top = 0.f, total = 0.f, mine = 0.f;
    int my_pick = 0;
    for (int k = 0; k < top_k; ++k) {
        float best = -INFINITY;
        int at = 0x7FFFFFFF;
        for (int i = lane; i < E; i += 32) {
            const float c = v[i];
            if (c > best || (c == best && i < at)) { best = c; at = i; }     // ascending i: the first maximum
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (k == 0) top = best;
        const float ex = expf(best - top);
        total += ex;
        if (lane == k) { mine = ex; my_pick = at; }
        if (lane == 0 && at < E) v[at] = -INFINITY;
        __syncwarp();
    }
    if (lane < top_k) {
        pick[(size_t)r * slots + lane] = my_pick;
        wts[(size_t)r * slots + lane] = bf2f(f2bf(mine / total));
    }
    if (lane == 0 && NE > E) {
        const float sg = bf2f(f2bf(logits[(size_t)r * NE + E]));
        pick[(size_t)r * slots + top_k] = E;
        wts[(size_t)r * slots + top_k] = bf2f(f2bf(1.0f / (1.0f + expf(-sg))));
    }
}

// ---- problem list: one CTA, one thread per expert id ----------------------------------------------
// exclusive prefix sum of one int per thread over the CTA's 1024 threads, fixed order
__device__ int scan1024(int v, int* warp_tot, int& total) {
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
    const int base = warp_tot[warp] + inc - v;
    total = warp_tot[32];
    __syncthreads();
    return base;
}

// Expert parallelism (world > 1): routed expert e lives on rank e / (E / world) as local weight slot
// e % (E / world); the shared expert (id E) is replicated as local slot E / world and its problems
// are dealt round-robin. Every rank builds the same global list and, besides, the ascending list
// prob_sel of the problems it owns; prob_expert then holds LOCAL weight slots (meaningful for owned
// problems only).
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* pick, int R, int slots, int NE, int max_probs, int* prob_expert,
                                                         int* prob_count, int* prob_rows, int* pair_loc, int E, int rank, int world,
                                                         int* prob_sel, int* sel_count) {
    extern __shared__ int sh_pick[];             // R * slots picks
    __shared__ int warp_tot[33];
    __shared__ int cnt_s[1024], base_s[1024], sel_s[1024];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pairs = R * slots, chunks = (pairs + 31) >> 5;
    for (int i = tid; i < pairs; i += 1024) sh_pick[i] = pick[i];
    __syncthreads();
    // members of each expert: a warp per expert (ids warp, warp + 32, ...), lanes over the pairs
    for (int e = warp; e < NE; e += 32) {
        int c = 0;
#pragma unroll 4
        for (int k = 0; k < chunks; ++k) {
            const int i = k * 32 + lane;
            c += __popc(__ballot_sync(0xffffffffu, i < pairs && sh_pick[i] == e));
        }
        if (lane == 0) cnt_s[e] = c;
    }
    __syncthreads();
    const int cnt = tid < NE ? cnt_s[tid] : 0;
    const int mine = (cnt + 7) >> 3;             // problems of expert `tid`
    int all;
    const int base = scan1024(mine, warp_tot, all);
    const int total = min(all, max_probs);
    if (tid == 0) prob_count[0] = total;
    const int per = world > 1 ? E / world : 0;
    // problems of an expert owned by this rank: all or none for a routed expert, every world-th for the shared one
    int owned = 0;
    if (world > 1 && tid < NE) owned = tid >= E ? (mine + world - 1 - rank) / world : (tid / per == rank ? mine : 0);
    int all_owned = 0;
    const int sel_base = world > 1 ? scan1024(owned, warp_tot, all_owned) : 0;
    if (world > 1 && tid == 0) sel_count[0] = all_owned;    // owned problems never exceed max_probs: they are a subset
    base_s[tid] = base;
    sel_s[tid] = sel_base;
    __syncthreads();
    // placement, in row order: a member's place is the count of earlier members of its expert
    for (int e = warp; e < NE; e += 32) {
        if (cnt_s[e] == 0) continue;
        const bool shared = e >= E;
        const int b0 = base_s[e];
        int j = 0;
#pragma unroll 2
        for (int k = 0; k < chunks; ++k) {
            const int i = k * 32 + lane;
            const bool hit = i < pairs && sh_pick[i] == e;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int jj = j + __popc(m & ((1u << lane) - 1u));
                const int pq = jj >> 3, p = b0 + pq;
                if (p < max_probs) {
                    const int row = i / slots, slot = i - row * slots;
                    prob_rows[p * 8 + (jj & 7)] = row * kMaxSlots + slot;
                    pair_loc[i] = p * 8 + (jj & 7);
                    if ((jj & 7) == 0) {
                        if (world == 1) {
                            prob_expert[p] = e;
                        } else {
                            prob_expert[p] = shared ? per : e % per;
                            if (shared) {
                                if (pq % world == rank) prob_sel[sel_s[e] + pq / world] = p;
                            } else if (e / per == rank) {
                                prob_sel[sel_s[e] + pq] = p;
                            }
                        }
                    }
                }
            }
            j += __popc(m);
        }
        const int pad = ((j + 7) & ~7) - j;      // absent members of the expert's last problem
        if (lane < pad) {
            const int jj = j + lane, p = b0 + (jj >> 3);
            if (p < max_probs) prob_rows[p * 8 + (jj & 7)] = -1;
        }
    }
}

// ---- gather + pack: problem p's 8 input rows in the matmul's packed form ---------------------------
// A member reads its window row of x [R, K]; absent members are zero rows.
template <int G>
__global__ void moe_pack_kernel(const __nv_bfloat16* x, size_t x_stride, const int* prob_rows, const int* prob_count, int max_probs,
                                uint8_t* xp, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int p = blockIdx.y;
    if (p >= min(prob_count[0], max_probs)) return;
    const int id = blockIdx.x * blockDim.x + threadIdx.x;
    const int chunks = 8 * (K >> 3);
    const int j = id / (K >> 3), c = id - j * (K >> 3);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id < chunks) {
        const int code = prob_rows[p * 8 + j];
        if (code >= 0) v = *reinterpret_cast<const uint4*>(x + (size_t)(code / kMaxSlots) * x_stride + 8 * c);
    }
    const float s = group_sum8<G>(v);
    if (id >= chunks) return;
    packed_store<G>(xp + (size_t)p * tf_packed_size(8, K, G), 8, j, c, v, s);
}

// ---- expert activation: act = bf16(silu(gate) * up) of problem p's rows, packed for the down matmul ---
template <int G>
__global__ void moe_act_kernel(const __nv_bfloat16* gate_up, const int* prob_count, int max_probs, uint8_t* act_packed, int I) {
    pdl_launch_dependents();
    pdl_wait();
    const int p = blockIdx.y;
    if (p >= min(prob_count[0], max_probs)) return;
    const int id = blockIdx.x * blockDim.x + threadIdx.x;
    const int chunks = 8 * (I >> 3);
    const int j = id / (I >> 3), c = id - j * (I >> 3);
    uint4 ov = make_uint4(0, 0, 0, 0);
    if (id < chunks) {
        const __nv_bfloat16* row = gate_up + ((size_t)p * 8 + j) * 2 * I;
        float g[8], u[8], o[8];
        unpack8(*reinterpret_cast<const uint4*>(row + 8 * c), g);
        unpack8(*reinterpret_cast<const uint4*>(row + I + 8 * c), u);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = g[i] * sigmoidf_(g[i]) * u[i];
        ov = pack8(o);
    }
    const float s = group_sum8<G>(ov);
    if (id >= chunks) return;
    packed_store<G>(act_packed + (size_t)p * tf_packed_size(8, I, G), 8, j, c, ov, s);
}

// ---- combine: out[r] = bf16( sum over slots in order of w[r,k] * y[pair (r,k)] ) --------------------
__global__ void moe_combine_kernel(const float* y, const int* pair_loc, const float* wts, int slots, __nv_bfloat16* out, int R, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= (D >> 2) || r >= R) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < slots; ++k) {
        const float w = wts[(size_t)r * slots + k];
        const float4 v = *reinterpret_cast<const float4*>(y + (size_t)pair_loc[r * slots + k] * D + 4 * c);
        acc.x = __fmaf_rn(w, v.x, acc.x);
        acc.y = __fmaf_rn(w, v.y, acc.y);
        acc.z = __fmaf_rn(w, v.z, acc.z);
        acc.w = __fmaf_rn(w, v.w, acc.w);
    }
    __nv_bfloat16* o = out + (size_t)r * D + 4 * c;
    *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(acc.x, acc.y);
    *reinterpret_cast<__nv_bfloat162*>(o + 2) = __floats2bfloat162_rn(acc.z, acc.w);
}

// ---- expert parallelism: results of a rank's own problems to every rank, then the combine --------------
// Packets as in the tensor-parallel exchange: 16 bytes {value, n, value, n}, n = the exchange number. A
// problem has one owner, so the data part of every rank's slot is one array indexed like the compact results
// ([problem * 8 + place][D / 2] packets) and nobody writes another's entries. The combine polls exactly
// the packets its pairs need (bounded) and adds a row's slots in slot order, as on one GPU.
//
// A slot starts with kPresenceBytes of presence cells, one 16-byte cell {n, n, n, n} per source rank. Every
// rank writes its cell into every rank's slot in EVERY exchange, also when it owns no problem, and a combine
// advances the exchange number only after it has seen all `world` cells carry n. So a rank that has passed
// combine n+1 knows that every rank has issued push n+1, which each issues only after its combine n completed:
// nobody still reads the slot of exchange n when exchange n+2 is pushed into it. The slot of an exchange is
// (n & 1), chosen on the device, so a captured graph with an odd number of exchanges still alternates.
constexpr size_t kPresenceBytes = 1024;      // 64 ranks x 16 bytes

__device__ __forceinline__ uint4 ld_volatile16(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile16(uint4* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__global__ void __launch_bounds__(256) moe_push_kernel(const float2* y, const int* prob_sel, const int* sel_count, int D2,
                                                       uint8_t* const* bufs, size_t slot_bytes, int rank, int world,
                                                       const uint32_t* seq) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(seq) + 1u;
    const size_t slot_off = (want & 1u) * slot_bytes;
    if (blockIdx.x == 0 && blockIdx.y == 0 && (int)threadIdx.x < world)
        st_volatile16(reinterpret_cast<uint4*>(bufs[threadIdx.x] + slot_off) + rank, make_uint4(want, want, want, want));
    const int n = sel_count[0];
    for (int q = blockIdx.y; q < n; q += gridDim.y) {
        const size_t base = (size_t)prob_sel[q] * 8 * D2;
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < 8 * D2; i += gridDim.x * blockDim.x) {
            const float2 v = y[base + i];
            const uint4 pkt = make_uint4(__float_as_uint(v.x), want, __float_as_uint(v.y), want);
            for (int peer = 0; peer < world; ++peer)
                st_volatile16(reinterpret_cast<uint4*>(bufs[peer] + slot_off + kPresenceBytes) + base + i, pkt);
        }
    }
}

__global__ void moe_combine_peer_kernel(const uint8_t* my_buf, size_t slot_bytes, const int* pair_loc, const float* wts, int slots,
                                        __nv_bfloat16* out, int R, int D, int world, uint32_t* seq, int* tickets, int* status,
                                        unsigned spin_limit) {
    __shared__ int is_last;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t want = *reinterpret_cast<volatile uint32_t*>(seq) + 1u;
    const uint4* cells = reinterpret_cast<const uint4*>(my_buf + (want & 1u) * slot_bytes);
    const uint4* packets = reinterpret_cast<const uint4*>(my_buf + (want & 1u) * slot_bytes + kPresenceBytes);
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;       // c: a pair of packets = 4 values
    // once a wait has run out anywhere in this process the exchange is lost: do not wait again
    bool stalled = status != nullptr && *reinterpret_cast<volatile int*>(status) != 0;
    if (c < (D >> 2) && r < R) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < slots; ++k) {
            const float w = wts[(size_t)r * slots + k];
            const uint4* src = packets + (size_t)pair_loc[r * slots + k] * (D >> 1) + 2 * c;
            uint4 a = ld_volatile16(src), b = ld_volatile16(src + 1);
            unsigned spins = 0;
            while ((a.y != want || a.w != want || b.y != want || b.w != want) && !stalled) {
                if (++spins > spin_limit) { stalled = true; break; }
                a = ld_volatile16(src);
                b = ld_volatile16(src + 1);
            }
            acc.x = __fmaf_rn(w, __uint_as_float(a.x), acc.x);
            acc.y = __fmaf_rn(w, __uint_as_float(a.z), acc.y);
            acc.z = __fmaf_rn(w, __uint_as_float(b.x), acc.z);
            acc.w = __fmaf_rn(w, __uint_as_float(b.z), acc.w);
        }
        __nv_bfloat16* o = out + (size_t)r * D + 4 * c;
        *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(acc.x, acc.y);
        *reinterpret_cast<__nv_bfloat162*>(o + 2) = __floats2bfloat162_rn(acc.z, acc.w);
    }
    if (stalled) report(status, TF_ESTALL);
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(tickets, 1) == (int)(gridDim.x * gridDim.y) - 1;
    __syncthreads();
    if (is_last) {
        // every rank's presence cell, also of ranks that sent this rank no data
        if ((int)threadIdx.x < world) {
            uint4 cell = ld_volatile16(cells + threadIdx.x);
            unsigned spins = 0;
            while ((cell.x != want || cell.y != want || cell.z != want || cell.w != want) && !stalled) {
                if (++spins > spin_limit) { stalled = true; break; }
                cell = ld_volatile16(cells + threadIdx.x);
            }
            if (stalled) report(status, TF_ESTALL);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            *tickets = 0;
            *reinterpret_cast<volatile uint32_t*>(seq) = want;
        }
    }
}

}  // namespace
}  // namespace tf

extern "C" {

int tf_moe_max_problems(int rows, int slots, int experts_total) {
    if (rows < 1 || slots < 1 || experts_total < 1) return 0;
    const int pairs = rows * slots;
    return (experts_total < pairs ? experts_total : pairs) + pairs / 8;
}

int tf_moe_router(const void* x, size_t x_stride, const void* router, float* logits, int rows, int D, int experts_total,
                  void* stream) {
    if (rows < 1 || D < 256 || D % 256 || experts_total < 1 || !x || !router || !logits || x_stride < (size_t)D) return TF_EINVAL;
    if (((uintptr_t)x | (uintptr_t)router | (x_stride * 2)) & 15) return TF_EALIGN;
    void* args[] = {&x, &x_stride, &router, &logits, &rows, &D, &experts_total};
    return tf::launch_pdl((const void*)tf::moe_router_kernel, dim3((experts_total + 3) / 4, (rows + 7) / 8), dim3(128), 0,
                          static_cast<cudaStream_t>(stream), args) == cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

int tf_moe_select(const float* logits, int rows, int experts_total, int experts, int top_k, int* pick, float* wts, void* stream) {
    if (rows < 1 || experts < 1 || experts > tf::kMaxExperts || top_k < 1 || top_k > experts || top_k + 1 > tf::kMaxSlots) return TF_EINVAL;
    if (experts_total != experts && experts_total != experts + 1) return TF_EINVAL;
    if (!logits || !pick || !wts) return TF_EINVAL;
    void* args[] = {&logits, &experts_total, &experts, &top_k, &pick, &wts};
    return tf::launch_pdl((const void*)tf::moe_select_kernel, dim3(rows), dim3(32), 0, static_cast<cudaStream_t>(stream), args) ==
                   cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

int tf_moe_group(const int* pick, int rows, int slots, int experts_total, int max_probs, int* prob_expert, int* prob_count,
                 int* prob_rows, int* pair_loc, int experts, int rank, int world, int* prob_sel, int* sel_count, void* stream) {
    if (rows < 1 || rows > 128 || slots < 1 || slots > tf::kMaxSlots || experts_total < 1 || experts_total > tf::kMaxExperts + 1) return TF_EINVAL;
    if (max_probs < 1 || !pick || !prob_expert || !prob_count || !prob_rows || !pair_loc) return TF_EINVAL;
    if (world < 1 || rank < 0 || rank >= world || experts < 1 || experts > experts_total) return TF_EINVAL;
    if (world > 1 && (experts % world || !prob_sel || !sel_count)) return TF_EINVAL;
    size_t smem = (size_t)rows * slots * sizeof(int);
    void* args[] = {&pick, &rows, &slots, &experts_total, &max_probs, &prob_expert, &prob_count, &prob_rows, &pair_loc,
                    &experts, &rank, &world, &prob_sel, &sel_count};
    return tf::launch_pdl((const void*)tf::moe_group_kernel, dim3(1), dim3(1024), smem, static_cast<cudaStream_t>(stream), args) ==
                   cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

int tf_moe_pack(const void* x, size_t x_stride, const int* prob_rows, const int* prob_count, int max_probs, void* x_packed, int K,
                int group, void* stream) {
    if (max_probs < 1 || max_probs > 65535 || K < 64 || K % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!x || !prob_rows || !prob_count || !x_packed || x_stride < (size_t)K) return TF_EINVAL;
    if (((uintptr_t)x | (uintptr_t)x_packed | (x_stride * 2)) & 15) return TF_EALIGN;
    void* args[] = {&x, &x_stride, &prob_rows, &prob_count, &max_probs, &x_packed, &K};
    const void* fn = group == 64 ? (const void*)tf::moe_pack_kernel<64> : (const void*)tf::moe_pack_kernel<32>;
    return tf::launch_pdl(fn, dim3((K + 255) / 256, max_probs), dim3(256), 0, static_cast<cudaStream_t>(stream), args) == cudaSuccess
               ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

int tf_moe_act(const void* gate_up, const int* prob_count, int max_probs, void* act_packed, int I, int group, void* stream) {
    if (max_probs < 1 || max_probs > 65535 || I < 64 || I % 64 || (group != 64 && group != 32)) return TF_EINVAL;
    if (!gate_up || !prob_count || !act_packed) return TF_EINVAL;
    if (((uintptr_t)gate_up | (uintptr_t)act_packed) & 15) return TF_EALIGN;
    void* args[] = {&gate_up, &prob_count, &max_probs, &act_packed, &I};
    const void* fn = group == 64 ? (const void*)tf::moe_act_kernel<64> : (const void*)tf::moe_act_kernel<32>;
    return tf::launch_pdl(fn, dim3((I + 255) / 256, max_probs), dim3(256), 0, static_cast<cudaStream_t>(stream), args) == cudaSuccess
               ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

int tf_moe_combine(const float* y, const int* pair_loc, const float* wts, int slots, void* out, int rows, int D, void* stream) {
    if (rows < 1 || rows > 65535 || slots < 1 || D < 8 || D % 8 || !y || !pair_loc || !wts || !out) return TF_EINVAL;
    if (((uintptr_t)y | (uintptr_t)out) & 15) return TF_EALIGN;
    void* args[] = {&y, &pair_loc, &wts, &slots, &out, &rows, &D};
    return tf::launch_pdl((const void*)tf::moe_combine_kernel, dim3((D / 4 + 255) / 256, rows), dim3(256), 0,
                          static_cast<cudaStream_t>(stream), args) == cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

size_t tf_moe_slot_bytes(int max_probs, int D) {
    if (max_probs < 1 || D < 4) return 0;
    return tf::kPresenceBytes + (size_t)max_probs * 8 * D * 8;      // presence cells, then a packet per two fp32 values
}

int tf_moe_push(const float* y, const int* prob_sel, const int* sel_count, int max_probs, int D, void* const* peer_bufs,
                size_t slot_bytes, int rank, int world, const void* seq, void* stream) {
    if (max_probs < 1 || D < 4 || D % 4 || world < 2 || world > 64 || rank < 0 || rank >= world) return TF_EINVAL;
    if (!y || !prob_sel || !sel_count || !peer_bufs || !seq || slot_bytes < tf_moe_slot_bytes(max_probs, D)) return TF_EINVAL;
    if (((uintptr_t)y | slot_bytes) & 15) return TF_EALIGN;
    const float2* src = reinterpret_cast<const float2*>(y);
    int d2 = D / 2;
    uint8_t* const* bufs = reinterpret_cast<uint8_t* const*>(peer_bufs);
    const uint32_t* seq_p = static_cast<const uint32_t*>(seq);
    int by = max_probs < 64 ? max_probs : 64;
    void* args[] = {&src, &prob_sel, &sel_count, &d2, &bufs, &slot_bytes, &rank, &world, &seq_p};
    return tf::launch_pdl((const void*)tf::moe_push_kernel, dim3(2, by), dim3(256), 0, static_cast<cudaStream_t>(stream), args) ==
                   cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

int tf_moe_combine_peer(const void* my_buf, size_t slot_bytes, const int* pair_loc, const float* wts, int slots, void* out, int rows,
                        int D, int world, void* seq, void* tickets, int* status, void* stream) {
    if (rows < 1 || rows > 65535 || slots < 1 || D < 8 || D % 8 || world < 2 || world > 64) return TF_EINVAL;
    if (!my_buf || !pair_loc || !wts || !out || !seq || !tickets || slot_bytes <= tf::kPresenceBytes) return TF_EINVAL;
    if (((uintptr_t)my_buf | (uintptr_t)out | slot_bytes) & 15) return TF_EALIGN;
    const uint8_t* buf = static_cast<const uint8_t*>(my_buf);
    uint32_t* seq_p = static_cast<uint32_t*>(seq);
    int* tick_p = static_cast<int*>(tickets);
    unsigned limit = tf::poll_limit_ref();
    void* args[] = {&buf, &slot_bytes, &pair_loc, &wts, &slots, &out, &rows, &D, &world, &seq_p, &tick_p, &status, &limit};
    return tf::launch_pdl((const void*)tf::moe_combine_peer_kernel, dim3((D / 4 + 255) / 256, rows), dim3(256), 0,
                          static_cast<cudaStream_t>(stream), args) == cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

}  // extern "C"
