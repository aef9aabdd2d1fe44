// Tensor-parallel exchange over peer memory (NVLink / NVSwitch): every rank ends up with all ranks'
// fp32 partials of a row-parallel projection, stacked in rank order, without a library collective.
//
// Each rank owns a buffer in symmetric memory: [flags: one 32-bit word per rank][two slots of
// world x rows x D fp32]. One exchange = one kernel per rank:
//   push    every CTA copies a share of the local partial into slot s, block `rank`, of EVERY rank's
//           buffer (plain 16-byte peer stores; its own buffer included), then fences at system scope
//           and takes a ticket;
//   signal  the last CTA writes the exchange number into flags[rank] of every rank (release, system);
//   wait    and spins (acquire, system; bounded) until its own flags show that number from every
//           rank, so the kernel that follows in the stream may read the gathered partials.
// The exchange number is a device counter that every rank advances identically; slots alternate
// (chosen by the host, fixed per launch) so that a fast rank's next push never lands in a block a
// slower rank is still reading: pushing exchange n+2 into the slot of exchange n requires having
// passed the wait of n+1, which every rank signals only after it consumed n.
// The sum itself (rank order, one rounding) is fused into the kernel that consumes the partials.
//
// No multicast of any kind is used: plain stores to peer addresses only.

#include "common.cuh"

namespace tf {
namespace {

constexpr unsigned kSpinLimit = 1u << 25;     // x ~100 ns: a few seconds, then TF_ESTALL is reported

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) peer_exchange_kernel(const float4* local, int n4, uint8_t* const* bufs, size_t dst_off,
                                                            size_t flags_off, int rank, int world, uint32_t* seq, int* tickets,
                                                            int* status) {
    __shared__ int is_last;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t want = *reinterpret_cast<volatile uint32_t*>(seq) + 1u;
    const int stride = gridDim.x * blockDim.x;
    for (int peer = 0; peer < world; ++peer) {
        float4* dst = reinterpret_cast<float4*>(bufs[peer] + dst_off);
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) dst[i] = local[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(tickets, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence_system();
    if (threadIdx.x < world) {
        st_release_sys(reinterpret_cast<uint32_t*>(bufs[threadIdx.x] + flags_off) + rank, want);
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(bufs[rank] + flags_off) + threadIdx.x;
        unsigned spins = 0;
        while ((int)(ld_acquire_sys(mine) - want) < 0) {
            if (++spins > kSpinLimit) { report(status, TF_ESTALL); break; }
            __nanosleep(64);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        *tickets = 0;
        *reinterpret_cast<volatile uint32_t*>(seq) = want;
    }
}

}  // namespace
}  // namespace tf

extern "C" {

int tf_peer_exchange(const float* local, int rows, int D, void* const* peer_bufs, size_t flags_off, size_t slot_off, int rank,
                     int world, void* seq, void* tickets, int* status, void* stream) {
    if (rows < 1 || D < 4 || D % 4 || world < 2 || world > 64 || rank < 0 || rank >= world) return TF_EINVAL;
    if (!local || !peer_bufs || !seq || !tickets) return TF_EINVAL;
    if (((uintptr_t)local | slot_off | flags_off) & 15) return TF_EALIGN;
    const float4* src = reinterpret_cast<const float4*>(local);
    int n4 = rows * (D / 4);
    size_t dst_off = slot_off + (size_t)rank * rows * D * sizeof(float);
    uint32_t* seq_p = static_cast<uint32_t*>(seq);
    int* tick_p = static_cast<int*>(tickets);
    uint8_t* const* bufs = reinterpret_cast<uint8_t* const*>(peer_bufs);
    int blocks = (n4 + 255) / 256;
    if (blocks > 32) blocks = 32;
    void* args[] = {&src, &n4, &bufs, &dst_off, &flags_off, &rank, &world, &seq_p, &tick_p, &status};
    return tf::launch_pdl((const void*)tf::peer_exchange_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                          args) == cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

}  // extern "C"
