// Tensor-parallel exchange over peer memory (NVLink / NVSwitch): every rank ends up with all ranks'
// fp32 partials of a row-parallel projection, stacked in rank order, without a library collective
// and without a fence or a round trip on the critical path.
//
// Each rank owns a buffer in symmetric memory with two "packet" slots. A packet is 16 bytes:
// {value, n, value, n} - two fp32 payload words, each followed by the exchange number n. One exchange =
// one kernel per rank:
//   push    every thread turns its share of the local partial into packets and stores them into
//           block `rank` of the slot in EVERY rank's buffer (plain 16-byte peer stores, own buffer
//           included). The payload carries its own arrival signal, so nothing else is sent.
//   gather  every thread then polls its share of the local slot, block by block in rank order, until
//           both exchange numbers of a packet read n (bounded spin), and writes the payload to the
//           plain [world, rows, D] fp32 array the next kernel reads.
// The exchange number is a device counter every rank advances identically; 8-byte halves of a packet
// are written atomically, and a stale packet carries an older number, so a reader never mixes
// exchanges. Slots alternate (chosen on the device from the exchange number, so a captured graph with an odd
// number of exchanges still alternates across replays): a rank can only push exchange
// n+2 into the slot of n after passing the gather of n+1, which needs every rank's push of n+1, which
// each rank issues only after it has consumed n.
// The sum itself (rank order, one rounding) is fused into the kernel that consumes the partials.
//
// No multicast of any kind is used: plain stores to peer addresses only.

#include "common.cuh"

namespace tf {
namespace {

__device__ __forceinline__ uint4 ld_volatile16(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile16(uint4* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// n2 = rows * D / 2 packets per rank block
__global__ void __launch_bounds__(256) peer_exchange_kernel(const float2* local, int n2, uint8_t* const* bufs, size_t slot_bytes,
                                                            float2* gathered, int rank, int world, uint32_t* seq, int* tickets,
                                                            int* status, unsigned spin_limit) {
    __shared__ int is_last;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t want = *reinterpret_cast<volatile uint32_t*>(seq) + 1u;
    const size_t slot_off = (want & 1u) * slot_bytes;      // consecutive exchanges alternate, whatever the host captured
    const int stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;
    for (int i = first; i < n2; i += stride) {
        const float2 v = local[i];
        const uint4 pkt = make_uint4(__float_as_uint(v.x), want, __float_as_uint(v.y), want);
        for (int peer = 0; peer < world; ++peer)
            st_volatile16(reinterpret_cast<uint4*>(bufs[peer] + slot_off) + (size_t)rank * n2 + i, pkt);
    }
    const uint4* mine = reinterpret_cast<const uint4*>(bufs[rank] + slot_off);
    // once a wait has run out anywhere in this process the exchange is lost: do not wait again
    bool stalled = status != nullptr && *reinterpret_cast<volatile int*>(status) != 0;
    for (int r = 0; r < world; ++r) {
        for (int i = first; i < n2; i += stride) {
            uint4 pkt = ld_volatile16(mine + (size_t)r * n2 + i);
            unsigned spins = 0;
            while ((pkt.y != want || pkt.w != want) && !stalled) {
                if (++spins > spin_limit) { stalled = true; break; }
                pkt = ld_volatile16(mine + (size_t)r * n2 + i);
            }
            gathered[(size_t)r * n2 + i] = make_float2(__uint_as_float(pkt.x), __uint_as_float(pkt.z));
        }
    }
    if (stalled) report(status, TF_ESTALL);
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(tickets, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (is_last && threadIdx.x == 0) {
        *tickets = 0;
        *reinterpret_cast<volatile uint32_t*>(seq) = want;
    }
}

}  // namespace
}  // namespace tf

extern "C" {

void tf_set_poll_limit(unsigned polls) { tf::poll_limit_ref() = polls ? polls : (1u << 22); }

size_t tf_peer_slot_bytes(int rows, int D, int world) {
    if (rows < 1 || D < 2 || world < 1) return 0;
    return (size_t)world * ((rows + 1) / 2) * D * 16;   // a 16-byte packet per two fp32 values (rows in pairs, rounded up)
}

int tf_peer_exchange(const float* local, int rows, int D, void* const* peer_bufs, size_t slot_bytes, float* gathered, int rank,
                     int world, void* seq, void* tickets, int* status, void* stream) {
    if (rows < 1 || D < 4 || D % 4 || world < 2 || world > 64 || rank < 0 || rank >= world) return TF_EINVAL;
    if (!local || !peer_bufs || !gathered || !seq || !tickets) return TF_EINVAL;
    if (((uintptr_t)local | (uintptr_t)gathered | slot_bytes) & 15) return TF_EALIGN;
    if (slot_bytes < (size_t)world * rows * D * 8) return TF_EINVAL;
    const float2* src = reinterpret_cast<const float2*>(local);
    float2* dst = reinterpret_cast<float2*>(gathered);
    int n2 = rows * (D / 2);
    uint32_t* seq_p = static_cast<uint32_t*>(seq);
    int* tick_p = static_cast<int*>(tickets);
    uint8_t* const* bufs = reinterpret_cast<uint8_t* const*>(peer_bufs);
    int blocks = (n2 + 255) / 256;
    if (blocks > 64) blocks = 64;      // few enough to be resident together beside the neighbouring kernels
    unsigned limit = tf::poll_limit_ref();
    void* args[] = {&src, &n2, &bufs, &slot_bytes, &dst, &rank, &world, &seq_p, &tick_p, &status, &limit};
    return tf::launch_pdl((const void*)tf::peer_exchange_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                          args) == cudaSuccess ? TF_OK : (cudaGetLastError(), TF_ECUDA);
}

}  // extern "C"
