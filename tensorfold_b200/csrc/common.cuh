// Shared device helpers for the lane-verify kernels (sm_100a).
//
// Every kernel in this library obeys one rule: an output row is a function of that row's own
// inputs only, computed by a chain of operations that does not depend on how many other rows
// ride in the same launch. That is what makes a verify window's rows bit-identical to serial
// one-row steps.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <stdint.h>

#include "../../include/tensorfold_b200.h"

namespace tf {

// ---- status word -----------------------------------------------------------------------------
// A bounded device-side wait that runs out records a code here and carries on; the host reads it
// when it next synchronises. Nothing in this library traps or spins without a limit.
__device__ __forceinline__ void report(int* status, int code) {
    if (status != nullptr) atomicCAS(status, 0, code);
}

// ---- bf16 helpers ----------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const uint32_t a = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo));
    const uint32_t b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi));
    return a | (b << 16);
}

// ---- eight bf16 values in a 16-byte chunk ------------------------------------------------------------
__device__ __forceinline__ void unpack8(uint4 v, float (&f)[8]) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = bf16_lo(u[i]); f[2 * i + 1] = bf16_hi(u[i]); }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---- packed activations -------------------------------------------------------------------------
// The lane matmul reads its input rows "packed": per k tile (64 inputs), Mp = M rounded up to its row
// bucket (8, 16, 32, 64 or 128) rows of 128 bytes each (16-byte chunk c of row r stored at chunk
// c ^ 4*(r&1); rows past M are zero), followed by the tile's group sums as [groups in the tile][Mp] fp32. Every kernel that produces matmul input writes this
// form directly with the two helpers below, so the sums are formed the same way everywhere.
__host__ __device__ constexpr int tf_padded_rows(int m) { return m <= 8 ? 8 : m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }
__host__ __device__ constexpr size_t tf_packed_size(int mp, int k, int group) { return (size_t)(k / 64) * mp * (128 + 4 * (64 / group)); }

// fp32 sum of a G-input group: each lane adds its 8 contiguous bf16 values in order, then the G/8
// lanes holding the group combine in a pairwise tree. Call with whole warps; every lane of the
// group gets the sum.
template <int G>
__device__ __forceinline__ float group_sum8(uint4 v) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { s += bf16_lo(u[i]); s += bf16_hi(u[i]); }
#pragma unroll
    for (int o = 1; o < G / 8; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    return s;
}

// Store chunk c (inputs 8c..8c+7) of `row` and, from the group's first lane, the group's sum.
template <int G>
__device__ __forceinline__ void packed_store(uint8_t* xp, int Mp, int row, int c, uint4 v, float sum) {
    constexpr int GPT = 64 / G;
    uint8_t* tile = xp + (size_t)(c >> 3) * Mp * (128 + 4 * GPT);
    *reinterpret_cast<uint4*>(tile + row * 128 + (((c & 7) * 16) ^ ((row & 1) << 6))) = v;
    if ((c & (G / 8 - 1)) == 0) reinterpret_cast<float*>(tile + Mp * 128)[((c / (G / 8)) % GPT) * Mp + row] = sum;
}

// ---- shared memory / mbarrier / bulk copy (TMA, untiled) --------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a hardware-defined slice),
// records TF_ESTALL and returns false. The caller carries on so that the kernel always terminates.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int limit = 1 << 22) {
    for (int i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    report(status, TF_ESTALL);
    return false;
}
// The same for a role that waits long and must not take issue slots from the warps that work meanwhile: each
// poll lets the hardware suspend the thread for up to `ns` nanoseconds (or until the phase completes).
__device__ __forceinline__ bool mbar_wait_idle(uint32_t bar, uint32_t parity, int* status, uint32_t ns = 2000, int limit = 1 << 20) {
    for (int i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(ns)
            : "memory");
        if (ok) return true;
    }
    report(status, TF_ESTALL);
    return false;
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier. Both addresses
// 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- tensor-core step: D(16x8, fp32) = A(16x16, bf16) * B(16x8, bf16) + C ----------------------
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                               const float (&c)[4]) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// (a & m) | c as ONE logic instruction; written with separate & and |, two constants make two.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t m, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(m), "r"(c));
    return d;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Programmatic dependent launch: wait for the producer grid's memory before touching inputs, and
// let the next grid start its prologue once this one has passed its own wait.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- bounded polling of memory another rank writes -----------------------------------------------
// Polls of one location before a kernel gives up and reports TF_ESTALL (each poll is a memory round trip:
// the default is seconds). tf_set_poll_limit changes it for later launches of this process, so that the
// run-out path can be exercised in milliseconds.
inline unsigned& poll_limit_ref() { static unsigned limit = 1u << 22; return limit; }

// ---- launches ------------------------------------------------------------------------------------
// Kernels can be launched with programmatic stream serialisation: a kernel may then become resident
// while its predecessor still runs, do its input-independent work (barrier setup, weight prefetch)
// and block in pdl_wait() until the predecessor's memory is visible. TF_PDL in the environment
// selects who gets the attribute: bit 0 the small kernels, bit 1 the matmuls, bit 2 the norm kernel,
// bit 3 the light elementwise steps; the default is all of them (15), the fastest setting measured on the
// 27B forward. Without the attribute pdl_wait() and pdl_launch_dependents() do nothing.
inline int pdl_mode() {
    static const int mode = [] { const char* e = std::getenv("TF_PDL"); return e ? atoi(e) : 15; }();
    return mode;
}
// kind: 0 a small kernel with a grid of its own weight (recurrence, attention, top-k, commits), 1 a matmul,
// 2 the residual-add + norm that feeds a matmul, 3 a light elementwise step between two matmuls
inline bool pdl_enabled(int kind = 0) { return (pdl_mode() >> kind) & 1; }

inline cudaError_t launch_pdl(const void* fn, dim3 grid, dim3 block, size_t smem, cudaStream_t st, void** args, int kind = 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled(kind) ? 1 : 0;
    return cudaLaunchKernelExC(&cfg, fn, args);
}

}  // namespace tf
