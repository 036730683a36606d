// Device-side helpers shared by the kernels: bf16 unpacking, mbarriers, bulk async copies, programmatic
// dependent launch, and the bounded waits every spin in this library goes through.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/plora.h"
#include "plora_internal.h"

// Kernel parameter and launch argument that exist in the range-checked build only
#ifdef PLORA_BOUNDS
#define PLORA_BOUNDS_PARAM , PloraBounds bnd
#define PLORA_BOUNDS_ARG(b) , b
#else
#define PLORA_BOUNDS_PARAM
#define PLORA_BOUNDS_ARG(b)
#endif

namespace {

#ifdef PLORA_BOUNDS
// Everything a few-token kernel will index with comes from `rec` (and K, the layer's input width): true when all of
// it stays inside what the launch may touch.
__device__ __forceinline__ bool rec_in_bounds(const PloraRec& rec, const PloraBounds& b, int K) {
    if (rec.cnt < 0 || rec.cnt > PLORA_WORK_TOKENS) return false;
    if (rec.cnt == 0 || rec.rank == 0) return true;  // nothing will be touched
    if (rec.rank < 0 || rec.rank > b.rmax || (rec.rank & 15)) return false;
    for (int t = 0; t < rec.cnt; t++)
        if (rec.tok[t] < 0 || rec.tok[t] >= b.rows) return false;
    if (rec.a < b.pool_lo || rec.a + (unsigned long long)rec.rank * (unsigned long long)K * 2ull > b.pool_hi || (rec.a & 15)) return false;
    for (int p = 0; p < PLORA_MAX_PARTS; p++) {
        const int r = rec.r[p];
        if (r == 0) continue;
        if (r < 0 || r > b.max_rank || (r & 15) || rec.r_off[p] < 0 || rec.r_off[p] + r > rec.rank) return false;
        if (rec.rows[p] <= 0 || (rec.rows[p] & 1) || rec.off[p] < 0 || (rec.off[p] & 1)) return false;
        if (b.ldy > 0 && rec.off[p] + rec.rows[p] > b.ldy) return false;
        if (rec.b[p] < b.pool_lo || rec.b[p] + (unsigned long long)rec.rows[p] * (unsigned long long)r * 2ull > b.pool_hi || (rec.b[p] & 15)) return false;
    }
    return true;
}
#endif

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    // a bf16 is the upper half of an f32
    f[0] = __uint_as_float(v.x << 16);
    f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16);
    f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16);
    f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16);
    f[7] = __uint_as_float(v.w & 0xffff0000u);
}

// ---- bulk async copies into shared memory, mbarriers, programmatic dependent launch ----

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for a phase of the barrier with an iteration limit; on running out it records PLORA_ERR_TIMEOUT in
// the status word and returns false, so the kernel can leave instead of hanging.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
    for (int i = 0; i < (1 << 20); i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicMax(status, PLORA_ERR_TIMEOUT);
    return false;
}

// global -> shared bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned), completion
// counted on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// ---- barrier arrival, proxy fence and the bulk-group calls that tensor stores are tracked with ----

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// makes this thread's ordinary shared-memory writes visible to the bulk-copy engine (which reads shared memory
// through the async proxy); to be followed by a barrier before another thread issues the copy
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's groups have read their shared-memory source (it may be overwritten)
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... and have been written to global memory
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
    return v;
}

// Programmatic dependent launch. Every kernel of the path waits for the kernels before it and only then
// lets the next one start its prologue, so a prologue may read anything written two or more kernels back
// (slabs, descriptors, the step's grouping) but nothing the kernel right before it writes.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A block that has nothing to do leaves at once, except block 0, which first waits for the kernels before:
// a grid completes only when all its blocks have, so every grid of the path outlasts its predecessors and
// "the kernel before me is done" keeps meaning "everything before me is done".
__device__ __forceinline__ void pdl_exit_idle() {
    if ((blockIdx.x | blockIdx.y | blockIdx.z) == 0) pdl_wait();
}

__device__ __forceinline__ uint4 lds16(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// 16 values per lane -> their 16 warp-wide sums in 16 shuffles; returns the sum of value (lane >> 1) & 15.
__device__ __forceinline__ float reduce16(float (&v)[16], int lane) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float send = (lane & 16) ? v[i] : v[i + 8];
        const float keep = (lane & 16) ? v[i + 8] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float send = (lane & 8) ? v[i] : v[i + 4];
        const float keep = (lane & 8) ? v[i + 4] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const float send = (lane & 4) ? v[i] : v[i + 2];
        const float keep = (lane & 4) ? v[i + 2] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    {
        const float send = (lane & 2) ? v[0] : v[1];
        const float keep = (lane & 2) ? v[1] : v[0];
        v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    }
    return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
}

// Hints that the 128-byte line holding `p` will be read soon: the line is brought into L2, no value is bound,
// so it is safe on memory an earlier kernel may still be writing.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// The same for `bytes` (a multiple of 16) from a 16-byte aligned address, as one request.
__device__ __forceinline__ void bulk_prefetch_l2(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

}  // namespace
