// Tensor-parallel exchange of the row-parallel shrink's partial sums, in one kernel per GPU (no counterpart
// in pocket-engine, which is single-GPU). Every rank holds the same step metadata and a partial S (its share
// of the K inputs). One launch per rank:
//
//   1. each block adds its rows' K-split planes (the local partial) and stores the result into slot `rank` of
//      the staging area of EVERY rank (plain stores through peer mappings over NVLink, its own included);
//   2. it then raises flag (rank, block) on every rank with a system-scope release store;
//   3. it waits, with a time limit, for the flags (p, block) of all ranks p in its own memory, and
//   4. adds the `world` partials of its rows in rank order (the same order everywhere: all ranks end with the
//      same bits) into plane 0 of S, which plora_expand_reduced reads.
//
// Data of a peer is read only after it has landed in local memory; there are no loads from peer memory and
// no bulk or tensor copies at all. Two staging buffers alternate by the parity of a device-side call counter
// (kept on the device so that a captured graph can be replayed): a rank can be at most one call ahead of
// another. A wait that runs out records PLORA_ERR_TIMEOUT and the block leaves.
//
// plora_xchg_all_ranks_kernel is the same body for every rank in ONE cooperative launch (grid y = rank), for
// machines with fewer GPUs than ranks: kernels that wait on one another must not be separate launches there.
#include <cuda_runtime.h>

#include "plora_internal.h"
#include "plora_device.cuh"

namespace {

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// this rank's partial of one group of four S values: gather rows add the site's K-split planes in order, tile
// rows add the tile path's planes as a balanced tree (the same sums plora_expand would form)
__device__ __forceinline__ float4 local_sum(const float* sp, size_t s_stride, int nplanes, bool tree) {
    if (!tree) {
        // all planes requested together (a layer has at most 16), then added in plane order
        float4 v[16];
#pragma unroll
        for (int s = 0; s < 16; s++)
            if (s < nplanes) v[s] = __ldcg(reinterpret_cast<const float4*>(sp + (size_t)s * s_stride));
        float4 acc = v[0];
#pragma unroll
        for (int s = 1; s < 16; s++)
            if (s < nplanes) acc = add4(acc, v[s]);
        for (int s = 16; s < nplanes; s++) acc = add4(acc, __ldcg(reinterpret_cast<const float4*>(sp + (size_t)s * s_stride)));
        return acc;
    }
    float4 v[PLORA_TILE_SPLIT_MAX];
#pragma unroll
    for (int a = 0; a < PLORA_TILE_SPLIT_MAX; a++)
        if (a < nplanes) v[a] = __ldcg(reinterpret_cast<const float4*>(sp + (size_t)a * s_stride));
#pragma unroll
    for (int stride = 1; stride < PLORA_TILE_SPLIT_MAX; stride <<= 1)
#pragma unroll
        for (int a = 0; a < PLORA_TILE_SPLIT_MAX; a += 2 * stride)
            if (a + stride < nplanes) v[a] = add4(v[a], v[a + stride]);
    return v[0];
}

__device__ void xchg_body(const PloraXchgCtx& c, int w, int nblocks) {
    __shared__ int s_fail;
    const int tid = threadIdx.x;
    const unsigned seq = *reinterpret_cast<volatile unsigned*>(&c.ctl[0]) + 1u;  // this call's number, the same on every rank
    const unsigned par = seq & 1u;
    // rows of this block: a gather work item, a tensor-core tile, or nothing
    int cnt = 0, rank_cols = 0, nplanes = 1, start = 0;
    const int* tok = nullptr;
    bool tree = false;
    if (w < c.work_cap) {
        if (w < c.segs[SEG_N_WORK]) {
            const int* work = c.segs + c.lay.work() + PLORA_WORK_WORDS * w;
            cnt = work[2];
            tok = work + 4;
            rank_cols = c.table[work[0]].rank;
            nplanes = c.nsplit;
        }
    } else if (w - c.work_cap < c.segs[SEG_N_MMA]) {
        const int* mt = c.segs + c.lay.mma() + 3 * (w - c.work_cap);
        start = mt[0];
        cnt = mt[1];
        rank_cols = c.table[mt[2]].rank;
        nplanes = rank_cols ? min(c.tile_split, plora_tile_chunks(c.K, rank_cols)) : 1;
        tree = true;
    }
    const bool live = cnt > 0 && rank_cols > 0;
    if (tid == 0) s_fail = 0;
    const int q4 = rank_cols >> 2;
    const size_t plane = (size_t)c.max_tokens * c.lds;                // one rank's slot of a staging buffer
    const size_t mine = ((size_t)par * c.world + c.rank) * plane;     // where this rank's partial goes, on every rank
    if (live) {
        for (int i = tid; i < cnt * q4; i += blockDim.x) {
            const int t = i / q4, j = i - t * q4;
            const size_t at = (size_t)(tok ? tok[t] : start + t) * c.lds + 4 * j;
            const float4 v = local_sum(c.S + at, c.s_stride, nplanes, tree);
            for (int p = 0; p < c.world; p++) *reinterpret_cast<float4*>(c.staging[p] + mine + at) = v;
        }
    }
    __syncthreads();
    if (live && tid < c.world) {
        __threadfence_system();
        st_release_sys(c.flags[tid] + ((size_t)par * c.world + c.rank) * c.max_blocks + w, seq);
        // and wait for rank `tid`'s flag for this block in local memory
        const unsigned* f = c.flags[c.rank] + ((size_t)par * c.world + tid) * c.max_blocks + w;
        const unsigned long long t0 = now_ns();
        bool ok = false;
        for (;;) {
            if (ld_acquire_sys(f) == seq) {
                ok = true;
                break;
            }
            if (now_ns() - t0 > c.timeout_ns) break;
            __nanosleep(40);
        }
        if (!ok) {
            atomicMax(c.status, PLORA_ERR_TIMEOUT);
            s_fail = 1;
        }
    }
    __syncthreads();
    if (live && !s_fail) {
        const float* local = c.staging[c.rank] + (size_t)par * c.world * plane;
        for (int i = tid; i < cnt * q4; i += blockDim.x) {
            const int t = i / q4, j = i - t * q4;
            const size_t at = (size_t)(tok ? tok[t] : start + t) * c.lds + 4 * j;
            float4 acc = __ldcg(reinterpret_cast<const float4*>(local + at));
            for (int p = 1; p < c.world; p++) acc = add4(acc, __ldcg(reinterpret_cast<const float4*>(local + p * plane + at)));
            *reinterpret_cast<float4*>(c.S + at) = acc;
        }
    }
    // the last block to finish closes the call: the counter moves on for the next launch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&c.ctl[1], 1u) == (unsigned)nblocks - 1u) {
            c.ctl[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(&c.ctl[0]) = seq;
        }
    }
}

__global__ void __launch_bounds__(128) plora_xchg_kernel(const __grid_constant__ PloraXchgCtx c) {
    pdl_wait();  // S comes from the shrink kernels before; the call counter from the exchange before
    pdl_trigger();
    xchg_body(c, blockIdx.x, gridDim.x);
}

__global__ void __launch_bounds__(128) plora_xchg_all_ranks_kernel(const PloraXchgCtx* __restrict__ ctxs) {
    xchg_body(ctxs[blockIdx.y], blockIdx.x, gridDim.x);
}

}  // namespace

cudaError_t plora_launch_xchg(const PloraXchgCtx& c, int nblocks, bool pdl, cudaStream_t st) {
    if (nblocks <= 0) return cudaSuccess;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)nblocks);
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, plora_xchg_kernel, c);
}

// All ranks of one process on one device in a single cooperative launch; `ctxs_dev` holds `world` contexts.
cudaError_t plora_launch_xchg_all_ranks(const PloraXchgCtx* ctxs_dev, int world, int nblocks, cudaStream_t st) {
    if (nblocks <= 0) return cudaSuccess;
    int per_sm = 0, dev = 0, sms = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, plora_xchg_all_ranks_kernel, 128, 0);
    if (e != cudaSuccess) return e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    if ((long long)nblocks * world > (long long)per_sm * sms) return cudaErrorCooperativeLaunchTooLarge;
    void* args[] = {(void*)&ctxs_dev};
    return cudaLaunchCooperativeKernel((const void*)plora_xchg_all_ranks_kernel, dim3((unsigned)nblocks, (unsigned)world),
                                       dim3(128), args, 0, st);
}
