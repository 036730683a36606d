// One kernel per layer for the gather path: a thread-block cluster of 8 blocks takes one work item (up to 16
// tokens of one slot). Block q of the cluster shrinks over the q-th eighth of the input features; the
// partial sums meet through distributed shared memory (no trip through global memory, no second launch);
// every block then expands its eighth of the output columns. All of the slot's A and B rows the cluster
// needs are requested by bulk async copies at kernel start, before the dependency wait, so that the slab
// traffic of this layer overlaps the tail of the kernel before. Replaces the lora_shrink + lora_expand pair
// of src/kernels/lora.cuh:23-126 when x and y are both ready at the call.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "plora_internal.h"
#include "plora_device.cuh"

typedef __nv_bfloat16 bf16;

PLORA_TRACE_SETTER(plora_trace_set_site)

#define SITE_CLUSTER 8
#define SITE_THREADS 256

namespace {

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// a float at the same shared-memory offset in block `rank` of the cluster
__device__ __forceinline__ float ld_peer_f32(const float* p, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}

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

struct SiteShape {
    int kchunk;   // input features per block of the cluster (a multiple of 8)
    int rmax;     // floats per S row in shared memory (parts * max_rank)
    int a_bytes;  // shared-memory bytes for the block's A rows
    int x_bytes;  // ... for the tokens' x chunks
    int b_bytes;  // ... for the block's share of B
};

__global__ void __cluster_dims__(SITE_CLUSTER, 1, 1) __launch_bounds__(SITE_THREADS)
    plora_site_gather_kernel(const bf16* __restrict__ X, int ldx, int K, const int* __restrict__ segs, SegLayout lay,
                             const plora_desc* __restrict__ table, void* Y, int ldy, int f32_out, SiteShape sh,
                             int* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ __align__(8) uint64_t bars[3];  // A rows, x chunks, B rows
    __shared__ int stok[PLORA_WORK_TOKENS];
    __shared__ int s_boff[PLORA_MAX_PARTS], s_lo[PLORA_MAX_PARTS], s_hi[PLORA_MAX_PARTS], s_cat[PLORA_MAX_PARTS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t crank = cluster_rank();
    unsigned char* As = dsm;
    unsigned char* Xs = As + sh.a_bytes;
    unsigned char* Bs = Xs + sh.x_bytes;
    float* Sp = reinterpret_cast<float*>(Bs + sh.b_bytes);  // this block's partial S [16][rmax]
    float* Ss = Sp + PLORA_WORK_TOKENS * sh.rmax;           // the summed S [16][rmax]
    const int n_work = segs[SEG_N_WORK];
    if (tid == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init(&bars[2], 1);
        mbar_fence_init();
    }
    bool waited = false;
    uint32_t ph_ax = 0, ph_b = 0;  // phases of the A/x barriers and of the B barrier (each flips only when used)
    bool alive = true;             // false once a bounded wait ran out: keep meeting the cluster, do no more work
    const int k0 = (int)crank * sh.kchunk;
    const int klen = max(0, min(sh.kchunk, K - k0));
    const uint32_t kbytes = (uint32_t)klen * 2u;
    for (int w = blockIdx.z; w < n_work; w += gridDim.z) {
        const int* work = segs + lay.work() + PLORA_WORK_WORDS * w;
        const int slot = work[0], cnt = work[2];
        const int mytok = work[4 + (lane & 15)];
        const plora_desc& d = table[slot];
        TRACE(0);
        const int R = d.rank;
        if (R == 0) continue;  // the same decision in every block of the cluster
        // this block's share of the slot's output columns, over the targeted parts laid end to end
        if (tid == 0) {
            int ntot = 0;
            for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                s_cat[p] = ntot;
                if (d.r[p] > 0) ntot += d.rows[p];
            }
            const int share = ((ntot + SITE_CLUSTER - 1) / SITE_CLUSTER + 1) & ~1;
            const int c_lo = min(ntot, (int)crank * share), c_hi = min(ntot, c_lo + share);
            int off = 0;
            for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                const int lo = max(c_lo, s_cat[p]) - s_cat[p];
                const int hi = d.r[p] > 0 ? min(c_hi, s_cat[p] + d.rows[p]) - s_cat[p] : 0;
                s_lo[p] = lo;
                s_hi[p] = hi > lo ? hi : lo;
                s_boff[p] = off;
                if (hi > lo) off += (hi - lo) * d.r[p] * 2;
            }
        }
        if (tid < PLORA_WORK_TOKENS) stok[tid] = mytok;
        __syncthreads();
        // ---- slab requests (before the dependency wait)
        if (warp == 0) {
            if (klen > 0) {
                const bf16* A = reinterpret_cast<const bf16*>(d.a) + k0;
                if (lane == 0) mbar_expect_tx(&bars[0], (uint32_t)R * kbytes);
                __syncwarp();
                for (int r = lane; r < R; r += 32) bulk_g2s(As + (size_t)r * kbytes, A + (size_t)r * K, kbytes, &bars[0]);
            }
            if (lane == 0) {
                uint32_t total = 0;
                for (int p = 0; p < PLORA_MAX_PARTS; p++) total += (uint32_t)(s_hi[p] - s_lo[p]) * (uint32_t)d.r[p] * 2u;
                if (total > 0) {
                    mbar_expect_tx(&bars[2], total);
                    for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                        const uint32_t bytes = (uint32_t)(s_hi[p] - s_lo[p]) * (uint32_t)d.r[p] * 2u;
                        if (bytes > 0)
                            bulk_g2s(Bs + s_boff[p], reinterpret_cast<const bf16*>(d.b[p]) + (size_t)s_lo[p] * d.r[p], bytes,
                                     &bars[2]);
                    }
                }
            }
        }
        if (!waited) {
            pdl_wait();
            pdl_trigger();
            waited = true;
        }
        TRACE(2);
        // ---- shrink over this block's eighth of the inputs
        if (klen > 0) {
            if (warp == 0) {
                if (lane == 0) mbar_expect_tx(&bars[1], (uint32_t)cnt * kbytes);
                __syncwarp();
                if (lane < cnt) bulk_g2s(Xs + (size_t)lane * kbytes, X + (size_t)mytok * ldx + k0, kbytes, &bars[1]);
            }
            if (alive) alive = mbar_wait(&bars[0], ph_ax, status) && mbar_wait(&bars[1], ph_ax, status);
            ph_ax ^= 1;
            TRACE(3);
            for (int tp = 0; alive && tp < cnt; tp += 4) {
                const int nt = min(4, cnt - tp);
                for (int n0 = warp * 4; n0 < R; n0 += 32) {
                    float acc[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) acc[i] = 0.f;
                    for (int k = lane * 8; k < klen; k += 256) {
                        float xf[4][8];
#pragma unroll
                        for (int t = 0; t < 4; t++)
                            unpack8(lds16(Xs + (size_t)(tp + min(t, nt - 1)) * kbytes + k * 2), xf[t]);
#pragma unroll
                        for (int r = 0; r < 4; r++) {
                            float af[8];
                            unpack8(lds16(As + (size_t)(n0 + r) * kbytes + k * 2), af);
#pragma unroll
                            for (int t = 0; t < 4; t++)
#pragma unroll
                                for (int e = 0; e < 8; e++) acc[r * 4 + t] = fmaf(xf[t][e], af[e], acc[r * 4 + t]);
                        }
                    }
                    const float v = reduce16(acc, lane);
                    if ((lane & 1) == 0) {
                        const int i = lane >> 1, r = i >> 2, t = i & 3;
                        if (t < nt) Sp[(tp + t) * sh.rmax + n0 + r] = v;
                    }
                }
            }
        } else {
            for (int i = tid; i < cnt * R; i += SITE_THREADS) Sp[(i / R) * sh.rmax + (i % R)] = 0.f;
        }
        // ---- the eight partials meet: block q's Sp is read by everyone, added in block order
        TRACE(4);
        cluster_arrive();
        cluster_wait();
        TRACE(5);
        for (int i = tid; i < cnt * R; i += SITE_THREADS) {
            const int t = i / R, j = i - t * R;
            const float* p = Sp + t * sh.rmax + j;
            float v[SITE_CLUSTER];
#pragma unroll
            for (int q = 0; q < SITE_CLUSTER; q++) v[q] = ld_peer_f32(p, q);
            float acc = v[0];
#pragma unroll
            for (int q = 1; q < SITE_CLUSTER; q++) acc += v[q];
            Ss[t * sh.rmax + j] = acc;
        }
        cluster_arrive();  // my reads of the others' partials are done
        __syncthreads();
        TRACE(6);
        // ---- expand over this block's share of the output columns
        bool okb = true;
        {
            int total = 0;
            for (int p = 0; p < PLORA_MAX_PARTS; p++) total += s_hi[p] - s_lo[p];
            if (total > 0) {
                if (alive) okb = mbar_wait(&bars[2], ph_b, status);
                ph_b ^= 1;
            }
        }
        if (!okb) alive = false;
        TRACE(7);
        if (alive) {
            for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                const int r = d.r[p];
                const int lo = s_lo[p], hi = s_hi[p];
                if (r == 0 || hi <= lo) continue;
                const int r_off = d.r_off[p];
                const unsigned char* bpart = Bs + s_boff[p];
                for (int c = lo + 2 * tid; c < hi; c += 2 * SITE_THREADS) {
                    const unsigned char* b0 = bpart + (size_t)(c - lo) * r * 2;
                    const unsigned char* b1 = b0 + (size_t)r * 2;
                    const size_t ycol = (size_t)d.off[p] + c;
                    for (int tg = 0; tg < cnt; tg += 4) {
                        float2 yv[4];
#pragma unroll
                        for (int t = 0; t < 4; t++) {
                            if (tg + t < cnt) {
                                const size_t at = (size_t)stok[tg + t] * ldy + ycol;
                                if (f32_out) yv[t] = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(Y) + at);
                                else
                                    yv[t] = __bfloat1622float2(
                                        *reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const bf16*>(Y) + at));
                            }
                        }
                        float acc[4][2];
#pragma unroll
                        for (int t = 0; t < 4; t++) acc[t][0] = acc[t][1] = 0.f;
                        for (int j = 0; j < r; j += 8) {
                            float f0[8], f1[8];
                            unpack8(lds16(b0 + j * 2), f0);
                            unpack8(lds16(b1 + j * 2), f1);
#pragma unroll
                            for (int t = 0; t < 4; t++) {
                                if (tg + t < cnt) {
                                    const float* sp = Ss + (tg + t) * sh.rmax + r_off + j;
                                    const float4 s0 = *reinterpret_cast<const float4*>(sp);
                                    const float4 s1 = *reinterpret_cast<const float4*>(sp + 4);
                                    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                                    for (int e = 0; e < 8; e++) {
                                        acc[t][0] = fmaf(sv[e], f0[e], acc[t][0]);
                                        acc[t][1] = fmaf(sv[e], f1[e], acc[t][1]);
                                    }
                                }
                            }
                        }
#pragma unroll
                        for (int t = 0; t < 4; t++) {
                            if (tg + t < cnt) {
                                const size_t at = (size_t)stok[tg + t] * ldy + ycol;
                                if (f32_out)
                                    *reinterpret_cast<float2*>(reinterpret_cast<float*>(Y) + at) =
                                        make_float2(yv[t].x + acc[t][0], yv[t].y + acc[t][1]);
                                else
                                    *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf16*>(Y) + at) =
                                        __floats2bfloat162_rn(yv[t].x + acc[t][0], yv[t].y + acc[t][1]);
                            }
                        }
                    }
                }
            }
        }
        cluster_wait();   // nobody reads my partials any more: they may be overwritten (or the block may leave)
        TRACE(8);
        __syncthreads();  // shared memory is reused by the next work item
    }
    if (!waited) pdl_exit_idle();
}

}  // namespace

// Shared-memory plan of the cluster kernel for one layer; returns 0 bytes when it does not fit.
size_t plora_site_plan(int K, int parts, int max_rank, int total_rows, int* kchunk, int* rmax, int* a_bytes,
                       int* x_bytes, int* b_bytes) {
    const int kc = (((K + SITE_CLUSTER - 1) / SITE_CLUSTER) + 7) & ~7;
    const int rm = parts * max_rank;
    const int share = ((total_rows + SITE_CLUSTER - 1) / SITE_CLUSTER + 1) & ~1;
    const size_t a = (size_t)rm * kc * 2, x = (size_t)PLORA_WORK_TOKENS * kc * 2;
    const size_t b = ((size_t)share * max_rank * 2 + 127) & ~(size_t)127;
    const size_t s = (size_t)2 * PLORA_WORK_TOKENS * rm * 4;
    const size_t total = a + x + b + s;
    if (total > 200 * 1024) return 0;
    *kchunk = kc;
    *rmax = rm;
    *a_bytes = (int)a;
    *x_bytes = (int)x;
    *b_bytes = (int)b;
    return total;
}

cudaError_t plora_site_init() {
    return cudaFuncSetAttribute(plora_site_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}

cudaError_t plora_launch_site(const void* x, int ldx, int K, const int32_t* segs, SegLayout lay, const plora_desc* table,
                              void* y, int ldy, int f32_out, int parts, int max_rank, int total_rows, int work_cap,
                              int* status, bool pdl, cudaStream_t st) {
    SiteShape sh;
    const size_t smem = plora_site_plan(K, parts, max_rank, total_rows, &sh.kchunk, &sh.rmax, &sh.a_bytes, &sh.x_bytes,
                                        &sh.b_bytes);
    if (smem == 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(SITE_CLUSTER, 1, (unsigned)(work_cap < 128 ? work_cap : 128));
    cfg.blockDim = dim3(SITE_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, plora_site_gather_kernel, reinterpret_cast<const bf16*>(x), ldx, K, segs, lay, table, y,
                              ldy, f32_out, sh, status);
}
