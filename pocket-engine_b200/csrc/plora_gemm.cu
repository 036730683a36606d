// One layer for prefill-sized steps as a single tensor-core kernel: the base matrix multiply (FP8 with
// per-token and per-output-channel scales, or bf16) and the adapter term of every long run of tokens, both on
// tcgen05 with accumulators in tensor memory, y written once (no read-modify-write). No counterpart in
// pocket-engine, whose expand is always a separate kernel after the layer's own GEMM (src/linear.rs:889-921).
//
// Block = 128 tokens x 256 output columns, 192 threads:
//   warp 0      producer: per step of 128 bytes of K, the x tile (16 KB) and the W tile (32 KB) as tensor copies
//               into a ring of three stages (128-byte swizzle)
//   warp 1      issues the MMAs: the base product into tensor-memory columns 0..255; after the last step, the
//               adapter passes into columns 256..511
//   warps 2..5  stage the adapter passes while the main loop runs, then the epilogue. A pass = one tensor-core
//               tile of the step's grouping (a run of one slot's tokens) that meets the block's rows x 64 columns
//               of the slot's rank: S rows (plane 0, other rows zero) split into bf16 high and low parts, and the
//               block's 256 rows of B_p, in the unswizzled core-matrix layout. Epilogue: y = s_t s_n acc + adapter
//               (or acc + adapter), staged in the idle ring in 128-byte-swizzled slots and written by tensor stores.
//
// Tokens outside long runs (decode tokens, short prompts) get only the base product here; the gather expand
// kernel adds their adapter term afterwards. Needs y 16-byte aligned with a 16-byte multiple pitch, and part
// boundaries at multiples of 256 columns (a block lies in one part). Every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "plora_internal.h"
#include "plora_device.cuh"
#include "plora_tc.cuh"

typedef __nv_bfloat16 bf16;

namespace {

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

#define G_BM 128
#define G_BN 256
#define G_BKB 128  // bytes of K per stage row
#define G_STAGES 3
#define G_STAGE_BYTES (G_BM * G_BKB + G_BN * G_BKB)
#define G_RC 64  // rank columns per adapter pass
#define G_AOP (G_BM * G_RC * 2)
#define G_BOP (G_BN * G_RC * 2)
#define G_MAX_PASS 16
#define G_SLOT 4096  // 32 rows x 128 bytes of y

struct GemmParts {
    int n;
    int off[PLORA_MAX_PARTS];
    int rows[PLORA_MAX_PARTS];
};

template <int KIND, bool F32>
__global__ void __launch_bounds__(192) plora_gemm_fused_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                const __grid_constant__ CUtensorMap wmap,
                                                                const __grid_constant__ CUtensorMap ymap,
                                                                const float* __restrict__ st, const float* __restrict__ sn,
                                                                int T, int N, int K, const int* __restrict__ segs,
                                                                SegLayout lay, const plora_desc* __restrict__ table,
                                                                GemmParts parts, const float* __restrict__ S, int lds,
                                                                int* __restrict__ status) {
    extern __shared__ unsigned char dsm_raw[];
    __shared__ __align__(8) uint64_t full[G_STAGES], empty[G_STAGES], acc_bar, meta_bar, ad_full, ad_empty;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_npass, p_row0[G_MAX_PASS], p_row1[G_MAX_PASS], p_slot[G_MAX_PASS], p_rc0[G_MAX_PASS], p_rw[G_MAX_PASS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * G_BN, m0 = blockIdx.y * G_BM;
    unsigned char* ring = dsm_raw + ((1024u - (smem_u32(dsm_raw) & 1023u)) & 1023u);
    unsigned char* Ahi = ring + G_STAGES * G_STAGE_BYTES;
    unsigned char* Alo = Ahi + G_AOP;
    unsigned char* Bop = Alo + G_AOP;
    float* sn_s = reinterpret_cast<float*>(Bop + G_BOP);  // the block's 256 column scales
    if (tid == 0) {
        for (int i = 0; i < G_STAGES; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(&acc_bar, 1);
        mbar_init(&meta_bar, 1);
        mbar_init(&ad_full, 1);
        mbar_init(&ad_empty, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const int kbytes = KIND == 0 ? K : 2 * K;
    const int nk = (kbytes + G_BKB - 1) / G_BKB;
    constexpr int KEL = KIND == 0 ? G_BKB : G_BKB / 2;  // elements of K per step
    pdl_wait();  // S, x and the scales come from the kernels before
    pdl_trigger();
    // the part this block's columns lie in
    int part = 0;
#pragma unroll
    for (int q = 1; q < PLORA_MAX_PARTS; q++)
        if (q < parts.n && n0 >= parts.off[q]) part = q;
    const int n_local = n0 - parts.off[part];  // first row of B_p for this block

    if (warp == 0) {
        if (elect_one()) {
            for (int ks = 0; ks < nk; ks++) {
                const int stg = ks % G_STAGES;
                if (ks >= G_STAGES && !mbar_wait(&empty[stg], ((ks / G_STAGES) - 1) & 1, status)) break;
                unsigned char* xs = ring + (size_t)stg * G_STAGE_BYTES;
                mbar_expect_tx(&full[stg], G_STAGE_BYTES);
                tma_load_2d(xs, &xmap, ks * KEL, m0, &full[stg]);
                tma_load_2d(xs + G_BM * G_BKB, &wmap, ks * KEL, n0, &full[stg]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (elect_one()) {
            // M 128, N 256, f32 accumulator, K-major operands; kind::f16 carries the bf16 formats in bits 7 and 10
            const uint32_t idesc_ad = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(G_BN >> 3) << 17) | ((uint32_t)(G_BM >> 4) << 24);
            const uint32_t idesc = KIND == 0 ? (1u << 4) | ((uint32_t)(G_BN >> 3) << 17) | ((uint32_t)(G_BM >> 4) << 24) : idesc_ad;
            bool ok = true;
            for (int ks = 0; ok && ks < nk; ks++) {
                const int stg = ks % G_STAGES;
                ok = mbar_wait(&full[stg], (ks / G_STAGES) & 1, status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t xs = smem_u32(ring + (size_t)stg * G_STAGE_BYTES);
                const uint32_t ws = xs + G_BM * G_BKB;
#pragma unroll
                for (int kk = 0; kk < G_BKB / 32; kk++)
                    umma<KIND>(tmem, umma_desc(xs + kk * 32, 16, 1024, 2), umma_desc(ws + kk * 32, 16, 1024, 2), idesc,
                               (ks | kk) != 0);
                umma_commit(&empty[stg]);
            }
            // the adapter passes, staged by warps 2..5 while the loop above ran
            if (ok) ok = mbar_wait_long(&meta_bar, 0, status);
            const int npass = ok ? s_npass : 0;
            for (int ps = 0; ok && ps < npass; ps++) {
                ok = mbar_wait_long(&ad_full, ps & 1, status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sbo = (uint32_t)p_rw[ps] * 16u;
                const uint32_t a_hi = smem_u32(Ahi), a_lo = smem_u32(Alo), b = smem_u32(Bop);
                for (int kk = 0; kk < p_rw[ps] / 16; kk++)
                    umma<1>(tmem + 256, umma_desc(a_hi + kk * 256, 128, sbo, 0), umma_desc(b + kk * 256, 128, sbo, 0), idesc_ad,
                            (ps | kk) != 0);
                for (int kk = 0; kk < p_rw[ps] / 16; kk++)
                    umma<1>(tmem + 256, umma_desc(a_lo + kk * 256, 128, sbo, 0), umma_desc(b + kk * 256, 128, sbo, 0), idesc_ad, 1);
                umma_commit(&ad_empty);
            }
            umma_commit(&acc_bar);
        }
        __syncwarp();
    } else {
        const int e = tid - 64;  // 0..127: token row of the block, and (twice) a row of B
        // ---- the block's adapter passes: tensor-core tiles of the grouping that meet its rows
        if (e == 0) {
            int np = 0;
            const int n_mma = segs[SEG_N_MMA];
            const int* mt = segs + lay.mma();
            int lo = 0, hi = n_mma;  // first tile that ends after the block's first row
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (mt[3 * mid] + mt[3 * mid + 1] > m0) hi = mid;
                else lo = mid + 1;
            }
            for (int t = lo; t < n_mma && mt[3 * t] < m0 + G_BM; t++) {
                const int start = mt[3 * t], len = mt[3 * t + 1], slot = mt[3 * t + 2];
                const int r = table[slot].r[part];
                for (int rc0 = 0; rc0 < r; rc0 += G_RC) {
                    if (np == G_MAX_PASS) {
                        atomicMax(status, PLORA_ERR_CAPACITY);
                        break;
                    }
                    p_row0[np] = max(start, m0) - m0;
                    p_row1[np] = min(start + len, m0 + G_BM) - m0;
                    p_slot[np] = slot;
                    p_rc0[np] = rc0;
                    p_rw[np] = min(G_RC, r - rc0);
                    np++;
                }
            }
            s_npass = np;
        }
        if (KIND == 0)
            for (int i = e; i < G_BN; i += 128) sn_s[i] = n0 + i < N ? sn[n0 + i] : 0.f;
        epi_sync();
        const int npass = s_npass;
        if (e == 0) mbar_arrive(&meta_bar);
        bool ok = true;
        for (int ps = 0; ok && ps < npass; ps++) {
            if (ps > 0) {  // the operands of the pass before are still being read until its MMAs complete
                ok = mbar_wait_long(&ad_empty, (ps - 1) & 1, status);
                if (!ok) break;
            }
            const plora_desc& d = table[p_slot[ps]];
            const int rw = p_rw[ps], rc0 = p_rc0[ps], r = d.r[part], P = rw >> 3;
            const uint32_t sbo = (uint32_t)rw * 16u;
            // rows of B_p for the block's columns: thread e copies rows e and e + 128
            const bf16* B = reinterpret_cast<const bf16*>(d.b[part]);
            for (int h = 0; h < 2; h++) {
                const int n = e + 128 * h;
                const bool valid = n_local + n < d.rows[part];
                const bf16* src = B + (size_t)(valid ? n_local + n : 0) * r + rc0;
                unsigned char* drow = Bop + (size_t)(n >> 3) * sbo + (n & 7) * 16;
                for (int j = 0; j < P; j++) cp_async16(drow + j * 128, src + j * 8, valid);
            }
            // this thread's token row of S (zero outside the pass's rows), as bf16 high and low parts
            {
                const bool valid = e >= p_row0[ps] && e < p_row1[ps];
                const float* sp = S + (size_t)(m0 + (valid ? e : 0)) * lds + d.r_off[part] + rc0;
                unsigned char* ahi = Ahi + (size_t)(e >> 3) * sbo + (e & 7) * 16;
                unsigned char* alo = Alo + (size_t)(e >> 3) * sbo + (e & 7) * 16;
                for (int j = 0; j < P; j++) {
                    float f[8];
                    if (valid) {
                        const float4 a = __ldcg(reinterpret_cast<const float4*>(sp + j * 8));
                        const float4 b = __ldcg(reinterpret_cast<const float4*>(sp + j * 8 + 4));
                        f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; q++) f[q] = 0.f;
                    }
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const __nv_bfloat162 h2 = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
                        const float2 hf = __bfloat1622float2(h2);
                        const __nv_bfloat162 l2 = __floats2bfloat162_rn(f[2 * q] - hf.x, f[2 * q + 1] - hf.y);
                        hi[q] = *reinterpret_cast<const uint32_t*>(&h2);
                        lo[q] = *reinterpret_cast<const uint32_t*>(&l2);
                    }
                    *reinterpret_cast<uint4*>(ahi + j * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(alo + j * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
            cp_async_wait_all();
            fence_async_smem();
            epi_sync();
            if (e == 0) mbar_arrive(&ad_full);
        }
        // ---- epilogue: the warp's 32 rows of both accumulators, scaled and added, into swizzled slots of the
        // idle ring, then tensor stores (clipped at the edges of y by the tensor map)
        if (ok) ok = mbar_wait_long(&acc_bar, 0, status);
        if (ok) {
            tc_fence_after();
            const int wq = warp & 3;  // tensor-memory lanes 32 wq .. 32 wq + 31
            const int row = m0 + wq * 32 + lane;
            constexpr int CW = F32 ? 32 : 64;     // y columns per slot
            constexpr int NSL = G_BN / CW;        // slots per warp
            unsigned char* slots = ring + (size_t)wq * NSL * G_SLOT;
            const float srow = KIND == 0 ? (row < T ? st[row] : 0.f) : 1.f;
            const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);
#pragma unroll 1
            for (int g = 0; g < G_BN / 32; g++) {  // 32 accumulator columns at a time
                uint32_t vb[32], va[32];
                tmem_ld32_nowait(lane_base + g * 32, vb);
                if (npass > 0) tmem_ld32_nowait(lane_base + 256 + g * 32, va);
                tmem_ld_wait();
                float o[32];
#pragma unroll
                for (int q = 0; q < 32; q++) {
                    const float base = KIND == 0 ? __uint_as_float(vb[q]) * (srow * sn_s[g * 32 + q]) : __uint_as_float(vb[q]);
                    o[q] = npass > 0 ? base + __uint_as_float(va[q]) : base;
                }
                if (F32) {
                    unsigned char* myrow = slots + (size_t)g * G_SLOT + lane * 128;
#pragma unroll
                    for (int c = 0; c < 8; c++)
                        *reinterpret_cast<float4*>(myrow + ((c ^ (lane & 7)) << 4)) =
                            make_float4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
                } else {
                    unsigned char* myrow = slots + (size_t)(g >> 1) * G_SLOT + lane * 128;
#pragma unroll
                    for (int c4 = 0; c4 < 4; c4++) {
                        uint32_t w[4];
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const __nv_bfloat162 b2 = __floats2bfloat162_rn(o[8 * c4 + 2 * q], o[8 * c4 + 2 * q + 1]);
                            w[q] = *reinterpret_cast<const uint32_t*>(&b2);
                        }
                        const int c = (g & 1) * 4 + c4;
                        *reinterpret_cast<uint4*>(myrow + ((c ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                for (int s = 0; s < NSL; s++)
                    if (n0 + s * CW < N) tma_store_2d(&ymap, n0 + s * CW, m0 + wq * 32, slots + (size_t)s * G_SLOT);
                bulk_commit();
                bulk_wait_all();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn g_encode = nullptr;

size_t gemm_smem() { return 1024 + (size_t)G_STAGES * G_STAGE_BYTES + 2 * G_AOP + G_BOP + G_BN * sizeof(float); }

template <typename... Params, typename... Args>
cudaError_t launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                       Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}

bool encode2d(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
              uint32_t box_inner, uint32_t box_outer) {
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t es[2] = {1, 1};
    return g_encode(m, dt, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t plora_gemm_init() {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (!fn || q != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        g_encode = reinterpret_cast<encode_tiled_fn>(fn);
    }
    cudaError_t e;
    const int smem = (int)gemm_smem();
    if ((e = plora_kernel_shared(reinterpret_cast<const void*>(plora_gemm_fused_kernel<0, false>), smem))) return e;
    if ((e = plora_kernel_shared(reinterpret_cast<const void*>(plora_gemm_fused_kernel<0, true>), smem))) return e;
    if ((e = plora_kernel_shared(reinterpret_cast<const void*>(plora_gemm_fused_kernel<1, false>), smem))) return e;
    return plora_kernel_shared(reinterpret_cast<const void*>(plora_gemm_fused_kernel<1, true>), smem);
}

// Whether a layer's shapes fit the kernel: parts starting at multiples of 256 columns (so does every block),
// and x, W, y meeting the alignment of tensor copies. kind 0 = e4m3 x and W with scales, 1 = bf16.
bool plora_gemm_fits(int kind, const void* x, const void* w, const void* y, int ldy, int f32_out, int K, int n_parts,
                     const int* part_off) {
    if (!g_encode) return false;
    const int el = kind == 0 ? 1 : 2, yel = f32_out ? 4 : 2;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)y & 15)) return false;
    if (((size_t)K * el) % 16 || ((size_t)ldy * yel) % 16) return false;
    for (int p = 0; p < n_parts; p++)
        if (part_off[p] % G_BN) return false;
    return true;
}

cudaError_t plora_launch_gemm_fused(int kind, const void* x, const float* st_, const void* w, const float* sn, int T, int N,
                                    int K, const int32_t* segs, SegLayout lay, const plora_desc* table, int n_parts,
                                    const int* part_off, const int* part_rows, const float* S, int lds, void* y, int ldy,
                                    int f32_out, int* status, bool pdl, cudaStream_t stream) {
    if (!g_encode) return cudaErrorNotSupported;
    CUtensorMap xmap, wmap, ymap;
    const CUtensorMapDataType dt = kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int el = kind == 0 ? 1 : 2;
    if (!encode2d(&xmap, dt, x, (uint64_t)K, (uint64_t)T, (uint64_t)K * el, G_BKB / el, G_BM)) return cudaErrorInvalidValue;
    if (!encode2d(&wmap, dt, w, (uint64_t)K, (uint64_t)N, (uint64_t)K * el, G_BKB / el, G_BN)) return cudaErrorInvalidValue;
    if (!encode2d(&ymap, f32_out ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, y, (uint64_t)N,
                  (uint64_t)T, (uint64_t)ldy * (f32_out ? 4 : 2), f32_out ? 32 : 64, 32))
        return cudaErrorInvalidValue;
    GemmParts parts;
    parts.n = n_parts;
    for (int p = 0; p < PLORA_MAX_PARTS; p++) {
        parts.off[p] = p < n_parts ? part_off[p] : 0;
        parts.rows[p] = p < n_parts ? part_rows[p] : 0;
    }
    dim3 grid((unsigned)((N + G_BN - 1) / G_BN), (unsigned)((T + G_BM - 1) / G_BM));
    const size_t smem = gemm_smem();
#define PLORA_GEMM_LAUNCH(KIND, F32)                                                                                        \
    return launch_pdl(plora_gemm_fused_kernel<KIND, F32>, grid, dim3(192), smem, stream, pdl, xmap, wmap, ymap, st_, sn, T, \
                      N, K, segs, lay, table, parts, S, lds, status)
    if (kind == 0) {
        if (f32_out) PLORA_GEMM_LAUNCH(0, true);
        PLORA_GEMM_LAUNCH(0, false);
    }
    if (f32_out) PLORA_GEMM_LAUNCH(1, true);
    PLORA_GEMM_LAUNCH(1, false);
#undef PLORA_GEMM_LAUNCH
}
