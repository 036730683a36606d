// Tensor-core tile path for long runs of contiguous tokens of one slot (prefill segments): tcgen05.mma with
// the accumulator in tensor memory, 128 tokens per tile.
//
//   plora_shrink_mma_kernel  S[128, R] = X[128, K] . A_slot[R, K]^T   x tiles and slab tiles by TMA (128-byte
//                            swizzle) from a producer thread, MMAs from another, a ring of stages, f32 in TMEM
//   plora_expand_mma_kernel  y[128, 128-column block] += S[128, r] . B_p[block, r]^T   S split into a bf16 high
//                            and low part (two accumulating MMAs, so S keeps ~16 bits of mantissa), operands in
//                            the unswizzled core-matrix layout, y read-modify-written from registers
//
// Every wait is bounded (mbar_wait); on a timeout the block records PLORA_ERR_TIMEOUT, frees its tensor
// memory and leaves. Replaces the reference's mma.sync tiles of 16 tokens (src/kernels/lora.cuh:23-126).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "plora_internal.h"
#include "plora_device.cuh"
#include "plora_tc.cuh"

typedef __nv_bfloat16 bf16;

namespace {

// ---- tcgen05 ----

// 8 consecutive columns, without the wait (several loads, then one tmem_ld_wait)
__device__ __forceinline__ void tmem_ld8_nowait(uint32_t taddr, float* v) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}

// v[0] = balanced binary tree sum of v[0..n), n a power of two <= 8 (W values per item)
template <int W>
__device__ __forceinline__ void tree_sum(float (&v)[PLORA_TILE_SPLIT_MAX][W], int n) {
#pragma unroll
    for (int stride = 1; stride < PLORA_TILE_SPLIT_MAX; stride <<= 1)
#pragma unroll
        for (int a = 0; a < PLORA_TILE_SPLIT_MAX; a += 2 * stride)
            if (a + stride < n)
#pragma unroll
                for (int q = 0; q < W; q++) v[a][q] += v[a + stride][q];
}

// Instruction descriptor, kind::f16: f32 accumulator, bf16 A and B, both K-major, M rows by N columns.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;  // a zero source size fills the 16 bytes with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Makes a tensor map that sits in global memory (written by a copy earlier in the stream) visible to this
// thread's tensor copies.
__device__ __forceinline__ void tmap_acquire(const CUtensorMap* map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(map) : "memory");
}

#define MMA_M 128
#define EXP_TPAD 66  // floats per row of the epilogue's transpose tile (64 columns + 2 of padding)

// ------------------------------------------------------------------------------------------------------
// Shrink of one 128-token tile. Grid (split, 1, tiles); 128 threads. The slot's K chunks (plora_tile_chunks) are
// shared evenly by min(split, chunks) blocks; each block accumulates its chunks in separate accumulators, adds
// them as a tree and writes plane blockIdx.x of S. K is walked in steps of 64 inputs through a ring of stages
// with two roles and no block-wide synchronisation in the loop: one thread of warp 0 issues, per step, the x
// tile and the slab's rows for the same 64 inputs as tensor copies (both in the 128-byte swizzle; the slab
// through the tensor map plora_upload encoded for the slot), waiting for a stage's MMAs before it refills it;
// one thread of warp 1 waits for a stage to land, issues its MMAs and commits them to the stage's "empty"
// barrier. Once the last MMAs are complete the f32 result leaves tensor memory one token row per thread.
#define SHR_KSTEP 64
#define SHR_X_BYTES (MMA_M * SHR_KSTEP * 2)
#define SHR_MAX_STAGES 8

__global__ void __launch_bounds__(128) plora_shrink_mma_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                const CUtensorMap* __restrict__ amaps, int K,
                                                                const int* __restrict__ segs, SegLayout lay,
                                                                const plora_desc* __restrict__ table,
                                                                float* __restrict__ S, size_t s_stride, int lds,
                                                                int ksplit, int nstage, int stage_bytes, int sub,
                                                                int late, int* __restrict__ status) {
    // late != 0: the kernel launched right before this one is the same layer's gather shrink, whose blocks let
    // this grid start only after they have themselves waited for the kernels before (or whose caller vouches
    // that x is older than those). x is then complete when this grid starts, the gather shrink writes other
    // rows of S, and only this grid's stores have to come after the dependency wait: the whole main loop runs
    // beside the gather shrink instead of behind it.
    // `sub` steps of 64 inputs share a stage (1 or 2): with two, a token row's two adjacent 128-byte pieces are
    // requested together. A stage is then [x box][x box][slab box][slab box] and stage_bytes covers all of it.
    extern __shared__ unsigned char dsm_raw[];
    __shared__ __align__(8) uint64_t full[SHR_MAX_STAGES], empty[SHR_MAX_STAGES], acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_fail;
    const int tile = blockIdx.z;
    const int n_mma = segs[SEG_N_MMA];
    const int* mt = segs + lay.mma() + 3 * tile;
    const int start = mt[0], len = mt[1], slot = mt[2];
    if (tile >= n_mma) return pdl_exit_idle();
    const plora_desc& d = table[slot];
    const int R = d.rank;
    if (R == 0) return pdl_exit_idle();
    const int n_chunks = plora_tile_chunks(K, R);
    const int s_eff = min(ksplit, n_chunks);
    if ((int)blockIdx.x >= s_eff) return pdl_exit_idle();
    const int n_acc = n_chunks / s_eff;  // accumulators (chunks) of this block
    const CUtensorMap* amap = amaps + slot;
    const int tid = threadIdx.x, warp = tid >> 5;
    // 1024-byte aligned stage ring: [x tile 16 KB][slab rows R x 128 B]
    unsigned char* ring = dsm_raw + ((1024u - (smem_u32(dsm_raw) & 1023u)) & 1023u);
    const uint32_t acc_cols = (uint32_t)plora_tile_cols(R);
    const uint32_t ncols = acc_cols * (uint32_t)n_acc;
    if (tid == 0) {
        for (int i = 0; i < nstage; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(&acc_bar, 1);
        mbar_fence_init();
        s_fail = 0;
    }
    if (warp == 0) tmem_alloc(&tmem_slot, ncols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const int nk_all = (K + SHR_KSTEP - 1) / SHR_KSTEP;
    const int spc = (nk_all + n_chunks - 1) / n_chunks;  // steps per chunk
    const int k_first = (int)blockIdx.x * n_acc * spc;
    const int nk1 = min(nk_all, k_first + n_acc * spc) - k_first;  // this block's steps of 64 inputs
    const int nk = (nk1 + sub - 1) / sub;                          // and its stages
    const uint32_t a_box_bytes = (uint32_t)R * 128u;
    // the slab's rows arrive as one box of R rows, or two of R / 2 when R is over the 256-row limit of a box
    const int nbox = R > 256 ? 2 : 1, box_rows = R / nbox;
    if (!late) pdl_wait();  // x comes from the kernels before
    pdl_trigger();

    if (warp == 0) {
        // producer: one thread feeds the ring, waiting for a stage's MMAs before refilling it
        if (elect_one()) {
            tmap_acquire(amap);
            // (both role threads are single threads whose instruction latencies are on the critical path: stage
            // index, barrier parity and chunk position are carried along instead of divided out every step)
            int st = 0;
            uint32_t par = 0;  // parity of the "empty" phase to wait for, from the ring's second round on
            bool round2 = false;
            int k0 = k_first * SHR_KSTEP;
            const uint32_t tx = (uint32_t)sub * (SHR_X_BYTES + a_box_bytes);
            for (int ks = 0; ks < nk; ks++) {
                if (ks >= nstage && !mbar_wait(&empty[st], par, status)) {
                    s_fail = 1;
                    break;
                }
                unsigned char* xs = ring + (size_t)st * stage_bytes;
                unsigned char* as = xs + (size_t)sub * SHR_X_BYTES;
                mbar_expect_tx(&full[st], tx);
                for (int u = 0; u < sub; u++)  // a step past the block's range reads zeros or unused columns
                    tma_load_2d(xs + (size_t)u * SHR_X_BYTES, &xmap, k0 + u * SHR_KSTEP, start, &full[st]);
                for (int u = 0; u < sub; u++)
                    for (int b = 0; b < nbox; b++)
                        tma_load_2d(as + (size_t)u * a_box_bytes + (size_t)b * box_rows * 128, amap, k0 + u * SHR_KSTEP,
                                    b * box_rows, &full[st]);
                k0 += sub * SHR_KSTEP;
                if (++st == nstage) {
                    st = 0;
                    if (round2) par ^= 1;
                    round2 = true;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // MMA issuer: a chunk of K starts a fresh accumulator
        if (elect_one()) {
            const uint32_t idesc_lo = umma_idesc_bf16(MMA_M, R > 256 ? 256 : R);
            const uint32_t idesc_hi = umma_idesc_bf16(MMA_M, R > 256 ? R - 256 : 16);
            // descriptors of stage 0's first x and slab boxes; every other operand is a constant number of 16-byte
            // units further on (the address field is the low 14 bits: shared memory is under 256 KB)
            const uint64_t dx0 = umma_desc(smem_u32(ring), 16, 1024, 2);
            const uint64_t da0 = umma_desc(smem_u32(ring) + (uint32_t)sub * SHR_X_BYTES, 16, 1024, 2);
            const uint32_t stage16 = (uint32_t)stage_bytes >> 4, abox16 = a_box_bytes >> 4;
            int st = 0, step = 0, first = 0;  // stage, 64-input step of this block, position inside the K chunk
            uint32_t par = 0, st16 = 0;
            uint32_t dacc = tmem;
            for (int it = 0; it < nk; it++) {
                if (!mbar_wait(&full[st], par, status)) {
                    s_fail = 1;
                    break;
                }
                tc_fence_after();
                for (int u = 0; u < sub && step < nk1; u++, step++) {
                    const uint64_t dx = dx0 + st16 + (uint32_t)u * (SHR_X_BYTES >> 4);
                    const uint64_t da = da0 + st16 + (uint32_t)u * abox16;
#pragma unroll
                    for (int kk = 0; kk < SHR_KSTEP / 16; kk++) {
                        umma<1>(dacc, dx + 2 * kk, da + 2 * kk, idesc_lo, (first | kk) != 0);
                        if (R > 256) umma<1>(dacc + 256, dx + 2 * kk, da + (256 * 128 >> 4) + 2 * kk, idesc_hi, (first | kk) != 0);
                    }
                    if (++first == spc) {  // the next step starts the next chunk's accumulator
                        first = 0;
                        dacc += acc_cols;
                    }
                }
                umma_commit(&empty[st]);
                if (it == nk - 1) umma_commit(&acc_bar);
                st16 += stage16;
                if (++st == nstage) {
                    st = 0;
                    st16 = 0;
                    par ^= 1;
                }
            }
        }
        __syncwarp();
    }
    // everyone: the accumulators are complete once the last commit has arrived
    bool ok = mbar_wait_long(&acc_bar, 0, status);
    __syncthreads();
    if (late) pdl_wait();  // before any store, and on every path: this grid must outlast the ones before it
    if (ok && !s_fail) {
        tc_fence_after();
        const int row = tid;
        float* out = S + (size_t)blockIdx.x * s_stride + (size_t)(start + row) * lds;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        for (int c = 0; n_acc > 1 && c < R; c += 8) {
            float v[PLORA_TILE_SPLIT_MAX][8];
#pragma unroll
            for (int a = 0; a < PLORA_TILE_SPLIT_MAX; a++)
                if (a < n_acc) tmem_ld8_nowait(lane_base + (uint32_t)a * acc_cols + c, v[a]);
            tmem_ld_wait();
            tree_sum<8>(v, n_acc);
            if (row < len) {
                *reinterpret_cast<float4*>(out + c) = make_float4(v[0][0], v[0][1], v[0][2], v[0][3]);
                *reinterpret_cast<float4*>(out + c + 4) = make_float4(v[0][4], v[0][5], v[0][6], v[0][7]);
            }
        }
        for (int c = 0; n_acc == 1 && c < R; c += 32) {
            uint32_t v[32];
            tmem_ld32(lane_base + c, v);
            if (row < len) {
#pragma unroll
                for (int q = 0; q < 32; q += 4)
                    if (c + q < R)
                        *reinterpret_cast<float4*>(out + c + q) =
                            make_float4(__uint_as_float(v[q]), __uint_as_float(v[q + 1]), __uint_as_float(v[q + 2]),
                                        __uint_as_float(v[q + 3]));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, ncols);
}

// ------------------------------------------------------------------------------------------------------
// Expand of one 128-token tile over `nb_per_cta` blocks of 128 output columns of one part. Grid (column
// groups, parts, tiles); 128 threads, thread t owns token row t. Operand layout: 8 x 16-byte core matrices,
// K direction 128 bytes apart, 8-row groups r * 16 bytes apart.
// 32 row segments of this lane's two columns, all requested before any is used
__device__ __forceinline__ void load_rows_bf16(uint32_t (&raw)[32], const bf16* y, int ldy, int nrows, bool colok) {
#pragma unroll
    for (int rr = 0; rr < 32; rr++)
        if (colok && rr < nrows) raw[rr] = *reinterpret_cast<const uint32_t*>(y + (size_t)rr * ldy);
}
__device__ __forceinline__ void load_rows_f32(float2 (&raw)[32], const float* y, int ldy, int nrows, bool colok) {
#pragma unroll
    for (int rr = 0; rr < 32; rr++)
        if (colok && rr < nrows) raw[rr] = *reinterpret_cast<const float2*>(y + (size_t)rr * ldy);
}

template <bool F32>
__global__ void __launch_bounds__(128) plora_expand_mma_kernel(const float* __restrict__ S, size_t s_stride, int lds,
                                                                int K, int ksplit,
                                                                const int* __restrict__ segs, SegLayout lay,
                                                                const plora_desc* __restrict__ table, void* Y,
                                                                int ldy, int nb_per_cta, int op_bytes,
                                                                int* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ __align__(8) uint64_t done;
    __shared__ uint32_t tmem_slot;
    const int tile = blockIdx.z;
    const int n_mma = segs[SEG_N_MMA];
    const int* mt = segs + lay.mma() + 3 * tile;
    const int start = mt[0], len = mt[1], slot = mt[2];
    if (tile >= n_mma) return pdl_exit_idle();
    const plora_desc& d = table[slot];
    const int p = blockIdx.y, r = d.r[p];
    if (r == 0) return pdl_exit_idle();
    const int rows = d.rows[p];
    const int cb0 = blockIdx.x * nb_per_cta;
    if (cb0 * 128 >= rows) return pdl_exit_idle();
    const int nblk = min(nb_per_cta, (rows - cb0 * 128 + 127) / 128);
    const int tid = threadIdx.x, warp = tid >> 5;
    unsigned char* Ahi = dsm;
    unsigned char* Alo = dsm + op_bytes;
    unsigned char* Bs[2] = {dsm + 2 * (size_t)op_bytes, dsm + 3 * (size_t)op_bytes};
    const bf16* B = reinterpret_cast<const bf16*>(d.b[p]);
    const uint32_t sbo = (uint32_t)r * 16u;  // 8-row group stride
    const int P = r >> 3;

    auto load_b = [&](int cb, unsigned char* dst) {
        const int n = tid;  // row of B = output column of the block
        const bool valid = cb * 128 + n < rows;
        const bf16* src = B + (size_t)(valid ? cb * 128 + n : 0) * r;
        unsigned char* drow = dst + (size_t)(n >> 3) * sbo + (n & 7) * 16;
        for (int j = 0; j < P; j++) cp_async16(drow + j * 128, src + j * 8, valid);
    };

    if (tid == 0) {
        mbar_init(&done, 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 128);
    load_b(cb0, Bs[0]);  // B is a slab: it may be fetched before the kernels ahead have finished
    cp_async_commit();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    pdl_wait();
    pdl_trigger();

    // this thread's token row of S, split into a bf16 high part and the bf16 of what is left
    {
        const int row = tid;
        const bool valid = row < len;
        const float* sp = S + (size_t)(start + (valid ? row : 0)) * lds + d.r_off[p];
        const int s_eff = min(ksplit, plora_tile_chunks(K, d.rank));  // planes the shrink wrote for this slot
        unsigned char* ahi = Ahi + (size_t)(row >> 3) * sbo + (row & 7) * 16;
        unsigned char* alo = Alo + (size_t)(row >> 3) * sbo + (row & 7) * 16;
        for (int j = 0; j < P; j++) {
            float f[8];
            if (valid && s_eff > 1) {
                float v[PLORA_TILE_SPLIT_MAX][8];
#pragma unroll
                for (int s = 0; s < PLORA_TILE_SPLIT_MAX; s++)
                    if (s < s_eff) {
                        const float* q = sp + (size_t)s * s_stride + j * 8;
                        const float4 a = __ldcg(reinterpret_cast<const float4*>(q));
                        const float4 b = __ldcg(reinterpret_cast<const float4*>(q + 4));
                        v[s][0] = a.x, v[s][1] = a.y, v[s][2] = a.z, v[s][3] = a.w;
                        v[s][4] = b.x, v[s][5] = b.y, v[s][6] = b.z, v[s][7] = b.w;
                    }
                tree_sum<8>(v, s_eff);
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] = v[0][e];
            } else if (valid) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(sp + j * 8));
                const float4 b = __ldcg(reinterpret_cast<const float4*>(sp + j * 8 + 4));
                f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
            } else {
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] = 0.f;
            }
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
                const float2 hf = __bfloat1622float2(h);
                const __nv_bfloat162 l = __floats2bfloat162_rn(f[2 * e] - hf.x, f[2 * e + 1] - hf.y);
                hi[e] = *reinterpret_cast<const uint32_t*>(&h);
                lo[e] = *reinterpret_cast<const uint32_t*>(&l);
            }
            *reinterpret_cast<uint4*>(ahi + j * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(alo + j * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
    }
    const uint32_t idesc = umma_idesc_bf16(MMA_M, 128);
    const int lane = tid & 31;
    // Epilogue layout: the accumulator leaves tensor memory one token row per thread, is transposed through a
    // warp-private shared-memory tile, and meets y with one 128-byte (bf16) or 256-byte (f32) row segment per
    // warp instruction: lane l owns columns 2l and 2l+1 of a 64-column chunk for each of the warp's 32 rows.
    float* T = reinterpret_cast<float*>(dsm + 4 * (size_t)op_bytes) + (size_t)warp * 32 * EXP_TPAD;
    const int wrow0 = warp * 32;
    const int nrows = max(0, min(32, len - wrow0));  // live rows of this warp
    const size_t ybase = (size_t)(start + wrow0) * ldy + d.off[p] + 2 * lane;
    bool ok = true;
    for (int nb = 0; nb < nblk; nb++) {
        const int cb = cb0 + nb;
        if (nb + 1 < nblk) load_b(cb + 1, Bs[(nb + 1) & 1]);
        cp_async_commit();
        cp_async_wait<1>();  // everything but the block just requested has landed
        fence_async_smem();
        __syncthreads();
        if (warp == 0) {
            if (elect_one()) {
                tc_fence_after();
                const uint32_t a_hi = smem_u32(Ahi), a_lo = smem_u32(Alo), b = smem_u32(Bs[nb & 1]);
                for (int kk = 0; kk < r / 16; kk++)
                    umma<1>(tmem, umma_desc(a_hi + kk * 256, 128, sbo, 0), umma_desc(b + kk * 256, 128, sbo, 0), idesc,
                              kk != 0);
                for (int kk = 0; kk < r / 16; kk++)
                    umma<1>(tmem, umma_desc(a_lo + kk * 256, 128, sbo, 0), umma_desc(b + kk * 256, 128, sbo, 0), idesc, 1);
                umma_commit(&done);
            }
            __syncwarp();
        }
        const int ncols = min(128, rows - cb * 128);
        // y is requested before the MMAs are waited for, as raw words so that all of a chunk's 32 row
        // segments are in flight together: both 64-column chunks for bf16, the first one for f32
        const size_t yblk = ybase + (size_t)cb * 128;
        uint32_t yb0[32], yb1[32];
        float2 yf[32];
        if (F32) {
            load_rows_f32(yf, reinterpret_cast<const float*>(Y) + yblk, ldy, nrows, 2 * lane < ncols);
        } else {
            load_rows_bf16(yb0, reinterpret_cast<const bf16*>(Y) + yblk, ldy, nrows, 2 * lane < ncols);
            load_rows_bf16(yb1, reinterpret_cast<const bf16*>(Y) + yblk + 64, ldy, nrows, 64 + 2 * lane < ncols);
        }
        ok = mbar_wait(&done, nb & 1, status);
        if (!__syncthreads_and(ok)) {
            ok = false;
            break;
        }
        tc_fence_after();
#pragma unroll
        for (int ch = 0; ch < 2; ch++) {
            if (ch * 64 >= ncols) break;
            {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)wrow0 << 16) + ch * 64, v);
#pragma unroll
                for (int q = 0; q < 32; q++) T[lane * EXP_TPAD + q] = __uint_as_float(v[q]);
                tmem_ld32(tmem + ((uint32_t)wrow0 << 16) + ch * 64 + 32, v);
#pragma unroll
                for (int q = 0; q < 32; q++) T[lane * EXP_TPAD + 32 + q] = __uint_as_float(v[q]);
            }
            __syncwarp();
            const bool colok = ch * 64 + 2 * lane < ncols;
            if (F32) {
                if (ch == 1) load_rows_f32(yf, reinterpret_cast<const float*>(Y) + yblk + 64, ldy, nrows, colok);
                float* yo = reinterpret_cast<float*>(Y) + yblk + ch * 64;
#pragma unroll
                for (int rr = 0; rr < 32; rr++) {
                    if (colok && rr < nrows) {
                        const float2 a = *reinterpret_cast<const float2*>(T + rr * EXP_TPAD + 2 * lane);
                        *reinterpret_cast<float2*>(yo + (size_t)rr * ldy) = make_float2(yf[rr].x + a.x, yf[rr].y + a.y);
                    }
                }
            } else {
                bf16* yo = reinterpret_cast<bf16*>(Y) + yblk + ch * 64;
#pragma unroll
                for (int rr = 0; rr < 32; rr++) {
                    if (colok && rr < nrows) {
                        const float2 a = *reinterpret_cast<const float2*>(T + rr * EXP_TPAD + 2 * lane);
                        const uint32_t raw = ch == 0 ? yb0[rr] : yb1[rr];
                        const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
                        *reinterpret_cast<__nv_bfloat162*>(yo + (size_t)rr * ldy) = __floats2bfloat162_rn(y.x + a.x, y.y + a.y);
                    }
                }
            }
            __syncwarp();
        }
        tc_fence_before();
        __syncthreads();  // the accumulator and this B buffer are free again
    }
    cp_async_wait<0>();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 128);
}

// ------------------------------------------------------------------------------------------------------
// The same expand with y moved by tensor copies, for outputs whose base, row pitch and part offsets are
// 16-byte aligned (every model width in practice; the kernel above stays for the rest). Eight adding warps and
// one more (two blocks per SM; sixteen and one, one block per SM, where the operands of a high maximum rank leave
// no room for two: measured slower at equal shared memory, 509 against 399 us on the widest prefill layer). The
// last warp copies the blocks' rows of B and issues the MMAs, up to two column blocks ahead (mbarriers tell it when S is
// staged and when an accumulator has been read); the other eight never meet at a block-wide barrier inside the
// loop. Each of them owns the 32 token rows tensor memory gives it (two warps per 32 rows, taking alternate
// slots of columns) and a private ring of 4 KB slots; a slot holds 32 rows x 128 bytes of y
// (64 bf16 or 32 f32 columns, 128-byte swizzle). Lane 0 keeps the ring full of loads; a landed slot gets the
// accumulator columns added in shared memory (thread = row: with the swizzle, eight rows cover all banks) and
// goes back with a tensor store, whose completion frees the slot for the next load. So the read-modify-write
// of y, which is most of the bytes of a prefill step, is asynchronous on both sides and many slots deep. The
// accumulator is double-buffered in tensor memory: the MMAs of the next column block run during this block's
// additions. Tensor maps are per part and end at the part's last column, so a box at the edge is clipped
// instead of touching the next part's columns. A warp whose 32 rows are not all inside the tile (the tail of
// a run) loads the same way but writes its live rows with plain stores: the other rows belong to other tokens.
struct ExpandYMaps {
    CUtensorMap m[PLORA_MAX_PARTS];
};
#define EXP_RING_MAX 8
#define EXP_SLOT_BYTES 4096

__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

template <bool F32, int WPQ>  // WPQ: warps per 32 rows (2 or 4)
__global__ void __launch_bounds__(32 * (4 * WPQ + 1)) plora_expand_tma_kernel(const float* __restrict__ S, size_t s_stride, int lds, int K,
                                                                int ksplit, const int* __restrict__ segs, SegLayout lay,
                                                                const plora_desc* __restrict__ table,
                                                                const __grid_constant__ ExpandYMaps ymaps, void* Y, int ldy,
                                                                int nb_per_cta, int op_bytes, int nst,
                                                                int* __restrict__ status) {
    extern __shared__ unsigned char dsm_raw[];
    __shared__ __align__(8) uint64_t done[2], acc_free[2], a_full, ybar[4 * WPQ][EXP_RING_MAX];
    __shared__ uint32_t tmem_slot;
    constexpr int CW = F32 ? 32 : 64;  // y columns per slot
    constexpr int CH = 128 / CW;       // slots per block of 128 columns
    const int tile = blockIdx.z;
    const int n_mma = segs[SEG_N_MMA];
    const int* mt = segs + lay.mma() + 3 * tile;
    const int start = mt[0], len = mt[1], slot = mt[2];
    if (tile >= n_mma) return pdl_exit_idle();
    const plora_desc& d = table[slot];
    const int p = blockIdx.y, r = d.r[p];
    if (r == 0) return pdl_exit_idle();
    const int rows = d.rows[p];
    const int cb0 = blockIdx.x * nb_per_cta;
    if (cb0 * 128 >= rows) return pdl_exit_idle();
    const int nblk = min(nb_per_cta, (rows - cb0 * 128 + 127) / 128);
    const int nchunks = min(nblk * CH, (rows - cb0 * 128 + CW - 1) / CW);  // slots this block fills, in column order
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char* dsm = dsm_raw + ((1024u - (smem_u32(dsm_raw) & 1023u)) & 1023u);
    unsigned char* ring = dsm + (size_t)warp * nst * EXP_SLOT_BYTES;  // this warp's slots
    constexpr int NW = 4 * WPQ;  // warps that add; warp NW copies B and issues the MMAs
    unsigned char* ops = dsm + (size_t)NW * nst * EXP_SLOT_BYTES;
    // Eight warps: warps w and w + 4 read the same 32 lanes of tensor memory (rows 32 (w % 4) ...) and take
    // the even and the odd slots of every column block.
    const int wq = warp & 3, wh = warp >> 2;
    unsigned char* Ahi = ops;
    unsigned char* Alo = ops + op_bytes;
    unsigned char* Bs[2] = {ops + 2 * (size_t)op_bytes, ops + 3 * (size_t)op_bytes};
    const bf16* B = reinterpret_cast<const bf16*>(d.b[p]);
    const uint32_t sbo = (uint32_t)r * 16u;  // 8-row group stride
    const int P = r >> 3;
    const CUtensorMap* ymap = &ymaps.m[p];

    // warp 8 alone copies the blocks' rows of B (four rows of the block per lane) and issues the MMAs
    auto load_b = [&](int cb, unsigned char* dst) {
        for (int n = lane; n < 128; n += 32) {  // row of B = output column of the block
            const bool valid = cb * 128 + n < rows;
            const bf16* src = B + (size_t)(valid ? cb * 128 + n : 0) * r;
            unsigned char* drow = dst + (size_t)(n >> 3) * sbo + (n & 7) * 16;
            for (int j = 0; j < P; j++) cp_async16(drow + j * 128, src + j * 8, valid);
        }
    };
    // warps that have rows of the tile and a slot in every full column block
    const int live_warps = (WPQ < CH ? WPQ : CH) * min(4, (len + 31) / 32);

    if (tid == 0) {
        mbar_init(&done[0], 1);
        mbar_init(&done[1], 1);
        mbar_init(&acc_free[0], live_warps);
        mbar_init(&acc_free[1], live_warps);
        mbar_init(&a_full, 32 * NW);
        for (int w = 0; w < NW; w++)
            for (int i = 0; i < nst; i++) mbar_init(&ybar[w][i], 1);
        mbar_fence_init();
    }
    if (warp == NW) {
        tmem_alloc(&tmem_slot, 256);
        load_b(cb0, Bs[0]);  // B is a slab: it may be fetched before the kernels ahead have finished
        cp_async_commit();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    pdl_wait();
    pdl_trigger();

    if (warp == NW) {
        // ---- B copies and MMAs, running up to two column blocks ahead of the additions
        const uint32_t idesc = umma_idesc_bf16(MMA_M, 128);
        bool ok = mbar_wait_long(&a_full, 0, status);  // S staged by the other warps
        for (int nb = 0; ok && nb < nblk; nb++) {
            cp_async_wait<0>();  // this warp's copies of block nb's rows of B
            fence_async_smem();
            __syncwarp();
            // the accumulator this block goes to was last read for block nb - 2
            if (nb >= 2) ok = mbar_wait_long(&acc_free[nb & 1], ((nb >> 1) - 1) & 1, status);
            if (!ok) break;
            if (elect_one()) {
                tc_fence_after();
                const uint32_t a_hi = smem_u32(Ahi), a_lo = smem_u32(Alo), b = smem_u32(Bs[nb & 1]);
                const uint32_t acc = tmem + (uint32_t)(nb & 1) * 128u;
                for (int kk = 0; kk < r / 16; kk++)
                    umma<1>(acc, umma_desc(a_hi + kk * 256, 128, sbo, 0), umma_desc(b + kk * 256, 128, sbo, 0), idesc, kk != 0);
                for (int kk = 0; kk < r / 16; kk++)
                    umma<1>(acc, umma_desc(a_lo + kk * 256, 128, sbo, 0), umma_desc(b + kk * 256, 128, sbo, 0), idesc, 1);
                umma_commit(&done[nb & 1]);
            }
            __syncwarp();
            if (nb + 1 < nblk) {
                // the other B buffer was read by block nb - 1's MMAs
                if (nb >= 1) ok = mbar_wait_long(&done[(nb - 1) & 1], ((nb - 1) >> 1) & 1, status);
                if (ok) load_b(cb0 + nb + 1, Bs[(nb + 1) & 1]);
            }
            cp_async_commit();
        }
        // every MMA has completed before the tensor memory goes back
        if (ok && nblk >= 1) mbar_wait_long(&done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, status);
        if (ok && nblk >= 2) mbar_wait_long(&done[(nblk - 2) & 1], ((nblk - 2) >> 1) & 1, status);
        cp_async_wait<0>();
        tc_fence_before();
        __syncthreads();
        tmem_dealloc(tmem, 256);
        return;
    }

    const int wrow0 = wq * 32;
    const bool live = wrow0 < len;            // the warp has rows of the tile
    const bool whole = wrow0 + 32 <= len;     // all its 32 rows are: results go back by tensor store
    const int ycol0 = d.off[p] + cb0 * 128;   // first y column of this block's range
    // the warp's i-th slot is slot q of the block's column range
    auto slot_of = [&](int i) { return wh + WPQ * i; };
    int my_n = 0;  // slots this warp handles
    while (slot_of(my_n) < nchunks) my_n++;
    auto load_y = [&](int i) {                // lane 0 only
        uint64_t* bar = &ybar[warp][i % nst];
        mbar_expect_tx(bar, EXP_SLOT_BYTES);
        tma_load_2d(ring + (size_t)(i % nst) * EXP_SLOT_BYTES, ymap, ycol0 + slot_of(i) * CW, start + wrow0, bar);
    };
    if (live && lane == 0)
        for (int i = 0; i < nst && i < my_n; i++) load_y(i);

    // this thread's token row of S, split into a bf16 high part and the bf16 of what is left
    {
        const int row = tid & 127;
        const bool valid = row < len;
        const float* sp = S + (size_t)(start + (valid ? row : 0)) * lds + d.r_off[p];
        const int s_eff = min(ksplit, plora_tile_chunks(K, d.rank));  // planes the shrink wrote for this slot
        unsigned char* ahi = Ahi + (size_t)(row >> 3) * sbo + (row & 7) * 16;
        unsigned char* alo = Alo + (size_t)(row >> 3) * sbo + (row & 7) * 16;
        for (int j = tid >> 7; j < P; j += WPQ) {
            float f[8];
            if (valid && s_eff > 1) {
                float v[PLORA_TILE_SPLIT_MAX][8];
#pragma unroll
                for (int s = 0; s < PLORA_TILE_SPLIT_MAX; s++)
                    if (s < s_eff) {
                        const float* q = sp + (size_t)s * s_stride + j * 8;
                        const float4 a = __ldcg(reinterpret_cast<const float4*>(q));
                        const float4 b = __ldcg(reinterpret_cast<const float4*>(q + 4));
                        v[s][0] = a.x, v[s][1] = a.y, v[s][2] = a.z, v[s][3] = a.w;
                        v[s][4] = b.x, v[s][5] = b.y, v[s][6] = b.z, v[s][7] = b.w;
                    }
                tree_sum<8>(v, s_eff);
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] = v[0][e];
            } else if (valid) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(sp + j * 8));
                const float4 b = __ldcg(reinterpret_cast<const float4*>(sp + j * 8 + 4));
                f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
            } else {
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] = 0.f;
            }
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
                const float2 hf = __bfloat1622float2(h);
                const __nv_bfloat162 l = __floats2bfloat162_rn(f[2 * e] - hf.x, f[2 * e + 1] - hf.y);
                hi[e] = *reinterpret_cast<const uint32_t*>(&h);
                lo[e] = *reinterpret_cast<const uint32_t*>(&l);
            }
            *reinterpret_cast<uint4*>(ahi + j * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(alo + j * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
    }
    // S is staged: tell the MMA warp (the writes above, made visible to the tensor cores first)
    fence_async_smem();
    mbar_arrive(&a_full);

    bool ok = true;
#pragma unroll 1
    for (int i = 0; ok && live && i < my_n; i++) {  // the warp's slots, in column order
        const int q = slot_of(i), nb = q / CH, ch = q % CH;
        if (ch < WPQ) {  // the warp's first slot of column block nb: its MMAs must be complete
            ok = mbar_wait_long(&done[nb & 1], (nb >> 1) & 1, status);
            if (!ok) break;
            tc_fence_after();
        }
        const uint32_t acc = tmem + ((uint32_t)wrow0 << 16) + (uint32_t)(nb & 1) * 128u;
        {
            unsigned char* sl = ring + (size_t)(i % nst) * EXP_SLOT_BYTES;
            if (!mbar_wait(&ybar[warp][i % nst], (i / nst) & 1, status)) {
                ok = false;
                break;
            }
            unsigned char* myrow = sl + lane * 128;
            const int col0 = (cb0 + nb) * 128 + ch * CW;  // first column of the slot within the part
            const bool mine = wrow0 + lane < len;
            if (F32) {
                uint32_t v[32];
                tmem_ld32(acc + ch * 32, v);
                float* yrow = reinterpret_cast<float*>(Y) + (size_t)(start + wrow0 + lane) * ldy + d.off[p] + col0;
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    float4* at = reinterpret_cast<float4*>(myrow + ((c ^ (lane & 7)) << 4));
                    float4 y = *at;
                    y.x += __uint_as_float(v[4 * c]), y.y += __uint_as_float(v[4 * c + 1]);
                    y.z += __uint_as_float(v[4 * c + 2]), y.w += __uint_as_float(v[4 * c + 3]);
                    if (whole) {
                        *at = y;
                    } else if (mine) {
                        if (col0 + 4 * c + 4 <= rows) {
                            *reinterpret_cast<float4*>(yrow + 4 * c) = y;
                        } else {
                            const float e[4] = {y.x, y.y, y.z, y.w};
                            for (int i = 0; i < 4; i++)
                                if (col0 + 4 * c + i < rows) yrow[4 * c + i] = e[i];
                        }
                    }
                }
            } else {
                bf16* yrow = reinterpret_cast<bf16*>(Y) + (size_t)(start + wrow0 + lane) * ldy + d.off[p] + col0;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t v[32];
                    tmem_ld32(acc + ch * 64 + h * 32, v);
#pragma unroll
                    for (int c4 = 0; c4 < 4; c4++) {
                        const int c = h * 4 + c4;
                        uint4* at = reinterpret_cast<uint4*>(myrow + ((c ^ (lane & 7)) << 4));
                        const uint4 raw = *at;
                        float f[8];
                        unpack8(raw, f);
                        uint32_t o[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const __nv_bfloat162 b2 = __floats2bfloat162_rn(f[2 * e] + __uint_as_float(v[8 * c4 + 2 * e]),
                                                                            f[2 * e + 1] + __uint_as_float(v[8 * c4 + 2 * e + 1]));
                            o[e] = *reinterpret_cast<const uint32_t*>(&b2);
                        }
                        if (whole) {
                            *at = make_uint4(o[0], o[1], o[2], o[3]);
                        } else if (mine) {
                            if (col0 + 8 * c + 8 <= rows) {
                                *reinterpret_cast<uint4*>(yrow + 8 * c) = make_uint4(o[0], o[1], o[2], o[3]);
                            } else {
                                const bf16* e = reinterpret_cast<const bf16*>(o);
                                for (int i = 0; i < 8; i++)
                                    if (col0 + 8 * c + i < rows) yrow[8 * c + i] = e[i];
                            }
                        }
                    }
                }
            }
            if (whole) fence_async_smem();  // the additions above, before the tensor store reads them
            __syncwarp();
            if (lane == 0) {
                if (whole) {
                    tma_store_2d(ymap, ycol0 + q * CW, start + wrow0, sl);
                    bulk_commit();
                    if (nst == 1) {  // one slot: wait for this store to have read it, then refill it
                        bulk_wait_read();
                        if (i + 1 < my_n) load_y(i + 1);
                    } else {  // the store before this one has read its slot: refill that slot
                        bulk_wait_read_1();
                        if (i >= 1 && i - 1 + nst < my_n) load_y(i - 1 + nst);
                    }
                } else if (i + nst < my_n) {
                    load_y(i + nst);  // plain stores: the slot is free at once
                }
            }
        }
        if (ch + WPQ >= CH) {  // the warp's last slot of column block nb: it is done with that accumulator
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_free[nb & 1]);
        }
    }
    if (lane == 0) bulk_wait_all();
    tc_fence_before();
    __syncthreads();
}

// cuTensorMapEncodeTiled, fetched from the driver once (no link-time dependency on libcuda)
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn g_encode = nullptr;

}  // namespace

cudaError_t plora_mma_init() {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (!fn || q != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        g_encode = reinterpret_cast<encode_tiled_fn>(fn);
    }
    cudaError_t e = plora_kernel_shared(reinterpret_cast<const void*>(plora_shrink_mma_kernel), 200 * 1024);
    if (e != cudaSuccess) return e;
    e = plora_kernel_shared(reinterpret_cast<const void*>(plora_expand_mma_kernel<false>), 172 * 1024);
    if (e != cudaSuccess) return e;
    e = plora_kernel_shared(reinterpret_cast<const void*>(plora_expand_mma_kernel<true>), 172 * 1024);
    if (e != cudaSuccess) return e;
    if ((e = plora_kernel_shared(reinterpret_cast<const void*>(plora_expand_tma_kernel<false, 2>), 220 * 1024))) return e;
    if ((e = plora_kernel_shared(reinterpret_cast<const void*>(plora_expand_tma_kernel<true, 2>), 220 * 1024))) return e;
    if ((e = plora_kernel_shared(reinterpret_cast<const void*>(plora_expand_tma_kernel<false, 4>), 220 * 1024))) return e;
    return plora_kernel_shared(reinterpret_cast<const void*>(plora_expand_tma_kernel<true, 4>), 220 * 1024);
}

namespace {
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
}  // namespace

// The tensor map of one slot's stacked A for one layer: [R, K] bf16 row-major, boxes of 64 inputs by R rows
// (R / 2 rows when R is over 256, the limit of a box), 128-byte swizzle.
cudaError_t plora_mma_encode_slab(void* out128, const void* a, int K, int R) {
    static_assert(sizeof(CUtensorMap) == sizeof(PloraTmap), "tensor map size");
    if (!g_encode) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)R};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {SHR_KSTEP, (cuuint32_t)(R > 256 ? R / 2 : R)};
    const cuuint32_t es[2] = {1, 1};
    if (g_encode(reinterpret_cast<CUtensorMap*>(out128), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a), dims,
                 strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    return cudaSuccess;
}

cudaError_t plora_launch_shrink_mma(const void* x, int rows, int ldx, int K, const int32_t* segs, SegLayout lay,
                                    const plora_desc* table, const PloraTmap* amaps, float* S, size_t s_stride_elems, int lds,
                                    int max_rank_total, int tile_cap, int tile_split, int* status, bool pdl, bool late,
                                    cudaStream_t st) {
    if (!g_encode) return cudaErrorNotSupported;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {SHR_KSTEP, MMA_M};
    const cuuint32_t es[2] = {1, 1};
    if (g_encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, es,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    int stage_bytes = SHR_X_BYTES + ((max_rank_total * 128 + 1023) / 1024) * 1024;
    // two steps of 64 inputs per stage where at least three such stages fit
    const int sub = 3 * 2 * stage_bytes <= 190 * 1024 ? 2 : 1;
    stage_bytes *= sub;
    int nstage = (190 * 1024) / stage_bytes;
    nstage = nstage > SHR_MAX_STAGES ? SHR_MAX_STAGES : nstage;
    if (nstage < 2) return cudaErrorInvalidValue;
    const size_t smem = (size_t)nstage * stage_bytes + 1024;
    return launch_pdl(plora_shrink_mma_kernel, dim3((unsigned)tile_split, 1, (unsigned)tile_cap), dim3(128), smem, st, pdl,
                      map, reinterpret_cast<const CUtensorMap*>(amaps), K, segs, lay, table, S, s_stride_elems, lds, tile_split,
                      nstage, stage_bytes, sub, late && pdl ? 1 : 0, status);
}

cudaError_t plora_launch_expand_mma(const float* S, size_t s_stride_elems, int lds, int K, int tile_split,
                                    const int32_t* segs, SegLayout lay, const plora_desc* table, void* y, int ldy,
                                    int f32_out, int parts, const int* part_off, const int* part_rows, int rows_total,
                                    int max_rows, int tile_cap, int* status, bool pdl, cudaStream_t st) {
    const int max_rank = lds / PLORA_MAX_PARTS;
    const int op_bytes = MMA_M * max_rank * 2;
    const int nblocks = (max_rows + 127) / 128;
    // Column blocks per thread block (one staging of its S tile each): the count, up to 16, that minimises
    // waves x (start-up + blocks walked) for the step's estimated tile count, two thread blocks per SM; start-up
    // (tensor-memory allocation, staging S, the first MMAs) costs about as much as two and a half column blocks.
    const long long tiles_est = (tile_cap + 1) / 2;  // tile_cap counts 64-token halves
    int nb_per_cta = 1;
    double best = 1e30;
    for (int nb = 1; nb <= 16; nb++) {
        long long groups = 0;
        for (int p = 0; p < parts; p++) groups += ((part_rows[p] + 127) / 128 + nb - 1) / nb;
        const long long waves = (tiles_est * groups + 2 * 148 - 1) / (2 * 148);
        const double cost = (double)waves * (2.5 + nb);
        if (cost < best) {
            best = cost;
            nb_per_cta = nb;
        }
    }
    if (nb_per_cta > nblocks) nb_per_cta = nblocks;
    dim3 grid((unsigned)((nblocks + nb_per_cta - 1) / nb_per_cta), (unsigned)parts, (unsigned)tile_cap);
    // y by tensor copies where its base, pitch and part offsets are 16-byte aligned
    const int elt = f32_out ? 4 : 2;
    bool aligned = g_encode && ((uintptr_t)y & 15) == 0 && ((size_t)ldy * elt) % 16 == 0 && rows_total > 0;
    for (int p = 0; p < parts; p++) aligned = aligned && ((size_t)part_off[p] * elt) % 16 == 0;
    // Two blocks per SM of eight adding warps with the ring slots that leaves room for; where the operands are too
    // large for that, one block per SM of sixteen adding warps.
    int wpq = 2;
    int nst = (111 * 1024 - 1024 - 4 * op_bytes) / (8 * EXP_SLOT_BYTES);
    if (nst < 1) {
        wpq = 4;
        nst = (216 * 1024 - 1024 - 4 * op_bytes) / (16 * EXP_SLOT_BYTES);
    }
    nst = nst > 4 ? 4 : nst;
    if (aligned && nst >= 1) {
        ExpandYMaps maps;
        memset(&maps, 0, sizeof(maps));
        const cuuint32_t es[2] = {1, 1};
        const cuuint32_t box[2] = {(cuuint32_t)(128 / elt), 32};
        const cuuint64_t strides[1] = {(cuuint64_t)ldy * elt};
        for (int p = 0; p < parts && aligned; p++) {
            // the map ends at the part's last column: a box over the edge is clipped
            const cuuint64_t dims[2] = {(cuuint64_t)(part_off[p] + part_rows[p]), (cuuint64_t)rows_total};
            aligned = g_encode(&maps.m[p], f32_out ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y,
                               dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        }
        if (aligned) {
            const size_t smem_tma = 1024 + (size_t)4 * wpq * nst * EXP_SLOT_BYTES + (size_t)4 * op_bytes;
            const dim3 block(32 * (4 * wpq + 1));
#define PLORA_EXPAND_TMA(F32, WPQ)                                                                                      \
    return launch_pdl(plora_expand_tma_kernel<F32, WPQ>, grid, block, smem_tma, st, pdl, S, s_stride_elems, lds, K, \
                      tile_split, segs, lay, table, maps, y, ldy, nb_per_cta, op_bytes, nst, status)
            if (wpq == 2) {
                if (f32_out) PLORA_EXPAND_TMA(true, 2);
                PLORA_EXPAND_TMA(false, 2);
            }
            if (f32_out) PLORA_EXPAND_TMA(true, 4);
            PLORA_EXPAND_TMA(false, 4);
#undef PLORA_EXPAND_TMA
        }
    }
    // at least 48 KB of shared memory per block: no more than four blocks, 128 tensor-memory columns each,
    // share an SM's 512 columns
    size_t smem = (size_t)4 * op_bytes + (size_t)4 * 32 * EXP_TPAD * sizeof(float);
    if (smem < 48 * 1024) smem = 48 * 1024;
    if (f32_out)
        return launch_pdl(plora_expand_mma_kernel<true>, grid, dim3(128), smem, st, pdl, S, s_stride_elems, lds, K,
                          tile_split, segs, lay, table, y, ldy, nb_per_cta, op_bytes, status);
    return launch_pdl(plora_expand_mma_kernel<false>, grid, dim3(128), smem, st, pdl, S, s_stride_elems, lds, K,
                      tile_split, segs, lay, table, y, ldy, nb_per_cta, op_bytes, status);
}
