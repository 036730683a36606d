// FP8 base layer with the adapter expand fused into its epilogue.
//
//   y[t, n] = s_t[t] * s_n[n] * sum_k e4m3(xq[t,k]) * e4m3(wq[n,k])  +  sum_j S[t, r_off_p + j] * B_slot(t),p[n - off_p, j]
//
// xq: per-token dynamically scaled activations, wq: per-output-channel scaled weights, both e4m3. The
// reference runs its FP8 layers through cuBLASLt (block-scaled layouts) and then lora_expand as a separate
// kernel that reads y back (src/linear.rs:428-849, src/kernels/lora.cuh:74-126); here y is written once.
//
//   plora_fp8_quant_rows_kernel  x (bf16) -> xq, s_t = amax_t / 448
//   plora_s_reduce_kernel        adds the shrink's K-split partials of the gather tokens into plane 0
//   plora_fp8_fused_kernel       128 tokens x 64 output columns per block: a TMA-fed ring of (x, W) stages,
//                                tcgen05.mma kind::f8f6f4 into tensor memory; meanwhile four warps build the
//                                adapter term for the tile on CUDA cores (tokens of the tile grouped by slot,
//                                every slot's rows of B streamed once through a ring of async copies); the
//                                same warps then scale the accumulator, add the adapter term and store y
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "plora_internal.h"
#include "plora_device.cuh"
#include "plora_tc.cuh"

typedef __nv_bfloat16 bf16;

namespace {

// K-major operand in 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

// ------------------------------------------------------------------------------------------------------
// Per-token dynamic quantisation: s_t = amax / 448 (1 for an all-zero row), xq = e4m3_satfinite(x / s_t).
// One block per token row.
__global__ void __launch_bounds__(256) plora_fp8_quant_rows_kernel(const bf16* __restrict__ X, int ldx, int K,
                                                                    uint8_t* __restrict__ Xq, float* __restrict__ st) {
    __shared__ float red[8];
    const int t = blockIdx.x;
    const bf16* x = X + (size_t)t * ldx;
    float amax = 0.f;
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(x + k), f);
#pragma unroll
        for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(f[e]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
    const float s = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
    if (threadIdx.x == 0) st[t] = s;
    uint8_t* q = Xq + (size_t)t * K;
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(x + k), f);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            lo |= (uint32_t)__nv_cvt_float_to_fp8(__fdiv_rn(f[e], s), __NV_SATFINITE, __NV_E4M3) << (8 * e);
            hi |= (uint32_t)__nv_cvt_float_to_fp8(__fdiv_rn(f[4 + e], s), __NV_SATFINITE, __NV_E4M3) << (8 * e);
        }
        *reinterpret_cast<uint2*>(q + k) = make_uint2(lo, hi);
    }
}

// Adds the K-split partial planes of every gather token into plane 0, in split order. Grid (work items).
__global__ void __launch_bounds__(128) plora_s_reduce_kernel(float* __restrict__ S, size_t s_stride, int lds, int nsplit,
                                                              const int* __restrict__ segs, SegLayout lay,
                                                              const plora_desc* __restrict__ table, int work_cap,
                                                              int tile_split, int K) {
    const int w = blockIdx.x;
    if (w >= work_cap) {
        // a tensor-core tile: the planes its shrink blocks wrote, added as a balanced tree
        const int tile = w - work_cap;
        if (tile >= segs[SEG_N_MMA]) return pdl_exit_idle();
        const int* mt = segs + lay.mma() + 3 * tile;
        const int start = mt[0], len = mt[1], rank = table[mt[2]].rank;
        const int s_eff = rank ? min(tile_split, plora_tile_chunks(K, rank)) : 1;
        if (s_eff <= 1) return pdl_exit_idle();
        pdl_wait();
        pdl_trigger();
        const int q4 = rank >> 2;
        for (int i = threadIdx.x; i < len * q4; i += 128) {
            const int t = i / q4, j = i - t * q4;
            float* sp = S + (size_t)(start + t) * lds + 4 * j;
            float v[PLORA_TILE_SPLIT_MAX][4];
#pragma unroll
            for (int a = 0; a < PLORA_TILE_SPLIT_MAX; a++)
                if (a < s_eff) {
                    const float4 f = __ldcg(reinterpret_cast<const float4*>(sp + (size_t)a * s_stride));
                    v[a][0] = f.x, v[a][1] = f.y, v[a][2] = f.z, v[a][3] = f.w;
                }
#pragma unroll
            for (int stride = 1; stride < PLORA_TILE_SPLIT_MAX; stride <<= 1)
#pragma unroll
                for (int a = 0; a < PLORA_TILE_SPLIT_MAX; a += 2 * stride)
                    if (a + stride < s_eff)
#pragma unroll
                        for (int q = 0; q < 4; q++) v[a][q] += v[a + stride][q];
            *reinterpret_cast<float4*>(sp) = make_float4(v[0][0], v[0][1], v[0][2], v[0][3]);
        }
        return;
    }
    const int n_work = segs[SEG_N_WORK];
    const int* work = segs + lay.work() + PLORA_WORK_WORDS * w;
    if (w >= n_work) return pdl_exit_idle();
    const int slot = work[0], cnt = work[2];
    const int rank = table[slot].rank;
    pdl_wait();
    pdl_trigger();
    for (int i = threadIdx.x; i < cnt * rank; i += 128) {
        const int t = i / rank, j = i - t * rank;
        float* sp = S + (size_t)work[4 + t] * lds + j;
        float acc = sp[0];
        int s = 1;
        for (; s + 4 <= nsplit; s += 4) {  // in split order, four loads in flight
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = __ldcg(sp + (size_t)(s + u) * s_stride);
#pragma unroll
            for (int u = 0; u < 4; u++) acc += v[u];
        }
        for (; s < nsplit; s++) acc += __ldcg(sp + (size_t)s * s_stride);
        sp[0] = acc;
    }
}

// ------------------------------------------------------------------------------------------------------
#define F8_BM 128
#define F8_BN 64
#define F8_BK 128  // bytes = e4m3 elements per stage row
#define F8_STAGES 3
#define F8_STAGE_BYTES (F8_BM * F8_BK + F8_BN * F8_BK)
#define F8_DPITCH (F8_BN + 1)  // floats per row of the adapter-term tile

struct Fp8Parts {
    int n;
    int off[PLORA_MAX_PARTS];
    int rows[PLORA_MAX_PARTS];
};

#define F8_NQ 8  // adapter work units in flight per block

// Warps: 0 = TMA producer of the GEMM ring, 1 = MMA issuer, 2..5 = adapter term + epilogue (128 threads, one
// output column each in two halves of 64), 6 = producer of the adapter ring (bulk copies of each unit's rows of
// B and S into a byte ring, first in first out).
template <bool F32>
__global__ void __launch_bounds__(224) plora_fp8_fused_kernel(const __grid_constant__ CUtensorMap xmap,
                                                               const __grid_constant__ CUtensorMap wmap,
                                                               const float* __restrict__ st,
                                                               const float* __restrict__ sn, int T, int N, int K,
                                                               const int* __restrict__ segs, SegLayout lay,
                                                               const plora_desc* __restrict__ table, Fp8Parts parts,
                                                               const float* __restrict__ S, int lds, void* Y, int ldy,
                                                               int ring_bytes, int* __restrict__ status) {
    extern __shared__ unsigned char dsm_raw[];
    __shared__ __align__(8) uint64_t full[F8_STAGES], empty[F8_STAGES], acc_bar, q_full[F8_NQ], q_empty[F8_NQ], lists_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_slot[F8_BM], o_row[F8_BM], o_slot[F8_BM], u_first[F8_BM], u_n[F8_BM], u_rank[F8_BM];
    __shared__ short u_r[F8_BM * PLORA_MAX_PARTS], u_roff[F8_BM * PLORA_MAX_PARTS];
    __shared__ uint64_t u_b[F8_BM * PLORA_MAX_PARTS];
    __shared__ int q_boff[F8_NQ * PLORA_MAX_PARTS], q_soff[F8_NQ];
    __shared__ int s_nunits, s_wsum[4];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * F8_BN, m0 = blockIdx.y * F8_BM;
    unsigned char* ring = dsm_raw + ((1024u - (smem_u32(dsm_raw) & 1023u)) & 1023u);
    float* delta = reinterpret_cast<float*>(ring + F8_STAGES * F8_STAGE_BYTES);
    unsigned char* bring = reinterpret_cast<unsigned char*>(delta + F8_BM * F8_DPITCH);
    if (tid == 0) {
        for (int i = 0; i < F8_STAGES; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < F8_NQ; i++) {
            mbar_init(&q_full[i], 1);
            mbar_init(&q_empty[i], 2);  // one arrival per warp of the half that consumed the unit
        }
        mbar_init(&acc_bar, 1);
        mbar_init(&lists_bar, 128);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_slot, F8_BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const int nk = (K + F8_BK - 1) / F8_BK;
    pdl_wait();  // S, xq and the scales come from the kernels before
    pdl_trigger();
    // columns of this tile inside each part: [p_lo, p_hi) relative to the part
    int p_lo[PLORA_MAX_PARTS], p_hi[PLORA_MAX_PARTS];
#pragma unroll
    for (int q = 0; q < PLORA_MAX_PARTS; q++) {
        const int lo = max(n0, parts.off[q]), hi = min(n0 + F8_BN, parts.off[q] + parts.rows[q]);
        p_lo[q] = q < parts.n && hi > lo ? lo - parts.off[q] : 0;
        p_hi[q] = q < parts.n && hi > lo ? hi - parts.off[q] : 0;
    }

    if (warp == 0) {
        // ---- producer: one lane feeds the GEMM ring with TMA
        if (lane == 0) {
            for (int ks = 0; ks < nk; ks++) {
                const int stg = ks % F8_STAGES;
                if (ks >= F8_STAGES && !mbar_wait(&empty[stg], ((ks / F8_STAGES) - 1) & 1, status)) break;
                unsigned char* xs = ring + (size_t)stg * F8_STAGE_BYTES;
                mbar_expect_tx(&full[stg], F8_STAGE_BYTES);
                tma_load_2d(xs, &xmap, ks * F8_BK, m0, &full[stg]);
                tma_load_2d(xs + F8_BM * F8_BK, &wmap, ks * F8_BK, n0, &full[stg]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (elect_one()) {
            // kind::f8f6f4: f32 accumulator, e4m3 A and B (format 0), K-major, M 128, N 64
            const uint32_t idesc = (1u << 4) | ((uint32_t)(F8_BN >> 3) << 17) | ((uint32_t)(F8_BM >> 4) << 24);
            for (int ks = 0; ks < nk; ks++) {
                const int stg = ks % F8_STAGES;
                if (!mbar_wait(&full[stg], (ks / F8_STAGES) & 1, status)) break;
                tc_fence_after();
                const uint32_t xs = smem_u32(ring + (size_t)stg * F8_STAGE_BYTES);
                const uint32_t ws = xs + F8_BM * F8_BK;
#pragma unroll
                for (int kk = 0; kk < F8_BK / 32; kk++)
                    umma<0>(tmem, umma_desc_sw128(xs + kk * 32), umma_desc_sw128(ws + kk * 32), idesc, (ks | kk) != 0);
                umma_commit(&empty[stg]);
            }
            umma_commit(&acc_bar);
        }
        __syncwarp();
    } else if (warp == 6) {
        // ---- producer of the adapter ring: each unit's rows of B (one contiguous block per part) and of S
        if (lane == 0 && mbar_wait(&lists_bar, 0, status)) {
            const int nunits = s_nunits;
            int head = 0, tail = 0, released = 0;
            int ent_off[F8_NQ];
            bool ok = true;
            for (int u = 0; ok && u < nunits; u++) {
                const int q = u % F8_NQ;
                int bbytes[PLORA_MAX_PARTS], size = 0;
#pragma unroll
                for (int pp = 0; pp < PLORA_MAX_PARTS; pp++) {
                    bbytes[pp] = (p_hi[pp] - p_lo[pp]) * (int)u_r[u * PLORA_MAX_PARTS + pp] * 2;
                    size += bbytes[pp];
                }
                const int srow_bytes = u_rank[u] * 4;
                size += u_n[u] * srow_bytes;
                int pos = -1;
                while (ok) {
                    // release the oldest units while the queue slot is taken or the bytes do not fit
                    const bool slot_free = u - released < F8_NQ;
                    if (released == u) head = tail = 0;
                    if (slot_free) {
                        if (head >= tail) {
                            if (head + size <= ring_bytes) pos = head;
                            else if (size < tail) pos = 0;
                        } else if (head + size < tail) {
                            pos = head;
                        }
                    }
                    if (pos >= 0) break;
                    if (released == u) {  // a single unit larger than the ring: cannot happen by construction
                        atomicMax(status, PLORA_ERR_CAPACITY);
                        ok = false;
                        break;
                    }
                    ok = mbar_wait(&q_empty[released % F8_NQ], (released / F8_NQ) & 1, status);
                    released++;
                    tail = released < u ? ent_off[released % F8_NQ] : head;
                }
                if (!ok) break;
                ent_off[q] = pos;
                head = pos + size;
                unsigned char* dst = bring + pos;
                int at = 0;
#pragma unroll
                for (int pp = 0; pp < PLORA_MAX_PARTS; pp++) {
                    q_boff[q * PLORA_MAX_PARTS + pp] = pos + at;
                    at += bbytes[pp];
                }
                q_soff[q] = pos + at;
                if (size > 0) {
                    mbar_expect_tx(&q_full[q], (uint32_t)size);
                    at = 0;
#pragma unroll
                    for (int pp = 0; pp < PLORA_MAX_PARTS; pp++) {
                        if (bbytes[pp] > 0) {
                            const int r = u_r[u * PLORA_MAX_PARTS + pp];
                            bulk_g2s(dst + at, reinterpret_cast<const bf16*>(u_b[u * PLORA_MAX_PARTS + pp]) + (size_t)p_lo[pp] * r,
                                     (uint32_t)bbytes[pp], &q_full[q]);
                            at += bbytes[pp];
                        }
                    }
                    for (int rr = 0; rr < u_n[u]; rr++)
                        bulk_g2s(dst + at + rr * srow_bytes, S + (size_t)(m0 + o_row[u_first[u] + rr]) * lds, (uint32_t)srow_bytes,
                                 &q_full[q]);
                } else {
                    mbar_arrive(&q_full[q]);
                }
            }
        }
    } else {
        // ---- adapter term of the tile, then the epilogue (threads 0..127 of this group)
        const int et = tid - 64;
        const int row = m0 + et;
        // tokens of the tile sorted by slot (stable); slot 0 (no adapter) and rows past T first
        const int myslot = row < T ? segs[lay.tslot() + row] : 0;
        s_slot[et] = myslot;
        for (int i = et; i < F8_BM * F8_DPITCH; i += 128) delta[i] = 0.f;
        epi_sync();
        int rank = 0;
        for (int j = 0; j < F8_BM; j++) {
            const int sj = s_slot[j];
            rank += (sj < myslot) || (sj == myslot && j < et);
        }
        o_row[rank] = et;
        o_slot[rank] = myslot;
        epi_sync();
        // units of work: the rows of one slot, four at a time. Entry et of the sorted list starts a unit when it is
        // the 1st, 5th, 9th ... row of its slot's group; unit numbers come from a prefix sum over the 128 entries.
        {
            const int sl = o_slot[et];
            int g0 = et;
            while (g0 > 0 && o_slot[g0 - 1] == sl) g0--;
            const int uhead = sl != 0 && ((et - g0) & 3) == 0;
            int incl = uhead;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int w4 = (et >> 5);
            if (lane == 31) s_wsum[w4] = incl;
            epi_sync();
            int base = 0;
            for (int q = 0; q < w4; q++) base += s_wsum[q];
            if (uhead) {
                const int u = base + incl - 1;
                int nrows = 1;
                while (nrows < 4 && et + nrows < F8_BM && o_slot[et + nrows] == sl) nrows++;
                u_first[u] = et;
                u_n[u] = nrows;
                // the unit's descriptor fields, fetched once
                const plora_desc& d = table[sl];
                u_rank[u] = d.rank;
                for (int q = 0; q < PLORA_MAX_PARTS; q++) {
                    u_r[u * PLORA_MAX_PARTS + q] = d.r[q];
                    u_roff[u * PLORA_MAX_PARTS + q] = d.r_off[q];
                    u_b[u * PLORA_MAX_PARTS + q] = d.b[q];
                }
            }
            if (et == 127) s_nunits = base + incl;
        }
        mbar_arrive(&lists_bar);  // the ring's producer may start
        epi_sync();
        const int nunits = s_nunits;
        // two halves of 64 threads: each thread owns one output column, each half every second unit
        const int half = et >> 6, c = et & 63;
        const int n = n0 + c;
        int p = -1;
        for (int q = 0; q < parts.n; q++)
            if (n >= parts.off[q] && n < parts.off[q] + parts.rows[q]) p = q;
        const int cl = p >= 0 ? n - parts.off[p] - p_lo[p] : 0;  // column inside the tile's block of part p
        bool alive = true;
        for (int u = half; u < nunits; u += 2) {
            const int q = u % F8_NQ;
            if (alive) alive = mbar_wait(&q_full[q], (u / F8_NQ) & 1, status);
            if (alive && p >= 0) {
                const int r = u_r[u * PLORA_MAX_PARTS + p], r_off = u_roff[u * PLORA_MAX_PARTS + p];
                const unsigned char* src = bring + q_boff[q * PLORA_MAX_PARTS + p] + (size_t)cl * r * 2;
                const int srow = u_rank[u];
                const float* sbase = reinterpret_cast<const float*>(bring + q_soff[q]) + r_off;
                const int nr = u_n[u];
                // Four rows at once, two partial sums each: eight independent chains, because each of these warps
                // runs alone on its scheduler and has nothing else to hide latencies with. Rows past nr repeat the
                // last row (their sums are dropped).
                float acc[4][2];
#pragma unroll
                for (int rr = 0; rr < 4; rr++) acc[rr][0] = acc[rr][1] = 0.f;
                const float* srow_p[4];
#pragma unroll
                for (int rr = 0; rr < 4; rr++) srow_p[rr] = sbase + min(rr, nr - 1) * srow;
                // Rows of B sit r * 2 bytes apart in the ring: walking them in step would put all lanes of a warp
                // on the same banks, so each column starts at its own 16-byte piece and wraps around.
                const int P = r >> 3;
                int jp = P > 0 ? c % P : 0;
#pragma unroll 2
                for (int qq = 0; qq < P; qq++) {
                    const int j = jp << 3;
                    jp = jp + 1 == P ? 0 : jp + 1;
                    float bf[8];
                    unpack8(*reinterpret_cast<const uint4*>(src + j * 2), bf);
                    float4 s0[4], s1[4];
#pragma unroll
                    for (int rr = 0; rr < 4; rr++) {
                        s0[rr] = *reinterpret_cast<const float4*>(srow_p[rr] + j);
                        s1[rr] = *reinterpret_cast<const float4*>(srow_p[rr] + j + 4);
                    }
#pragma unroll
                    for (int rr = 0; rr < 4; rr++) {
                        acc[rr][0] = fmaf(s0[rr].x, bf[0], acc[rr][0]);
                        acc[rr][1] = fmaf(s0[rr].y, bf[1], acc[rr][1]);
                        acc[rr][0] = fmaf(s0[rr].z, bf[2], acc[rr][0]);
                        acc[rr][1] = fmaf(s0[rr].w, bf[3], acc[rr][1]);
                        acc[rr][0] = fmaf(s1[rr].x, bf[4], acc[rr][0]);
                        acc[rr][1] = fmaf(s1[rr].y, bf[5], acc[rr][1]);
                        acc[rr][0] = fmaf(s1[rr].z, bf[6], acc[rr][0]);
                        acc[rr][1] = fmaf(s1[rr].w, bf[7], acc[rr][1]);
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 4; rr++)
                    if (rr < nr && r > 0) delta[o_row[u_first[u] + rr] * F8_DPITCH + c] = acc[rr][0] + acc[rr][1];  // each row: one unit
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_empty[q]);  // this warp is done with the unit's bytes
        }
        epi_sync();
        // ---- epilogue: accumulator row by row out of tensor memory, scaled, plus the adapter term
        const bool ok = mbar_wait(&acc_bar, 0, status) && alive;
        tc_fence_after();
        const int q4 = warp & 3;  // this warp's quarter of the 128 tensor-memory lanes
        const int lrow = q4 * 32 + lane;
        const float srow_scale = (m0 + lrow) < T ? st[m0 + lrow] : 0.f;
        if (ok) {
#pragma unroll
            for (int cc = 0; cc < F8_BN; cc += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + cc, v);
#pragma unroll
                for (int q = 0; q < 32; q++) {
                    const int col = n0 + cc + q;
                    const float sc = col < N ? __ldg(sn + col) : 0.f;
                    float* dp = delta + lrow * F8_DPITCH + cc + q;
                    *dp = fmaf(__uint_as_float(v[q]), srow_scale * sc, *dp);
                }
            }
        }
        __syncwarp();
        // coalesced store: the warp's 32 rows, lane l writes columns 2l and 2l + 1
        if (ok) {
            const int col = n0 + 2 * lane;
            if (col < N) {
                for (int rr = 0; rr < 32; rr++) {
                    const int grow = m0 + q4 * 32 + rr;
                    if (grow >= T) break;
                    const float a = delta[(q4 * 32 + rr) * F8_DPITCH + 2 * lane];
                    const float b = delta[(q4 * 32 + rr) * F8_DPITCH + 2 * lane + 1];
                    const size_t at = (size_t)grow * ldy + col;
                    if (F32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(Y) + at) = make_float2(a, b);
                    else *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf16*>(Y) + at) = __floats2bfloat162_rn(a, b);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, F8_BN);
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn g_encode = nullptr;

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

// Shared memory: GEMM stages, the adapter-term tile, and whatever is left (up to the launch limit) as the byte
// ring of the adapter units.
size_t fused_smem() { return (size_t)212 * 1024; }
int fused_ring_bytes() {
    return (int)(fused_smem() - 1024 - (size_t)F8_STAGES * F8_STAGE_BYTES - (size_t)F8_BM * F8_DPITCH * 4);
}

}  // namespace

cudaError_t plora_fp8_init(int max_rank) {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (!fn || q != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        g_encode = reinterpret_cast<encode_tiled_fn>(fn);
    }
    // the largest unit (64 columns x 4 parts' worst rank + 4 rows of S) must fit the ring a few times over
    if ((size_t)F8_BN * max_rank * 2 + (size_t)4 * PLORA_MAX_PARTS * max_rank * 4 > (size_t)fused_ring_bytes() / 2)
        return cudaErrorInvalidValue;
    const int smem = (int)fused_smem();
    // the two small kernels that run right before the layer kernel ask for the same split of the SM
    cudaError_t e0 = plora_kernel_shared(reinterpret_cast<const void*>(plora_fp8_quant_rows_kernel), 0);
    if (e0 == cudaSuccess) e0 = plora_kernel_shared(reinterpret_cast<const void*>(plora_s_reduce_kernel), 0);
    if (e0 != cudaSuccess) return e0;
    cudaError_t e = plora_kernel_shared(reinterpret_cast<const void*>(plora_fp8_fused_kernel<false>), smem);
    if (e != cudaSuccess) return e;
    return plora_kernel_shared(reinterpret_cast<const void*>(plora_fp8_fused_kernel<true>), smem);
}

cudaError_t plora_launch_fp8_quant(const void* x, int rows, int ldx, int K, void* xq, float* st, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    plora_fp8_quant_rows_kernel<<<rows, 256, 0, stream>>>(reinterpret_cast<const bf16*>(x), ldx, K,
                                                          reinterpret_cast<uint8_t*>(xq), st);
    return cudaGetLastError();
}

cudaError_t plora_launch_s_reduce(float* S, size_t s_stride_elems, int lds, int nsplit, const int32_t* segs,
                                  SegLayout lay, const plora_desc* table, int work_cap, int tile_cap, int tile_split,
                                  int K, bool pdl, cudaStream_t st) {
    if (tile_split <= 1) tile_cap = 0;
    if (nsplit <= 1 && tile_cap == 0) return cudaSuccess;
    if (work_cap + tile_cap == 0) return cudaSuccess;
    return launch_pdl(plora_s_reduce_kernel, dim3((unsigned)(work_cap + tile_cap)), dim3(128), 0, st, pdl, S, s_stride_elems,
                      lds, nsplit, segs, lay, table, work_cap, tile_split, K);
}

cudaError_t plora_launch_fp8_fused(const void* xq, const float* st_, const void* wq, const float* sn, int T, int N, int K,
                                   const int32_t* segs, SegLayout lay, const plora_desc* table, int n_parts,
                                   const int* part_off, const int* part_rows, const float* S, int lds, void* y, int ldy,
                                   int f32_out, int max_rank, int* status, bool pdl, cudaStream_t stream) {
    if (!g_encode) return cudaErrorNotSupported;
    CUtensorMap xmap, wmap;
    const cuuint32_t es[2] = {1, 1};
    {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)T};
        const cuuint64_t strides[1] = {(cuuint64_t)K};
        const cuuint32_t box[2] = {F8_BK, F8_BM};
        if (g_encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(xq), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
        const cuuint64_t strides[1] = {(cuuint64_t)K};
        const cuuint32_t box[2] = {F8_BK, F8_BN};
        if (g_encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(wq), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    Fp8Parts parts;
    parts.n = n_parts;
    for (int i = 0; i < PLORA_MAX_PARTS; i++) {
        parts.off[i] = i < n_parts ? part_off[i] : 0;
        parts.rows[i] = i < n_parts ? part_rows[i] : 0;
    }
    (void)max_rank;
    dim3 grid((unsigned)((N + F8_BN - 1) / F8_BN), (unsigned)((T + F8_BM - 1) / F8_BM));
    const size_t smem = fused_smem();
    const int ring_bytes = fused_ring_bytes();
    if (f32_out)
        return launch_pdl(plora_fp8_fused_kernel<true>, grid, dim3(224), smem, stream, pdl, xmap, wmap, st_, sn, T, N, K,
                          segs, lay, table, parts, S, lds, y, ldy, ring_bytes, status);
    return launch_pdl(plora_fp8_fused_kernel<false>, grid, dim3(224), smem, stream, pdl, xmap, wmap, st_, sn, T, N, K, segs,
                      lay, table, parts, S, lds, y, ldy, ring_bytes, status);
}
