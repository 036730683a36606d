// Tensor-core tiles of the few-token expand, shared by the cluster kernel (one kernel per layer) and the gather
// expand of the shrink / expand bracket: S as bf16 terms in shared memory times rows of B in shared memory, y
// updated in global memory. 16-token tiles on the warp-level instruction (m16n8k16, bf16 in, f32 accumulate); the
// f32 intermediate enters as three bf16 terms (high, middle, low part), whose products with bf16 B are exact in
// f32, so no precision is given up against an f32 multiply-add chain.
#pragma once
#include <cuda_bf16.h>

#include <type_traits>

#include "plora_device.cuh"

#define PLORA_TILE_WARPS 8  // warps of a block that share the columns of an expand

namespace {

typedef __nv_bfloat16 bf16;

// four 8x8 bf16 matrices from shared memory: lane l gives the address of row (l % 8) of matrix l / 8
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// D (16 x 8, f32) += A (16 x 16, bf16, row-major) . B (16 x 8, bf16, column-major)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// y of one 16-column step: the lane's two token rows (g and g + 8) times its two column pairs
template <bool F32>
struct YStep {
    float2 v[2][2];
};

// One part's share of the output columns: y[tok, off + lo + c] += S3[tok, r_off ..] . B[c, :]^T for c in [0, ncols).
// NK: 16-wide steps over the part's rank held as fragments in registers (0: fetched from shared memory per step).
template <int NK, bool F32>
__device__ __forceinline__ void expand_part(uint32_t s3_part, uint32_t plane_bytes, uint32_t bs_lane, int r, int ncols,
                                            void* Y, int ldy, size_t ybase, int tok0, int tok1, int warp, int t2) {
    typedef typename std::conditional<F32, float, bf16>::type ytype;
    const int nk = NK > 0 ? NK : r >> 4;
    uint32_t sa[NK > 0 ? NK : 1][3][4];
    if (NK > 0) {
#pragma unroll
        for (int ks = 0; ks < NK; ks++)
#pragma unroll
            for (int pl = 0; pl < 3; pl++) ldmatrix_x4(sa[ks][pl], s3_part + (uint32_t)pl * plane_bytes + (uint32_t)ks * 32u);
    }
    ytype* y0 = tok0 >= 0 ? reinterpret_cast<ytype*>(Y) + (size_t)tok0 * ldy + ybase + t2 : nullptr;
    ytype* y1 = tok1 >= 0 ? reinterpret_cast<ytype*>(Y) + (size_t)tok1 * ldy + ybase + t2 : nullptr;
    auto load = [&](YStep<F32>& q, int c) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const ytype* yp = h ? y1 : y0;
#pragma unroll
            for (int n = 0; n < 2; n++) {
                if (yp != nullptr && c + n * 8 + t2 < ncols) {
                    if (F32) q.v[h][n] = *reinterpret_cast<const float2*>(yp + c + n * 8);
                    else q.v[h][n] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(yp + c + n * 8));
                }
            }
        }
    };
    // 16 columns (two tiles of 8) per step; warp q takes the steps q, q + 8, ...; y is fetched two steps ahead
    int c = warp * 16;
    YStep<F32> q0, q1, q2;
    load(q0, c);
    load(q1, c + PLORA_TILE_WARPS * 16);
    for (; c < ncols; c += PLORA_TILE_WARPS * 16) {
        load(q2, c + 2 * PLORA_TILE_WARPS * 16);
        float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < (NK > 0 ? NK : 8); ks++) {
            if (ks < nk) {
                uint32_t bb[4];
                ldmatrix_x4(bb, bs_lane + (uint32_t)c * (uint32_t)r * 2u + (uint32_t)ks * 32u);
                // low, middle, high term: the small ones first
#pragma unroll
                for (int pl = 2; pl >= 0; pl--) {
                    if (NK > 0) {
                        mma_16816(d0, sa[ks][pl], bb[0], bb[1]);
                        mma_16816(d1, sa[ks][pl], bb[2], bb[3]);
                    } else {
                        uint32_t st[4];
                        ldmatrix_x4(st, s3_part + (uint32_t)pl * plane_bytes + (uint32_t)ks * 32u);
                        mma_16816(d0, st, bb[0], bb[1]);
                        mma_16816(d1, st, bb[2], bb[3]);
                    }
                }
            }
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            ytype* yp = h ? y1 : y0;
#pragma unroll
            for (int n = 0; n < 2; n++) {
                if (yp != nullptr && c + n * 8 + t2 < ncols) {
                    const float* d = n ? d1 : d0;
                    const float v0 = q0.v[h][n].x + d[2 * h], v1 = q0.v[h][n].y + d[2 * h + 1];
                    if (F32) *reinterpret_cast<float2*>(yp + c + n * 8) = make_float2(v0, v1);
                    else *reinterpret_cast<__nv_bfloat162*>(yp + c + n * 8) = __floats2bfloat162_rn(v0, v1);
                }
            }
        }
        q0 = q1;
        q1 = q2;
    }
}

// The same for work items of at most 8 tokens whose y rows can move in 16-byte pieces (the common decoding case):
// 32 columns per step. Rows 0-7 of the token tile carry one bf16 term of S and rows 8-15 another, so the three terms
// take two multiplies per 8-column tile ([high | middle], [low | zero]) and a lane adds its two rows. The B rows
// are fed to the step's four tiles in an order that leaves every lane with 8 adjacent columns of its token row:
// y is read and written as 16-byte pieces, 64 contiguous bytes per row and instruction (bf16).
template <int NK, bool F32>
__device__ __forceinline__ void expand_fast(uint32_t s3_part, uint32_t sp_pad, uint32_t plane_bytes, uint32_t bs_part, int r,
                                            int ncols, void* Y, int ldy, size_t ybase, int tok, int warp, int lane, bool pre,
                                            uint4 pre0, uint4 pre1) {
    typedef typename std::conditional<F32, float, bf16>::type ytype;
    const int nk = NK > 0 ? NK : r >> 4;
    const uint32_t a_lane = s3_part + (uint32_t)(lane & 7) * sp_pad + (uint32_t)((lane >> 3) & 1) * plane_bytes + (uint32_t)(lane >> 4) * 16u;
    uint32_t sa[NK > 0 ? NK : 1][2][4];
    if (NK > 0) {
#pragma unroll
        for (int ks = 0; ks < NK; ks++) {
            ldmatrix_x4(sa[ks][0], a_lane + (uint32_t)ks * 32u);
            ldmatrix_x4(sa[ks][1], a_lane + 2u * plane_bytes + (uint32_t)ks * 32u);
        }
    }
    const bool live = tok >= 0;
    ytype* y = reinterpret_cast<ytype*>(Y) + (size_t)(live ? tok : 0) * ldy + ybase + 8 * (lane & 3);
    // four-matrix load: matrices 0,1 = tile n (inputs 0-7, 8-15 of the step), matrices 2,3 = tile n + 1; row j of tile
    // n is column 8 (j / 2) + 2 n + (j % 2) of the step
    const int j = lane & 7, half = (lane >> 3) & 1, tsel = lane >> 4;
    const uint32_t b01 = bs_part + (uint32_t)(8 * (j >> 1) + 2 * tsel + (j & 1)) * (uint32_t)r * 2u + (uint32_t)half * 16u;
    const uint32_t b23 = b01 + 4u * (uint32_t)r * 2u;
    const int c8 = 8 * (lane & 3);
    int c = warp * 32;
    uint4 q0 = make_uint4(0u, 0u, 0u, 0u), q1 = q0, n0 = q0, n1 = q0;
    auto fetch = [&](uint4& a, uint4& b, int cc) {
        if (live && cc + c8 < ncols) {
            a = __ldcg(reinterpret_cast<const uint4*>(y + cc));
            if (F32) b = __ldcg(reinterpret_cast<const uint4*>(y + cc) + 1);
        }
    };
    if (pre) {  // the first step's y was asked for right after the dependency wait
        q0 = pre0;
        q1 = pre1;
    } else {
        fetch(q0, q1, c);
    }
    for (; c < ncols; c += PLORA_TILE_WARPS * 32) {
        fetch(n0, n1, c + PLORA_TILE_WARPS * 32);
        float d[4][4];
#pragma unroll
        for (int n = 0; n < 4; n++) d[n][0] = d[n][1] = d[n][2] = d[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < (NK > 0 ? NK : 8); ks++) {
            if (ks < nk) {
                uint32_t ba[4], bc[4];
                ldmatrix_x4(ba, b01 + (uint32_t)c * (uint32_t)r * 2u + (uint32_t)ks * 32u);
                ldmatrix_x4(bc, b23 + (uint32_t)c * (uint32_t)r * 2u + (uint32_t)ks * 32u);
                // [low | zero] first, then [high | middle]
#pragma unroll
                for (int f = 1; f >= 0; f--) {
                    uint32_t st[4];
                    if (NK == 0) ldmatrix_x4(st, a_lane + (uint32_t)f * 2u * plane_bytes + (uint32_t)ks * 32u);
                    const uint32_t(&a)[4] = NK > 0 ? sa[NK > 0 ? ks : 0][f] : st;
                    mma_16816(d[0], a, ba[0], ba[1]);
                    mma_16816(d[1], a, ba[2], ba[3]);
                    mma_16816(d[2], a, bc[0], bc[1]);
                    mma_16816(d[3], a, bc[2], bc[3]);
                }
            }
        }
        if (live && c + c8 < ncols) {
            if (F32) {
                const float4 a = *reinterpret_cast<const float4*>(&q0), b = *reinterpret_cast<const float4*>(&q1);
                *reinterpret_cast<float4*>(y + c) = make_float4(a.x + (d[0][0] + d[0][2]), a.y + (d[0][1] + d[0][3]),
                                                                 a.z + (d[1][0] + d[1][2]), a.w + (d[1][1] + d[1][3]));
                *(reinterpret_cast<float4*>(y + c) + 1) = make_float4(b.x + (d[2][0] + d[2][2]), b.y + (d[2][1] + d[2][3]),
                                                                       b.z + (d[3][0] + d[3][2]), b.w + (d[3][1] + d[3][3]));
            } else {
                const uint32_t w[4] = {q0.x, q0.y, q0.z, q0.w};
                uint32_t o[4];
#pragma unroll
                for (int n = 0; n < 4; n++) {
                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[n]));
                    const __nv_bfloat162 v = __floats2bfloat162_rn(f.x + (d[n][0] + d[n][2]), f.y + (d[n][1] + d[n][3]));
                    o[n] = *reinterpret_cast<const uint32_t*>(&v);
                }
                *reinterpret_cast<uint4*>(y + c) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        q0 = n0;
        q1 = n1;
    }
}

}  // namespace
