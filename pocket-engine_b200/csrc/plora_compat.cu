// Drop-in kernel image for an UNMODIFIED pocket-engine: the engine fetches `lora_shrink` and `lora_expand` by
// name from whatever fatbin POCKET_KERNELS points at (src/gpu.rs:451-468,552-564; src/lora.rs:510-521) and
// launches them with its own grids (src/linear.rs:862-884,900-920):
//   lora_shrink  grid (min(max_tiles, rows), ceil(parts * max_rank / 32), ceil(K / 256)), 128 threads
//   lora_expand  grid (min(max_tiles, rows), ceil(max part rows / 128), parts),            128 threads
// The signatures, the 112-byte LoraDesc, the tile words and the two-buffer S choreography (shrink accumulates
// into a zeroed S; block (y=0, z=0) of the expand zeroes the tile's rows of the other buffer) are the
// reference's (src/kernels/lora.cuh:7-126). The bodies are new: CUDA-core code with 128-bit loads and warp
// shuffles instead of mma.sync fragments fetched 4 bytes at a time, and S is not rounded to bf16.
// Build: nvcc --fatbin -gencode arch=compute_100a,code=sm_100a plora_compat.cu -o plora_compat.fatbin
#include <cuda_bf16.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

struct LoraDesc {
    const bf16* a;     // [rank, K]
    const bf16* b[4];  // per part [rows, r]
    int rank;          // total, 0 when the adapter leaves this layer alone
    int r[4];          // per part, 0 when untargeted
    int r_off[4];      // per part, its first column of S
    int off[4];        // per part, its first output column
    int rows[4];
    int pad_;
};

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x << 16);
    f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16);
    f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16);
    f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16);
    f[7] = __uint_as_float(v.w & 0xffff0000u);
}

// 32 values per lane -> their warp-wide sums; lane l returns the sum of value l.
__device__ __forceinline__ float reduce32(float (&v)[32], int lane) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
#pragma unroll
        for (int i = 0; i < s; i++) {
            const float send = (lane & s) ? v[i] : v[i + s];
            const float keep = (lane & s) ? v[i + s] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
        }
    }
    return v[0];
}

// Each block adds 32 columns of S for one tile over 256 inputs. Warp w takes S columns n0 + 8w .. + 7, its lanes
// 8 inputs each; tokens go four at a time (8 columns x 4 tokens = 32 sums per pass).
extern "C" __global__ void __launch_bounds__(128) lora_shrink(const bf16* __restrict__ X, int ldx, int K,
                                                              const int* __restrict__ tiles,
                                                              const LoraDesc* __restrict__ table,
                                                              float* __restrict__ S, int lds) {
    const int tile = blockIdx.x;
    if (tile >= tiles[0]) return;
    const int t0 = tiles[1 + 3 * tile], len = tiles[2 + 3 * tile], slot = tiles[3 + 3 * tile];
    const LoraDesc& d = table[slot];
    const int n0 = blockIdx.y * 32;
    if (n0 >= d.rank) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k = blockIdx.z * 256 + 8 * lane;
    const bool kin = k < K;  // K is a multiple of 16
    const int nw = n0 + 8 * warp;
    float af[8][8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int n = min(nw + j, d.rank - 1);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (kin) v = __ldg(reinterpret_cast<const uint4*>(d.a + (size_t)n * K + k));
        unpack8(v, af[j]);
    }
    for (int tp = 0; tp < len; tp += 4) {
        float acc[32];
#pragma unroll
        for (int t = 0; t < 4; t++) {
            float xf[8];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (kin && tp + t < len) v = __ldg(reinterpret_cast<const uint4*>(X + (size_t)(t0 + tp + t) * ldx + k));
            unpack8(v, xf);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < 8; e++) s = fmaf(xf[e], af[j][e], s);
                acc[t * 8 + j] = s;
            }
        }
        const float v = reduce32(acc, lane);
        // step s of the butterfly keeps bit s of the value index equal to bit s of the lane: lane l ends with value l
        const int t = lane >> 3, j = lane & 7;
        if (tp + t < len && nw + j < d.rank) atomicAdd(&S[(size_t)(t0 + tp + t) * lds + nw + j], v);
    }
}

// Each block adds 128 output columns of one part for one tile (thread = column) and, for (y=0, z=0), zeroes the
// tile's rows of the other S buffer.
extern "C" __global__ void __launch_bounds__(128) lora_expand(const float* __restrict__ S, int lds,
                                                              float* __restrict__ next,
                                                              const int* __restrict__ tiles,
                                                              const LoraDesc* __restrict__ table, void* Y, int ldy,
                                                              int f32_out) {
    __shared__ float ss[16][128 + 4];
    const int tile = blockIdx.x;
    if (tile >= tiles[0]) return;
    const int t0 = tiles[1 + 3 * tile], len = tiles[2 + 3 * tile], slot = tiles[3 + 3 * tile];
    if (blockIdx.y == 0 && blockIdx.z == 0)
        for (int i = threadIdx.x; i < len * lds; i += 128) next[(size_t)t0 * lds + i] = 0.f;
    const LoraDesc& d = table[slot];
    const int p = blockIdx.z, r = d.r[p];
    if (r == 0) return;
    const int rows = d.rows[p];
    if (blockIdx.y * 128 >= rows) return;
    const int col = blockIdx.y * 128 + threadIdx.x;
    const bf16* b = d.b[p] + (size_t)min(col, rows - 1) * r;
    float acc[16];
#pragma unroll
    for (int t = 0; t < 16; t++) acc[t] = 0.f;
    for (int k0 = 0; k0 < r; k0 += 128) {
        const int kn = min(128, r - k0);
        __syncthreads();
        for (int i = threadIdx.x; i < len * kn; i += 128) {
            const int t = i / kn, k = i - t * kn;
            ss[t][k] = S[(size_t)(t0 + t) * lds + d.r_off[p] + k0 + k];
        }
        __syncthreads();
        for (int k = 0; k < kn; k += 8) {
            float bf[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(b + k0 + k)), bf);
#pragma unroll
            for (int t = 0; t < 16; t++) {
                if (t < len) {
#pragma unroll
                    for (int e = 0; e < 8; e++) acc[t] = fmaf(ss[t][k + e], bf[e], acc[t]);
                }
            }
        }
    }
    if (col >= rows) return;
#pragma unroll
    for (int t = 0; t < 16; t++) {
        if (t < len) {
            const size_t at = (size_t)(t0 + t) * ldy + d.off[p] + col;
            if (f32_out) ((float*)Y)[at] += acc[t];
            else ((bf16*)Y)[at] = __float2bfloat16_rn(__bfloat162float(((bf16*)Y)[at]) + acc[t]);
        }
    }
}
