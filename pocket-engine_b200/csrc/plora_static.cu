// plora_site_apply_static: one layer's adapter application (shrink, then expand) for callers that
// cannot allocate device memory.
//
// Who that is: a host that swaps this library's kernels into an engine whose memory is fully claimed at
// start-up (pocket-engine sizes its pools once and never allocates inside Linear::forward), so a later
// cudaMalloc can simply fail, and plugin hosts that forbid their plugins to allocate after initialisation. They still own x, y, the tile words and the descriptor table;
// what they lack is a place for the f32 intermediate S. Here that intermediate lives in a file-scope
// device array of fixed size, so the entry point calls no cudaMalloc, cudaFree or any allocating routine.
//
// Limits and rules:
//   * nsplit * rows * lds * 4 bytes must fit PLORA_STATIC_SCRATCH_BYTES (8 MiB); larger calls are
//     rejected with PLORA_ERR_CAPACITY and nothing is launched.
//   * Every GPU that loads this library holds the 8 MiB array until the process exits.
//   * All calls on a device share the array and it keeps the previous call's contents. Nothing in it has
//     to start at zero: the shrink writes every element the expand reads (each token, each row of the
//     slot's stacked A, each K-split) before the expand runs, so no clearing is done. Two calls whose
//     kernels overlap on the GPU (different streams without ordering) race on it: order them.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) with that
//     device current; make that first call before any stream capture begins.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "../../include/plora.h"

typedef __nv_bfloat16 bf16;

#define PLORA_STATIC_SCRATCH_BYTES (8u << 20)

// In host code this name is only a stand-in for the symbol, never a device address: the address comes
// from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[PLORA_STATIC_SCRATCH_BYTES / 4];
// how many tiles the kernels refused since the library was loaded (see tile_ok); read by plora_static_bad_tiles
static __device__ unsigned int g_static_bad_tiles = 0;

namespace {

thread_local std::string g_static_err;
std::mutex g_setup_mutex;
float* g_scratch_ptr[64] = {nullptr};

int sfail(int code, const std::string& text) {
    g_static_err = text;
    return code;
}

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

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

// 16 values per lane -> 16 warp-wide sums; the caller's lane holds the sum of value (lane >> 1) & 15.
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

// The tile words and the descriptor come from the caller, unchecked by any grouping kernel: a tile is used only
// if its token rows lie inside [0, rows), it has 1..16 tokens, its slot is not negative and the slot's ranks fit
// the intermediate's row (lds floats). A refused tile is skipped by both kernels (y keeps its value for those
// tokens) and counted; nothing is read or written through its numbers.
__device__ __forceinline__ bool tile_ok(int t0, int cnt, int slot, int rows) {
    return t0 >= 0 && cnt >= 1 && cnt <= PLORA_TILE && t0 <= rows - cnt && slot >= 0;
}
__device__ __forceinline__ bool desc_ok(const plora_desc& d, int lds) {
    if (d.rank < 0 || d.rank > lds) return false;
#pragma unroll
    for (int p = 0; p < PLORA_MAX_PARTS; p++)
        if (d.r[p] < 0 || d.r_off[p] < 0 || d.r_off[p] + d.r[p] > d.rank || d.r[p] > lds / PLORA_MAX_PARTS || (d.r[p] & 7)) return false;
    return true;
}

// Shrink straight from the engine's tile words: grid (tiles, K-splits), 128 threads. Writes
// S[split][token][row] for every token of the tile and every row of the slot's stacked A.
__global__ void __launch_bounds__(128) plora_static_shrink_kernel(const bf16* __restrict__ X, int ldx, int K,
                                                                   const int* __restrict__ tiles,
                                                                   const plora_desc* __restrict__ table,
                                                                   float* __restrict__ S, size_t s_stride, int lds,
                                                                   int kchunk, int rows) {
    const int w = blockIdx.x;
    if (w >= tiles[0]) return;
    const int t0 = tiles[1 + 3 * w], cnt = tiles[2 + 3 * w], slot = tiles[3 + 3 * w];
    if (!tile_ok(t0, cnt, slot, rows)) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicAdd(&g_static_bad_tiles, 1u);
        return;
    }
    const plora_desc& d = table[slot];
    const int rank = d.rank;
    if (rank == 0) return;
    if (!desc_ok(d, lds)) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicAdd(&g_static_bad_tiles, 1u);
        return;
    }
    const bf16* A = reinterpret_cast<const bf16*>(d.a);
    const int k0 = blockIdx.y * kchunk, k1 = min(K, k0 + kchunk);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* Sout = S + (size_t)blockIdx.y * s_stride;
    for (int tp = 0; tp < cnt; tp += 4) {
        const int nt = min(4, cnt - tp);
        for (int n0 = warp * 4; n0 < rank; n0 += 16) {
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = 0.f;
            for (int k = k0 + lane * 8; k < k1; k += 256) {
                uint4 av[4], xv[4];
#pragma unroll
                for (int r = 0; r < 4; r++) av[r] = ldg16(A + (size_t)(n0 + r) * K + k);
#pragma unroll
                for (int t = 0; t < 4; t++) xv[t] = ldg16(X + (size_t)(t0 + tp + min(t, nt - 1)) * ldx + k);
                float xf[4][8];
#pragma unroll
                for (int t = 0; t < 4; t++) unpack8(xv[t], xf[t]);
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    float af[8];
                    unpack8(av[r], af);
#pragma unroll
                    for (int t = 0; t < 4; t++)
#pragma unroll
                        for (int e = 0; e < 8; e++) acc[r * 4 + t] = fmaf(xf[t][e], af[e], acc[r * 4 + t]);
                }
            }
            const float v = reduce16(acc, lane);
            if ((lane & 1) == 0) {
                const int i = lane >> 1, r = i >> 2, t = i & 3;
                if (t < nt) Sout[(size_t)(t0 + tp + t) * lds + n0 + r] = v;
            }
        }
    }
}

// Expand straight from the tile words: grid (tiles, ceil(max part rows / 256), parts), 128 threads, two
// adjacent output columns per thread; adds the K-split partials in split order.
__global__ void __launch_bounds__(128) plora_static_expand_kernel(const float* __restrict__ S, size_t s_stride,
                                                                   int lds, int nsplit, const int* __restrict__ tiles,
                                                                   const plora_desc* __restrict__ table, void* Y,
                                                                   int ldy, int f32_out, int n_rows) {
    extern __shared__ float ss[];  // [16][r]
    const int w = blockIdx.x;
    if (w >= tiles[0]) return;
    const int t0 = tiles[1 + 3 * w], cnt = tiles[2 + 3 * w], slot = tiles[3 + 3 * w];
    if (!tile_ok(t0, cnt, slot, n_rows)) return;  // counted by the shrink
    const plora_desc& d = table[slot];
    if (d.rank == 0 || !desc_ok(d, lds)) return;
    const int p = blockIdx.z, r = d.r[p];
    if (r == 0) return;
    // two columns per thread: a part's width and offset must be even (the registry enforces it for its own tables)
    const int rows = d.rows[p] & ~1, c0 = blockIdx.y * 256;
    if (c0 >= rows || (d.off[p] & 1) || d.off[p] < 0 || d.off[p] + d.rows[p] > ldy) return;
    const int r_off = d.r_off[p];
    for (int i = threadIdx.x; i < cnt * r; i += 128) {
        const int t = i / r, j = i - t * r;
        const float* sp = S + (size_t)(t0 + t) * lds + r_off + j;
        float acc = sp[0];
        for (int s = 1; s < nsplit; s++) acc += sp[(size_t)s * s_stride];
        ss[i] = acc;
    }
    __syncthreads();
    const int c = c0 + 2 * threadIdx.x;
    if (c >= rows) return;
    const bf16* b = reinterpret_cast<const bf16*>(d.b[p]) + (size_t)c * r;
    const int col = d.off[p] + c;
    for (int t = 0; t < cnt; t++) {
        float a0 = 0.f, a1 = 0.f;
        for (int j = 0; j < r; j += 8) {
            float f0[8], f1[8];
            unpack8(ldg16(b + j), f0);
            unpack8(ldg16(b + r + j), f1);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                a0 = fmaf(ss[t * r + j + e], f0[e], a0);
                a1 = fmaf(ss[t * r + j + e], f1[e], a1);
            }
        }
        const size_t at = (size_t)(t0 + t) * ldy + col;
        if (f32_out) {
            float2* py = reinterpret_cast<float2*>(reinterpret_cast<float*>(Y) + at);
            float2 v = *py;
            v.x += a0;
            v.y += a1;
            *py = v;
        } else {
            __nv_bfloat162* py = reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf16*>(Y) + at);
            const float2 v = __bfloat1622float2(*py);
            *py = __floats2bfloat162_rn(v.x + a0, v.y + a1);
        }
    }
}

// Once per device, with that device current: the device address of the static array.
int static_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return sfail(PLORA_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return sfail(PLORA_ERR_ARG, "device index out of range");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return sfail(PLORA_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return PLORA_OK;
}

}  // namespace

extern "C" {

uint64_t plora_static_scratch_bytes(void) { return PLORA_STATIC_SCRATCH_BYTES; }

const char* plora_static_error(void) { return g_static_err.c_str(); }

// Tiles refused on the current device since the library was loaded (a bad row range, token count, slot or
// descriptor). Waits for the device; allocates nothing. -1 on a CUDA error.
long long plora_static_bad_tiles(void) {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_static_bad_tiles, sizeof(v)) != cudaSuccess) return -1;
    return (long long)v;
}

// K-splits of the intermediate for a layer of `cols` inputs: a call needs splits * rows * lds * 4 bytes of scratch
int plora_static_splits(int cols) {
    if (cols <= 0) return 0;
    const int few = cols + 511 < 512 * 16 ? (cols + 511) / 512 : 16;
    const int want = (cols + 2047) / 2048 > few ? (cols + 2047) / 2048 : few;
    const int kchunk = ((cols + want - 1) / want + 255) / 256 * 256;
    return (cols + kchunk - 1) / kchunk;
}

int plora_site_apply_static(uint64_t x, int rows, int cols, uint64_t tiles, int max_tiles, uint64_t table, int parts,
                            int max_rows, int lds, uint64_t y, int ldy, int f32_out, void* stream) {
    if (!x || !tiles || !table || !y) return sfail(PLORA_ERR_ARG, "null device address");
    if ((x & 15) || cols <= 0 || (cols & 7)) return sfail(PLORA_ERR_ARG, "x must be 16-byte aligned and cols a multiple of 8");
    if ((y & (f32_out ? 7 : 3)) || (ldy & 1)) return sfail(PLORA_ERR_ARG, "y must be aligned to two elements and ldy even");
    if (rows < 0 || max_tiles < 0 || parts < 1 || parts > PLORA_MAX_PARTS || max_rows <= 0 || lds <= 0 || (lds & 63))
        return sfail(PLORA_ERR_ARG, "rows, max_tiles, parts, max_rows or lds out of range");
    // the same K-split rule the handle-based path fixes per layer: chunks of at least 512 inputs, at most 16
    // of them, but never wider than 2048
    const int few = cols + 511 < 512 * 16 ? (cols + 511) / 512 : 16;
    const int want = (cols + 2047) / 2048 > few ? (cols + 2047) / 2048 : few;
    const int kchunk = ((cols + want - 1) / want + 255) / 256 * 256;
    const int nsplit = (cols + kchunk - 1) / kchunk;
    const size_t need = (size_t)nsplit * (size_t)rows * (size_t)lds * 4;
    if (need > PLORA_STATIC_SCRATCH_BYTES)
        return sfail(PLORA_ERR_CAPACITY, "the f32 intermediate needs " + std::to_string(need) + " bytes; the static scratch holds " +
                                             std::to_string(PLORA_STATIC_SCRATCH_BYTES));
    if ((size_t)16 * (size_t)(lds / PLORA_MAX_PARTS) * 4 > 48 * 1024) return sfail(PLORA_ERR_CAPACITY, "rank over 768");
    const int ntiles = max_tiles < rows ? max_tiles : rows;
    if (ntiles == 0) return PLORA_OK;
    float* S = nullptr;
    int rc = static_scratch(&S);
    if (rc != PLORA_OK) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const size_t s_stride = (size_t)rows * (size_t)lds;
    plora_static_shrink_kernel<<<dim3((unsigned)ntiles, (unsigned)nsplit), 128, 0, st>>>(
        reinterpret_cast<const bf16*>(x), cols, cols, reinterpret_cast<const int*>(tiles),
        reinterpret_cast<const plora_desc*>(table), S, s_stride, lds, kchunk, rows);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return sfail(PLORA_ERR_CUDA, std::string("shrink: ") + cudaGetErrorString(e));
    const size_t smem = (size_t)16 * (size_t)(lds / PLORA_MAX_PARTS) * 4;
    plora_static_expand_kernel<<<dim3((unsigned)ntiles, (unsigned)((max_rows + 255) / 256), (unsigned)parts), 128, smem, st>>>(
        S, s_stride, lds, nsplit, reinterpret_cast<const int*>(tiles), reinterpret_cast<const plora_desc*>(table),
        reinterpret_cast<void*>(y), ldy, f32_out, rows);
    e = cudaGetLastError();
    if (e != cudaSuccess) return sfail(PLORA_ERR_CUDA, std::string("expand: ") + cudaGetErrorString(e));
    return PLORA_OK;
}

}  // extern "C"
