// sm_100a kernels of the adapter path and their launchers.
//
//   plora_meta_tiles_kernel  cu[], seq_slot[] -> the engine's tile words (src/sched.rs:1096-1104), on the device
//   plora_meta_group_kernel  tile words -> tokens regrouped by slot (gather work items) and long runs cut
//                            into tensor-core tiles; stable, so results do not depend on scheduling
//   plora_shrink_gather      S_split[t, :] = x[t, k-chunk] . A_slot[:, k-chunk]^T   (replaces lora.cuh:23-67)
//   plora_expand_gather      y[t, off_p + n] += sum_j S[t, r_off_p + j] B_p[n, j]   (replaces lora.cuh:74-126)
//
// The shrink writes one partial per K-split instead of accumulating with float atomics; the expand adds
// the partials in split order, so S needs no zeroing and the result is reproducible bit for bit.
#include <cuda_bf16.h>

#include "plora_internal.h"

typedef __nv_bfloat16 bf16;

namespace {

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

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

// Exclusive scan of one int per thread over a block of 1024 threads. `sh` holds 33 ints.
__device__ __forceinline__ int block_scan_excl(int v, int& total, int* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    if (lane == 31) sh[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int t = sh[lane], ti = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int u = __shfl_up_sync(0xffffffffu, ti, o);
            if (lane >= o) ti += u;
        }
        sh[lane] = ti - t;
        if (lane == 31) sh[32] = ti;
    }
    __syncthreads();
    const int r = incl - v + sh[warp];
    total = sh[32];
    __syncthreads();
    return r;
}

// ---------------------------------------------------------------------------------------------
// Tile words from the step's sequences: for each sequence in order with a slot, chunks of 16 tokens
// (start, len, slot); word 0 is the count. One block of 1024 threads.
__global__ void __launch_bounds__(1024) plora_meta_tiles_kernel(const int* __restrict__ cu,
                                                                 const int* __restrict__ seq_slot, int n_seqs,
                                                                 int* __restrict__ tiles, int cap_tiles,
                                                                 int* __restrict__ status) {
    __shared__ int sh[33];
    __shared__ int s_first[1024], s_start[1024], s_n[1024], s_slot[1024];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int carry = 0;
    for (int base = 0; base < n_seqs; base += 1024) {
        const int i = base + tid;
        int start = 0, n = 0, slot = 0, nt = 0;
        if (i < n_seqs) {
            start = cu[i];
            n = cu[i + 1] - start;
            slot = seq_slot[i];
            if (n < 0) n = 0;
            nt = slot != 0 ? (n + PLORA_TILE - 1) / PLORA_TILE : 0;
        }
        int total;
        const int excl = block_scan_excl(nt, total, sh);
        s_first[tid] = carry + excl;
        s_start[tid] = start;
        s_n[tid] = n;
        s_slot[tid] = slot;
        __syncthreads();
        const int here = min(1024, n_seqs - base);
        for (int q = warp; q < here; q += 32) {
            const int qs = s_slot[q];
            if (qs == 0) continue;
            const int qn = s_n[q], q0 = s_start[q], qf = s_first[q];
            const int qt = (qn + PLORA_TILE - 1) / PLORA_TILE;
            for (int k = lane; k < qt; k += 32) {
                const int idx = qf + k;
                if (idx < cap_tiles) {
                    tiles[1 + 3 * idx] = q0 + k * PLORA_TILE;
                    tiles[2 + 3 * idx] = min(qn - k * PLORA_TILE, PLORA_TILE);
                    tiles[3 + 3 * idx] = qs;
                }
            }
        }
        carry += total;
        __syncthreads();
    }
    if (tid == 0) {
        if (carry > cap_tiles) {
            tiles[0] = 0;
            atomicMax(status, PLORA_ERR_CAPACITY);
        } else {
            tiles[0] = carry;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Regroup the tile words by slot. Runs = maximal ranges of contiguous tokens of one slot. Runs of at
// least lay.run_min tokens become tensor-core tiles; the rest are gathered by slot: perm lists their
// token rows ordered by (slot, position in the tile list), cut into work items of <= 16 tokens.
__global__ void __launch_bounds__(1024) plora_meta_group_kernel(const int* __restrict__ tiles, int* __restrict__ segs,
                                                                 SegLayout lay, int* __restrict__ status) {
    extern __shared__ int sm[];
    __shared__ int sh[33];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cap = lay.cap_tiles, S1 = lay.max_slots + 1;
    int* run_start = sm;
    int* run_len = run_start + cap;
    int* run_slot = run_len + cap;
    int* run_pos = run_slot + cap;
    int* cnt = run_pos + cap;
    int* seg_base = cnt + S1;
    int* fill = seg_base + S1;
    int* whist = fill + S1;  // [32][S1]

    int n_tiles = tiles[0];
    bool bad = false;
    if (n_tiles < 0 || n_tiles > cap) {
        n_tiles = 0;
        bad = true;
    }
    for (int i = tid; i < n_tiles; i += 1024) run_len[i] = 0;
    for (int i = tid; i < S1; i += 1024) {
        cnt[i] = 0;
        fill[i] = 0;
        seg_base[i] = 0;
    }
    __syncthreads();

    // runs
    int n_runs = 0;
    for (int base = 0; base < n_tiles; base += 1024) {
        const int i = base + tid;
        int head = 0, start = 0, len = 0, slot = 0;
        if (i < n_tiles) {
            start = tiles[1 + 3 * i];
            len = tiles[2 + 3 * i];
            slot = tiles[3 + 3 * i];
            if (slot < 0 || slot > lay.max_slots || len < 1 || len > PLORA_TILE || start < 0 ||
                start + len > lay.max_tokens) {
                bad = true;
                slot = 0;
                len = 0;
                start = 0;
            }
            if (i == 0) head = 1;
            else {
                const int ps = tiles[1 + 3 * (i - 1)], pl = tiles[2 + 3 * (i - 1)], pslot = tiles[3 + 3 * (i - 1)];
                head = !(pslot == slot && ps + pl == start);
            }
        }
        int total;
        const int excl = block_scan_excl(head, total, sh);
        const int rid = n_runs + excl + head - 1;
        if (i < n_tiles) {
            if (head) {
                run_start[rid] = start;
                run_slot[rid] = slot;
            }
            atomicAdd(&run_len[rid], len);
        }
        n_runs += total;
        __syncthreads();
    }

    // classify runs; tensor-core tiles
    int n_mma = 0;
    for (int base = 0; base < n_runs; base += 1024) {
        const int r = base + tid;
        int nm = 0, len = 0, slot = 0, start = 0;
        if (r < n_runs) {
            len = run_len[r];
            slot = run_slot[r];
            start = run_start[r];
            if (slot == 0 || len == 0) run_pos[r] = -1;
            else if (len >= lay.run_min) {
                nm = (len + PLORA_MMA_TOKENS - 1) / PLORA_MMA_TOKENS;
                run_pos[r] = -1;
            } else {
                run_pos[r] = -2;
                atomicAdd(&cnt[slot], len);
            }
        }
        int total;
        const int excl = block_scan_excl(nm, total, sh);
        int* mma = segs + lay.mma();
        for (int q = 0; q < nm; q++) {
            const int at = n_mma + excl + q;
            mma[3 * at] = start + q * PLORA_MMA_TOKENS;
            mma[3 * at + 1] = min(PLORA_MMA_TOKENS, len - q * PLORA_MMA_TOKENS);
            mma[3 * at + 2] = slot;
        }
        n_mma += total;
    }
    __syncthreads();

    // slots with gather tokens, ascending; their offsets into perm; work items
    int n_act, n_gather, n_work;
    {
        const int s = tid;
        const int c = (s >= 1 && s < S1) ? cnt[s] : 0;
        const int flag = c > 0;
        const int nw = (c + PLORA_WORK_TOKENS - 1) / PLORA_WORK_TOKENS;
        const int aidx = block_scan_excl(flag, n_act, sh);
        const int off = block_scan_excl(c, n_gather, sh);
        const int woff = block_scan_excl(nw, n_work, sh);
        if (flag) {
            segs[lay.act() + aidx] = s;
            segs[lay.seg_off() + aidx] = off;
            seg_base[s] = off;
            int* work = segs + lay.work();
            for (int q = 0; q < nw; q++) {
                work[3 * (woff + q)] = s;
                work[3 * (woff + q) + 1] = off + q * PLORA_WORK_TOKENS;
                work[3 * (woff + q) + 2] = min(PLORA_WORK_TOKENS, c - q * PLORA_WORK_TOKENS);
            }
        }
        if (tid == 0) segs[lay.seg_off() + n_act] = n_gather;
    }
    __syncthreads();

    // stable position of every gather run inside its slot's segment
    for (int base = 0; base < n_runs; base += 1024) {
        const int r = base + tid;
        int key = 0, w = 0;
        if (r < n_runs && run_pos[r] == -2) {
            key = run_slot[r];
            w = run_len[r];
        }
        for (int i = tid; i < 32 * S1; i += 1024) whist[i] = 0;
        __syncthreads();
        int sum = 0;
        bool last = true;
#pragma unroll 8
        for (int j = 0; j < 32; j++) {
            const int wj = __shfl_sync(0xffffffffu, w, j);
            const int kj = __shfl_sync(0xffffffffu, key, j);
            if (kj == key) {
                if (j < lane) sum += wj;
                if (j > lane) last = false;
            }
        }
        if (key != 0 && last) whist[warp * S1 + key] = sum + w;
        __syncthreads();
        if (key != 0) {
            int pre = 0;
            for (int q = 0; q < warp; q++) pre += whist[q * S1 + key];
            run_pos[r] = seg_base[key] + fill[key] + pre + sum;
        }
        __syncthreads();
        for (int s = tid; s < S1; s += 1024) {
            int tot = 0;
            for (int q = 0; q < 32; q++) tot += whist[q * S1 + s];
            fill[s] += tot;
        }
        __syncthreads();
    }

    // perm
    int* perm = segs + lay.perm();
    for (int r = tid; r < n_runs; r += 1024) {
        const int pos = run_pos[r];
        if (pos < 0) continue;
        const int start = run_start[r], len = run_len[r];
        for (int k = 0; k < len; k++) perm[pos + k] = start + k;
    }
    const int any_bad = __syncthreads_or(bad);
    if (any_bad && tid == 0) atomicMax(status, PLORA_ERR_ARG);
    if (tid == 0) {
        segs[SEG_N_ACT] = n_act;
        segs[SEG_N_WORK] = n_work;
        segs[SEG_N_MMA] = n_mma;
        segs[SEG_N_GATHER] = n_gather;
        segs[SEG_N_TILES] = n_tiles;
        segs[SEG_STATUS] = any_bad ? PLORA_ERR_ARG : 0;
    }
}

// ---------------------------------------------------------------------------------------------
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

// Shrink over gather work items. Grid (work items, K-splits); 128 threads. A work item is up to 16 tokens
// of one slot; each warp takes 4 of every 16 rows of the slot's stacked A and 4 tokens at a time, its
// lanes 8 inputs each per 256-wide step; sums cross the warp by shuffles. Every (token, row, split) is
// written exactly once.
__global__ void __launch_bounds__(128) plora_shrink_gather_kernel(const bf16* __restrict__ X, int ldx, int K,
                                                                   const int* __restrict__ segs, SegLayout lay,
                                                                   const plora_desc* __restrict__ table,
                                                                   float* __restrict__ S, size_t s_stride, int lds,
                                                                   int kchunk) {
    const int w = blockIdx.x;
    if (w >= segs[SEG_N_WORK]) return;
    const int* work = segs + lay.work() + 3 * w;
    const int slot = work[0], p0 = work[1], cnt = work[2];
    const plora_desc& d = table[slot];
    const int rank = d.rank;
    if (rank == 0) return;
    const bf16* A = reinterpret_cast<const bf16*>(d.a);
    const int k0 = blockIdx.y * kchunk, k1 = min(K, k0 + kchunk);
    const int* perm = segs + lay.perm() + p0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* Sout = S + (size_t)blockIdx.y * s_stride;
    for (int tp = 0; tp < cnt; tp += 4) {
        const int nt = min(4, cnt - tp);
        int tok[4];
#pragma unroll
        for (int t = 0; t < 4; t++) tok[t] = perm[tp + min(t, nt - 1)];
        for (int n0 = warp * 4; n0 < rank; n0 += 16) {
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = 0.f;
            for (int k = k0 + lane * 8; k < k1; k += 256) {
                uint4 av[4], xv[4];
#pragma unroll
                for (int r = 0; r < 4; r++) av[r] = ldg16(A + (size_t)(n0 + r) * K + k);
#pragma unroll
                for (int t = 0; t < 4; t++) xv[t] = ldg16(X + (size_t)tok[t] * ldx + k);
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
                if (t < nt) Sout[(size_t)tok[t] * lds + n0 + r] = v;
            }
        }
    }
}

// Expand over gather work items. Grid (work items, ceil(max part rows / 256), parts); 128 threads, two
// adjacent output columns each. The work item's S rows (partials added in split order) sit in shared
// memory; every thread streams its two rows of B once and updates y for each token.
template <int TOKS>
__device__ __forceinline__ void expand_body(const float* ss, const int* stok, int cnt, int r, const bf16* b, void* Y,
                                            int ldy, int col, int f32_out) {
    float acc[TOKS][2];
#pragma unroll
    for (int t = 0; t < TOKS; t++) acc[t][0] = acc[t][1] = 0.f;
    for (int j = 0; j < r; j += 8) {
        float f0[8], f1[8];
        unpack8(ldg16(b + j), f0);
        unpack8(ldg16(b + r + j), f1);
#pragma unroll
        for (int t = 0; t < TOKS; t++) {
            if (t < cnt) {
                const float4 s0 = *reinterpret_cast<const float4*>(ss + t * r + j);
                const float4 s1 = *reinterpret_cast<const float4*>(ss + t * r + j + 4);
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
    for (int t = 0; t < TOKS; t++) {
        if (t < cnt) {
            const size_t at = (size_t)stok[t] * ldy + col;
            if (f32_out) {
                float2* p = reinterpret_cast<float2*>(reinterpret_cast<float*>(Y) + at);
                float2 v = *p;
                v.x += acc[t][0];
                v.y += acc[t][1];
                *p = v;
            } else {
                __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf16*>(Y) + at);
                const float2 v = __bfloat1622float2(*p);
                *p = __floats2bfloat162_rn(v.x + acc[t][0], v.y + acc[t][1]);
            }
        }
    }
}

__global__ void __launch_bounds__(128) plora_expand_gather_kernel(const float* __restrict__ S, size_t s_stride,
                                                                   int lds, int nsplit, const int* __restrict__ segs,
                                                                   SegLayout lay,
                                                                   const plora_desc* __restrict__ table, void* Y,
                                                                   int ldy, int f32_out) {
    extern __shared__ float ss[];  // [16][r]
    __shared__ int stok[PLORA_WORK_TOKENS];
    const int w = blockIdx.x;
    if (w >= segs[SEG_N_WORK]) return;
    const int* work = segs + lay.work() + 3 * w;
    const int slot = work[0], p0 = work[1], cnt = work[2];
    const plora_desc& d = table[slot];
    const int p = blockIdx.z, r = d.r[p];
    if (r == 0) return;
    const int rows = d.rows[p], c0 = blockIdx.y * 256;
    if (c0 >= rows) return;
    const int* perm = segs + lay.perm() + p0;
    if (threadIdx.x < cnt) stok[threadIdx.x] = perm[threadIdx.x];
    const int r_off = d.r_off[p];
    for (int i = threadIdx.x; i < cnt * r; i += 128) {
        const int t = i / r, j = i - t * r;
        const float* sp = S + (size_t)perm[t] * lds + r_off + j;
        float acc = sp[0];
        for (int s = 1; s < nsplit; s++) acc += sp[(size_t)s * s_stride];
        ss[i] = acc;
    }
    __syncthreads();
    const int c = c0 + 2 * threadIdx.x;
    if (c >= rows) return;
    const bf16* b = reinterpret_cast<const bf16*>(d.b[p]) + (size_t)c * r;
    const int col = d.off[p] + c;
    if (cnt <= 4) expand_body<4>(ss, stok, cnt, r, b, Y, ldy, col, f32_out);
    else expand_body<PLORA_WORK_TOKENS>(ss, stok, cnt, r, b, Y, ldy, col, f32_out);
}

}  // namespace

// ---------------------------------------------------------------------------------------------

cudaError_t plora_launch_meta_tiles(const int32_t* cu, const int32_t* seq_slot, int n_seqs, int32_t* tiles,
                                    int cap_tiles, int* status, cudaStream_t st) {
    plora_meta_tiles_kernel<<<1, 1024, 0, st>>>(cu, seq_slot, n_seqs, tiles, cap_tiles, status);
    return cudaGetLastError();
}

size_t plora_meta_group_smem(const SegLayout& lay) {
    return (size_t)(4 * lay.cap_tiles + 3 * (lay.max_slots + 1) + 32 * (lay.max_slots + 1)) * sizeof(int);
}

cudaError_t plora_launch_meta_group(const int32_t* tiles, int32_t* segs, SegLayout lay, int* status,
                                    cudaStream_t st) {
    const size_t smem = plora_meta_group_smem(lay);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(plora_meta_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    plora_meta_group_kernel<<<1, 1024, smem, st>>>(tiles, segs, lay, status);
    return cudaGetLastError();
}

cudaError_t plora_launch_shrink(const void* x, int ldx, int K, const int32_t* segs, SegLayout lay,
                                const plora_desc* table, float* S, size_t s_stride_elems, int lds, int kchunk,
                                int nsplit, int work_cap, int max_rank_total, int* status, cudaStream_t st) {
    (void)max_rank_total;
    (void)status;
    dim3 grid((unsigned)work_cap, (unsigned)nsplit, 1);
    plora_shrink_gather_kernel<<<grid, 128, 0, st>>>(reinterpret_cast<const bf16*>(x), ldx, K, segs, lay, table, S,
                                                     s_stride_elems, lds, kchunk);
    return cudaGetLastError();
}

cudaError_t plora_launch_expand(const float* S, size_t s_stride_elems, int lds, int nsplit, const int32_t* segs,
                                SegLayout lay, const plora_desc* table, void* y, int ldy, int f32_out, int parts,
                                int max_rows, int work_cap, int* status, cudaStream_t st) {
    (void)status;
    dim3 grid((unsigned)work_cap, (unsigned)((max_rows + 255) / 256), (unsigned)parts);
    const size_t smem = (size_t)PLORA_WORK_TOKENS * (size_t)(lds / PLORA_MAX_PARTS) * sizeof(float);
    plora_expand_gather_kernel<<<grid, 128, smem, st>>>(S, s_stride_elems, lds, nsplit, segs, lay, table, y, ldy,
                                                        f32_out);
    return cudaGetLastError();
}
