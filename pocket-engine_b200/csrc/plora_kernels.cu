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
#include "plora_device.cuh"

typedef __nv_bfloat16 bf16;


namespace {

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
// One launch record: gather work item w resolved against one layer's descriptor table, so that the kernels of
// that layer make one metadata fetch per block. `o` is the record's 16 uint4.
__device__ __forceinline__ void write_record(uint4* o, const int* segs, const SegLayout& lay, const plora_desc* table, int w,
                                             int cols, int pieces) {
    const uint4* work = reinterpret_cast<const uint4*>(segs + lay.work() + PLORA_WORK_WORDS * w);
    const uint4 head = work[0];  // slot, perm start, count, 0
    const int slot = (int)head.x;
    const uint4* d = reinterpret_cast<const uint4*>(table + slot);  // 112 bytes: a, b[4], rank, r, r_off, off, rows
    uint4 dv[7];
#pragma unroll
    for (int i = 0; i < 7; i++) dv[i] = d[i];
    // Desc: a | b0 b1 | b2 b3 | rank r0 r1 r2 | r3 ro0 ro1 ro2 | ro3 o0 o1 o2 | o3 rows0 rows1 rows2 | rows3 pad
    const uint32_t* dw = reinterpret_cast<const uint32_t*>(dv);
    o[0] = make_uint4(head.z, head.x, dw[10], (uint32_t)cols);  // cnt, slot, rank, cols
    o[1] = make_uint4(dw[0], dw[1], dw[2], dw[3]);              // a, b[0]
    o[2] = make_uint4(dw[4], dw[5], dw[6], dw[7]);              // b[1], b[2]
    o[3] = make_uint4(dw[8], dw[9], dw[11], dw[12]);            // b[3], r[0], r[1]
    o[4] = make_uint4(dw[13], dw[14], dw[15], dw[16]);          // r[2], r[3], r_off[0], r_off[1]
    o[5] = make_uint4(dw[17], dw[18], dw[19], dw[20]);          // r_off[2], r_off[3], off[0], off[1]
    o[6] = make_uint4(dw[21], dw[22], dw[23], dw[24]);          // off[2], off[3], rows[0], rows[1]
    // the slot's output columns over its targeted parts laid end to end, and the even share of them that
    // one block of the layer's cluster kernel expands
    uint32_t cat[PLORA_MAX_PARTS], ntot = 0;
#pragma unroll
    for (int p = 0; p < PLORA_MAX_PARTS; p++) {
        cat[p] = ntot;
        if ((int)dw[11 + p] > 0) ntot += dw[23 + p];
    }
    const uint32_t share = pieces > 0 ? (((ntot + pieces - 1) / pieces + 1) & ~1u) : 0u;
    o[7] = make_uint4(dw[25], dw[26], ntot, share);             // rows[2], rows[3], ntot, share
    o[8] = work[1];                                             // the token rows
    o[9] = work[2];
    o[10] = work[3];
    o[11] = work[4];
    o[12] = make_uint4(cat[0], cat[1], cat[2], cat[3]);
}

// ---------------------------------------------------------------------------------------------
// Regroup the tile words by slot. Runs = maximal ranges of contiguous tokens of one slot. Runs of at
// least lay.run_min tokens become tensor-core tiles; the rest are gathered by slot: perm lists their
// token rows ordered by (slot, position in the tile list), cut into work items of <= 16 tokens.
//
// The same block then writes the step's launch records: every gather work item resolved against every layer's
// descriptor table. The list of a layer ends with records whose cnt is 0.
__global__ void __launch_bounds__(1024) plora_meta_group_kernel(const int* __restrict__ tiles, int* __restrict__ segs,
                                                                 SegLayout lay, int* __restrict__ status,
                                                                 const plora_desc* __restrict__ tables,
                                                                 const int* __restrict__ site_cols, int n_sites,
                                                                 PloraRec* __restrict__ recs, int rec_cap) {
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
    for (int i = tid; i < lay.max_tokens; i += 1024) segs[lay.tslot() + i] = 0;
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
            for (int k = 0; k < len; k++) segs[lay.tslot() + start + k] = slot;
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
            if (at >= cap) break;  // tiles that overlap can add up to more rows than the step has: flagged below
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
        // Tiles that overlap one another pass the per-tile checks but name more token rows than the step has: the
        // regrouped rows would not fit their region. Such a list is refused as a whole.
        if (n_gather > lay.max_tokens || n_work > cap || n_mma > cap) bad = true;
        const bool over = n_gather > lay.max_tokens || n_work > cap || n_mma > cap;
        if (flag && !over) {
            segs[lay.act() + aidx] = s;
            segs[lay.seg_off() + aidx] = off;
            seg_base[s] = off;
            int* work = segs + lay.work();
            for (int q = 0; q < nw; q++) {
                int* wi = work + PLORA_WORK_WORDS * (woff + q);
                wi[0] = s;
                wi[1] = off + q * PLORA_WORK_TOKENS;
                wi[2] = min(PLORA_WORK_TOKENS, c - q * PLORA_WORK_TOKENS);
                wi[3] = 0;
            }
            cnt[s] = woff;  // from here on: the slot's first work item
        }
        if (tid == 0 && !over) segs[lay.seg_off() + n_act] = n_gather;
        if (over) n_act = n_gather = n_work = n_mma = n_runs = 0;
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

    // perm, and the same token rows inside the work items
    int* perm = segs + lay.perm();
    int* work = segs + lay.work();
    for (int r = tid; r < n_runs; r += 1024) {
        const int pos = run_pos[r];
        if (pos < 0) continue;
        const int start = run_start[r], len = run_len[r], slot = run_slot[r];
        const int rel0 = pos - seg_base[slot], w0 = cnt[slot];
        for (int k = 0; k < len; k++) {
            perm[pos + k] = start + k;
            const int rel = rel0 + k;
            work[PLORA_WORK_WORDS * (w0 + rel / PLORA_WORK_TOKENS) + 4 + rel % PLORA_WORK_TOKENS] = start + k;
        }
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
    // launch records (the barrier above made the work items, written by other threads of this block, visible)
    if (recs != nullptr) {
        const int nw = min(n_work, rec_cap - 1), end = min(rec_cap, nw + PLORA_REC_TERM);
        for (int i = tid; i < n_sites * end; i += 1024) {
            const int site = i / end, w = i - site * end;
            uint4* o = reinterpret_cast<uint4*>(recs + (size_t)site * (size_t)rec_cap + w);
            const int cols = site_cols[2 * site];
            if (w >= nw) o[0] = make_uint4(0u, 0u, 0u, (uint32_t)cols);
            else write_record(o, segs, lay, tables + (size_t)site * (size_t)(lay.max_slots + 1), w, cols, site_cols[2 * site + 1]);
        }
    }
}

// Shrink over gather work items. Grid (K-splits x row tiles, 1, work items); 128 threads. A work item is up
// to 16 tokens of one slot, described by one launch record. The block's rows of the slot's stacked A (one
// K-chunk wide) arrive in shared memory by bulk async copies issued before the dependency wait; the tokens'
// x chunks follow right after it. Each warp takes 4 of every 16 rows and 4 tokens at a time, its lanes 8
// inputs each per 256-wide step; sums cross the warp by shuffles. Every (token, row, split) is written
// exactly once.
__global__ void __launch_bounds__(128) plora_shrink_gather_kernel(const bf16* __restrict__ X, int ldx, int K,
                                                                   const PloraRec* __restrict__ recs, int rec_cap,
                                                                   float* __restrict__ S, size_t s_stride, int lds,
                                                                   int kchunk, int rps, int rt_max, int early, int early_x,
                                                                   int* __restrict__ status PLORA_BOUNDS_PARAM) {
    // early != 0: dependents are released at kernel start (every store of the path comes after a wait).
    // early_x != 0: the caller vouches that x is older than every kernel still in flight, so x is fetched and
    // the partial sums computed before the dependency wait; only the stores into S (which the expand before may
    // still be reading) come after it.
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ PloraRec srec;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (early) pdl_trigger();
    if (threadIdx.x == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_fence_init();
    }
    bool waited = false;
    uint32_t phase = 0;
    const int split = blockIdx.x / rt_max, rt = blockIdx.x - split * rt_max;
    const int row0 = rt * rps;
    const int k0 = split * kchunk, klen = min(kchunk, K - k0);
    const uint32_t kbytes = (uint32_t)klen * 2u;
    // the grid's z extent is capped: a block walks the work items z, z + gridDim.z, ...
    for (int w = blockIdx.z; w < rec_cap; w += gridDim.z) {
    if (threadIdx.x < 12) reinterpret_cast<uint4*>(&srec)[threadIdx.x] = __ldg(reinterpret_cast<const uint4*>(recs + w) + threadIdx.x);
    __syncthreads();
    const int cnt = srec.cnt, rank = srec.rank;
    if (cnt == 0) break;
#ifdef PLORA_BOUNDS
    if (!rec_in_bounds(srec, bnd, K)) {
        if (threadIdx.x == 0) atomicMax(status, PLORA_ERR_ARG);
        __syncthreads();
        continue;
    }
#endif
    if (row0 >= rank) {
        __syncthreads();
        continue;
    }
    const int rows = min(rps, rank - row0);
    unsigned char* As = dsm;
    unsigned char* Xs = dsm + (size_t)rps * kchunk * 2;
    if (warp == 0) {
        const bf16* A = reinterpret_cast<const bf16*>(srec.a) + (size_t)row0 * K + k0;
        if (lane == 0) mbar_expect_tx(&bars[0], (uint32_t)rows * kbytes);
        __syncwarp();
        for (int r = lane; r < rows; r += 32) bulk_g2s(As + (size_t)r * kbytes, A + (size_t)r * K, kbytes, &bars[0]);
    } else if (!waited && !early_x) {
        // hint only: the x lines this block will copy once the kernel before is done
        const int lines = (int)((kbytes + 127) / 128);
        for (int i = threadIdx.x - 32; i < cnt * lines; i += 96) {
            const int t = i / lines, l = i - t * lines;
            prefetch_l2(reinterpret_cast<const unsigned char*>(X + (size_t)srec.tok[t] * ldx + k0) + (size_t)l * 128);
        }
    }
    if (!early_x && !waited) {
        pdl_wait();
        if (!early) pdl_trigger();
        waited = true;
    }
    if (warp == 0) {
        if (lane == 0) mbar_expect_tx(&bars[1], (uint32_t)cnt * kbytes);
        __syncwarp();
        if (lane < cnt) bulk_g2s(Xs + (size_t)lane * kbytes, X + (size_t)srec.tok[lane] * ldx + k0, kbytes, &bars[1]);
    }
    if (!mbar_wait(&bars[0], phase, status)) return;
    if (!mbar_wait(&bars[1], phase, status)) return;
    phase ^= 1;
    float* Sout = S + (size_t)split * s_stride;
    float res[PLORA_WORK_TOKENS / 4];  // rows == 16: one 4-row group per warp, one value per token pass
#pragma unroll
    for (int tq = 0; tq < PLORA_WORK_TOKENS / 4; tq++) {
        const int tp = 4 * tq;
        res[tq] = 0.f;
        if (tp >= cnt) continue;
        const int nt = min(4, cnt - tp);
        {
            const int n0 = warp * 4;
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = 0.f;
            for (int k = lane * 8; k < klen; k += 256) {
                float xf[4][8];
#pragma unroll
                for (int t = 0; t < 4; t++) unpack8(lds16(Xs + (size_t)(tp + min(t, nt - 1)) * kbytes + k * 2), xf[t]);
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
            res[tq] = reduce16(acc, lane);
        }
    }
    if (!waited) {
        pdl_wait();
        if (!early) pdl_trigger();
        waited = true;
    }
    if ((lane & 1) == 0) {
        const int i = lane >> 1, r = i >> 2, t = i & 3;
#pragma unroll
        for (int tq = 0; tq < PLORA_WORK_TOKENS / 4; tq++)
            if (4 * tq + t < cnt) Sout[(size_t)srec.tok[4 * tq + t] * lds + row0 + warp * 4 + r] = res[tq];
    }
    __syncthreads();  // shared memory is reused by the next work item
    }
    if (!waited) pdl_exit_idle();
}

// Expand over gather work items. Grid (column blocks, parts, work items); 128 threads, two adjacent output
// columns each. The block's rows of B arrive in shared memory by one bulk async copy issued before the
// dependency wait, together with L2 prefetch hints for its y lines. After the wait, the work item's S rows
// (K-split partials, all in flight together, added in split order) go to shared memory while the y values are
// on their way; every thread then walks its two rows of B once per group of 4 tokens and writes y back.
#define EXP_SPAD 12  // floats per 8-wide piece of an S row in shared memory (conflict-free for rotated reads)

// PASSES: whether the tile buffer is smaller than a block's columns at the maximum rank. NH: column pairs per
// thread, half a block's width apart (2 for the 512-column blocks of wide layers: 128 threads instead of 256
// hold the block's registers, so more blocks, and more bytes in flight, share an SM).
template <bool PASSES, int NH>
__global__ void __launch_bounds__(256 / NH, 4 * NH) plora_expand_gather_kernel(const float* __restrict__ S, size_t s_stride,
                                                                      int lds, int nsplit,
                                                                      const PloraRec* __restrict__ recs, int rec_cap,
                                                                      void* Y, int ldy, int f32_out, int nc, int bs_bytes,
                                                                      int early, int* __restrict__ status PLORA_BOUNDS_PARAM) {
    // early != 0: dependents are released at kernel start. No value of y is bound before the dependency wait
    // (the kernel before, the layer's matrix multiply, may still be writing it): only L2 prefetch hints.
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ PloraRec srec;
    if (early) pdl_trigger();
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    bool waited = false;
    uint32_t phase = 0;
    const int esize = f32_out ? 4 : 2;
    // the grid's z extent is capped: a block walks the work items z, z + gridDim.z, ...
    for (int w = blockIdx.z; w < rec_cap; w += gridDim.z) {
    if (threadIdx.x < 12) reinterpret_cast<uint4*>(&srec)[threadIdx.x] = __ldg(reinterpret_cast<const uint4*>(recs + w) + threadIdx.x);
    __syncthreads();
    const int cnt = srec.cnt;
    if (cnt == 0) break;
#ifdef PLORA_BOUNDS
    if (!rec_in_bounds(srec, bnd, srec.cols)) {
        if (threadIdx.x == 0) atomicMax(status, PLORA_ERR_ARG);
        __syncthreads();
        continue;
    }
#endif
    const int p = blockIdx.y, r = srec.r[p];
    const int rows = srec.rows[p], c0 = blockIdx.x * nc;
    if (r == 0 || c0 >= rows) {
        __syncthreads();
        continue;
    }
    const int ncols_all = min(nc, rows - c0);
    // The tile buffer holds bs_bytes of B: all the block's columns for ranks up to bs_bytes / (2 nc), fewer
    // columns per pass (a multiple of 32) for higher ranks, so that a high maximum rank does not cost every
    // block, whatever its slot's rank, the shared memory that limits how many blocks share an SM.
    const int sub = PASSES ? min(nc, max(32, (bs_bytes / (2 * r)) & ~31)) : nc;
    int ncols = min(sub, ncols_all);
    unsigned char* Bs = dsm;
    float* ss = reinterpret_cast<float*>(dsm + bs_bytes);
    const bf16* Bp = reinterpret_cast<const bf16*>(srec.b[p]);
    if (threadIdx.x == 0) {
        const uint32_t bytes = (uint32_t)ncols * (uint32_t)r * 2u;
        mbar_expect_tx(&bar, bytes);
        bulk_g2s(Bs, Bp + (size_t)c0 * r, bytes, &bar);
    }
    const int r_off = srec.r_off[p];
    const int c = 2 * threadIdx.x;       // the thread's first column pair; pair h is h * HALF columns further
    const int HALF = 2 * blockDim.x;
    size_t ycol = (size_t)srec.off[p] + c0 + c;
    if (!waited) {
        // hints for the block's y lines, then the dependency wait
        const size_t len = (size_t)ncols_all * esize;
        const int lines = (int)((len + 127) / 128) + 1;
        for (int i = threadIdx.x; i < cnt * lines; i += blockDim.x) {
            const int t = i / lines, l = i - t * lines;
            const size_t start = ((size_t)srec.tok[t] * ldy + srec.off[p] + c0) * esize;
            const size_t at = (start & ~(size_t)127) + (size_t)l * 128;
            if (at < start + len) prefetch_l2(reinterpret_cast<const unsigned char*>(Y) + at);
        }
        pdl_wait();
        if (!early) pdl_trigger();
        waited = true;
    }
    // y of a group of 4 tokens, all of the thread's pairs
    float2 yv[4][NH];
    auto load_y = [&](int tg) {
#pragma unroll
        for (int h = 0; h < NH; h++) {
            if (c + h * HALF < ncols) {
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    if (tg + t < cnt) {
                        const size_t at = (size_t)srec.tok[tg + t] * ldy + ycol + h * HALF;
                        if (f32_out) yv[t][h] = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(Y) + at);
                        else yv[t][h] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const bf16*>(Y) + at));
                    }
                }
            }
        }
    };
    // y of the first token group: on its way before anything else is waited for
    load_y(0);
    const int P = r >> 3;  // 16-byte pieces per row of B
    for (int i = threadIdx.x; i < cnt * r; i += blockDim.x) {
        const int t = i / r, j = i - t * r;
        const float* sp = S + (size_t)srec.tok[t] * lds + r_off + j;
        float acc = 0.f;
        for (int s0 = 0; s0 < nsplit; s0 += 8) {
            float v[8];
#pragma unroll
            for (int s = 0; s < 8; s++) v[s] = s0 + s < nsplit ? __ldcg(sp + (size_t)(s0 + s) * s_stride) : 0.f;
#pragma unroll
            for (int s = 0; s < 8; s++)
                if (s0 + s < nsplit) acc = s0 + s == 0 ? v[s] : acc + v[s];
        }
        ss[t * P * EXP_SPAD + (j >> 3) * EXP_SPAD + (j & 7)] = acc;
    }
    __syncthreads();
    for (int cs = 0; cs < ncols_all; cs += sub) {
    if (cs > 0) {
        // the next columns of the block: the tile buffer is free once every thread is through the pass before
        __syncthreads();
        ncols = min(sub, ncols_all - cs);
        if (threadIdx.x == 0) {
            const uint32_t bytes = (uint32_t)ncols * (uint32_t)r * 2u;
            mbar_expect_tx(&bar, bytes);
            bulk_g2s(Bs, Bp + (size_t)(c0 + cs) * r, bytes, &bar);
        }
        ycol = (size_t)srec.off[p] + c0 + cs + c;
        load_y(0);
    }
    if (!mbar_wait(&bar, phase, status)) return;
    phase ^= 1;
    const int rot = (P >= 8 ? threadIdx.x : threadIdx.x >> 1) % P;
    const int sstride = P * EXP_SPAD;
    for (int tg = 0; tg < cnt; tg += 4) {
        if (tg > 0) load_y(tg);
#pragma unroll
        for (int h = 0; h < NH; h++) {
            if (c + h * HALF >= ncols) continue;
            const unsigned char* b0 = Bs + (size_t)(c + h * HALF) * r * 2;
            const unsigned char* b1 = b0 + (size_t)r * 2;
            float acc[4][2];
#pragma unroll
            for (int t = 0; t < 4; t++) acc[t][0] = acc[t][1] = 0.f;
            int jp = rot;
            for (int q = 0; q < P; q++) {
                float f0[8], f1[8];
                unpack8(lds16(b0 + jp * 16), f0);
                unpack8(lds16(b1 + jp * 16), f1);
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    if (tg + t < cnt) {
                        const float* sp = ss + (tg + t) * sstride + jp * EXP_SPAD;
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
                jp = jp + 1 == P ? 0 : jp + 1;
            }
#pragma unroll
            for (int t = 0; t < 4; t++) {
                if (tg + t < cnt) {
                    const size_t at = (size_t)srec.tok[tg + t] * ldy + ycol + h * HALF;
                    if (f32_out)
                        *reinterpret_cast<float2*>(reinterpret_cast<float*>(Y) + at) =
                            make_float2(yv[t][h].x + acc[t][0], yv[t][h].y + acc[t][1]);
                    else
                        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf16*>(Y) + at) =
                            __floats2bfloat162_rn(yv[t][h].x + acc[t][0], yv[t][h].y + acc[t][1]);
                }
            }
        }
    }
    }
    __syncthreads();  // shared memory is reused by the next work item
    }
    if (!waited) pdl_exit_idle();
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

// One-time function attributes (dynamic shared memory above 48 KB). Called from plora_create, never from
// the launch path, so launches stay legal inside a stream capture.
static int g_sms = 148;  // SMs of the device the kernels were set up for

cudaError_t plora_kernels_init(const SegLayout& lay) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(plora_meta_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)plora_meta_group_smem(lay) > 48 * 1024 ? (int)plora_meta_group_smem(lay)
                                                                                       : 48 * 1024);
    if (e != cudaSuccess) return e;
    // The few-token kernels overlap with their neighbours in the stream (programmatic dependent launch), and an SM's
    // split between L1 and shared memory is fixed while any block runs on it: all of them ask for the largest
    // split, so that a block of the next kernel finds room beside the blocks of this one.
    const void* fns[5] = {reinterpret_cast<const void*>(plora_shrink_gather_kernel),
                          reinterpret_cast<const void*>(plora_expand_gather_kernel<false, 1>),
                          reinterpret_cast<const void*>(plora_expand_gather_kernel<true, 1>),
                          reinterpret_cast<const void*>(plora_expand_gather_kernel<false, 2>),
                          reinterpret_cast<const void*>(plora_expand_gather_kernel<true, 2>)};
    for (int i = 0; i < 5 && e == cudaSuccess; i++) {
        e = cudaFuncSetAttribute(fns[i], cudaFuncAttributeMaxDynamicSharedMemorySize, i == 0 ? 136 * 1024 : 112 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fns[i], cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    }
    return e;
}

cudaError_t plora_launch_meta_group(const int32_t* tiles, int32_t* segs, SegLayout lay, int* status, const plora_desc* tables,
                                    const int32_t* site_cols, int n_sites, PloraRec* recs, int rec_cap, cudaStream_t st) {
    plora_meta_group_kernel<<<1, 1024, plora_meta_group_smem(lay), st>>>(tiles, segs, lay, status, tables, site_cols, n_sites, recs,
                                                                         rec_cap);
    return cudaGetLastError();
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

#define PLORA_GRID_Z_CAP 64  // blocks along the work-item axis; more work items are walked in a loop

// rows of A per block: 16 (one 4-row group per warp), so that a slot's rows spread over many blocks and
// each block's copies are issued and consumed quickly
int plora_shrink_rps(int kchunk) {
    (void)kchunk;
    return 16;
}

cudaError_t plora_launch_shrink(const void* x, int ldx, int K, const PloraRec* recs, int rec_cap, float* S,
                                size_t s_stride_elems, int lds, int kchunk, int nsplit, int work_cap, int max_rank_total,
                                const PloraBounds& bnd, int* status, bool pdl, bool early, bool early_x, cudaStream_t st) {
    (void)bnd;
    const int rps = plora_shrink_rps(kchunk);
    const int rt_max = (max_rank_total + rps - 1) / rps;
    dim3 grid((unsigned)(nsplit * rt_max), 1, (unsigned)(work_cap < PLORA_GRID_Z_CAP ? work_cap : PLORA_GRID_Z_CAP));
    const size_t smem = (size_t)(rps + PLORA_WORK_TOKENS) * (size_t)kchunk * 2;
    return launch_pdl(plora_shrink_gather_kernel, grid, dim3(128), smem, st, pdl, reinterpret_cast<const bf16*>(x), ldx,
                      K, recs, rec_cap, S, s_stride_elems, lds, kchunk, rps, rt_max, early ? 1 : 0, early_x ? 1 : 0, status PLORA_BOUNDS_ARG(bnd));
}

// output columns per block (two per thread): 512 for wide layers so the grid stays near one wave, 256
// otherwise, fewer when a row of B is so long that the block's rows would pass 64 KB of shared memory
int plora_expand_nc(int max_rank, int max_rows) {
    int nc = max_rows >= 8192 ? 512 : 256;
    while (nc > 32 && nc * max_rank * 2 > 64 * 1024) nc >>= 1;
    return nc;
}

cudaError_t plora_launch_expand(const float* S, size_t s_stride_elems, int lds, int nsplit, const PloraRec* recs,
                                int rec_cap, void* y, int ldy, int f32_out, int parts, int max_rows, int work_cap,
                                const PloraBounds& bnd, int* status, bool pdl, bool early, cudaStream_t st) {
    (void)bnd;
    const int max_rank = lds / PLORA_MAX_PARTS;
    const int nc = plora_expand_nc(max_rank, max_rows);
    // tile buffer: all of a block's columns at the maximum rank, up to 32 KB; blocks of higher-rank slots take
    // their columns in passes
    const int bs_bytes = nc * max_rank * 2 < 32 * 1024 ? nc * max_rank * 2 : 32 * 1024;
    dim3 grid((unsigned)((max_rows + nc - 1) / nc), (unsigned)parts,
              (unsigned)(work_cap < PLORA_GRID_Z_CAP ? work_cap : PLORA_GRID_Z_CAP));
    const size_t smem = (size_t)bs_bytes + (size_t)PLORA_WORK_TOKENS * (size_t)(max_rank / 8) * EXP_SPAD * sizeof(float);
    // 512-column blocks take two column pairs per thread (128 threads instead of 256) where that makes the whole
    // launch resident at once (8 such blocks of 64 registers per thread share an SM, shared memory permitting):
    // a launch this small is a chain of dependent fetches per block, and a second wave of blocks pays it again.
    // Larger launches are bound by their arithmetic and keep one pair per thread.
    const bool passes = bs_bytes < nc * max_rank * 2;
    int per_sm = (int)((size_t)(227 * 1024) / (smem + 1024));
    if (per_sm > 8) per_sm = 8;
    const int nh = nc >= 512 && (long long)grid.x * grid.y * grid.z <= (long long)per_sm * g_sms ? 2 : 1;
    const dim3 block((unsigned)(nc / (2 * nh)));
#define PLORA_EXPAND_ARGS S, s_stride_elems, lds, nsplit, recs, rec_cap, y, ldy, f32_out, nc, bs_bytes, early ? 1 : 0, status PLORA_BOUNDS_ARG(bnd)
    if (nh == 2)
        return passes ? launch_pdl(plora_expand_gather_kernel<true, 2>, grid, block, smem, st, pdl, PLORA_EXPAND_ARGS)
                      : launch_pdl(plora_expand_gather_kernel<false, 2>, grid, block, smem, st, pdl, PLORA_EXPAND_ARGS);
    return passes ? launch_pdl(plora_expand_gather_kernel<true, 1>, grid, block, smem, st, pdl, PLORA_EXPAND_ARGS)
                  : launch_pdl(plora_expand_gather_kernel<false, 1>, grid, block, smem, st, pdl, PLORA_EXPAND_ARGS);
#undef PLORA_EXPAND_ARGS
}
