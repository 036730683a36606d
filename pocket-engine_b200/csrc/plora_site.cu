// One kernel per layer for the few-token work items: a thread-block cluster of 8 blocks takes one work item (up
// to 16 tokens of one slot, 8 at a time) and one group of its output columns. Block q of the cluster shrinks over the q-th
// eighth of the input features; the partial sums meet through distributed shared memory (no trip through global
// memory, no second launch); every block then expands its eighth of the cluster's columns. Replaces the
// lora_shrink + lora_expand pair of src/kernels/lora.cuh:23-126 when x and y are both ready at the call (after
// the layer's own matrix multiply).
//
// Order of events in a block, chosen so that nothing that can be known early waits for anything:
//   1. (when the caller vouched for x) the next kernel of the stream is released at once;
//   2. one fetch of the work item's launch record (descriptor and token rows, written once per step);
//   3. bulk async copies of the block's rows of A and of its share of B into shared memory, L2 prefetch hints
//      for the x and y lines it will touch (and, when asked for, an L2 prefetch of the same work item's slabs of
//      the next layer);
//   4. the dependency wait (the kernel before, typically the layer's matrix multiply, wrote y);
//   5. x into shared memory, shrink, release of the next kernel of the stream (its prologue, steps 2 and 3, then
//      overlaps this kernel's exchange and expand), exchange, expand, y read-modify-write.
// Nothing before step 4 binds a value of x or y, unless the caller vouched for x (early_x). The release point was
// measured: released at kernel start, the next layer's blocks take the places that this layer's own late clusters
// need (a B200 holds about 33 clusters of this kernel, two neighbouring layers can need 48) and sit in their wait.
//
// Arithmetic: tiles of the warp-level tensor-core instruction (m16n8k16, bf16 in, f32 accumulate), the shape the
// engine's own kernels use for their 16-token tiles; here a tile carries 8 tokens, and in the expand its other 8
// rows carry a second term of S (plora_tiles.cuh). On the CUDA cores the step is bound by
// instruction issue (one conversion per bf16 element plus one multiply-add per token), not by memory; a 128-row
// tcgen05 tile would spend 1/8 or less of its rows on a work item. The f32 intermediate enters the expand as
// three bf16 terms (high, middle, low part), whose products with bf16 B are exact in f32, so no precision is
// given up against an f32 multiply-add chain.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "plora_internal.h"
#include "plora_device.cuh"
#include "plora_tiles.cuh"

#define SITE_CLUSTER 8
#define SITE_THREADS 256
#define SITE_WARPS PLORA_TILE_WARPS
#define SITE_TOK 8  // tokens per pass over a work item

namespace {

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// a float at the same shared-memory offset in block `rank` of the cluster
__device__ __forceinline__ float ld_peer_f32(const float* p, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}

struct SiteShape {
    int kchunk;    // input features per block of the cluster (a multiple of 8)
    int kb_pad;    // bytes between rows of the A and x tiles in shared memory (an odd number of 16-byte pieces)
    int rmax;      // floats per partial S row in shared memory (parts * max_rank)
    int sp_pad;    // bytes between rows of a bf16 plane of the summed S
    int aw_bytes;  // shared-memory bytes for the block's A rows, reused for the warps' partial sums
    int g_rows;    // rows of A per group (64, or all of them when there are fewer)
    int g_stride;  // bytes between groups: room for g_rows rows of A and for the 8 warps' partials of those rows
    int x_bytes;   // ... for the tokens' x chunks
    int b_bytes;   // ... for the block's share of B
    int nsub;      // column groups per work item (grid y): each is one cluster
};

// this block's share [lo, hi) of each part's output columns, and where its rows of B start in shared memory
struct Share {
    int lo[PLORA_MAX_PARTS], hi[PLORA_MAX_PARTS], boff[PLORA_MAX_PARTS];
};

// The slot's output columns, over the targeted parts laid end to end (rec.cat, rec.ntot), are cut into even shares of
// rec.share columns, one per block of the cluster kernel. Run by lanes 0..3 of one warp, lane p for part p.
__device__ __forceinline__ void column_share(const PloraRec& rec, int piece, int p, Share& s) {
    const int c_lo = min(rec.ntot, piece * rec.share), c_hi = min(rec.ntot, c_lo + rec.share);
    const int lo = max(c_lo, rec.cat[p]) - rec.cat[p];
    int hi = rec.r[p] > 0 ? min(c_hi, rec.cat[p] + rec.rows[p]) - rec.cat[p] : 0;
    hi = hi > lo ? hi : lo;
    const int bytes = (hi - lo) * rec.r[p] * 2;
    // where the part's rows of B start in shared memory: the bytes of the parts before it
    int off = 0;
#pragma unroll
    for (int q = 0; q < PLORA_MAX_PARTS - 1; q++) {
        const int b = __shfl_sync(0xfu, bytes, q);
        if (q < p) off += b;
    }
    s.lo[p] = lo;
    s.hi[p] = hi;
    s.boff[p] = off;
}

// L2 prefetch of this block's eighth of `bytes` at `base` (both multiples of 16), 32 KB per request, one warp
__device__ __forceinline__ void prefetch_eighth(uint64_t base, uint64_t bytes, uint32_t crank, int lane) {
    const uint64_t per = ((bytes / SITE_CLUSTER) + 15) & ~(uint64_t)15;
    const uint64_t lo = min(bytes, per * crank), hi = min(bytes, lo + per);
    for (uint64_t o = lo + (uint64_t)lane * 32768; o < hi; o += 32 * 32768) {
        const uint32_t n = (uint32_t)min((uint64_t)32768, hi - o) & ~15u;
        if (n) bulk_prefetch_l2(reinterpret_cast<const unsigned char*>(base) + o, n);
    }
}

// remote arrival on the same barrier in block `rank` of the cluster, releasing this thread's (and, through the
// block barrier before it, the block's) shared-memory writes to the cluster
__device__ __forceinline__ void mbar_arrive_peer(uint64_t* bar, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(bar)), "r"(rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(a) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, int* status) {
    for (int i = 0; i < (1 << 20); i++)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    atomicMax(status, PLORA_ERR_TIMEOUT);
    return false;
}
// "my reads of your shared memory are done": no memory ordering is asked of the arrival itself
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }

// The shrink's inner loop for one warp: n 16-wide steps, SITE_WARPS steps apart, over PAIRS pairs of 8-row tiles of A
template <int PAIRS>
__device__ __forceinline__ void shrink_steps(float (&acc)[8][4], uint32_t xs_w, uint32_t as_w, uint32_t kb_pad, int n) {
#pragma unroll 2
    for (int i = 0; i < n; i++) {
        uint32_t xa[4];
        ldmatrix_x4(xa, xs_w + (uint32_t)i * (SITE_WARPS * 32u));
#pragma unroll
        for (int pr = 0; pr < PAIRS; pr++) {
            uint32_t bb[4];
            ldmatrix_x4(bb, as_w + (uint32_t)(pr * 16) * kb_pad + (uint32_t)i * (SITE_WARPS * 32u));
            mma_16816(acc[2 * pr], xa, bb[0], bb[1]);
            mma_16816(acc[2 * pr + 1], xa, bb[2], bb[3]);
        }
    }
}

template <bool F32>
__global__ void __cluster_dims__(SITE_CLUSTER, 1, 1) __launch_bounds__(SITE_THREADS, 2)
    plora_site_gather_kernel(const bf16* __restrict__ X, int ldx, int K, const PloraRec* __restrict__ recs, int rec_cap,
                             const PloraRec* __restrict__ next_recs, void* Y, int ldy, SiteShape sh, int mode,
                             int* __restrict__ status PLORA_BOUNDS_PARAM) {
    extern __shared__ __align__(128) unsigned char dsm[];
    __shared__ __align__(8) uint64_t bars[4];  // A rows, x chunks, B rows, the cluster's partials
    __shared__ PloraRec srec;
    __shared__ Share sshare;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t crank = cluster_rank();
    // A rows in groups of g_rows: group q at q * g_stride, its rows kb_pad apart. Once a group's rows are used up,
    // the warps' partial sums of those rows [warp][16][g_rows] take their place.
    unsigned char* As = dsm;
    unsigned char* Xs = As + sh.aw_bytes;                   // x chunks [8][kb_pad]
    unsigned char* Bs = Xs + sh.x_bytes;                    // this block's rows of B, part after part
    float* Sp = reinterpret_cast<float*>(Bs + sh.b_bytes);  // this block's partial S [16][rmax]
    // the summed S as three bf16 planes [16][sp_pad] (high, middle, low term) and a fourth plane that stays zero
    unsigned char* S3 = reinterpret_cast<unsigned char*>(Sp + PLORA_WORK_TOKENS * sh.rmax);
    const uint32_t plane_bytes = PLORA_WORK_TOKENS * (uint32_t)sh.sp_pad;
    for (uint32_t i = tid * 16u; i < plane_bytes; i += SITE_THREADS * 16u)
        *reinterpret_cast<uint4*>(S3 + 3u * plane_bytes + i) = make_uint4(0u, 0u, 0u, 0u);
    // The kernels after this one may start their prologues now: before their own waits they touch slabs and
    // launch records only (and x, where their caller vouched for it); every store of the path comes after a
    // wait, and every grid waits for its predecessor before it completes.
    // mode: bit 0 = the caller vouched for x; bits 1-3 = when the next kernel of the stream is released (0: at
    // once, 1: after the shrink, 2: after the exchange); bit 4 = ask L2 for the next layer's slabs too
    const int early_x = mode & 1, release_at = (mode >> 1) & 7;  // (3, 4: after the wait, after A and x landed)
    bool triggered = release_at == 0;
    if (triggered) pdl_trigger();
    if (tid == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init(&bars[2], 1);
        mbar_init(&bars[3], SITE_CLUSTER);  // one arrival per block of the cluster
        mbar_fence_init();
    }
    cluster_arrive_relaxed();  // the barriers exist (published by the init fence); met before the first remote arrival
    bool met = false, waited = false;
    uint32_t ph_ax = 0, ph_b = 0, ph_s = 0;  // barrier phases (each flips only when its barrier was used)
    bool alive = true;                       // false once a bounded wait ran out: keep meeting the cluster, do no more work
    const int k0 = (int)crank * sh.kchunk;
    const int klen = max(0, min(sh.kchunk, K - k0));
    const uint32_t kbytes = (uint32_t)klen * 2u;
    const int nks = (klen + 15) >> 4;  // 16-wide steps over this block's inputs (a half step reads zeros)
    const int esize = F32 ? 4 : 2;
    // fragment coordinates of the tensor-core tile: this lane holds rows g and g + 8, columns 2 t and 2 t + 1
    const int g = lane >> 2, t2 = (lane & 3) * 2;
    // row and 16-byte piece this lane names in a four-matrix load: A-side (16 rows x 16 inputs) and B-side (two
    // 8-row tiles x 16 inputs)
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_piece = lane >> 4;
    const int b_row = (lane & 7) + (lane >> 4) * 8, b_piece = (lane >> 3) & 1;
    // (the x tile has 8 rows: rows 8-15 of the multiply's token tile repeat them and their results are dropped)
    const uint32_t xs_lane = smem_u32(Xs) + (uint32_t)(a_row & 7) * (uint32_t)sh.kb_pad + (uint32_t)a_piece * 16u;
    const uint32_t as_lane = smem_u32(As) + (uint32_t)b_row * (uint32_t)sh.kb_pad + (uint32_t)b_piece * 16u;
    const uint32_t s3_lane = smem_u32(S3) + (uint32_t)a_row * (uint32_t)sh.sp_pad + (uint32_t)a_piece * 16u;
    for (int w = blockIdx.z; w < rec_cap; w += gridDim.z) {
        // ---- the one metadata fetch: the record's 208 live bytes into shared memory
        if (tid < 13) reinterpret_cast<uint4*>(&srec)[tid] = __ldg(reinterpret_cast<const uint4*>(recs + w) + tid);
        __syncthreads();
        const int cnt = srec.cnt, R = srec.rank;
        if (cnt == 0) break;  // end of the list: the same decision in every block of the cluster
#ifdef PLORA_BOUNDS
        if (!rec_in_bounds(srec, bnd, K) || srec.cols != K) {  // the same decision in every block that reads this record
            if (tid == 0) atomicMax(status, PLORA_ERR_ARG);
            __syncthreads();
            continue;
        }
#endif
        if (R == 0) {         // the slot's adapter skips this layer
            __syncthreads();
            continue;
        }
        // the work item's tokens, 8 at a time (a decoding batch rarely has more of one slot): the x tile has 8 rows,
        // which is what lets the layers with the longest inputs keep their whole share of B in one block
        for (int t0 = 0; t0 < cnt; t0 += SITE_TOK) {
            const int cn = min(SITE_TOK, cnt - t0);
            const int* tok = srec.tok + t0;
            // warp 1: the block's share of the output columns (lane p takes part p), then the copies of its rows of B
            if (warp == 1 && t0 == 0) {
                if (lane < PLORA_MAX_PARTS) column_share(srec, (int)blockIdx.y * SITE_CLUSTER + (int)crank, lane, sshare);
                __syncwarp();
                if (lane == 0) {
                    uint32_t total = 0;
    #pragma unroll
                    for (int p = 0; p < PLORA_MAX_PARTS; p++)
                        total += (uint32_t)(sshare.hi[p] - sshare.lo[p]) * (uint32_t)srec.r[p] * 2u;
                    if (total > 0) {
                        mbar_expect_tx(&bars[2], total);
    #pragma unroll
                        for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                            const uint32_t bytes = (uint32_t)(sshare.hi[p] - sshare.lo[p]) * (uint32_t)srec.r[p] * 2u;
                            if (bytes > 0)
                                bulk_g2s(Bs + sshare.boff[p],
                                         reinterpret_cast<const bf16*>(srec.b[p]) + (size_t)sshare.lo[p] * srec.r[p], bytes, &bars[2]);
                        }
                    }
                }
            }
            // ---- slab requests (before the dependency wait): the block's rows of A, one bulk copy per row. The copies
            // of the lanes of one warp are issued one after another, so the rows go round the warps: row r is lane
            // r / 8 of warp r % 8. (The barrier's one arrival carries the whole byte count; copies that land before it
            // only run the count down early.)
            if (klen > 0) {
                const bf16* A = reinterpret_cast<const bf16*>(srec.a) + k0;
                if (tid == 0) mbar_expect_tx(&bars[0], (uint32_t)R * kbytes);
                for (int r = warp + SITE_WARPS * lane; r < R; r += SITE_THREADS)
                    bulk_g2s(As + (size_t)(r >> 6) * sh.g_stride + (size_t)(r & 63) * sh.kb_pad, A + (size_t)r * K, kbytes, &bars[0]);
            }
            // a half step at the end of the rows multiplies zeros
            if ((klen & 15) != 0)
                for (int r = tid; r < R + SITE_TOK; r += SITE_THREADS)
                    *reinterpret_cast<uint4*>((r < R ? As + (size_t)(r >> 6) * sh.g_stride + (size_t)(r & 63) * sh.kb_pad
                                                     : Xs + (size_t)(r - R) * sh.kb_pad) + kbytes) = make_uint4(0u, 0u, 0u, 0u);
            __syncthreads();  // the share is known to every warp
            // ---- hints: the x and y lines this block will touch, and the next layer's slabs of this work item
            if (!waited && warp >= 2) {
                const int t1 = tid - 64, n1 = SITE_THREADS - 64;
                if (klen > 0 && !early_x) {
                    const int lines = (int)((kbytes + 127) / 128);
                    for (int i = t1; i < cn * lines; i += n1) {
                        const int t = i / lines, l = i - t * lines;
                        prefetch_l2(reinterpret_cast<const unsigned char*>(X + (size_t)tok[t] * ldx + k0) + (size_t)l * 128);
                    }
                }
    #pragma unroll 1
                for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                    const int ncol = sshare.hi[p] - sshare.lo[p];
                    if (ncol <= 0) continue;
                    const size_t len = (size_t)ncol * esize;
                    const int lines = (int)((len + 127) / 128) + 1;
                    for (int i = t1; i < cn * lines; i += n1) {
                        const int t = i / lines, l = i - t * lines;
                        const size_t start = ((size_t)tok[t] * ldy + srec.off[p] + sshare.lo[p]) * esize;
                        const size_t at = (start & ~(size_t)127) + (size_t)l * 128;
                        if (at < start + len) prefetch_l2(reinterpret_cast<const unsigned char*>(Y) + at);
                    }
                }
            }
            if (next_recs != nullptr && warp == 1 && blockIdx.y == 0 && t0 == 0) {
                // the same work item's launch record at the next layer (the records are written for all layers at
                // once) is asked into L2, and, when the caller wants it, an eighth of each of its slabs
                const PloraRec* nr = next_recs + w;
                if (crank == 0 && lane < 2) prefetch_l2(reinterpret_cast<const unsigned char*>(nr) + 128 * lane);
                if (mode & 16) {
                    const int4 head = __ldg(reinterpret_cast<const int4*>(nr));  // cn, slot, rank, cols
                    if (head.x > 0 && head.z > 0) {
                        prefetch_eighth(__ldg(&nr->a), (uint64_t)head.z * (uint64_t)head.w * 2u, crank, lane);
    #pragma unroll 1
                        for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                            const int rp = __ldg(&nr->r[p]);
                            if (rp > 0) prefetch_eighth(__ldg(&nr->b[p]), (uint64_t)__ldg(&nr->rows[p]) * (uint64_t)rp * 2u, crank, lane);
                        }
                    }
                }
            }
            if (!waited && !early_x) {
                pdl_wait();
                waited = true;
            }
            if (!triggered && release_at == 3) {
                pdl_trigger();
                triggered = true;
            }
            // y of this lane's first expand step (first part of the share), on its way while the shrink and the exchange run
            uint4 pre0 = make_uint4(0u, 0u, 0u, 0u), pre1 = pre0;
            int pre_part = -1;
            if (waited) {
    #pragma unroll
                for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                    if (pre_part < 0 && srec.r[p] > 0 && sshare.hi[p] > sshare.lo[p]) {
                        pre_part = p;
                        const size_t ybase = (size_t)srec.off[p] + sshare.lo[p];
                        const int ncols = sshare.hi[p] - sshare.lo[p];
                        const bool fast = cn <= 8 && (ncols & 7) == 0 &&
                                          ((reinterpret_cast<uintptr_t>(Y) | ((size_t)ldy * esize) | (ybase * esize)) & 15) == 0;
                        const int c = warp * 32 + 8 * (lane & 3);
                        if (fast && g < cn && c < ncols) {
                            const unsigned char* yp = reinterpret_cast<const unsigned char*>(Y) + ((size_t)tok[g] * ldy + ybase + c) * esize;
                            pre0 = __ldcg(reinterpret_cast<const uint4*>(yp));
                            if (F32) pre1 = __ldcg(reinterpret_cast<const uint4*>(yp) + 1);
                        }
                    }
                }
            }
            // ---- shrink over this block's eighth of the inputs: warp q takes the 16-wide steps q, q + 8, ...
            if (klen > 0) {
                if (warp == 0) {
                    if (lane == 0) mbar_expect_tx(&bars[1], (uint32_t)cn * kbytes);
                    __syncwarp();
                    if (lane < cn) bulk_g2s(Xs + (size_t)lane * sh.kb_pad, X + (size_t)tok[lane] * ldx + k0, kbytes, &bars[1]);
                }
                if (alive) alive = mbar_wait(&bars[0], ph_ax, status) && mbar_wait(&bars[1], ph_ax, status);
                ph_ax ^= 1;
            }
            if (!triggered && release_at == 4) {
                pdl_trigger();
                triggered = true;
            }
            // rows of A in groups of 64 (8 tiles of 8): 32 accumulators per lane
            for (int j0 = 0; j0 < R; j0 += 64) {
                float acc[8][4];
    #pragma unroll
                for (int i = 0; i < 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
                const int pairs = min(4, (R - j0) >> 4);  // 16-row pairs of tiles in this group
                const uint32_t grp = (uint32_t)(j0 >> 6) * (uint32_t)sh.g_stride;
                if (alive && klen > 0) {
                    const uint32_t xs_w = xs_lane + (uint32_t)warp * 32u, as_w = as_lane + grp + (uint32_t)warp * 32u;
                    const int n = (nks - warp + SITE_WARPS - 1) / SITE_WARPS;  // this warp's steps
                    if (pairs == 1) shrink_steps<1>(acc, xs_w, as_w, (uint32_t)sh.kb_pad, n);
                    else if (pairs == 2) shrink_steps<2>(acc, xs_w, as_w, (uint32_t)sh.kb_pad, n);
                    else if (pairs == 3) shrink_steps<3>(acc, xs_w, as_w, (uint32_t)sh.kb_pad, n);
                    else shrink_steps<4>(acc, xs_w, as_w, (uint32_t)sh.kb_pad, n);
                }
                __syncthreads();  // every warp is through with this group's rows of A: their place takes the partials
                float* wp = reinterpret_cast<float*>(As + grp) + (size_t)warp * PLORA_WORK_TOKENS * sh.g_rows + t2;
    #pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (i < 2 * pairs) {
                        if (g < cn) *reinterpret_cast<float2*>(wp + g * sh.g_rows + i * 8) = make_float2(acc[i][0], acc[i][1]);
                    }
                }
            }
            __syncthreads();
            // the eight warps' partials, added in warp order: warp q takes the token rows q, q + 8
            for (int t = warp; t < cn; t += SITE_WARPS) {
                for (int j = lane; j < R; j += 32) {
                    const float* p = reinterpret_cast<const float*>(As + (size_t)(j >> 6) * sh.g_stride) + t * sh.g_rows + (j & 63);
                    float acc = p[0];
    #pragma unroll
                    for (int q = 1; q < SITE_WARPS; q++) acc += p[(size_t)q * PLORA_WORK_TOKENS * sh.g_rows];
                    Sp[t * sh.rmax + j] = acc;
                }
            }
            if (!triggered && release_at == 1) {
                pdl_trigger();
                triggered = true;
            }
            // ---- the eight partials meet: every block tells every block that its Sp is written, then reads all
            // eight and adds them in block order
            __syncthreads();
            if (!met) {
                cluster_wait();  // everybody's barriers exist
                met = true;
            }
            if (tid < SITE_CLUSTER) mbar_arrive_peer(&bars[3], (uint32_t)tid);
            if (alive) alive = mbar_wait_cluster(&bars[3], ph_s, status);
            ph_s ^= 1;
            for (int t = warp; t < cn; t += SITE_WARPS) {
                for (int j = lane; j < R; j += 32) {
                    const float* p = Sp + t * sh.rmax + j;
                    float v[SITE_CLUSTER];
    #pragma unroll
                    for (int q = 0; q < SITE_CLUSTER; q++) v[q] = ld_peer_f32(p, q);
                    float acc = v[0];
    #pragma unroll
                    for (int q = 1; q < SITE_CLUSTER; q++) acc += v[q];
                    // three bf16 terms whose sum is the f32 value
                    const bf16 hi = __float2bfloat16_rn(acc);
                    const float r1 = acc - __bfloat162float(hi);
                    const bf16 mid = __float2bfloat16_rn(r1);
                    const bf16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
                    unsigned char* s3 = S3 + (size_t)t * sh.sp_pad + (size_t)j * 2;
                    *reinterpret_cast<bf16*>(s3) = hi;
                    *reinterpret_cast<bf16*>(s3 + plane_bytes) = mid;
                    *reinterpret_cast<bf16*>(s3 + 2 * plane_bytes) = lo;
                }
            }
            cluster_arrive_relaxed();  // my reads of the others' partials are done
            if (!triggered) {
                pdl_trigger();
                triggered = true;
            }
            if (!waited) {             // early_x: everything so far ran ahead of the kernel before; y must not
                pdl_wait();
                waited = true;
            }
            __syncthreads();
            // ---- expand over this block's share of the output columns
            bool okb = true;
            {
                int total = 0;
    #pragma unroll
                for (int p = 0; p < PLORA_MAX_PARTS; p++) total += sshare.hi[p] - sshare.lo[p];
                if (total > 0 && t0 == 0) {  // (a later pass finds the rows of B in place)
                    if (alive) okb = mbar_wait(&bars[2], ph_b, status);
                    ph_b ^= 1;
                }
            }
            if (!okb) alive = false;
            if (alive) {
                const int tok0 = g < cn ? tok[g] : -1, tok1 = g + 8 < cn ? tok[g + 8] : -1;
    #pragma unroll 1
                for (int p = 0; p < PLORA_MAX_PARTS; p++) {
                    const int r = srec.r[p];
                    const int lo = sshare.lo[p], hi = sshare.hi[p];
                    if (r == 0 || hi <= lo) continue;
                    const uint32_t s3_part = s3_lane + (uint32_t)srec.r_off[p] * 2u;
                    const uint32_t bs_lane = smem_u32(Bs) + (uint32_t)sshare.boff[p] + (uint32_t)b_row * (uint32_t)r * 2u + (uint32_t)b_piece * 16u;
                    const size_t ybase = (size_t)srec.off[p] + lo;
                    // fast form: at most 8 tokens, and y rows that move in 16-byte pieces
                    const bool fast = cn <= 8 && ((hi - lo) & 7) == 0 && ((reinterpret_cast<uintptr_t>(Y) | ((size_t)ldy * esize) | (ybase * esize)) & 15) == 0;
                    if (fast) {
                        const int tk = g < cn ? tok[g] : -1;
                        const uint32_t s3p = smem_u32(S3) + (uint32_t)srec.r_off[p] * 2u, bsp = smem_u32(Bs) + (uint32_t)sshare.boff[p];
                        const bool pre = p == pre_part;
                        if (r == 16) expand_fast<1, F32>(s3p, (uint32_t)sh.sp_pad, plane_bytes, bsp, r, hi - lo, Y, ldy, ybase, tk, warp, lane, pre, pre0, pre1);
                        else if (r == 32) expand_fast<2, F32>(s3p, (uint32_t)sh.sp_pad, plane_bytes, bsp, r, hi - lo, Y, ldy, ybase, tk, warp, lane, pre, pre0, pre1);
                        else expand_fast<0, F32>(s3p, (uint32_t)sh.sp_pad, plane_bytes, bsp, r, hi - lo, Y, ldy, ybase, tk, warp, lane, pre, pre0, pre1);
                    } else if (r == 16) expand_part<1, F32>(s3_part, plane_bytes, bs_lane, r, hi - lo, Y, ldy, ybase, tok0, tok1, warp, t2);
                    else expand_part<0, F32>(s3_part, plane_bytes, bs_lane, r, hi - lo, Y, ldy, ybase, tok0, tok1, warp, t2);
                }
            }
            cluster_wait();   // nobody reads my partials any more: they may be overwritten (or the block may leave)
            __syncthreads();  // shared memory is reused by the next pass or work item
        }
    }
    if (!met) cluster_wait();  // a block must not leave while a peer may still be arriving at the start-up barrier
    // A grid completes only after the grids before it. Blocks with work have waited; of the blocks that found none,
    // one waits for all (a grid is complete only when every block has left), so that the others give their places
    // on the SMs back at once instead of holding them until the kernel before has finished.
    if (!waited && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) pdl_wait();
}

struct Plan {
    SiteShape sh;
    size_t smem;
};

// Shared-memory plan for `nsub` column groups
Plan plan_for(int K, int parts, int max_rank, int total_rows, int nsub) {
    Plan pl;
    SiteShape& s = pl.sh;
    s.kchunk = (((K + SITE_CLUSTER - 1) / SITE_CLUSTER) + 7) & ~7;
    const int pieces = s.kchunk / 8;                          // 16-byte pieces per row
    s.kb_pad = s.kchunk * 2 + ((pieces + 1) % 2 ? 16 : 32);   // an odd number of pieces between rows
    s.rmax = parts * max_rank;
    s.sp_pad = (s.rmax + 8) * 2;
    s.g_rows = s.rmax < 64 ? s.rmax : 64;
    const size_t a = (size_t)s.g_rows * s.kb_pad, wsum = (size_t)SITE_WARPS * PLORA_WORK_TOKENS * s.g_rows * 4;
    s.g_stride = (int)(((a > wsum ? a : wsum) + 127) & ~(size_t)127);
    s.aw_bytes = s.g_stride * ((s.rmax + 63) / 64);
    s.x_bytes = (int)(((size_t)SITE_TOK * s.kb_pad + 127) & ~(size_t)127);
    const int share = ((total_rows + nsub * SITE_CLUSTER - 1) / (nsub * SITE_CLUSTER) + 1) & ~1;
    // the tile loads of the last columns of a part may run up to 31 rows past the share
    s.b_bytes = (int)((((size_t)share + 32 * parts) * max_rank * 2 + 127) & ~(size_t)127);
    s.nsub = nsub;
    pl.smem = (size_t)s.aw_bytes + s.x_bytes + s.b_bytes + (size_t)PLORA_WORK_TOKENS * s.rmax * 4 +
              (size_t)4 * PLORA_WORK_TOKENS * s.sp_pad;
    return pl;
}

}  // namespace

// Plan of the cluster kernel for one layer: the fewest column groups (1, 2 or 4) with which two blocks share an
// SM (one SM cannot take a whole cluster of 8, and a B200 has room for only 15 clusters of 8 at one block per
// SM), else one block per SM with 4 groups. Returns the dynamic shared memory per block, 0 when nothing fits.
size_t plora_site_plan(int K, int parts, int max_rank, int total_rows, int* nsub) {
    if (parts * max_rank > 256) return 0;  // the shrink keeps at most 4 x 64 rows of A in flight per pass
    for (int n = 1; n <= 4; n *= 2) {
        const Plan pl = plan_for(K, parts, max_rank, total_rows, n);
        if (pl.smem <= 111 * 1024) {
            *nsub = n;
            return pl.smem;
        }
    }
    const Plan pl = plan_for(K, parts, max_rank, total_rows, 4);
    if (pl.smem > 200 * 1024) return 0;
    *nsub = 4;
    return pl.smem;
}

cudaError_t plora_site_init() {
    // The split of an SM's memory between L1 and shared memory is fixed while any block runs on it. Layers of
    // different widths ask for different amounts of shared memory per block; left to itself the driver would pick
    // a split per launch, and a block of the next layer would then find no room beside the blocks still running
    // under a smaller split. Every launch of this kernel asks for the largest split.
    cudaError_t e = cudaSuccess;
    for (int f32 = 0; f32 < 2 && e == cudaSuccess; f32++) {
        const void* fn = f32 ? reinterpret_cast<const void*>(plora_site_gather_kernel<true>)
                             : reinterpret_cast<const void*>(plora_site_gather_kernel<false>);
        e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    }
    return e;
}

// How many clusters of the layer's plan the device runs at once (0 on failure)
int plora_site_max_clusters(int K, int parts, int max_rank, int total_rows) {
    int nsub = 1;
    const size_t smem = plora_site_plan(K, parts, max_rank, total_rows, &nsub);
    if (smem == 0) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(SITE_CLUSTER, (unsigned)nsub, 16);
    cfg.blockDim = dim3(SITE_THREADS);
    cfg.dynamicSmemBytes = smem;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, plora_site_gather_kernel<false>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

cudaError_t plora_launch_site(const void* x, int ldx, int K, const PloraRec* recs, int rec_cap, const PloraRec* next_recs,
                              void* y, int ldy, int f32_out, int parts, int max_rank, int total_rows, int work_cap,
                              int max_clusters, int mode, const PloraBounds& bnd, int* status, bool pdl, cudaStream_t st) {
    (void)bnd;
    int nsub = 1;
    const size_t smem = plora_site_plan(K, parts, max_rank, total_rows, &nsub);
    if (smem == 0) return cudaErrorInvalidValue;
    const Plan pl = plan_for(K, parts, max_rank, total_rows, nsub);
    // one wave: work items beyond the clusters the device runs at once are walked in a loop, so that every block
    // of the grid starts (and releases the next kernel) at once
    int z = work_cap < PLORA_REC_TERM ? work_cap : PLORA_REC_TERM;
    if (max_clusters >= nsub && z > max_clusters / nsub) z = max_clusters / nsub;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(SITE_CLUSTER, (unsigned)nsub, (unsigned)z);
    cfg.blockDim = dim3(SITE_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (f32_out)
        return cudaLaunchKernelEx(&cfg, plora_site_gather_kernel<true>, reinterpret_cast<const bf16*>(x), ldx, K, recs, rec_cap,
                                  next_recs, y, ldy, pl.sh, mode, status PLORA_BOUNDS_ARG(bnd));
    return cudaLaunchKernelEx(&cfg, plora_site_gather_kernel<false>, reinterpret_cast<const bf16*>(x), ldx, K, recs, rec_cap,
                              next_recs, y, ldy, pl.sh, mode, status PLORA_BOUNDS_ARG(bnd));
}
