// Internal declarations shared by the host registry (plora_host.cpp) and the
// kernel launchers (plora_kernels.cu). Not part of the public C ABI.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/plora.h"

// ---- device metadata produced once per step by the grouping kernel ("segs") ----
// All int32 words. Gather path: tokens of short runs regrouped by slot and cut into work items of at
// most PLORA_WORK_TOKENS tokens of one slot. Tile path: runs of contiguous tokens of one slot that are
// at least PLORA_RUN_MIN long, cut into tensor-core tiles of PLORA_MMA_TOKENS tokens.
#define PLORA_WORK_TOKENS 16
#define PLORA_WORK_WORDS 32
#define PLORA_MMA_TOKENS 128
#define PLORA_RUN_MIN_DEFAULT 64
#define PLORA_XCHG_MAX_WORLD 8  // ranks of a tensor-parallel exchange

#define SEG_N_ACT 0    // slots that have gather tokens
#define SEG_N_WORK 1   // gather work items
#define SEG_N_MMA 2    // tensor-core tiles
#define SEG_N_GATHER 3 // tokens on the gather path
#define SEG_N_TILES 4  // tile count the grouping consumed
#define SEG_STATUS 5   // 0, or PLORA_ERR_* found while grouping
#define SEG_HDR 8

struct SegLayout {
    int max_slots, max_tokens, cap_tiles;
    int run_min;  // runs at least this long take the tensor-core tile path
    // word offsets
    __host__ __device__ int act() const { return SEG_HDR; }                            // [max_slots] slot ids, ascending
    __host__ __device__ int seg_off() const { return act() + max_slots; }              // [max_slots + 1] by active index
    __host__ __device__ int perm() const { return seg_off() + max_slots + 1; }         // [max_tokens] token rows by slot
    // [cap_tiles][PLORA_WORK_WORDS]: slot, perm start, count, 0, then the count token rows themselves, so
    // one 128-byte line tells a block everything about its work item
    __host__ __device__ int work() const { return (perm() + max_tokens + 31) / 32 * 32; }
    __host__ __device__ int mma() const { return work() + PLORA_WORK_WORDS * cap_tiles; }  // [cap_tiles][3] start, len, slot
    __host__ __device__ int tslot() const { return mma() + 3 * cap_tiles; }  // [max_tokens] slot of every token row, 0 = none
    __host__ __device__ int words() const { return tslot() + max_tokens; }
};

// ---- per-step launch records: one per (layer, gather work item), written once per step by the records
// kernel right after the grouping. A record carries everything a block of the few-token kernels needs about
// its work item (the slot's resolved descriptor and the token rows), so the block makes one metadata fetch
// and then issues its slab copies, instead of walking header -> work item -> descriptor table -> slab.
// Record w of a layer is valid while cnt > 0; the grouping kernel ends the list with cnt == 0.
#define PLORA_REC_TERM 128  // cleared records after the last valid one (>= the z extent of every grid that walks them)
struct alignas(256) PloraRec {
    int32_t cnt, slot, rank, cols;  // tokens (1..16), slot, stacked rows of A, the layer's input width
    uint64_t a;
    uint64_t b[PLORA_MAX_PARTS];
    int32_t r[PLORA_MAX_PARTS], r_off[PLORA_MAX_PARTS], off[PLORA_MAX_PARTS], rows[PLORA_MAX_PARTS];
    int32_t ntot, share;  // output columns over the targeted parts; columns per block of the layer's cluster kernel
    int32_t tok[PLORA_WORK_TOKENS];
    int32_t cat[PLORA_MAX_PARTS];  // where each targeted part starts when the targeted parts are laid end to end
    int32_t pad2[12];
};
static_assert(sizeof(PloraRec) == 256, "one record is two 128-byte lines");

// Range-checked build (-DPLORA_BOUNDS, libplora_bounds.so): what a launch may touch. The few-token kernels take
// every index they use from a launch record and from these launch arguments, so they check each record against
// this before using it: a record that names a token row outside [0, rows), a slab outside the slot pool, ranks
// that do not fit the intermediate's row, or output columns past the pitch of y is skipped by every block that
// sees it and PLORA_ERR_ARG is recorded in the status word; nothing is read or written through its numbers and
// nothing traps. In the ordinary build the struct is passed along and ignored.
struct PloraBounds {
    unsigned long long pool_lo, pool_hi;  // the slot pool [lo, hi)
    int rows;                             // token rows of x and y the caller named
    int ldy;                              // pitch of y in elements (0: the launch does not touch y)
    int rmax;                             // parts * max_rank: the longest stacked A, the live part of an S row
    int max_rank;
};

struct alignas(64) PloraTmap {  // a CUtensorMap, opaque to the host registry
    unsigned char b[128];
};

struct SiteInfo {
    int layer = 0, cols = 0;
    int col_heads_start = -1, col_heads_block = 0;
    struct Part {
        std::string module;
        int rows = 0, off = 0, heads_start = -1, heads_block = 0;
    };
    std::vector<Part> parts;
    int max_rows() const {
        int m = 0;
        for (auto& p : parts) m = p.rows > m ? p.rows : m;
        return m;
    }
    int part_off[PLORA_MAX_PARTS] = {0, 0, 0, 0}, part_rows[PLORA_MAX_PARTS] = {0, 0, 0, 0};  // copies of parts[]
    // K-split of the shrink: fixed per site so results do not depend on the batch
    int kchunk = 0, nsplit = 1;
    bool cluster_ok = false;  // the one-kernel-per-layer cluster path fits this layer's shapes
    int max_clusters = 0;     // clusters of that kernel the device runs at once
};

struct SiteData {  // src/lora.rs:74-79
    size_t a = 0;
    int rank = 0;
    size_t b_off[PLORA_MAX_PARTS] = {0, 0, 0, 0};
    int r_off[PLORA_MAX_PARTS] = {0, 0, 0, 0};
    int r[PLORA_MAX_PARTS] = {0, 0, 0, 0};
};

struct plora_adapter {  // src/lora.rs:82-88
    std::string name;
    int rank = 0;
    uint8_t* data = nullptr;  // pinned when a device is present, else plain host memory
    bool pinned = false;
    size_t len = 0;
    std::vector<SiteData> sites;
};

struct plora {
    std::vector<SiteInfo> sites;
    bool base_gguf = false;
    int hk = 0, hv = 0;
    int max_slots = 0, max_rank = 0, max_tokens = 0, max_seqs = 0, device = 0;
    size_t slot_bytes = 0;
    uint8_t* pool = nullptr;
    plora_desc* tables = nullptr;       // device
    plora_desc* host_tables = nullptr;  // pinned mirror
    size_t table_bytes = 0;
    PloraTmap* amaps = nullptr;       // device: per (layer, slot) tensor map of the stacked A (tile path)
    PloraTmap* host_amaps = nullptr;  // pinned mirror
    std::unordered_map<uint32_t, plora_adapter*> adapters;
    std::map<std::string, uint32_t> names;
    uint32_t next_id = 1;
    float* s = nullptr;
    size_t s_bytes = 0, s_stride = 0;
    int lds = 0, nsplit_max = 1;
    int32_t* meta = nullptr;  // device: tile words, then segs
    PloraRec* recs = nullptr;  // device: [sites][rec_cap] launch records of the step
    int rec_cap = 0;
    int32_t* host_meta = nullptr;  // pinned staging for plora_meta_upload
    int32_t* site_cols = nullptr;  // device: per layer {input width, column pieces of the cluster kernel} (for the launch records)
    int cap_tiles = 0;
    SegLayout seg;
    int* status = nullptr;  // device status word
    cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
    mutable std::string err;
    int sm_count = 148;
    bool pdl = true;        // launch with programmatic stream serialization
    // tensor-parallel exchange (plora_exchange_create): one device allocation holding the staging buffers, the
    // flags, the call counters and room for the contexts of an all-ranks launch
    uint8_t* xchg = nullptr;
    size_t xchg_bytes = 0, xchg_flags_off = 0, xchg_ctl_off = 0, xchg_ctx_off = 0;
    int xchg_world = 0, xchg_rank = 0, xchg_max_blocks = 0;
    unsigned long long xchg_timeout_ns = 0;
    uint8_t* xchg_peer[PLORA_XCHG_MAX_WORLD] = {};   // base of every rank's allocation as mapped in this process
    bool xchg_ipc[PLORA_XCHG_MAX_WORLD] = {};        // opened from an IPC handle (closed on destroy)
    int tile_split_force = 0;  // plora_set_tile_split: 0 = chosen per launch
    int apply_mode = 1;     // plora_apply: 0 = shrink / expand pair, 1 = one cluster kernel per layer where it fits
    bool early_x = false;   // plora_set_early_x: plora_apply may read x ahead of its dependency wait
    int site_release = -1;  // when the cluster kernel releases the next kernel (-1: chosen by mode)
    bool prefetch_next = false;  // the cluster kernel asks L2 for the next layer's slabs of its work item (PLORA_PREFETCH_NEXT=1: on)
    bool site_ok = false;   // the cluster kernel's attributes were set
    bool fp8_ok = false;    // the fused FP8 layer can run
    bool gemm_ok = false;   // the one-kernel layer for prefill-sized steps can run
    int fused_tile_rows = 1;  // steps with at least this many rows take it (plora_set_fused_tile_rows)
    bool tile_late = true;    // the tile shrink runs beside the gather shrink launched right before it (PLORA_TILE_LATE=0: behind it)
    bool mma_ok = false;    // the tensor-core tile kernels can run (max_rank <= 128 and the driver entry point exists)
    bool pdl_armed = false;  // false right after the step's grouping kernel: the next launch is a plain one
    // plora_profile_begin / _end: one pair of events per kernel launch while a profile is open
    struct ProfEntry {
        const char* what;
        cudaEvent_t a, b;
    };
    bool prof_on = false;
    std::vector<ProfEntry> prof;
};

size_t plora_meta_group_smem(const SegLayout& lay);

// ---- tensor-parallel exchange of the shrink partials (plora_xchg.cu) ----
struct PloraXchgCtx {
    float* S;
    size_t s_stride;  // floats between K-split planes
    int lds, nsplit;
    const int32_t* segs;
    SegLayout lay;
    const plora_desc* table;
    int work_cap, tile_split, K;
    int world, rank, max_tokens, max_blocks;
    float* staging[PLORA_XCHG_MAX_WORLD];    // every rank's staging area [2][world][max_tokens][lds], as mapped here
    unsigned* flags[PLORA_XCHG_MAX_WORLD];   // every rank's flags [2][world][max_blocks]
    unsigned* ctl;                           // local: [0] calls completed, [1] blocks finished in this call
    int* status;
    unsigned long long timeout_ns;
};
cudaError_t plora_launch_xchg(const PloraXchgCtx& c, int nblocks, bool pdl, cudaStream_t st);
cudaError_t plora_launch_xchg_all_ranks(const PloraXchgCtx* ctxs_dev, int world, int nblocks, cudaStream_t st);

// The tensor-core tile path cuts a site's K inputs into `chunks` ranges that are accumulated separately (each in
// its own tensor-memory accumulator, inputs in order) and then added as a balanced binary tree. The count is a
// function of the site and of the slot's total rank only, so a token's result never depends on the batch; a
// launch may hand the chunks to 1, 2, 4 or 8 blocks (each an aligned subtree, one plane of S per block, the
// planes tree-summed by the reader) and every such choice gives the same bits. At most 256 accumulator
// columns per block, so that two blocks share an SM's tensor memory, and at least 8 steps of 64 inputs per chunk.
#define PLORA_TILE_SPLIT_MAX 8
__host__ __device__ inline int plora_tile_cols(int R) { return R <= 32 ? 32 : R <= 64 ? 64 : R <= 128 ? 128 : R <= 256 ? 256 : 512; }
__host__ __device__ inline int plora_tile_chunks(int K, int R) {
    const int nk = (K + 63) / 64, rc = plora_tile_cols(R);
    int c = PLORA_TILE_SPLIT_MAX;
    while (c > 1 && (c * 8 > nk || c * rc > 256)) c >>= 1;
    return c;
}

// ---- kernel launchers (plora_kernels.cu); each returns a cudaError_t from the launch ----
cudaError_t plora_launch_meta_tiles(const int32_t* cu, const int32_t* seq_slot, int n_seqs, int32_t* tiles,
                                    int cap_tiles, int* status, cudaStream_t st);
// Groups the step's tiles by slot and writes the launch records of every layer (recs may be null: grouping only).
// site_info: per layer {input width, blocks that share a work item's output columns in the cluster kernel (0: none)}
cudaError_t plora_launch_meta_group(const int32_t* tiles, int32_t* segs, SegLayout lay, int* status, const plora_desc* tables,
                                    const int32_t* site_info, int n_sites, PloraRec* recs, int rec_cap, cudaStream_t st);
// Dynamic shared-memory limit of a kernel together with a request for the largest shared-memory split of the SM.
// Kernels of this library overlap with their neighbours in the stream (programmatic dependent launch); an SM's
// split between L1 and shared memory is fixed while any block runs on it, so kernels that each let the driver
// pick their own split would keep each other's blocks off the SMs.
inline cudaError_t plora_kernel_shared(const void* fn, int max_dynamic_bytes) {
    cudaError_t e = cudaSuccess;
    if (max_dynamic_bytes > 0) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, max_dynamic_bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return e;
}
cudaError_t plora_kernels_init(const SegLayout& lay);
cudaError_t plora_site_init();
size_t plora_site_plan(int K, int parts, int max_rank, int total_rows, int* nsub);
int plora_site_max_clusters(int K, int parts, int max_rank, int total_rows);
cudaError_t plora_launch_site(const void* x, int ldx, int K, const PloraRec* recs, int rec_cap, const PloraRec* next_recs,
                              void* y, int ldy, int f32_out, int parts, int max_rank, int total_rows, int work_cap,
                              int max_clusters, int mode, const PloraBounds& bnd, int* status, bool pdl, cudaStream_t st);
cudaError_t plora_mma_init();
cudaError_t plora_fp8_init(int max_rank);
cudaError_t plora_launch_fp8_quant(const void* x, int rows, int ldx, int K, void* xq, float* st, cudaStream_t stream);
cudaError_t plora_launch_s_reduce(float* S, size_t s_stride_elems, int lds, int nsplit, const int32_t* segs,
                                  SegLayout lay, const plora_desc* table, int work_cap, int tile_cap, int tile_split,
                                  int K, bool pdl, cudaStream_t st);
cudaError_t plora_launch_fp8_fused(const void* xq, const float* st_, const void* wq, const float* sn, int T, int N, int K,
                                   const int32_t* segs, SegLayout lay, const plora_desc* table, int n_parts,
                                   const int* part_off, const int* part_rows, const float* S, int lds, void* y, int ldy,
                                   int f32_out, int max_rank, int* status, bool pdl, cudaStream_t stream);
cudaError_t plora_gemm_init();
bool plora_gemm_fits(int kind, const void* x, const void* w, const void* y, int ldy, int f32_out, int K, int n_parts,
                     const int* part_off);
cudaError_t plora_launch_gemm_fused(int kind, const void* x, const float* st_, const void* w, const float* sn, int T, int N,
                                    int K, const int32_t* segs, SegLayout lay, const plora_desc* table, int n_parts,
                                    const int* part_off, const int* part_rows, const float* S, int lds, void* y, int ldy,
                                    int f32_out, int* status, bool pdl, cudaStream_t stream);
cudaError_t plora_mma_encode_slab(void* out128, const void* a, int K, int R);
cudaError_t plora_launch_shrink_mma(const void* x, int rows, int ldx, int K, const int32_t* segs, SegLayout lay,
                                    const plora_desc* table, const PloraTmap* amaps, float* S, size_t s_stride_elems, int lds,
                                    int max_rank_total, int tile_cap, int tile_split, int* status, bool pdl, bool late,
                                    cudaStream_t st);
cudaError_t plora_launch_expand_mma(const float* S, size_t s_stride_elems, int lds, int K, int tile_split,
                                    const int32_t* segs, SegLayout lay, const plora_desc* table, void* y, int ldy,
                                    int f32_out, int parts, const int* part_off, const int* part_rows, int rows_total,
                                    int max_rows, int tile_cap, int* status, bool pdl, cudaStream_t st);
// early: dependents are released at kernel start and slabs are requested ahead of the dependency wait (used by
// plora_apply, whose kernels follow one another); early_x: x too may be read ahead of the wait
cudaError_t plora_launch_shrink(const void* x, int ldx, int K, const PloraRec* recs, int rec_cap, float* S,
                                size_t s_stride_elems, int lds, int kchunk, int nsplit, int work_cap, int max_rank_total,
                                const PloraBounds& bnd, int* status, bool pdl, bool early, bool early_x, cudaStream_t st);
cudaError_t plora_launch_expand(const float* S, size_t s_stride_elems, int lds, int nsplit, const PloraRec* recs,
                                int rec_cap, void* y, int ldy, int f32_out, int parts, int max_rows, int work_cap,
                                const PloraBounds& bnd, int* status, bool pdl, bool early, cudaStream_t st);
