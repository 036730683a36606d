// Host side of the adapter path behind the C ABI: the adapter registry (pocket-engine's
// src/lora.rs), the scheduler's slot policy and tile rule (src/sched.rs), and the bracket
// Linear::forward puts around a layer's own matrix multiply (src/linear.rs:428-443,844-921).
// Device work is launched through plora_kernels.cu; nothing here computes on the CPU.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "plora_internal.h"

namespace {

thread_local std::string g_create_err;
thread_local std::string g_adapter_err;

int fail(const plora_t* h, int code, const std::string& text) {
    if (h) h->err = text;
    else g_create_err = text;
    return code;
}

int cuda_fail(const plora_t* h, const char* what, cudaError_t e) {
    return fail(h, PLORA_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

#define CU(h, what, call)                                    \
    do {                                                     \
        cudaError_t e_ = (call);                             \
        if (e_ != cudaSuccess) return cuda_fail(h, what, e_); \
    } while (0)

// A kernel launch of the path. While a profile is being collected (plora_profile_begin) and the stream is not
// capturing, the launch is bracketed by a pair of events on its stream (src/gpu.rs:321-332, 809-822 do the same
// under POCKET_PROFILE); plora_profile_end sums the pairs per name.
#define CUK(h, what, call)                                                        \
    do {                                                                          \
        cudaEvent_t pa_ = nullptr, pb_ = nullptr;                                 \
        const bool prof_ = prof_open(h, as_stream(stream), &pa_, &pb_);           \
        if (prof_) cudaEventRecord(pa_, as_stream(stream));                       \
        cudaError_t e_ = (call);                                                  \
        if (prof_) {                                                              \
            cudaEventRecord(pb_, as_stream(stream));                              \
            (h)->prof.push_back({what, pa_, pb_});                                \
        }                                                                         \
        if (e_ != cudaSuccess) return cuda_fail(h, what, e_);                     \
    } while (0)

// a pair of timing events for one launch, or false when no profile is open, the stream is capturing, or the
// profile is full (it holds at most 65536 launches)
bool prof_open(plora_t* h, cudaStream_t st, cudaEvent_t* a, cudaEvent_t* b) {
    if (!h || !h->prof_on || h->prof.size() >= 65536) return false;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return false;
    }
    if (cudaEventCreate(a) != cudaSuccess) return false;
    if (cudaEventCreate(b) != cudaSuccess) {
        cudaEventDestroy(*a);
        return false;
    }
    return true;
}

int next_mult(int x, int m) { return (x + m - 1) / m * m; }

// words the tile list [count, (start, len, slot) x cap_tiles] takes at the head of the step metadata, rounded up
// so that the grouping output behind it (and with it every 32-word work item) starts on a 128-byte line
size_t tile_words(const plora_t* h) { return (size_t)next_mult(1 + 3 * h->cap_tiles, 32); }

// bf16 with round-to-nearest-even, as half::bf16::from_f32 does for finite values (src/lora.rs:141-145)
inline uint16_t bf16_bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// src/lora.rs:98-101
std::vector<int> tiled_order(int hk, int hv) {
    std::vector<int> o((size_t)hv);
    int per = hv / hk;
    for (int t = 0; t < hv; t++) o[(size_t)t] = (t % hk) * per + t / hk;
    return o;
}

// src/lora.rs:105-113
void permute_blocks(float* v, size_t start, size_t block, const std::vector<int>& order, bool inverse) {
    size_t n = order.size();
    float* span = v + start;
    std::vector<float> old(span, span + n * block);
    for (size_t t = 0; t < n; t++) {
        size_t g = (size_t)order[t];
        size_t dst = inverse ? g : t, src = inverse ? t : g;
        memcpy(span + dst * block, old.data() + src * block, sizeof(float) * block);
    }
}

const plora_module* find_module(const plora_module* m, int n, int layer, const std::string& name) {
    for (int i = 0; i < n; i++)
        if (m[i].layer == layer && m[i].module && name == m[i].module) return &m[i];
    return nullptr;
}

// The descriptor of one (site, slot) for an adapter whose slab starts at `base` (src/lora.rs:597-615).
plora_desc desc_for(const SiteInfo& site, const SiteData& sd, uint64_t base) {
    plora_desc d;
    memset(&d, 0, sizeof(d));
    if (sd.rank == 0) return d;
    d.a = base + sd.a;
    d.rank = sd.rank;
    for (size_t pi = 0; pi < site.parts.size(); pi++) {
        d.b[pi] = base + sd.b_off[pi];
        d.r[pi] = sd.r[pi];
        d.r_off[pi] = sd.r_off[pi];
        d.off[pi] = site.parts[pi].off;
        d.rows[pi] = site.parts[pi].rows;
    }
    return d;
}

cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

}  // namespace

static_assert(sizeof(plora_desc) == 112, "Desc is 112 bytes (src/lora.rs:59-70)");

// for the readers in plora_read.cpp: the text plora_adapter_error returns on this thread
void plora_set_adapter_error(const std::string& text) { g_adapter_err = text; }

extern "C" {

// ------------------------------------------------------------------ registry

int plora_create(const plora_site* sites, int n_sites, int base_gguf, int key_heads, int value_heads,
                 int max_slots, int max_rank, int max_tokens, int max_seqs, int device, plora_t** out) {
    if (!out) return fail(nullptr, PLORA_ERR_ARG, "out is null");
    *out = nullptr;
    if (!sites || n_sites <= 0 || max_slots <= 0 || max_rank <= 0 || max_tokens <= 0 || max_seqs <= 0)
        return fail(nullptr, PLORA_ERR_ARG, "sites, max_slots, max_rank, max_tokens and max_seqs must be positive");
    plora_t* h = new plora();
    h->base_gguf = base_gguf != 0;
    h->hk = key_heads;
    h->hv = value_heads;
    h->max_slots = max_slots;
    h->max_rank = next_mult(max_rank, PLORA_RANK_STEP);  // src/lora.rs:481
    h->max_tokens = max_tokens;
    h->max_seqs = max_seqs;
    h->device = device;
    h->lds = PLORA_MAX_PARTS * h->max_rank;  // src/lora.rs:491
    for (int i = 0; i < n_sites; i++) {
        const plora_site& s = sites[i];
        if (s.n_parts < 1 || s.n_parts > PLORA_MAX_PARTS || s.cols <= 0 || s.cols % 8 != 0) {
            delete h;
            return fail(nullptr, PLORA_ERR_CONFIG, "site " + std::to_string(i) + ": 1..4 parts and cols a multiple of 8");
        }
        SiteInfo si;
        si.layer = s.layer;
        si.cols = s.cols;
        si.col_heads_start = s.col_heads_start;
        si.col_heads_block = s.col_heads_block;
        for (int p = 0; p < s.n_parts; p++) {
            SiteInfo::Part part;
            part.module = s.parts[p].module ? s.parts[p].module : "";
            part.rows = s.parts[p].rows;
            part.off = s.parts[p].off;
            part.heads_start = s.parts[p].heads_start;
            part.heads_block = s.parts[p].heads_block;
            if (part.rows <= 0 || part.rows % 2 != 0 || part.off < 0 || part.off % 2 != 0) {
                delete h;
                return fail(nullptr, PLORA_ERR_CONFIG,
                            "site " + std::to_string(i) + ": part rows and offsets must be positive and even");
            }
            si.parts.push_back(part);
        }
        // K-split of the shrink, a function of the site alone: chunks of at least 512 inputs, at most 16
        // of them, but never wider than 2048 (what one block stages in shared memory).
        int want = std::max((si.cols + 2047) / 2048, std::min(16, std::max(1, (si.cols + 511) / 512)));
        si.kchunk = next_mult((si.cols + want - 1) / want, 256);
        si.nsplit = (si.cols + si.kchunk - 1) / si.kchunk;
        h->nsplit_max = std::max(h->nsplit_max, si.nsplit);
        for (size_t p = 0; p < si.parts.size() && p < PLORA_MAX_PARTS; p++) {
            si.part_off[p] = si.parts[p].off;
            si.part_rows[p] = si.parts[p].rows;
        }
        h->sites.push_back(si);
    }
    // src/lora.rs:482-488
    for (auto& s : h->sites) {
        h->slot_bytes += s.parts.size() * (size_t)h->max_rank * (size_t)s.cols * 2;
        for (auto& p : s.parts) h->slot_bytes += (size_t)p.rows * (size_t)h->max_rank * 2;
    }
    h->cap_tiles = max_tokens / PLORA_TILE + max_seqs;  // src/model.rs:1346-1348
    h->seg.max_slots = max_slots;
    h->seg.max_tokens = max_tokens;
    h->seg.cap_tiles = h->cap_tiles;
    h->seg.run_min = 1 << 30;  // every run takes the gather path unless the tile path can run (set below)
    if (max_slots > 1023 || h->max_rank > 512 || plora_meta_group_smem(h->seg) > 200 * 1024) {
        delete h;
        return fail(nullptr, PLORA_ERR_CAPACITY,
                    "limits: max_slots <= 1023, max_rank <= 512, and max_tokens/16 + max_seqs tiles must fit the "
                    "grouping kernel's shared memory");
    }
    size_t entries = h->sites.size() * (size_t)(max_slots + 1);  // src/lora.rs:489
    h->table_bytes = entries * sizeof(plora_desc);
    h->s_stride = (size_t)max_tokens * (size_t)h->lds * 4;  // src/model.rs:1613
    h->s_bytes = h->s_stride * (size_t)std::max(PLORA_TILE_SPLIT_MAX, h->nsplit_max);
    if (device < 0) {
        // Layout-only handle: adapters can be prepared and inspected, nothing can be uploaded or run.
        h->host_tables = (plora_desc*)calloc(entries, sizeof(plora_desc));
        *out = h;
        return PLORA_OK;
    }
    int rc = PLORA_OK;
    auto check = [&](const char* what, cudaError_t e) {
        if (rc == PLORA_OK && e != cudaSuccess) rc = cuda_fail(nullptr, what, e);
        return e == cudaSuccess;
    };
    cudaDeviceProp prop;
    if (check("cudaSetDevice", cudaSetDevice(device)) &&
        check("cudaGetDeviceProperties", cudaGetDeviceProperties(&prop, device))) {
        if (prop.major != 10) {
            rc = fail(nullptr, PLORA_ERR_CUDA,
                      std::string("device is sm_") + std::to_string(prop.major * 10 + prop.minor) +
                          "; this library holds sm_100a code only");
        } else {
            h->sm_count = prop.multiProcessorCount;
            size_t meta_words = tile_words(h) + (size_t)h->seg.words();
            check("alloc pool", cudaMalloc((void**)&h->pool, h->slot_bytes * (size_t)max_slots));
            check("alloc tables", cudaMalloc((void**)&h->tables, h->table_bytes));
            check("pinned tables", cudaMallocHost((void**)&h->host_tables, h->table_bytes));
            const size_t amap_bytes = sizeof(PloraTmap) * h->sites.size() * (size_t)(max_slots + 1);
            check("alloc slab tensor maps", cudaMalloc((void**)&h->amaps, amap_bytes));
            check("pinned slab tensor maps", cudaMallocHost((void**)&h->host_amaps, amap_bytes));
            if (rc == PLORA_OK) {
                memset(h->host_amaps, 0, amap_bytes);
                check("zero slab tensor maps", cudaMemset(h->amaps, 0, amap_bytes));
            }
            check("alloc S", cudaMalloc((void**)&h->s, h->s_bytes));
            check("alloc meta", cudaMalloc((void**)&h->meta, meta_words * 4));
            check("pinned meta", cudaMallocHost((void**)&h->host_meta, (size_t)(1 + 3 * h->cap_tiles) * 4));
            // launch records: at most one gather work item per slot plus one per 16 tokens, never more than tiles
            h->rec_cap = std::min(h->cap_tiles, max_slots + max_tokens / PLORA_WORK_TOKENS) + 1;
            const size_t rec_bytes = sizeof(PloraRec) * h->sites.size() * (size_t)h->rec_cap;
            check("alloc launch records", cudaMalloc((void**)&h->recs, rec_bytes));
            check("alloc layer widths", cudaMalloc((void**)&h->site_cols, 2 * h->sites.size() * sizeof(int32_t)));
            if (rc == PLORA_OK) check("zero launch records", cudaMemset(h->recs, 0, rec_bytes));
            check("alloc status", cudaMalloc((void**)&h->status, 64));
            check("kernel attributes", plora_kernels_init(h->seg));
            if (rc == PLORA_OK && h->max_rank <= 128) h->mma_ok = plora_mma_init() == cudaSuccess;
            if (rc == PLORA_OK) h->site_ok = plora_site_init() == cudaSuccess;
            std::vector<int32_t> info;
            for (auto& s : h->sites) {
                int nsub = 1, total = 0;
                for (auto& p : s.parts) total += p.rows;
                s.cluster_ok = h->site_ok && plora_site_plan(s.cols, (int)s.parts.size(), h->max_rank, total, &nsub) > 0;
                if (s.cluster_ok) {
                    s.max_clusters = plora_site_max_clusters(s.cols, (int)s.parts.size(), h->max_rank, total);
                    if (s.max_clusters < nsub) s.cluster_ok = false;
                }
                info.push_back(s.cols);
                info.push_back(s.cluster_ok ? 8 * nsub : 0);
            }
            if (rc == PLORA_OK)
                check("upload layer widths", cudaMemcpy(h->site_cols, info.data(), info.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
            if (rc == PLORA_OK && h->max_rank <= 128) h->fp8_ok = plora_fp8_init(h->max_rank) == cudaSuccess;
            if (rc == PLORA_OK && h->mma_ok) h->gemm_ok = plora_gemm_init() == cudaSuccess;
            // runs of 64 or more contiguous tokens of one slot take the tensor-core tile kernels
            if (h->mma_ok) h->seg.run_min = PLORA_RUN_MIN_DEFAULT;
            if (const char* e = getenv("PLORA_PDL")) h->pdl = e[0] != '0';
            if (const char* e = getenv("PLORA_FUSED_TILE_ROWS")) h->fused_tile_rows = std::max(1, atoi(e));
            if (const char* e = getenv("PLORA_TILE_LATE")) h->tile_late = e[0] != '0';
            if (const char* e = getenv("PLORA_PREFETCH_NEXT")) h->prefetch_next = e[0] != '0';
            if (const char* e = getenv("PLORA_SITE_RELEASE")) h->site_release = atoi(e);
            if (rc == PLORA_OK) {
                memset(h->host_tables, 0, h->table_bytes);
                check("zero tables", cudaMemset(h->tables, 0, h->table_bytes));  // src/lora.rs:494
                check("zero S", cudaMemset(h->s, 0, h->s_bytes));                // src/lora.rs:508
                check("zero meta", cudaMemset(h->meta, 0, meta_words * 4));
                check("zero status", cudaMemset(h->status, 0, 64));
                check("event", cudaEventCreateWithFlags(&h->fork_ev, cudaEventDisableTiming));
                check("event", cudaEventCreateWithFlags(&h->join_ev, cudaEventDisableTiming));
                check("sync", cudaDeviceSynchronize());
            }
        }
    }
    if (rc != PLORA_OK) {
        std::string keep = g_create_err;
        plora_destroy(h);
        g_create_err = keep;
        return rc;
    }
    *out = h;
    return PLORA_OK;
}

void plora_destroy(plora_t* h) {
    if (!h) return;
    for (auto& kv : h->adapters) plora_adapter_drop(kv.second);
    if (h->device >= 0) {
        cudaSetDevice(h->device);
        if (h->pool) cudaFree(h->pool);
        if (h->tables) cudaFree(h->tables);
        if (h->host_tables) cudaFreeHost(h->host_tables);
        if (h->amaps) cudaFree(h->amaps);
        if (h->host_amaps) cudaFreeHost(h->host_amaps);
        if (h->s) cudaFree(h->s);
        if (h->meta) cudaFree(h->meta);
        if (h->recs) cudaFree(h->recs);
        if (h->site_cols) cudaFree(h->site_cols);
        if (h->host_meta) cudaFreeHost(h->host_meta);
        if (h->status) cudaFree(h->status);
        for (int p = 0; p < PLORA_XCHG_MAX_WORLD; p++)
            if (h->xchg_ipc[p] && h->xchg_peer[p]) cudaIpcCloseMemHandle(h->xchg_peer[p]);
        if (h->xchg) cudaFree(h->xchg);
        for (auto& e : h->prof) {
            cudaEventDestroy(e.a);
            cudaEventDestroy(e.b);
        }
        if (h->fork_ev) cudaEventDestroy(h->fork_ev);
        if (h->join_ev) cudaEventDestroy(h->join_ev);
    } else {
        free(h->host_tables);
    }
    delete h;
}

int plora_abi_version(void) { return PLORA_ABI_VERSION; }

// 1 in the range-checked build (-DPLORA_BOUNDS), else 0
int plora_bounds_build(void) {
#ifdef PLORA_BOUNDS
    return 1;
#else
    return 0;
#endif
}

const char* plora_last_error(const plora_t* h) { return h ? h->err.c_str() : g_create_err.c_str(); }

uint64_t plora_bytes(const plora_t* h) {  // src/lora.rs:526-528
    if (!h) return 0;
    return (uint64_t)(h->slot_bytes * (size_t)h->max_slots + h->table_bytes + h->s_bytes);
}
uint64_t plora_slot_bytes(const plora_t* h) { return h ? (uint64_t)h->slot_bytes : 0; }
uint64_t plora_pool_ptr(const plora_t* h) { return h ? (uint64_t)(uintptr_t)h->pool : 0; }
uint64_t plora_tables_ptr(const plora_t* h) { return h ? (uint64_t)(uintptr_t)h->tables : 0; }
uint64_t plora_s_ptr(const plora_t* h) { return h ? (uint64_t)(uintptr_t)h->s : 0; }
uint64_t plora_recs_ptr(const plora_t* h) { return h ? (uint64_t)(uintptr_t)h->recs : 0; }
uint64_t plora_tiles_ptr(const plora_t* h) { return h ? (uint64_t)(uintptr_t)h->meta : 0; }
int plora_max_lora_tiles(const plora_t* h) { return h ? h->cap_tiles : 0; }
int plora_site_splits(const plora_t* h, int site) {
    if (!h || site < 0 || site >= (int)h->sites.size()) return -1;
    return h->sites[(size_t)site].nsplit;
}

// Prep::prepare, src/lora.rs:307-411
int plora_adapter_prepare(const plora_t* h, const char* name, const plora_module* modules, int n_modules,
                          int tiled_file, plora_adapter_t** out) {
    auto bad = [&](int code, const std::string& text) {
        g_adapter_err = text;
        return code;
    };
    if (!h || !name || !out || (n_modules > 0 && !modules)) return bad(PLORA_ERR_ARG, "null argument");
    *out = nullptr;
    std::string nm(name);
    if (tiled_file && !h->base_gguf)  // :308-312
        return bad(PLORA_ERR_CONFIG, nm + ": GGUF adapters need a GGUF base (their value heads are reordered)");
    // PEFT adapters on a GGUF base move value heads to the base's order (:315)
    std::vector<int> order;
    if (h->base_gguf && !tiled_file && h->hk != h->hv && h->hk > 0) order = tiled_order(h->hk, h->hv);
    int rank = 0;
    size_t len = 0;
    std::vector<SiteData> sds;
    sds.reserve(h->sites.size());
    int placed = 0;
    for (auto& site : h->sites) {  // :320-355 layout first
        SiteData sd;
        int r_total = 0;
        for (size_t pi = 0; pi < site.parts.size(); pi++) {
            const plora_module* f = find_module(modules, n_modules, site.layer, site.parts[pi].module);
            if (!f) continue;
            placed++;
            if (f->r <= 0 || f->a_len != (uint64_t)f->r * (uint64_t)site.cols ||
                f->b_len != (uint64_t)site.parts[pi].rows * (uint64_t)f->r)  // :325-330
                return bad(PLORA_ERR_CONFIG, nm + ": layer " + std::to_string(site.layer) + " " +
                                                 site.parts[pi].module + ": shapes do not match the model");
            int rp = next_mult(f->r, PLORA_RANK_STEP);  // :331
            if (rp > h->max_rank)                       // :332-337
                return bad(PLORA_ERR_RANK, nm + ": rank " + std::to_string(f->r) + " is over --max-lora-rank " +
                                               std::to_string(h->max_rank));
            rank = std::max(rank, f->r);
            sd.r_off[pi] = r_total;
            sd.r[pi] = rp;
            r_total += rp;
        }
        sd.rank = r_total;
        if (r_total > 0) {
            sd.a = len;
            len += (size_t)r_total * (size_t)site.cols * 2;
            for (size_t pi = 0; pi < site.parts.size(); pi++)
                if (sd.r[pi] > 0) {
                    sd.b_off[pi] = len;
                    len += (size_t)site.parts[pi].rows * (size_t)sd.r[pi] * 2;
                }
        }
        sds.push_back(sd);
    }
    if (placed == 0 || placed < n_modules)  // :356-372
        return bad(PLORA_ERR_CONFIG, nm + ": " + std::to_string(placed) + " of its " + std::to_string(n_modules) +
                                         " modules match this model's layers");
    plora_adapter_t* a = new plora_adapter();
    a->name = nm;
    a->rank = rank;
    a->len = len;
    a->sites = sds;
    size_t alloc = std::max<size_t>(len, 1);
    if (h->device >= 0) {
        // the Pinner of src/gpu.rs:85-110: make the device current on this (possibly worker) thread
        cudaError_t e = cudaSetDevice(h->device);
        if (e == cudaSuccess) e = cudaMallocHost((void**)&a->data, alloc);
        if (e != cudaSuccess) {
            delete a;
            return bad(PLORA_ERR_CUDA, std::string("pinned adapter buffer: ") + cudaGetErrorString(e));
        }
        a->pinned = true;
    } else {
        a->data = (uint8_t*)malloc(alloc);
    }
    memset(a->data, 0, alloc);  // :375
    for (size_t si = 0; si < h->sites.size(); si++) {  // :376-403 fill
        const SiteInfo& site = h->sites[si];
        const SiteData& sd = sds[si];
        for (size_t pi = 0; pi < site.parts.size(); pi++) {
            int rp = sd.r[pi];
            if (rp == 0) continue;
            const plora_module* f = find_module(modules, n_modules, site.layer, site.parts[pi].module);
            const float* fa = f->a;
            const float* fb = f->b;
            std::vector<float> pa, pb;
            if (!order.empty()) {  // Factors::permute, :115-135
                const auto& part = site.parts[pi];
                if (part.heads_start >= 0) {
                    pb.assign(f->b, f->b + f->b_len);
                    permute_blocks(pb.data(), (size_t)part.heads_start * (size_t)f->r,
                                   (size_t)part.heads_block * (size_t)f->r, order, false);
                    fb = pb.data();
                }
                if (site.col_heads_start >= 0) {
                    pa.assign(f->a, f->a + f->a_len);
                    for (int row = 0; row < f->r; row++)
                        permute_blocks(pa.data() + (size_t)row * (size_t)site.cols, (size_t)site.col_heads_start,
                                       (size_t)site.col_heads_block, order, false);
                    fa = pa.data();
                }
            }
            // A rows r_off .. r_off + r of the stacked A; padding rows stay zero (:388-393)
            uint16_t* adst = (uint16_t*)(a->data + sd.a + (size_t)sd.r_off[pi] * (size_t)site.cols * 2);
            size_t na = (size_t)f->r * (size_t)site.cols;
            for (size_t i = 0; i < na; i++) adst[i] = bf16_bits(fa[i]);
            // B [rows, rp], the last rp - r columns zero (:394-401)
            for (int row = 0; row < site.parts[pi].rows; row++) {
                uint16_t* bdst = (uint16_t*)(a->data + sd.b_off[pi] + (size_t)row * (size_t)rp * 2);
                const float* src = fb + (size_t)row * (size_t)f->r;
                for (int j = 0; j < f->r; j++) bdst[j] = bf16_bits(src[j]);
            }
        }
    }
    *out = a;
    return PLORA_OK;
}

void plora_adapter_drop(plora_adapter_t* a) {
    if (!a) return;
    if (a->data) {
        if (a->pinned) cudaFreeHost(a->data);
        else free(a->data);
    }
    delete a;
}

int plora_adapter_rank(const plora_adapter_t* a) { return a ? a->rank : -1; }
uint64_t plora_adapter_len(const plora_adapter_t* a) { return a ? (uint64_t)a->len : 0; }
const uint8_t* plora_adapter_data(const plora_adapter_t* a) { return a ? a->data : nullptr; }
const char* plora_adapter_error(void) { return g_adapter_err.c_str(); }

// The descriptor an upload of `a` at slab address `base` would write for `site` (src/lora.rs:597-615).
int plora_adapter_desc(const plora_t* h, const plora_adapter_t* a, int site, uint64_t base, plora_desc* out) {
    if (!h || !a || !out || site < 0 || site >= (int)h->sites.size() || a->sites.size() != h->sites.size())
        return PLORA_ERR_ARG;
    *out = desc_for(h->sites[(size_t)site], a->sites[(size_t)site], base);
    return PLORA_OK;
}

// src/lora.rs:562-574
int plora_insert(plora_t* h, plora_adapter_t* a, uint32_t* id) {
    if (!h || !a || !id) return fail(h, PLORA_ERR_ARG, "null argument");
    if (a->sites.size() != h->sites.size()) return fail(h, PLORA_ERR_CONFIG, "adapter was prepared for another model");
    if (h->names.count(a->name)) return fail(h, PLORA_ERR_DUPLICATE, "adapter " + a->name + " is already loaded");
    *id = h->next_id++;
    h->names[a->name] = *id;
    h->adapters[*id] = a;
    return PLORA_OK;
}

// src/lora.rs:578-580
int plora_retire(plora_t* h, const char* name, uint32_t* id) {
    if (!h || !name) return PLORA_ERR_ARG;
    auto it = h->names.find(name);
    if (it == h->names.end()) return fail(h, PLORA_ERR_UNKNOWN_ID, std::string("adapter ") + name + " is not loaded");
    if (id) *id = it->second;
    h->names.erase(it);
    return PLORA_OK;
}

// src/lora.rs:583-585
int plora_free(plora_t* h, uint32_t id) {
    if (!h) return PLORA_ERR_ARG;
    auto it = h->adapters.find(id);
    if (it == h->adapters.end()) return PLORA_OK;
    plora_adapter_drop(it->second);
    h->adapters.erase(it);
    return PLORA_OK;
}

// src/lora.rs:540-542
int plora_id(const plora_t* h, const char* name, uint32_t* id) {
    if (!h || !name || !id) return PLORA_ERR_ARG;
    auto it = h->names.find(name);
    if (it == h->names.end()) return PLORA_ERR_UNKNOWN_ID;
    *id = it->second;
    return PLORA_OK;
}

// src/lora.rs:544-548
int plora_names(const plora_t* h, char* buf, size_t cap) {
    if (!h) return 0;
    std::string all;
    for (auto& kv : h->names) {  // std::map iterates sorted
        if (!all.empty()) all += "\n";
        all += kv.first;
    }
    if (buf && cap > 0) {
        size_t n = std::min(cap - 1, all.size());
        memcpy(buf, all.data(), n);
        buf[n] = 0;
    }
    return (int)h->names.size();
}

// src/lora.rs:625-627
const plora_adapter_t* plora_adapter_of(const plora_t* h, uint32_t id) {
    if (!h) return nullptr;
    auto it = h->adapters.find(id);
    return it == h->adapters.end() ? nullptr : it->second;
}

// src/lora.rs:589-623
int plora_upload(plora_t* h, int slot, uint32_t id, void* stream) {
    if (!h) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device to upload to");
    if (slot < 1 || slot > h->max_slots) return fail(h, PLORA_ERR_ARG, "slot " + std::to_string(slot) + " is out of range");
    auto it = h->adapters.find(id);
    if (it == h->adapters.end()) return fail(h, PLORA_ERR_UNKNOWN_ID, "adapter " + std::to_string(id) + " is not loaded");
    const plora_adapter* a = it->second;
    if (a->len > h->slot_bytes) return fail(h, PLORA_ERR_CONFIG, "adapter is larger than a slot");
    CU(h, "cudaSetDevice", cudaSetDevice(h->device));
    cudaStream_t st = as_stream(stream);
    uint8_t* base = h->pool + (size_t)(slot - 1) * h->slot_bytes;
    if (a->len > 0) CU(h, "upload slab", cudaMemcpyAsync(base, a->data, a->len, cudaMemcpyHostToDevice, st));
    for (size_t si = 0; si < h->sites.size(); si++)
        h->host_tables[si * (size_t)(h->max_slots + 1) + (size_t)slot] =
            desc_for(h->sites[si], a->sites[si], (uint64_t)(uintptr_t)base);
    // one copy per site's entry for this slot (:616-621)
    for (size_t si = 0; si < h->sites.size(); si++) {
        size_t at = si * (size_t)(h->max_slots + 1) + (size_t)slot;
        CU(h, "upload descriptor",
           cudaMemcpyAsync(h->tables + at, h->host_tables + at, sizeof(plora_desc), cudaMemcpyHostToDevice, st));
        const plora_desc& d = h->host_tables[at];
        if (h->mma_ok && d.rank > 0) {  // the tile path's view of the stacked A
            CU(h, "encode slab tensor map",
               plora_mma_encode_slab(&h->host_amaps[at], (const void*)(uintptr_t)d.a, h->sites[si].cols, d.rank));
            CU(h, "upload slab tensor map",
               cudaMemcpyAsync(h->amaps + at, h->host_amaps + at, sizeof(PloraTmap), cudaMemcpyHostToDevice, st));
        }
    }
    return PLORA_OK;
}

// src/lora.rs:530-538
int plora_hook_of(const plora_t* h, int site, plora_hook* out) {
    if (!h || !out || site < 0 || site >= (int)h->sites.size()) return PLORA_ERR_ARG;
    const SiteInfo& s = h->sites[(size_t)site];
    out->table = (uint64_t)(uintptr_t)(h->tables + (size_t)site * (size_t)(h->max_slots + 1));
    out->parts = (int32_t)s.parts.size();
    out->max_rows = s.max_rows();
    out->parity = site % 2;
    out->cols = s.cols;
    out->site = site;
    out->pad_ = 0;
    return PLORA_OK;
}

int plora_desc_of(const plora_t* h, int site, int slot, plora_desc* out) {
    if (!h || !out || site < 0 || site >= (int)h->sites.size() || slot < 0 || slot > h->max_slots) return PLORA_ERR_ARG;
    *out = h->host_tables[(size_t)site * (size_t)(h->max_slots + 1) + (size_t)slot];
    return PLORA_OK;
}

// -------------------------------------------------------------- slot policy

struct plora_slots {
    std::vector<uint32_t> held;  // 0 = none; adapter ids start at 1 (src/lora.rs:507)
    std::vector<size_t> refs;
    std::vector<uint64_t> used;
    uint64_t clock = 0;
    std::vector<std::pair<int, uint32_t>> loads;
};

plora_slots_t* plora_slots_new(int slots) {
    if (slots < 0) return nullptr;
    plora_slots_t* s = new plora_slots();
    s->held.assign((size_t)slots + 1, 0);
    s->refs.assign((size_t)slots + 1, 0);
    s->used.assign((size_t)slots + 1, 0);
    return s;
}
void plora_slots_free(plora_slots_t* s) { delete s; }

int plora_slots_holding(const plora_slots_t* s, uint32_t a) {
    if (!s) return 0;
    for (size_t i = 1; i < s->held.size(); i++)
        if (s->held[i] == a) return (int)i;
    return 0;
}

int plora_slots_can_place(const plora_slots_t* s, uint32_t a) {
    if (!s) return 0;
    if (plora_slots_holding(s, a)) return 1;
    for (size_t i = 1; i < s->held.size(); i++)
        if (s->refs[i] == 0) return 1;
    return 0;
}

// The slot holding the adapter, else among slots nobody runs on: an empty one first, then the least
// recently placed; the first of equals (src/sched.rs:430-448).
int plora_slots_place(plora_slots_t* s, uint32_t a) {
    if (!s || !plora_slots_can_place(s, a)) return -1;
    s->clock += 1;
    int i = plora_slots_holding(s, a);
    if (!i) {
        int best = 0;
        for (size_t j = 1; j < s->held.size(); j++) {
            if (s->refs[j] != 0) continue;
            auto key = [&](size_t q) { return std::make_pair(s->held[q] != 0, s->used[q]); };
            if (!best || key(j) < key((size_t)best)) best = (int)j;
        }
        i = best;
        s->held[(size_t)i] = a;
        s->loads.push_back({i, a});
    }
    s->refs[(size_t)i] += 1;
    s->used[(size_t)i] = s->clock;
    return i;
}

void plora_slots_release(plora_slots_t* s, int slot) {
    if (s && slot > 0 && (size_t)slot < s->refs.size() && s->refs[(size_t)slot] > 0) s->refs[(size_t)slot] -= 1;
}

void plora_slots_forget(plora_slots_t* s, uint32_t a) {
    if (!s) return;
    int i = plora_slots_holding(s, a);
    if (i) s->held[(size_t)i] = 0;
}

int plora_slots_take_loads(plora_slots_t* s, int32_t* slot_out, uint32_t* id_out, int cap) {
    if (!s || !slot_out || !id_out || cap <= 0) return 0;
    int n = std::min<int>(cap, (int)s->loads.size());
    for (int i = 0; i < n; i++) {
        slot_out[i] = s->loads[(size_t)i].first;
        id_out[i] = s->loads[(size_t)i].second;
    }
    s->loads.erase(s->loads.begin(), s->loads.begin() + n);
    return n;
}

// ---------------------------------------------------------------- tile rule

int plora_plan_tiles(const int32_t* row_n, const int32_t* row_slot, int n_rows) {
    if (n_rows > 0 && (!row_n || !row_slot)) return -1;
    int tiles = 0;
    for (int i = 0; i < n_rows; i++) {
        if (row_n[i] < 0) return -1;
        if (row_slot[i] != 0) tiles += (row_n[i] + PLORA_TILE - 1) / PLORA_TILE;
    }
    return tiles;
}

int plora_fill_tiles(const int32_t* row_n, const int32_t* row_slot, int n_rows, int32_t* words, int cap_tiles) {
    if (!words || (n_rows > 0 && (!row_n || !row_slot))) return -1;
    int tiles = 0, t = 0;
    for (int i = 0; i < n_rows; i++) {
        const int n = row_n[i];
        if (n < 0) return -1;
        if (row_slot[i] != 0)
            for (int k = 0; k < n; k += PLORA_TILE) {
                if (tiles >= cap_tiles) return -1;
                words[1 + 3 * tiles] = t + k;
                words[2 + 3 * tiles] = std::min(n - k, PLORA_TILE);
                words[3 + 3 * tiles] = row_slot[i];
                tiles++;
            }
        t += n;
    }
    words[0] = tiles;
    return tiles;
}

// --------------------------------------------------------------------- step

int plora_meta_build(plora_t* h, uint64_t cu_dev, uint64_t seq_slot_dev, int n_seqs, void* stream) {
    if (!h) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (n_seqs < 0 || n_seqs > h->max_seqs) return fail(h, PLORA_ERR_CAPACITY, "more sequences than max_seqs");
    if (!cu_dev || !seq_slot_dev) return fail(h, PLORA_ERR_ARG, "null device pointer");
    CUK(h, "meta_tiles", plora_launch_meta_tiles((const int32_t*)(uintptr_t)cu_dev, (const int32_t*)(uintptr_t)seq_slot_dev,
                                                n_seqs, h->meta, h->cap_tiles, h->status, as_stream(stream)));
    return PLORA_OK;
}

int plora_meta_upload(plora_t* h, const int32_t* words, void* stream) {
    if (!h || !words) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    int count = words[0];
    if (count < 0 || count > h->cap_tiles) return fail(h, PLORA_ERR_CAPACITY, "more tiles than the metadata holds");
    CU(h, "upload tiles", cudaMemcpyAsync(h->meta, words, (size_t)(1 + 3 * count) * 4, cudaMemcpyHostToDevice,
                                          as_stream(stream)));
    return PLORA_OK;
}

int plora_step_begin(plora_t* h, int max_tiles, int decode, void* stream, plora_step* out) {
    if (!h || !out) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (max_tiles < 0) return fail(h, PLORA_ERR_ARG, "max_tiles is negative");
    int32_t* segs = h->meta + tile_words(h);
    h->pdl_armed = false;
    SegLayout lay = h->seg;
    if (decode) lay.run_min = 1 << 30;
    CUK(h, "meta_group", plora_launch_meta_group(h->meta, segs, lay, h->status, h->tables, h->site_cols, (int)h->sites.size(),
                                                 h->recs, h->rec_cap, as_stream(stream)));
    out->run_min = lay.run_min;
    out->pad_ = 0;
    out->tiles = (uint64_t)(uintptr_t)h->meta;
    out->s = (uint64_t)(uintptr_t)h->s;
    out->s_stride = (uint64_t)h->s_stride;
    out->segs = (uint64_t)(uintptr_t)segs;
    out->max_tiles = std::min(max_tiles, h->cap_tiles);
    out->lds = h->lds;
    return PLORA_OK;
}

// ------------------------------------------------------------------ bracket

// How many blocks share the K chunks of one tensor-core tile: enough to fill the SMs when a step has few
// tiles (prompt chunks inside a decode batch), one when there are plenty. Any value gives the same bits.
static int tile_split(const plora_t* h, int rows) {
    if (h->tile_split_force) return h->tile_split_force;
    const int est = std::max(1, rows / PLORA_MMA_TOKENS);
    int s = 1;
    while (s < PLORA_TILE_SPLIT_MAX && 2 * s * est <= h->sm_count) s <<= 1;
    return s;
}

static int shrink_impl(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t x, int rows, bool early,
                       bool early_x, void* stream);

int plora_shrink(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t x, int rows, void* stream) {
    return shrink_impl(h, hook, step, x, rows, false, false, stream);
}

// what a launch over `rows` token rows may touch (checked by the kernels of the -DPLORA_BOUNDS build only)
static PloraBounds bounds_of(const plora_t* h, const plora_hook* hook, int rows, int ldy) {
    PloraBounds b;
    b.pool_lo = (unsigned long long)(uintptr_t)h->pool;
    b.pool_hi = b.pool_lo + (unsigned long long)h->slot_bytes * (unsigned long long)h->max_slots;
    b.rows = rows;
    b.ldy = ldy;
    b.rmax = hook->parts * h->max_rank;
    b.max_rank = h->max_rank;
    return b;
}

// the launch records of a layer for this step
static const PloraRec* recs_of(const plora_t* h, int site) { return h->recs + (size_t)site * (size_t)h->rec_cap; }

static int shrink_impl(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t x, int rows, bool early,
                       bool early_x, void* stream) {
    if (!h || !hook || !step) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (hook->site < 0 || hook->site >= (int)h->sites.size()) return fail(h, PLORA_ERR_ARG, "hook names no site");
    if (rows < 0 || rows > h->max_tokens) return fail(h, PLORA_ERR_CAPACITY, "more rows than max_tokens");
    if (!x || (x & 15)) return fail(h, PLORA_ERR_ARG, "x must be a 16-byte aligned device address");
    const SiteInfo& site = h->sites[(size_t)hook->site];
    // src/linear.rs:862 bounds the grid by min(max_tiles, rows); grouped by slot, the work items are also
    // at most one per slot plus one per 16 tokens
    int work_cap = std::min(std::min(step->max_tiles, rows), h->max_slots + rows / PLORA_WORK_TOKENS);
    if (work_cap == 0) return PLORA_OK;
    const bool pdl = h->pdl && h->pdl_armed;
    h->pdl_armed = true;
    CUK(h, "shrink",
       plora_launch_shrink((const void*)(uintptr_t)x, site.cols, site.cols, recs_of(h, hook->site), h->rec_cap,
                           (float*)(uintptr_t)step->s, (size_t)(step->s_stride / 4), step->lds, site.kchunk, site.nsplit,
                           work_cap, hook->parts * h->max_rank, bounds_of(h, hook, rows, 0), h->status, pdl, early, early_x,
                           as_stream(stream)));
    if (h->mma_ok && rows >= step->run_min)
        CUK(h, "shrink (tile path)",
           plora_launch_shrink_mma((const void*)(uintptr_t)x, rows, site.cols, site.cols, (const int32_t*)(uintptr_t)step->segs,
                                   h->seg, (const plora_desc*)(uintptr_t)hook->table,
                                   h->amaps + (size_t)hook->site * (size_t)(h->max_slots + 1), (float*)(uintptr_t)step->s,
                                   (size_t)(step->s_stride / 4), step->lds, hook->parts * h->max_rank, std::max(1, rows / 64),
                                   tile_split(h, rows), h->status, h->pdl, h->tile_late && (!early || early_x),
                                   as_stream(stream)));
    return PLORA_OK;
}

static int expand_impl(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, uint64_t y, int ldy,
                       int f32_out, bool reduced, bool early, void* stream);


int plora_expand(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, uint64_t y, int ldy,
                 int f32_out, void* stream) {
    return expand_impl(h, hook, step, rows, y, ldy, f32_out, false, false, stream);
}

int plora_expand_reduced(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, uint64_t y, int ldy,
                         int f32_out, void* stream) {
    return expand_impl(h, hook, step, rows, y, ldy, f32_out, true, false, stream);
}

// Shrink and expand of one layer in one call, for callers whose x and y are both ready (after the layer's own
// matrix multiply): the gather tokens go through the cluster kernel where the layer's shapes fit it.
int plora_apply(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t x, int rows, uint64_t y, int ldy,
                int f32_out, void* stream) {
    if (!h || !hook || !step) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (hook->site < 0 || hook->site >= (int)h->sites.size()) return fail(h, PLORA_ERR_ARG, "hook names no site");
    const SiteInfo& site = h->sites[(size_t)hook->site];
    if (!site.cluster_ok || h->apply_mode == 0) {
        // x and y are both older than the kernel before each launch: fetch them ahead of the dependency waits
        int rc = shrink_impl(h, hook, step, x, rows, true, h->early_x, stream);
        return rc != PLORA_OK ? rc : expand_impl(h, hook, step, rows, y, ldy, f32_out, false, true, stream);
    }
    if (rows < 0 || rows > h->max_tokens) return fail(h, PLORA_ERR_CAPACITY, "more rows than max_tokens");
    if (!x || (x & 15)) return fail(h, PLORA_ERR_ARG, "x must be a 16-byte aligned device address");
    if (!y || (y & (f32_out ? 7 : 3)) || (ldy & 1)) return fail(h, PLORA_ERR_ARG, "y must be aligned to two elements and ldy even");
    int work_cap = std::min(std::min(step->max_tiles, rows), h->max_slots + rows / PLORA_WORK_TOKENS);
    if (work_cap == 0) return PLORA_OK;
    const bool pdl = h->pdl && h->pdl_armed;
    h->pdl_armed = true;
    int total = 0;
    for (auto& p : site.parts) total += p.rows;
    CUK(h, "site kernel",
       plora_launch_site((const void*)(uintptr_t)x, site.cols, site.cols, recs_of(h, hook->site), h->rec_cap,
                         hook->site + 1 < (int)h->sites.size() ? recs_of(h, hook->site + 1) : nullptr,
                         (void*)(uintptr_t)y, ldy, f32_out, (int)site.parts.size(), h->max_rank, total, work_cap,
                         site.max_clusters, (h->early_x ? 1 : 0) | ((h->site_release >= 0 && h->site_release <= 4 ? h->site_release : (h->early_x ? 0 : 1)) << 1) |
                             (h->prefetch_next ? 16 : 0),
                         bounds_of(h, hook, rows, ldy), h->status, pdl, as_stream(stream)));
    if (h->mma_ok && rows >= step->run_min) {
        CUK(h, "shrink (tile path)",
           plora_launch_shrink_mma((const void*)(uintptr_t)x, rows, site.cols, site.cols, (const int32_t*)(uintptr_t)step->segs,
                                   h->seg, (const plora_desc*)(uintptr_t)hook->table,
                                   h->amaps + (size_t)hook->site * (size_t)(h->max_slots + 1), (float*)(uintptr_t)step->s,
                                   (size_t)(step->s_stride / 4), step->lds, hook->parts * h->max_rank, std::max(1, rows / 64),
                                   tile_split(h, rows), h->status, h->pdl, false, as_stream(stream)));
        CUK(h, "expand (tile path)",
           plora_launch_expand_mma((const float*)(uintptr_t)step->s, (size_t)(step->s_stride / 4), step->lds, site.cols,
                                   tile_split(h, rows), (const int32_t*)(uintptr_t)step->segs, h->seg,
                                   (const plora_desc*)(uintptr_t)hook->table, (void*)(uintptr_t)y, ldy, f32_out, hook->parts,
                                   site.part_off, site.part_rows, rows, hook->max_rows, std::max(1, rows / 64), h->status,
                                   h->pdl, as_stream(stream)));
    }
    return PLORA_OK;
}

int plora_s_reduce(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, void* stream) {
    if (!h || !hook || !step) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (hook->site < 0 || hook->site >= (int)h->sites.size()) return fail(h, PLORA_ERR_ARG, "hook names no site");
    if (rows < 0 || rows > h->max_tokens) return fail(h, PLORA_ERR_CAPACITY, "more rows than max_tokens");
    const SiteInfo& site = h->sites[(size_t)hook->site];
    int work_cap = std::min(std::min(step->max_tiles, rows), h->max_slots + rows / PLORA_WORK_TOKENS);
    const bool pdl = h->pdl && h->pdl_armed;
    h->pdl_armed = true;
    CUK(h, "S reduce", plora_launch_s_reduce((float*)(uintptr_t)step->s, (size_t)(step->s_stride / 4), step->lds, site.nsplit,
                                            (const int32_t*)(uintptr_t)step->segs, h->seg,
                                            (const plora_desc*)(uintptr_t)hook->table, work_cap,
                                            h->mma_ok && rows >= step->run_min ? std::max(1, rows / 64) : 0,
                                            tile_split(h, rows), site.cols, pdl, as_stream(stream)));
    return PLORA_OK;
}

static int expand_impl(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, uint64_t y, int ldy,
                       int f32_out, bool reduced, bool early, void* stream) {
    if (!h || !hook || !step) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (hook->site < 0 || hook->site >= (int)h->sites.size()) return fail(h, PLORA_ERR_ARG, "hook names no site");
    if (rows < 0 || rows > h->max_tokens) return fail(h, PLORA_ERR_CAPACITY, "more rows than max_tokens");
    if (!y || (y & (f32_out ? 7 : 3)) || (ldy & 1))
        return fail(h, PLORA_ERR_ARG, "y must be aligned to two elements and ldy even");
    const SiteInfo& site = h->sites[(size_t)hook->site];
    int work_cap = std::min(std::min(step->max_tiles, rows), h->max_slots + rows / PLORA_WORK_TOKENS);  // src/linear.rs:900
    if (work_cap == 0) return PLORA_OK;
    const bool pdl = h->pdl && h->pdl_armed;
    h->pdl_armed = true;
    CUK(h, "expand",
       plora_launch_expand((const float*)(uintptr_t)step->s, (size_t)(step->s_stride / 4), step->lds,
                           reduced ? 1 : site.nsplit, recs_of(h, hook->site), h->rec_cap,
                           (void*)(uintptr_t)y, ldy, f32_out, hook->parts, hook->max_rows, work_cap,
                           bounds_of(h, hook, rows, ldy), h->status, pdl, early, as_stream(stream)));
    if (h->mma_ok && rows >= step->run_min)
        CUK(h, "expand (tile path)",
           plora_launch_expand_mma((const float*)(uintptr_t)step->s, (size_t)(step->s_stride / 4), step->lds, site.cols,
                                   reduced ? 1 : tile_split(h, rows), (const int32_t*)(uintptr_t)step->segs, h->seg,
                                   (const plora_desc*)(uintptr_t)hook->table, (void*)(uintptr_t)y, ldy, f32_out, hook->parts,
                                   site.part_off, site.part_rows, rows, hook->max_rows, std::max(1, rows / 64), h->status,
                                   h->pdl, as_stream(stream)));
    return PLORA_OK;
}

int plora_fp8_quant_rows(plora_t* h, uint64_t x, int rows, int cols, uint64_t xq, uint64_t st, void* stream) {
    if (!h) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (!x || !xq || !st || (x & 15) || (xq & 7) || cols <= 0 || (cols & 7) || rows < 0)
        return fail(h, PLORA_ERR_ARG, "x, xq, st must be aligned device addresses and cols a multiple of 8");
    CUK(h, "fp8 quantise", plora_launch_fp8_quant((const void*)(uintptr_t)x, rows, cols, cols, (void*)(uintptr_t)xq,
                                                 (float*)(uintptr_t)st, as_stream(stream)));
    h->pdl_armed = false;
    return PLORA_OK;
}

// The one-kernel layer (plora_gemm.cu) followed by the gather expand from plane 0 for the tokens outside long
// runs. The caller has already reduced S to plane 0.
static int gemm_layer(plora_t* h, const plora_hook* hook, const plora_step* step, int kind, uint64_t x, uint64_t st,
                      uint64_t w, uint64_t sn, int rows, int width, uint64_t y, int ldy, int f32_out, int work_cap,
                      void* stream) {
    const SiteInfo& site = h->sites[(size_t)hook->site];
    const bool pdl = h->pdl && h->pdl_armed;
    h->pdl_armed = true;
    // the kernel reads the long runs' S from plane 0: fold the tile path's planes (the gather tokens' K-split
    // planes are added by the gather expand itself)
    CUK(h, "S reduce (tiles)",
       plora_launch_s_reduce((float*)(uintptr_t)step->s, (size_t)(step->s_stride / 4), step->lds, 1,
                             (const int32_t*)(uintptr_t)step->segs, h->seg, (const plora_desc*)(uintptr_t)hook->table, 0,
                             h->mma_ok && rows >= step->run_min ? std::max(1, rows / 64) : 0, tile_split(h, rows),
                             site.cols, pdl, as_stream(stream)));
    CUK(h, "fused layer (tensor-core adapter term)",
       plora_launch_gemm_fused(kind, (const void*)(uintptr_t)x, (const float*)(uintptr_t)st, (const void*)(uintptr_t)w,
                               (const float*)(uintptr_t)sn, rows, width, site.cols, (const int32_t*)(uintptr_t)step->segs,
                               h->seg, (const plora_desc*)(uintptr_t)hook->table, (int)site.parts.size(), site.part_off,
                               site.part_rows, (const float*)(uintptr_t)step->s, step->lds, (void*)(uintptr_t)y, ldy, f32_out,
                               h->status, h->pdl, as_stream(stream)));
    if (work_cap > 0)
        CUK(h, "expand (tokens outside long runs)",
           plora_launch_expand((const float*)(uintptr_t)step->s, (size_t)(step->s_stride / 4), step->lds, site.nsplit,
                               recs_of(h, hook->site), h->rec_cap, (void*)(uintptr_t)y, ldy, f32_out, hook->parts,
                               hook->max_rows, work_cap, bounds_of(h, hook, rows, ldy), h->status, h->pdl, false,
                               as_stream(stream)));
    return PLORA_OK;
}

int plora_linear_bf16_fused(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t x, uint64_t w, int rows,
                            uint64_t y, int ldy, int f32_out, void* stream) {
    if (!h || !hook || !step) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (!h->gemm_ok) return fail(h, PLORA_ERR_CONFIG, "the fused layer needs max_rank <= 128");
    if (hook->site < 0 || hook->site >= (int)h->sites.size()) return fail(h, PLORA_ERR_ARG, "hook names no site");
    if (rows < 0 || rows > h->max_tokens) return fail(h, PLORA_ERR_CAPACITY, "more rows than max_tokens");
    const SiteInfo& site = h->sites[(size_t)hook->site];
    if (rows == 0) return PLORA_OK;
    int width = 0;
    for (auto& p : site.parts) width = std::max(width, p.off + p.rows);
    if (!x || !w || !y ||
        !plora_gemm_fits(1, (const void*)(uintptr_t)x, (const void*)(uintptr_t)w, (const void*)(uintptr_t)y, ldy, f32_out,
                         site.cols, (int)site.parts.size(), site.part_off))
        return fail(h, PLORA_ERR_ARG,
                    "x, w and y must be 16-byte aligned with 16-byte multiple pitches, and parts must start at multiples of 256 columns");
    int work_cap = std::min(std::min(step->max_tiles, rows), h->max_slots + rows / PLORA_WORK_TOKENS);
    return gemm_layer(h, hook, step, 1, x, 0, w, 0, rows, width, y, ldy, f32_out, work_cap, stream);
}

int plora_set_fused_tile_rows(plora_t* h, int rows) {
    if (!h || rows < 1) return PLORA_ERR_ARG;
    h->fused_tile_rows = rows;
    return PLORA_OK;
}

int plora_linear_fp8_fused(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t xq, uint64_t st,
                           uint64_t wq, uint64_t sn, int rows, uint64_t y, int ldy, int f32_out, void* stream) {
    if (!h || !hook || !step) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (!h->fp8_ok) return fail(h, PLORA_ERR_CONFIG, "the fused FP8 layer needs max_rank <= 128");
    if (hook->site < 0 || hook->site >= (int)h->sites.size()) return fail(h, PLORA_ERR_ARG, "hook names no site");
    if (rows < 0 || rows > h->max_tokens) return fail(h, PLORA_ERR_CAPACITY, "more rows than max_tokens");
    const SiteInfo& site = h->sites[(size_t)hook->site];
    if (!xq || !st || !wq || !sn || (xq & 15) || (wq & 15) || (site.cols & 15))
        return fail(h, PLORA_ERR_ARG, "xq and wq must be 16-byte aligned and cols a multiple of 16");
    if (!y || (y & (f32_out ? 7 : 3)) || (ldy & 1)) return fail(h, PLORA_ERR_ARG, "y must be aligned to two elements and ldy even");
    if (rows == 0) return PLORA_OK;
    int off[PLORA_MAX_PARTS] = {0, 0, 0, 0}, prow[PLORA_MAX_PARTS] = {0, 0, 0, 0}, width = 0;
    for (size_t p = 0; p < site.parts.size(); p++) {
        off[p] = site.parts[p].off;
        prow[p] = site.parts[p].rows;
        width = std::max(width, off[p] + prow[p]);
    }
    int work_cap = std::min(std::min(step->max_tiles, rows), h->max_slots + rows / PLORA_WORK_TOKENS);
    // base product and the long runs' adapter term on the tensor cores in one kernel, then the gather kernel for
    // the tokens outside long runs
    if (h->gemm_ok && rows >= h->fused_tile_rows &&
        plora_gemm_fits(0, (const void*)(uintptr_t)xq, (const void*)(uintptr_t)wq, (const void*)(uintptr_t)y, ldy, f32_out,
                        site.cols, (int)site.parts.size(), off))
        return gemm_layer(h, hook, step, 0, xq, st, wq, sn, rows, width, y, ldy, f32_out, work_cap, stream);
    const bool pdl = h->pdl && h->pdl_armed;
    h->pdl_armed = true;
    CUK(h, "S reduce", plora_launch_s_reduce((float*)(uintptr_t)step->s, (size_t)(step->s_stride / 4), step->lds, site.nsplit,
                                            (const int32_t*)(uintptr_t)step->segs, h->seg,
                                            (const plora_desc*)(uintptr_t)hook->table, work_cap,
                                            h->mma_ok && rows >= step->run_min ? std::max(1, rows / 64) : 0,
                                            tile_split(h, rows), site.cols, pdl, as_stream(stream)));
    CUK(h, "fused fp8 layer",
       plora_launch_fp8_fused((const void*)(uintptr_t)xq, (const float*)(uintptr_t)st, (const void*)(uintptr_t)wq,
                              (const float*)(uintptr_t)sn, rows, width, site.cols, (const int32_t*)(uintptr_t)step->segs,
                              h->seg, (const plora_desc*)(uintptr_t)hook->table, (int)site.parts.size(), off, prow,
                              (const float*)(uintptr_t)step->s, step->lds, (void*)(uintptr_t)y, ldy, f32_out, h->max_rank,
                              h->status, h->pdl, as_stream(stream)));
    return PLORA_OK;
}

// src/gpu.rs:849-858: the side stream waits for everything queued on the main stream
int plora_fork(plora_t* h, void* main_stream, void* side_stream) {
    if (!h) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    CU(h, "fork record", cudaEventRecord(h->fork_ev, as_stream(main_stream)));
    CU(h, "fork wait", cudaStreamWaitEvent(as_stream(side_stream), h->fork_ev, 0));
    return PLORA_OK;
}

// src/gpu.rs:861-870: the main stream waits for the side stream's work
int plora_join(plora_t* h, void* main_stream, void* side_stream) {
    if (!h) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    CU(h, "join record", cudaEventRecord(h->join_ev, as_stream(side_stream)));
    CU(h, "join wait", cudaStreamWaitEvent(as_stream(main_stream), h->join_ev, 0));
    return PLORA_OK;
}

// ---- where the time went: src/gpu.rs:1741-1791 (POCKET_PROFILE) ----

int plora_profile_begin(plora_t* h) {
    if (!h) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    for (auto& e : h->prof) {
        cudaEventDestroy(e.a);
        cudaEventDestroy(e.b);
    }
    h->prof.clear();
    h->prof_on = true;
    return PLORA_OK;
}

int plora_profile_end(plora_t* h, char* buf, size_t cap) {
    if (!h) return -PLORA_ERR_ARG;
    h->prof_on = false;
    std::map<std::string, std::pair<int, double>> sum;  // name -> launches, microseconds
    cudaError_t bad = cudaSuccess;
    for (auto& e : h->prof) {
        float ms = 0.f;
        cudaError_t r = cudaEventSynchronize(e.b);
        if (r == cudaSuccess) r = cudaEventElapsedTime(&ms, e.a, e.b);
        if (r != cudaSuccess) bad = r;
        else {
            auto& s = sum[e.what];
            s.first += 1;
            s.second += 1e3 * ms;
        }
        cudaEventDestroy(e.a);
        cudaEventDestroy(e.b);
    }
    h->prof.clear();
    if (bad != cudaSuccess) return -cuda_fail(h, "profile events", bad);  // negative: a count is expected
    std::string out;
    for (auto& kv : sum) {
        char line[160];
        snprintf(line, sizeof line, "%s\t%d\t%.3f\n", kv.first.c_str(), kv.second.first, kv.second.second);
        out += line;
    }
    if (buf && cap) {
        const size_t n = out.size() < cap - 1 ? out.size() : cap - 1;
        memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return (int)sum.size();
}

int plora_set_apply_mode(plora_t* h, int mode) {
    if (!h || mode < 0 || mode > 1) return PLORA_ERR_ARG;
    h->apply_mode = mode;
    return PLORA_OK;
}

int plora_set_early_x(plora_t* h, int on) {
    if (!h) return PLORA_ERR_ARG;
    h->early_x = on != 0;
    return PLORA_OK;
}

int plora_set_run_min(plora_t* h, int tokens) {
    if (!h || tokens < 64) return fail(h, PLORA_ERR_ARG, "run_min must be at least 64 tokens");
    if (!h->mma_ok && tokens < (1 << 30))
        return fail(h, PLORA_ERR_CONFIG, "the tile path needs a device handle and max_rank <= 128");
    h->seg.run_min = tokens;
    return PLORA_OK;
}

// ------------------------------------------------------------------ tensor-parallel exchange

int plora_exchange_create(plora_t* h, int world, int rank, int timeout_ms) {
    if (!h) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    if (world < 1 || world > PLORA_XCHG_MAX_WORLD || rank < 0 || rank >= world || timeout_ms < 1)
        return fail(h, PLORA_ERR_ARG, "exchange: world 1..8, rank inside it, timeout at least 1 ms");
    if (h->xchg) return fail(h, PLORA_ERR_ARG, "exchange already created");
    CU(h, "cudaSetDevice", cudaSetDevice(h->device));
    const int work_cap = h->max_slots + h->max_tokens / PLORA_WORK_TOKENS + 1;
    h->xchg_max_blocks = work_cap + std::max(1, h->max_tokens / 64);
    const size_t staging = (size_t)2 * world * h->max_tokens * h->lds * 4;
    h->xchg_flags_off = (staging + 255) / 256 * 256;
    h->xchg_ctl_off = h->xchg_flags_off + ((size_t)2 * world * h->xchg_max_blocks * 4 + 255) / 256 * 256;
    h->xchg_ctx_off = h->xchg_ctl_off + 256;
    h->xchg_bytes = h->xchg_ctx_off + (size_t)PLORA_XCHG_MAX_WORLD * sizeof(PloraXchgCtx);
    h->xchg_bytes = (h->xchg_bytes + ((size_t)2 << 20) - 1) / ((size_t)2 << 20) * ((size_t)2 << 20);
    CU(h, "alloc exchange", cudaMalloc((void**)&h->xchg, h->xchg_bytes));
    CU(h, "zero exchange", cudaMemset(h->xchg, 0, h->xchg_bytes));
    CU(h, "sync", cudaDeviceSynchronize());
    h->xchg_world = world;
    h->xchg_rank = rank;
    h->xchg_timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    h->xchg_peer[rank] = h->xchg;
    return PLORA_OK;
}

// After a wait ran out (a peer that never arrived), the ranks disagree on the call number: the rank that timed out
// counted the call, the absent one did not. This puts one rank back to the state right after
// plora_exchange_create: flags and call counters zero, stream-ordered. Every rank calls it, and no rank starts
// its next plora_s_exchange before all have (a host-side barrier between the two): a peer's late store from
// the failed call must not land after the reset.
int plora_exchange_reset(plora_t* h, void* stream) {
    if (!h) return PLORA_ERR_ARG;
    if (!h->xchg) return fail(h, PLORA_ERR_ARG, "exchange not created");
    CU(h, "reset exchange flags and counters",
       cudaMemsetAsync(h->xchg + h->xchg_flags_off, 0, h->xchg_ctx_off - h->xchg_flags_off, as_stream(stream)));
    return PLORA_OK;
}

int plora_exchange_export(plora_t* h, void* handle64) {
    if (!h || !handle64) return PLORA_ERR_ARG;
    if (!h->xchg) return fail(h, PLORA_ERR_ARG, "exchange not created");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t hd;
    CU(h, "cudaSetDevice", cudaSetDevice(h->device));
    CU(h, "export exchange memory", cudaIpcGetMemHandle(&hd, h->xchg));
    memcpy(handle64, &hd, 64);
    return PLORA_OK;
}

int plora_exchange_import(plora_t* h, int peer, const void* handle64) {
    if (!h || !handle64) return PLORA_ERR_ARG;
    if (!h->xchg) return fail(h, PLORA_ERR_ARG, "exchange not created");
    if (peer < 0 || peer >= h->xchg_world || peer == h->xchg_rank || h->xchg_peer[peer])
        return fail(h, PLORA_ERR_ARG, "exchange: peer out of range, self, or already imported");
    cudaIpcMemHandle_t hd;
    memcpy(&hd, handle64, 64);
    void* p = nullptr;
    CU(h, "cudaSetDevice", cudaSetDevice(h->device));
    CU(h, "open peer exchange memory", cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess));
    h->xchg_peer[peer] = (uint8_t*)p;
    h->xchg_ipc[peer] = true;
    return PLORA_OK;
}

int plora_exchange_import_local(plora_t* h, int peer, plora_t* other) {
    if (!h || !other) return PLORA_ERR_ARG;
    if (!h->xchg || !other->xchg) return fail(h, PLORA_ERR_ARG, "exchange not created");
    if (peer < 0 || peer >= h->xchg_world || peer == h->xchg_rank || h->xchg_peer[peer] || other->xchg_rank != peer ||
        other->xchg_world != h->xchg_world || other->xchg_bytes != h->xchg_bytes)
        return fail(h, PLORA_ERR_ARG, "exchange: peer handle does not match (rank, world or sizes)");
    if (other->device != h->device) {
        CU(h, "cudaSetDevice", cudaSetDevice(h->device));
        cudaError_t e = cudaDeviceEnablePeerAccess(other->device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        else if (e != cudaSuccess) return cuda_fail(h, "enable peer access", e);
    }
    h->xchg_peer[peer] = other->xchg;
    return PLORA_OK;
}

static int xchg_ctx(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, PloraXchgCtx* c, int* nblocks) {
    if (!h || !hook || !step) return PLORA_ERR_ARG;
    if (!h->xchg) return fail(h, PLORA_ERR_ARG, "exchange not created");
    if (hook->site < 0 || hook->site >= (int)h->sites.size()) return fail(h, PLORA_ERR_ARG, "hook names no site");
    if (rows < 0 || rows > h->max_tokens) return fail(h, PLORA_ERR_CAPACITY, "more rows than max_tokens");
    for (int p = 0; p < h->xchg_world; p++)
        if (!h->xchg_peer[p]) return fail(h, PLORA_ERR_ARG, "exchange: rank " + std::to_string(p) + " was not imported");
    const SiteInfo& site = h->sites[(size_t)hook->site];
    const int work_cap = std::min(std::min(step->max_tiles, rows), h->max_slots + rows / PLORA_WORK_TOKENS);
    const int tile_cap = h->mma_ok && rows >= step->run_min ? std::max(1, rows / 64) : 0;
    *nblocks = work_cap + tile_cap;
    if (*nblocks > h->xchg_max_blocks) return fail(h, PLORA_ERR_CAPACITY, "exchange: more blocks than flags");
    c->S = (float*)(uintptr_t)step->s;
    c->s_stride = (size_t)(step->s_stride / 4);
    c->lds = step->lds;
    c->nsplit = site.nsplit;
    c->segs = (const int32_t*)(uintptr_t)step->segs;
    c->lay = h->seg;
    c->table = (const plora_desc*)(uintptr_t)hook->table;
    c->work_cap = work_cap;
    c->tile_split = tile_split(h, rows);
    c->K = site.cols;
    c->world = h->xchg_world;
    c->rank = h->xchg_rank;
    c->max_tokens = h->max_tokens;
    c->max_blocks = h->xchg_max_blocks;
    for (int p = 0; p < PLORA_XCHG_MAX_WORLD; p++) {
        c->staging[p] = p < h->xchg_world ? (float*)h->xchg_peer[p] : nullptr;
        c->flags[p] = p < h->xchg_world ? (unsigned*)(h->xchg_peer[p] + h->xchg_flags_off) : nullptr;
    }
    c->ctl = (unsigned*)(h->xchg + h->xchg_ctl_off);
    c->status = h->status;
    c->timeout_ns = h->xchg_timeout_ns;
    return PLORA_OK;
}

int plora_s_exchange(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, void* stream) {
    PloraXchgCtx c;
    int nblocks = 0;
    int rc = xchg_ctx(h, hook, step, rows, &c, &nblocks);
    if (rc != PLORA_OK) return rc;
    const bool pdl = h->pdl && h->pdl_armed;
    h->pdl_armed = true;
    CUK(h, "S exchange", plora_launch_xchg(c, nblocks, pdl, as_stream(stream)));
    return PLORA_OK;
}

int plora_s_exchange_all_ranks(plora_t* const* hs, const plora_hook* const* hooks, const plora_step* const* steps,
                               int world, int rows, void* stream) {
    if (!hs || !hooks || !steps || world < 1 || world > PLORA_XCHG_MAX_WORLD || !hs[0]) return PLORA_ERR_ARG;
    plora_t* h0 = hs[0];
    PloraXchgCtx cs[PLORA_XCHG_MAX_WORLD];
    int nblocks = 0;
    for (int r = 0; r < world; r++) {
        if (!hs[r] || hs[r]->device != h0->device || hs[r]->xchg_world != world || hs[r]->xchg_rank != r)
            return fail(h0, PLORA_ERR_ARG, "all-ranks exchange: handle r must be rank r of this world on one device");
        int nb = 0;
        int rc = xchg_ctx(hs[r], hooks[r], steps[r], rows, &cs[r], &nb);
        if (rc != PLORA_OK) return rc;
        if (r && nb != nblocks) return fail(h0, PLORA_ERR_ARG, "all-ranks exchange: ranks disagree on the step's shape");
        nblocks = nb;
        hs[r]->pdl_armed = false;  // a cooperative launch: the next kernel of each rank starts plain
    }
    CU(h0, "cudaSetDevice", cudaSetDevice(h0->device));
    PloraXchgCtx* dev = (PloraXchgCtx*)(h0->xchg + h0->xchg_ctx_off);
    CU(h0, "upload contexts",
       cudaMemcpyAsync(dev, cs, sizeof(PloraXchgCtx) * (size_t)world, cudaMemcpyHostToDevice, as_stream(stream)));
    CU(h0, "S exchange (all ranks)", plora_launch_xchg_all_ranks(dev, world, nblocks, as_stream(stream)));
    return PLORA_OK;
}

int plora_set_tile_split(plora_t* h, int blocks) {
    if (!h || (blocks != 0 && blocks != 1 && blocks != 2 && blocks != 4 && blocks != 8))
        return fail(h, PLORA_ERR_ARG, "tile split must be 0 (automatic), 1, 2, 4 or 8");
    h->tile_split_force = blocks;
    return PLORA_OK;
}

int plora_device_status(plora_t* h) {
    if (!h) return PLORA_ERR_ARG;
    if (h->device < 0) return fail(h, PLORA_ERR_CUDA, "layout-only handle: no device");
    int v = 0;
    CU(h, "sync", cudaDeviceSynchronize());
    CU(h, "read status", cudaMemcpy(&v, h->status, 4, cudaMemcpyDeviceToHost));
    if (v != 0) {
        cudaMemset(h->status, 0, 4);
        return fail(h, v, "a kernel recorded status " + std::to_string(v));
    }
    return PLORA_OK;
}

}  // extern "C"
