/* plora — B200 (sm_100a) implementation of pocket-engine's batched multi-adapter
 * LoRA path behind a C ABI.
 *
 * Every entry point names the pocket-engine interface it replaces (file:line in
 * the pocket-engine source tree). The binding a pocket-engine maintainer would
 * add on the Rust side is a plain `extern "C"` block over these signatures; all
 * device addresses are uint64_t like the engine's own `u64` pointers, streams are
 * the CUstream / cudaStream_t handle passed as void*.
 *
 * Threading: a handle is driven from the one thread that created it (as
 * src/gpu.rs:1-3 requires of the engine); plora_adapter_prepare may run on any
 * thread (src/lora.rs:283-305).
 *
 * Stream semantics: plora_shrink / plora_expand / plora_step_begin /
 * plora_meta_build issue no host synchronisation and no allocation
 * (src/linear.rs:425-426), so a step can be captured into a CUDA graph.
 *
 * There is no CPU fallback: every compute entry point fails with
 * PLORA_ERR_CUDA when no sm_100 device is usable.
 */
#ifndef PLORA_H
#define PLORA_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Bumped whenever a struct layout or a signature below changes; a binding compares it with
 * plora_abi_version() of the library it loaded before making any other call. */
#define PLORA_ABI_VERSION 2
int plora_abi_version(void);
/* 1 when the library was built with -DPLORA_BOUNDS (libplora_bounds.so): its few-token kernels check every launch
 * record against the launch's arguments (token rows inside [0, rows), slabs inside the slot pool, ranks inside the
 * intermediate's row, output columns inside y's pitch) and skip what does not fit, recording PLORA_ERR_ARG in the
 * device status word instead of reading or writing through it. The stand-in, on this path, for running the suite
 * under a memory checker. 0 in the ordinary build. */
int plora_bounds_build(void);

#define PLORA_MAX_PARTS 4  /* src/lora.rs:14 */
#define PLORA_RANK_STEP 16 /* src/lora.rs:16 */
#define PLORA_TILE 16      /* src/lora.rs:18 */

/* Error::Cuda / Error::Config of the engine (src/gpu.rs:19-35) as integer codes. */
enum {
    PLORA_OK = 0,
    PLORA_ERR_CUDA = 1,       /* a CUDA call failed; text in plora_last_error */
    PLORA_ERR_CONFIG = 2,     /* malformed adapter or site description */
    PLORA_ERR_RANK = 3,       /* rank over max_rank (src/lora.rs:332-337) */
    PLORA_ERR_UNKNOWN_ID = 4, /* adapter id is not loaded (src/lora.rs:590-593) */
    PLORA_ERR_DUPLICATE = 5,  /* name already loaded (src/lora.rs:563-568) */
    PLORA_ERR_NO_SLOT = 6,    /* no GPU slot can take the adapter now */
    PLORA_ERR_TIMEOUT = 7,    /* a bounded device-side wait ran out */
    PLORA_ERR_ARG = 8,        /* bad argument (null, misaligned, out of range) */
    PLORA_ERR_CAPACITY = 9    /* more tokens / tiles / sequences than the handle was made for */
};

typedef struct plora plora_t;                 /* src/lora.rs:416-442  Loras */
typedef struct plora_adapter plora_adapter_t; /* src/lora.rs:82-88    Adapter */
typedef struct plora_slots plora_slots_t;     /* src/sched.rs:410-420 LoraSlots */
typedef struct plora_manager plora_manager_t; /* the adapter lifecycle of src/engine.rs:490-655 */

/* src/lora.rs:33-41 SitePart. heads_start < 0 is Heads::None (src/lora.rs:23-31). */
typedef struct {
    const char* module;
    int32_t rows;
    int32_t off;
    int32_t heads_start;
    int32_t heads_block;
} plora_site_part;

/* src/lora.rs:43-50 Site */
typedef struct {
    int32_t layer;
    int32_t cols;
    int32_t n_parts;
    int32_t col_heads_start;
    int32_t col_heads_block;
    plora_site_part parts[PLORA_MAX_PARTS];
} plora_site;

/* src/lora.rs:91-95 Factors, keyed as in Modules (src/lora.rs:139): f32, scale already folded into b
 * (src/lora.rs:225-228). a_len / b_len carry the element counts so shape mismatches are caught
 * (src/lora.rs:325-330). */
typedef struct {
    int32_t layer;
    int32_t r;
    const char* module;
    const float* a;
    const float* b;
    uint64_t a_len;
    uint64_t b_len;
} plora_module;

/* src/lora.rs:59-70 Desc == src/kernels/lora.cuh:7-16 LoraDesc; 112 bytes. */
typedef struct {
    uint64_t a;
    uint64_t b[PLORA_MAX_PARTS];
    int32_t rank;
    int32_t r[PLORA_MAX_PARTS];
    int32_t r_off[PLORA_MAX_PARTS];
    int32_t off[PLORA_MAX_PARTS];
    int32_t rows[PLORA_MAX_PARTS];
    int32_t pad_;
} plora_desc;

/* src/lora.rs:445-452 Hook (+ the layer's input width, which Linear keeps itself: src/linear.rs:44-45) */
typedef struct {
    uint64_t table;
    int32_t parts;
    int32_t max_rows;
    int32_t parity;
    int32_t cols;
    int32_t site;
    int32_t pad_;
} plora_hook;

/* src/lora.rs:455-467 StepLora. `segs` is new: the step's tokens regrouped by slot on the device. */
typedef struct {
    uint64_t tiles;
    uint64_t s;
    uint64_t s_stride;
    uint64_t segs;
    int32_t max_tiles;
    int32_t lds;
    int32_t run_min; /* runs at least this long were routed to the tensor-core tile kernels in this step */
    int32_t pad_;
} plora_step;

/* ---- registry: src/lora.rs ---- */

/* Loras::new (src/lora.rs:470-523). max_seqs sizes the tile region as Meta::max_lora_tiles does
 * (src/model.rs:1346-1348). Unlike the engine, an odd number of sites is accepted. */
int plora_create(const plora_site* sites, int n_sites, int base_gguf, int key_heads, int value_heads,
                 int max_slots, int max_rank, int max_tokens, int max_seqs, int device, plora_t** out);
void plora_destroy(plora_t* h);
/* text of the last failure on this handle (h may be NULL for plora_create failures) */
const char* plora_last_error(const plora_t* h);
/* Loras::bytes (src/lora.rs:526-528) */
uint64_t plora_bytes(const plora_t* h);
uint64_t plora_slot_bytes(const plora_t* h);
/* device addresses the tests and multi-GPU callers need: pool, tables, S */
uint64_t plora_pool_ptr(const plora_t* h);
uint64_t plora_tables_ptr(const plora_t* h);
uint64_t plora_s_ptr(const plora_t* h);
int plora_max_lora_tiles(const plora_t* h);
/* how many K-splits the shrink of `site` writes (each [max_tokens, lds] f32, s_stride bytes apart) */
int plora_site_splits(const plora_t* h, int site);

/* Prep::prepare (src/lora.rs:307-411); tiled_file is read_gguf's flag (src/lora.rs:280). Thread-safe. */
int plora_adapter_prepare(const plora_t* h, const char* name, const plora_module* modules, int n_modules,
                          int tiled_file, plora_adapter_t** out);
void plora_adapter_drop(plora_adapter_t* a);
/* Adapter.rank / len / the host image of the slot, for inspection */
int plora_adapter_rank(const plora_adapter_t* a);
uint64_t plora_adapter_len(const plora_adapter_t* a);
const uint8_t* plora_adapter_data(const plora_adapter_t* a);
const char* plora_adapter_error(void); /* thread-local text of the last failed prepare */
/* the Desc that Loras::upload would write for `site` with the slab at `base` (src/lora.rs:597-615) */
int plora_adapter_desc(const plora_t* h, const plora_adapter_t* a, int site, uint64_t base, plora_desc* out);

/* Loras::insert / retire / free / id / names (src/lora.rs:540-585). insert takes ownership. */
int plora_insert(plora_t* h, plora_adapter_t* a, uint32_t* id);
int plora_retire(plora_t* h, const char* name, uint32_t* id);
int plora_free(plora_t* h, uint32_t id);
int plora_id(const plora_t* h, const char* name, uint32_t* id);
/* names, sorted, '\n'-separated into buf; returns the count */
int plora_names(const plora_t* h, char* buf, size_t cap);
/* Loras::adapter (src/lora.rs:625-627): the registered adapter, still owned by the registry (valid until
 * plora_free of that id; never pass it to plora_adapter_drop), or NULL when the id is not loaded */
const plora_adapter_t* plora_adapter_of(const plora_t* h, uint32_t id);
/* Loras::upload (src/lora.rs:589-623): slab and descriptors, stream-ordered */
int plora_upload(plora_t* h, int slot, uint32_t id, void* stream);
/* Loras::hook (src/lora.rs:530-538) */
int plora_hook_of(const plora_t* h, int site, plora_hook* out);
/* the pinned mirror of one descriptor (src/lora.rs:596-615), for inspection */
int plora_desc_of(const plora_t* h, int site, int slot, plora_desc* out);

/* Prep::read (src/lora.rs:298-306): reads an adapter from a PEFT directory (adapter_config.json + *.safetensors,
 * src/lora.rs:148-233) or a llama.cpp GGUF adapter file (src/lora.rs:237-281) and lays it out as its GPU slot will
 * hold it. Same rejections as the engine (DoRA, modules_to_save, trained biases, alpha_pattern, vision modules;
 * `.mtp.` modules skipped), scale = alpha / r (alpha / sqrt(r) with use_rslora; alpha defaults to 8) folded into B
 * in f32. Callable from any thread; errors in plora_adapter_error(). */
int plora_adapter_read(const plora_t* h, const char* name, const char* path, plora_adapter_t** out);

/* ---- adapter lifecycle: Engine::{start_load, finish_loads, evict, unload_adapter, submit} (src/engine.rs:490-655).
 * plora_manager_load starts a worker thread that reads the adapter (plora_adapter_read) and returns a ticket;
 * plora_manager_finish_loads, called from the engine thread between steps, registers what the workers finished,
 * answers the tickets (plora_manager_poll), drops the least recently used idle on-demand adapters beyond
 * max_cpu_loras (0 = no limit), and frees unloaded adapters once no request uses them. `slots` may be NULL; when
 * given, a freed adapter also leaves its GPU slot (Scheduler::forget_adapter, src/sched.rs:569-585). Requests
 * are counted with plora_manager_submit / plora_manager_release. All calls except the worker's read belong to the
 * thread that owns the handle. */
plora_manager_t* plora_manager_new(plora_t* h, plora_slots_t* slots, int max_cpu_loras);
void plora_manager_free(plora_manager_t* m); /* joins the worker threads */
const char* plora_manager_error(const plora_manager_t* m);
int plora_manager_load(plora_manager_t* m, const char* name, const char* path, int on_demand, uint64_t* ticket);
int plora_manager_finish_loads(plora_manager_t* m); /* returns how many adapters it registered */
int plora_manager_wait(plora_manager_t* m, int timeout_ms); /* 1 = a worker has finished something */
int plora_manager_poll(plora_manager_t* m, uint64_t ticket, int* done, int* status, char* text, int text_cap);
int plora_manager_loading(const plora_manager_t* m);
int plora_manager_unload(plora_manager_t* m, const char* name);
int plora_manager_submit(plora_manager_t* m, uint32_t adapter);
void plora_manager_release(plora_manager_t* m, uint32_t adapter);
int plora_manager_resident_on_demand(const plora_manager_t* m);

/* ---- scheduler side: src/sched.rs ---- */

/* Scheduler::with_lora_slots (src/sched.rs:550-558) */
plora_slots_t* plora_slots_new(int slots);
void plora_slots_free(plora_slots_t* s);
int plora_slots_holding(const plora_slots_t* s, uint32_t adapter);   /* src/sched.rs:422-424; 0 = none */
int plora_slots_can_place(const plora_slots_t* s, uint32_t adapter); /* src/sched.rs:425-427 */
int plora_slots_place(plora_slots_t* s, uint32_t adapter);           /* src/sched.rs:430-448; -1 = cannot */
void plora_slots_release(plora_slots_t* s, int slot);                /* src/sched.rs:846-849 */
void plora_slots_forget(plora_slots_t* s, uint32_t adapter);         /* src/sched.rs:569-572 */
/* step.lora_loads = take(loads) (src/sched.rs:1018) */
int plora_slots_take_loads(plora_slots_t* s, int32_t* slot_out, uint32_t* id_out, int cap);

/* Scheduler::plan's tile count (src/sched.rs:1019-1025) */
int plora_plan_tiles(const int32_t* row_n, const int32_t* row_slot, int n_rows);
/* Scheduler::fill's tile words (src/sched.rs:1096-1104,1189): [count,(start,len,slot) x count];
 * returns the count or -1 when it would pass cap_tiles */
int plora_fill_tiles(const int32_t* row_n, const int32_t* row_slot, int n_rows, int32_t* words, int cap_tiles);

/* ---- the step: src/model.rs:1603-1618 Act::lora_step and the metadata it points into ---- */

/* Device-side replacement of the tile part of Scheduler::fill + Act::upload_meta: from the step's
 * cumulative token offsets cu[n_seqs+1] and each sequence's slot (both i32, on the device) write the
 * tile words into the handle's metadata, bit-exact with plora_fill_tiles. No host round trip. */
int plora_meta_build(plora_t* h, uint64_t cu_dev, uint64_t seq_slot_dev, int n_seqs, void* stream);
/* The engine's own route: tile words written on the host (pinned or pageable), copied stream-ordered. */
int plora_meta_upload(plora_t* h, const int32_t* words, void* stream);
/* Act::lora_step(l, max_tiles, decode): regroups the handle's tile words by slot on the device (once per
 * step, before the first layer), resolves every few-token work item against each layer's descriptor table into
 * the step's launch records, and returns the per-step handle. Slot uploads of a step therefore come before
 * its plora_step_begin on the stream, as in the engine (src/lora.rs:589-623: "before the next step"). max_tiles bounds the launch grids
 * (src/engine.rs:448-451). decode != 0 says the step holds only tiles of a few tokens (the decoding graphs),
 * so the tensor-core tile kernels are neither fed nor launched. */
int plora_step_begin(plora_t* h, int max_tiles, int decode, void* stream, plora_step* out);
uint64_t plora_tiles_ptr(const plora_t* h);
/* the step's launch records [sites][plora_max_lora_tiles-bounded] of 256 bytes each, for inspection */
uint64_t plora_recs_ptr(const plora_t* h);

/* ---- Linear::forward's bracket: src/linear.rs:428-443,844-921 ---- */

/* Linear::lora_shrink (src/linear.rs:853-885): S = x A^T for every slot present, all parts at once.
 * x: [rows, cols] bf16 row-major, 16-byte aligned. Launches on `stream` (the engine's side stream). */
int plora_shrink(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t x, int rows, void* stream);
/* Linear::lora_expand (src/linear.rs:889-921): y[:, off_p ..] += S_p B_p^T per part, bf16 (one rounding
 * of f32(y)+acc) or f32 in place. */
int plora_expand(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, uint64_t y, int ldy,
                 int f32_out, void* stream);
/* FP8 layer with the adapter expand fused into its epilogue (builder-defined layout: e4m3 activations with one
 * f32 scale per token, e4m3 weights [width, cols] with one f32 scale per output channel). The engine's own FP8
 * layers go through cuBLASLt and are followed by lora_expand as a separate pass over y
 * (src/linear.rs:428-849, src/gpu.rs:1183-1277); here y is written once:
 *   y[t, n] = st[t] * sn[n] * sum_k xq[t,k] * wq[n,k]  +  the adapter term of token t's slot.
 * Call plora_shrink on the bf16 activations first (as Linear::forward does: src/linear.rs:440-443). */
int plora_fp8_quant_rows(plora_t* h, uint64_t x, int rows, int cols, uint64_t xq, uint64_t st, void* stream);
int plora_linear_fp8_fused(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t xq, uint64_t st,
                           uint64_t wq, uint64_t sn, int rows, uint64_t y, int ldy, int f32_out, void* stream);
/* The same for a bf16 layer: y = x w^T + adapter term, x [rows, cols] and w [width, cols] bf16 row-major, y
 * written once. The engine runs its bf16 matrix multiply and then lora_expand as a read-modify-write pass over y
 * (src/linear.rs:844-847, 889-921). One kernel does the base product and the adapter term of every long run of
 * tokens on the tensor cores; tokens outside long runs get their term from the gather kernel afterwards.
 * Needs x, w, y 16-byte aligned, pitches that are multiples of 16 bytes, and every part starting at a multiple
 * of 256 columns (PLORA_ERR_ARG otherwise). Call plora_shrink first. */
int plora_linear_bf16_fused(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t x, uint64_t w, int rows,
                            uint64_t y, int ldy, int f32_out, void* stream);
/* plora_linear_fp8_fused uses that same form (with the FP8 scales) for steps of at least this many rows, where the
 * layer's shapes meet the conditions above; smaller steps, and layers that do not meet them, take the
 * decode-shaped kernel, which builds the adapter term of all tokens on the CUDA cores inside 128 x 64 tiles and
 * writes y once. Default 1: on B200 the tensor-core form followed by the gather kernel is faster at every size
 * measured (256 mixed decode tokens over 4096 -> 12288: 65 us against 204 us). */
int plora_set_fused_tile_rows(plora_t* h, int rows); /* PLORA_FUSED_TILE_ROWS in the environment sets it at plora_create */

/* Shrink and expand of one layer in one call, for callers whose x and y are both ready (that is, after the
 * layer's own matrix multiply, where Linear::forward issues lora_expand: src/linear.rs:844-847). Same results
 * as plora_shrink + plora_expand (bitwise in mode 0; within the stated tolerance in mode 1, whose summation
 * order differs); deterministic.
 *
 * What runs ahead of the kernel before. The kernels of this call are launched with programmatic stream
 * serialization and release their own dependents at once, so consecutive calls overlap: before its dependency
 * wait a kernel reads only slabs and the step's launch records and sends L2 prefetch hints for the x and y
 * lines it will touch. It binds no value of x or y and stores nothing until the kernel launched before it on
 * the stream (typically the matrix multiply that wrote y) has completed. So any producer of x and y is safe,
 * whether or not it releases its dependents early itself. */
int plora_apply(plora_t* h, const plora_hook* hook, const plora_step* step, uint64_t x, int rows, uint64_t y, int ldy,
                int f32_out, void* stream);
/* How plora_apply runs the few-token work items: 1 (default) = one cluster kernel per layer where the layer's
 * shapes fit its shared memory, else as mode 0; 0 = the shrink / expand pair. */
int plora_set_apply_mode(plora_t* h, int mode);
/* on != 0: the caller vouches that x, at every later plora_apply, was complete before the kernel launched right
 * before plora_apply STARTED (true when that kernel is the layer's matrix multiply launched in plain stream
 * order, which reads x itself): x is then also read ahead of the dependency wait and only the y update comes
 * after it. Default off. y is never read early. */
int plora_set_early_x(plora_t* h, int on);

/* Tensor-parallel row-parallel layers (no counterpart in the single-GPU engine): plora_s_reduce adds the
 * shrink's K-split partials into plane 0 of S ([max_tokens, lds] f32 at plora_s_ptr), the caller all-reduces
 * the first `rows` rows of that plane over its ranks, and plora_expand_reduced expands from plane 0 alone. */
int plora_s_reduce(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, void* stream);
int plora_expand_reduced(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, uint64_t y, int ldy,
                         int f32_out, void* stream);

/* The same exchange in one kernel per GPU instead of a collective library call (no counterpart in the
 * engine). Every rank stores its partial into a staging slot on every rank through peer mappings (NVLink),
 * raises a flag there, waits (at most timeout_ms, then PLORA_ERR_TIMEOUT in the device status word) for the
 * flags of all ranks in its own memory and adds the partials in rank order, so all ranks end with the same
 * bits in plane 0. Set-up: plora_exchange_create on every rank (same world, max_tokens, max_rank, max_slots
 * everywhere), then hand every other rank's 64-byte handle from plora_exchange_export to
 * plora_exchange_import (another process; CUDA IPC) or its plora_t to plora_exchange_import_local (same
 * process). All ranks must then make the same sequence of plora_s_exchange calls on steps with identical
 * metadata; follow each with plora_expand_reduced. Graph-capturable: the call counter lives on the device. */
int plora_exchange_create(plora_t* h, int world, int rank, int timeout_ms);
/* Back to the state right after plora_exchange_create (flags and call counters zero, stream-ordered) after a
 * wait ran out: the rank that timed out counted the call, the absent peer did not, so without this every later
 * exchange would time out too. Every rank calls it; no rank starts its next plora_s_exchange before all have. */
int plora_exchange_reset(plora_t* h, void* stream);
int plora_exchange_export(plora_t* h, void* handle64);
int plora_exchange_import(plora_t* h, int peer, const void* handle64);
int plora_exchange_import_local(plora_t* h, int peer, plora_t* other);
int plora_s_exchange(plora_t* h, const plora_hook* hook, const plora_step* step, int rows, void* stream);
/* All ranks of one process on ONE device in a single cooperative launch, for machines with fewer GPUs than
 * ranks (kernels that wait on one another must not be separate launches on one GPU). hs[r] is rank r. */
int plora_s_exchange_all_ranks(plora_t* const* hs, const plora_hook* const* hooks, const plora_step* const* steps,
                               int world, int rows, void* stream);

/* Gpu::fork / Gpu::join (src/gpu.rs:849-901): order `side` after `main`, and `main` after `side`. */
int plora_fork(plora_t* h, void* main_stream, void* side_stream);
int plora_join(plora_t* h, void* main_stream, void* side_stream);

/* Runs of contiguous tokens of one slot at least this long leave the gather kernels for the
 * tensor-core tile kernels (no counterpart in the engine, whose tiles are always 16 tokens). */
int plora_set_run_min(plora_t* h, int tokens);

/* The tile kernels cut a layer's inputs into a fixed number of ranges (a function of the layer's width and
 * the adapter's rank alone), accumulate each on its own and add the results as a balanced tree, so that a
 * token's result does not depend on what else is in the batch. `blocks` = 1, 2, 4 or 8 fixes how many thread
 * blocks share the ranges of one 128-token tile; 0 (the default) lets the library choose from the step's row
 * count. Every value gives bit-identical results. No counterpart in the engine. */
int plora_set_tile_split(plora_t* h, int blocks);

/* No counterpart in pocket-engine. One layer's adapter application (shrink, then expand, straight from the
 * engine's tile words and descriptor table) for callers that cannot allocate device memory: an engine whose
 * memory is fully claimed at start-up (a later cudaMalloc may fail), a plugin host that forbids allocation
 * after initialisation. The f32 intermediate lives in a fixed 8 MiB device array inside the
 * library (held by every GPU that loads it, until exit), so this call allocates nothing. Calls with
 * nsplit * rows * lds * 4 bytes over plora_static_scratch_bytes() are rejected with PLORA_ERR_CAPACITY.
 * All calls on a device share that array: order them on the GPU, overlapping calls race. The first call on
 * a device resolves the array's address; make it before any stream capture begins.
 * x [rows, cols] bf16; tiles = [count,(start,len,slot) x count] i32; table = the layer's Desc table;
 * y [rows, ldy] bf16 or f32, updated in place. Error text: plora_static_error().
 * The tile words and descriptors are the caller's: every slot in the tile words must index `table`, and every
 * part's width (Desc.rows) and offset (Desc.off) must be even, as the registry enforces for its own tables. The
 * kernels check what they can see: a tile whose rows leave [0, rows), whose token count is not 1..16, whose slot
 * is negative, or whose descriptor's ranks do not fit lds is skipped (y keeps its value for those tokens) and
 * counted in plora_static_bad_tiles(). nsplit = plora_static_splits(cols). */
int plora_site_apply_static(uint64_t x, int rows, int cols, uint64_t tiles, int max_tiles, uint64_t table, int parts,
                            int max_rows, int lds, uint64_t y, int ldy, int f32_out, void* stream);
uint64_t plora_static_scratch_bytes(void);
int plora_static_splits(int cols);
long long plora_static_bad_tiles(void); /* refused tiles on the current device so far; waits for the device */
const char* plora_static_error(void);

/* Where the time went (the engine's POCKET_PROFILE, src/gpu.rs:321-332, 809-822, 1741-1791). Between begin and end
 * every kernel launch of this handle is bracketed by a pair of CUDA events on its stream (not while the stream is
 * capturing; at most 65536 launches per profile). plora_profile_end waits for them and writes one line per kernel
 * name, "name<TAB>launches<TAB>microseconds", into buf (truncated to cap); returns the number of names, or minus
 * a PLORA_ERR_* code. Event pairs
 * keep consecutive launches from overlapping, so the sum is an upper bound of the time inside a graph. */
int plora_profile_begin(plora_t* h);
int plora_profile_end(plora_t* h, char* buf, size_t cap);

/* Device status word: 0, or the PLORA_ERR_* a kernel recorded (bounded wait ran out, capacity).
 * Synchronises the device. */
int plora_device_status(plora_t* h);

#ifdef __cplusplus
}
#endif
#endif
