/* TEST INFRASTRUCTURE — CPU restatement of pocket-engine's batched multi-adapter
 * LoRA path, used only as the checker for the CUDA library and as the timed CPU
 * baseline of the benchmark. Nothing in the product library includes, links or
 * calls this file.
 *
 * Parity status: the reference's own tests hold only two known-answer checks that
 * touch this path at its own boundary (src/lora.rs:640-659: tiled_order(2,6) and a
 * permute_blocks round trip); both are checked in tests/test_oracle.py. The
 * arithmetic of the kernels is pinned against the reference's own lora_shrink /
 * lora_expand (compiled from the reference's sources into oracle/_ref/) by the
 * GPU tests and by the fixtures under tests/golden/ that were produced by running
 * those kernels.
 *
 * Every function cites the reference file:line it follows (paths are relative to
 * the pocket-engine source tree).
 */
#ifndef PLORA_ORACLE_H
#define PLORA_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PO_MAX_PARTS 4 /* src/lora.rs:14 */
#define PO_RANK_STEP 16 /* src/lora.rs:16 */
#define PO_TILE 16      /* src/lora.rs:18 */

/* src/lora.rs:59-70 == src/kernels/lora.cuh:7-16 (112 bytes). */
typedef struct {
    uint64_t a;
    uint64_t b[PO_MAX_PARTS];
    int32_t rank;
    int32_t r[PO_MAX_PARTS];
    int32_t r_off[PO_MAX_PARTS];
    int32_t off[PO_MAX_PARTS];
    int32_t rows[PO_MAX_PARTS];
    int32_t pad_;
} po_desc;

/* src/lora.rs:23-50 (Heads::None is start < 0). */
typedef struct {
    int32_t layer;
    int32_t cols;
    int32_t n_parts;
    int32_t rows[PO_MAX_PARTS];
    int32_t off[PO_MAX_PARTS];
    int32_t heads_start[PO_MAX_PARTS];
    int32_t heads_block[PO_MAX_PARTS];
    int32_t col_heads_start;
    int32_t col_heads_block;
    const char* module[PO_MAX_PARTS];
} po_site;

/* src/lora.rs:91-95: one module's factors, scale already folded into b (f32). */
typedef struct {
    int32_t layer;
    int32_t r;
    const char* module;
    const float* a; /* [r, cols] */
    const float* b; /* [rows, r] */
} po_module;

/* src/lora.rs:74-79. */
typedef struct {
    uint64_t a;
    int32_t rank;
    uint64_t b_off[PO_MAX_PARTS];
    int32_t r_off[PO_MAX_PARTS];
    int32_t r[PO_MAX_PARTS];
} po_site_data;

/* ---- number formats ---- */
uint16_t po_bf16_from_f32(float x);
float po_bf16_to_f32(uint16_t h);
void po_bf16_from_f32_n(const float* src, uint16_t* dst, size_t n);
void po_bf16_to_f32_n(const uint16_t* src, float* dst, size_t n);
uint8_t po_e4m3_from_f32(float x); /* saturating-finite, round to nearest even */
float po_e4m3_to_f32(uint8_t v);

/* ---- GGUF value-head order, src/lora.rs:98-113 ---- */
void po_tiled_order(int hk, int hv, int32_t* out);
void po_permute_blocks(float* v, size_t start, size_t block, const int32_t* order, int n, int inverse);

/* ---- step tiles ---- */
/* src/sched.rs:1019-1025 */
int po_plan_tiles(const int32_t* row_n, const int32_t* row_slot, int n_rows);
/* src/sched.rs:1096-1104,1189; words = [count,(start,len,slot) x count]; -1 when over cap */
int po_fill_tiles(const int32_t* row_n, const int32_t* row_slot, int n_rows, int32_t* words, int cap_tiles);
/* src/model.rs:1346-1348 */
int po_max_lora_tiles(int max_tokens, int max_seqs);

/* ---- GPU slot policy, src/sched.rs:410-449,846-849,569-572 ---- */
typedef struct po_slots po_slots;
po_slots* po_slots_new(int slots);
void po_slots_free(po_slots*);
int po_slots_holding(const po_slots*, uint32_t adapter); /* 0 when none */
int po_slots_can_place(const po_slots*, uint32_t adapter);
int po_slots_place(po_slots*, uint32_t adapter); /* slot (1-based), -1 if it cannot */
void po_slots_release(po_slots*, int slot);
void po_slots_forget(po_slots*, uint32_t adapter);
int po_slots_take_loads(po_slots*, int32_t* slot_out, uint32_t* id_out, int cap);

/* ---- host slab layout ---- */
/* src/lora.rs:482-488 */
size_t po_slot_bytes(const po_site* sites, int n_sites, int max_rank);
/* src/lora.rs:307-411. Two-phase: bytes == NULL computes only layout and length.
 * Returns the length in bytes (>= 0) or a negative code:
 * -1 shapes do not match, -2 rank over max_rank, -3 modules that match no site / none placed,
 * -4 buffer too small, -5 tiled (GGUF) file on a non-GGUF base. */
long po_prepare(const po_site* sites, int n_sites, const po_module* modules, int n_modules, int max_rank,
                int base_gguf, int tiled_file, int hk, int hv, po_site_data* out, uint8_t* bytes, size_t cap,
                int* adapter_rank);
/* src/lora.rs:597-615 */
void po_desc_for(const po_site* site, const po_site_data* sd, uint64_t base, po_desc* out);

/* ---- arithmetic of one linear layer's adapter application ----
 * X [T, ldx] bf16 bits; tiles as above; table[slot] with HOST addresses in a / b[];
 * only rows that some tile covers are touched. */

/* fp64, no intermediate rounding: Y64[t, off_p+n] += sum_j (sum_k x[t,k] A[r_off_p+j,k]) B_p[n,j]
 * (src/kernels/lora.cuh:23-126 for which elements take part; scripts/accuracy.py:15-35 for the statement) */
void po_site_f64(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, double* Y64,
                 int ldy);

/* The reference kernels' rounding points: S summed then held in f32, rounded to bf16 before it meets B
 * (lora.cuh:96-102), f32 accumulate, then bf16(f32(y)+acc) or y_f32 += acc (lora.cuh:115-125). */
void po_site_emul(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, void* Y, int ldy,
                  int f32_out);

/* f32 S (no bf16 rounding of S), f32 accumulate, one rounding of the result: the arithmetic of the
 * new CUDA kernels, evaluated with fp64 sums so it is order-free. */
void po_site_f32s(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, void* Y, int ldy,
                  int f32_out);

/* Multithreaded f32 implementation (the timed CPU baseline). S [T, lds] scratch. Returns threads used. */
int po_site_mt(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, float* S, int lds,
               void* Y, int ldy, int f32_out, int n_threads);

/* FP8 base layer with per-token activation scales and per-output-channel weight scales, fp64:
 * Y64[t,n] = st[t]*sn[n]*sum_k e4m3(Xq[t,k])*e4m3(Wq[n,k])   (all T rows, N columns) */
void po_fp8_base_f64(const uint8_t* Xq, const float* st, const uint8_t* Wq, const float* sn, int T, int K, int N,
                     double* Y64, int ldy, int n_threads);
/* per-token dynamic quantisation: st[t] = amax_t/448 (1 when the row is zero), Xq = e4m3(x/st) */
void po_fp8_quant_rows(const uint16_t* X, int ldx, int T, int K, uint8_t* Xq, float* st);

int po_hw_threads(void);

#ifdef __cplusplus
}
#endif
#endif
