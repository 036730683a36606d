/* TEST INFRASTRUCTURE — see plora_oracle.h. CPU restatement of pocket-engine's
 * batched multi-adapter LoRA path (src/lora.rs, src/sched.rs tile rule,
 * src/kernels/lora.cuh arithmetic). Not part of the product library. */
#include "plora_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ------------------------------------------------------------------ formats */

/* Round to nearest even, as __float2bfloat16_rn (qwen35.cu:27) and half::bf16::from_f32
 * (src/lora.rs:141-145) do for every finite value. */
uint16_t po_bf16_from_f32(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float po_bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

void po_bf16_from_f32_n(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = po_bf16_from_f32(src[i]);
}

void po_bf16_to_f32_n(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = po_bf16_to_f32(src[i]);
}

float po_e4m3_to_f32(uint8_t v) {
    int s = v >> 7, e = (v >> 3) & 15, m = v & 7;
    float f;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) f = ldexpf((float)m, -9);
    else f = ldexpf((float)(8 + m), e - 10);
    return s ? -f : f;
}

/* __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3) (src/kernels/fp8.cuh:12): round to nearest
 * even on the e4m3 grid, magnitudes above 448 (and infinities) clamp to 448, NaN -> 0x7f. */
uint8_t po_e4m3_from_f32(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    uint8_t s = (uint8_t)((u >> 24) & 0x80);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7f;
    float a = fabsf(x);
    if (a >= 448.0f) return s | 0x7e;
    if (a < ldexpf(1.0f, -10)) return s; /* below half of the least subnormal: also the tie, to even (0) */
    int e;
    (void)frexpf(a, &e); /* a = f * 2^e, f in [0.5,1) */
    int ex = e - 1;      /* a in [2^ex, 2^(ex+1)) */
    if (ex < -6) ex = -6; /* subnormal grid */
    float step = ldexpf(1.0f, ex - 3);
    float q = a / step; /* exact: power-of-two scaling */
    float r = nearbyintf(q); /* default mode: ties to even */
    float v = r * step;
    if (v >= 448.0f) return s | 0x7e;
    /* encode v */
    if (v < ldexpf(1.0f, -6)) return s | (uint8_t)(int)(v * 512.0f);
    int e2;
    float f2 = frexpf(v, &e2); /* v = f2 * 2^e2, f2 in [0.5,1) */
    int m = (int)(f2 * 16.0f) - 8;
    return s | (uint8_t)(((e2 - 1 + 7) << 3) | m);
}

int po_hw_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n < 1 ? 1 : (int)n;
}

/* ------------------------------------------------- GGUF value-head ordering */

/* src/lora.rs:98-101 */
void po_tiled_order(int hk, int hv, int32_t* out) {
    int per = hv / hk;
    for (int t = 0; t < hv; t++) out[t] = (t % hk) * per + t / hk;
}

/* src/lora.rs:105-113 */
void po_permute_blocks(float* v, size_t start, size_t block, const int32_t* order, int n, int inverse) {
    float* span = v + start;
    float* old = (float*)malloc(sizeof(float) * block * (size_t)n);
    memcpy(old, span, sizeof(float) * block * (size_t)n);
    for (int t = 0; t < n; t++) {
        int g = order[t];
        int dst = inverse ? g : t, src = inverse ? t : g;
        memcpy(span + (size_t)dst * block, old + (size_t)src * block, sizeof(float) * block);
    }
    free(old);
}

/* -------------------------------------------------------------------- tiles */

/* src/sched.rs:1019-1025 */
int po_plan_tiles(const int32_t* row_n, const int32_t* row_slot, int n_rows) {
    int tiles = 0;
    for (int i = 0; i < n_rows; i++)
        if (row_slot[i] != 0) tiles += (row_n[i] + PO_TILE - 1) / PO_TILE;
    return tiles;
}

/* src/sched.rs:1096-1104 (the tile loop inside fill) and :1189 (the count) */
int po_fill_tiles(const int32_t* row_n, const int32_t* row_slot, int n_rows, int32_t* words, int cap_tiles) {
    int tiles = 0, t = 0;
    for (int i = 0; i < n_rows; i++) {
        int n = row_n[i];
        if (row_slot[i] != 0) {
            for (int k = 0; k < n; k += PO_TILE) {
                if (tiles >= cap_tiles) return -1;
                int32_t* at = words + 1 + 3 * tiles;
                at[0] = t + k;
                at[1] = (n - k) < PO_TILE ? (n - k) : PO_TILE;
                at[2] = row_slot[i];
                tiles++;
            }
        }
        t += n;
    }
    words[0] = tiles;
    return tiles;
}

/* src/model.rs:1346-1348 */
int po_max_lora_tiles(int max_tokens, int max_seqs) { return max_tokens / PO_TILE + max_seqs; }

/* -------------------------------------------------------------- slot policy */

struct po_slots {
    int n; /* slots + 1; index 0 unused */
    uint32_t* held; /* 0 = None (adapter ids start at 1, src/lora.rs:507) */
    size_t* refs;
    uint64_t* used;
    uint64_t clock;
    int n_loads, cap_loads;
    int32_t* load_slot;
    uint32_t* load_id;
};

/* src/sched.rs:550-558 */
po_slots* po_slots_new(int slots) {
    po_slots* s = (po_slots*)calloc(1, sizeof(po_slots));
    s->n = slots + 1;
    s->held = (uint32_t*)calloc((size_t)s->n, sizeof(uint32_t));
    s->refs = (size_t*)calloc((size_t)s->n, sizeof(size_t));
    s->used = (uint64_t*)calloc((size_t)s->n, sizeof(uint64_t));
    return s;
}

void po_slots_free(po_slots* s) {
    if (!s) return;
    free(s->held);
    free(s->refs);
    free(s->used);
    free(s->load_slot);
    free(s->load_id);
    free(s);
}

/* src/sched.rs:422-424 */
int po_slots_holding(const po_slots* s, uint32_t a) {
    for (int i = 1; i < s->n; i++)
        if (s->held[i] == a) return i;
    return 0;
}

/* src/sched.rs:425-427 */
int po_slots_can_place(const po_slots* s, uint32_t a) {
    if (po_slots_holding(s, a)) return 1;
    for (int i = 1; i < s->n; i++)
        if (s->refs[i] == 0) return 1;
    return 0;
}

/* src/sched.rs:430-448: the holder, else the free slot that is empty first, then least recently used
 * (min_by_key keeps the first of equal keys). */
int po_slots_place(po_slots* s, uint32_t a) {
    if (!po_slots_can_place(s, a)) return -1;
    s->clock += 1;
    int i = po_slots_holding(s, a);
    if (!i) {
        int best = 0;
        for (int j = 1; j < s->n; j++) {
            if (s->refs[j] != 0) continue;
            if (!best) {
                best = j;
                continue;
            }
            int kj = s->held[j] != 0, kb = s->held[best] != 0;
            if (kj < kb || (kj == kb && s->used[j] < s->used[best])) best = j;
        }
        i = best;
        s->held[i] = a;
        if (s->n_loads == s->cap_loads) {
            s->cap_loads = s->cap_loads ? 2 * s->cap_loads : 8;
            s->load_slot = (int32_t*)realloc(s->load_slot, sizeof(int32_t) * (size_t)s->cap_loads);
            s->load_id = (uint32_t*)realloc(s->load_id, sizeof(uint32_t) * (size_t)s->cap_loads);
        }
        s->load_slot[s->n_loads] = i;
        s->load_id[s->n_loads] = a;
        s->n_loads++;
    }
    s->refs[i] += 1;
    s->used[i] = s->clock;
    return i;
}

/* src/sched.rs:846-849 */
void po_slots_release(po_slots* s, int slot) {
    if (slot > 0 && slot < s->n && s->refs[slot] > 0) s->refs[slot] -= 1;
}

/* src/sched.rs:569-572 */
void po_slots_forget(po_slots* s, uint32_t a) {
    int i = po_slots_holding(s, a);
    if (i) s->held[i] = 0;
}

/* src/sched.rs:1018 (step.lora_loads = take(loads)) */
int po_slots_take_loads(po_slots* s, int32_t* slot_out, uint32_t* id_out, int cap) {
    int n = s->n_loads < cap ? s->n_loads : cap;
    for (int i = 0; i < n; i++) {
        slot_out[i] = s->load_slot[i];
        id_out[i] = s->load_id[i];
    }
    s->n_loads = 0;
    return n;
}

/* -------------------------------------------------------------- slab layout */

static int next_mult(int x, int m) { return (x + m - 1) / m * m; }

/* src/lora.rs:482-488 (max_rank already rounded up by the caller, :481) */
size_t po_slot_bytes(const po_site* sites, int n_sites, int max_rank) {
    size_t total = 0;
    max_rank = next_mult(max_rank, PO_RANK_STEP);
    for (int i = 0; i < n_sites; i++) {
        const po_site* s = &sites[i];
        total += (size_t)s->n_parts * (size_t)max_rank * (size_t)s->cols * 2;
        for (int p = 0; p < s->n_parts; p++) total += (size_t)s->rows[p] * (size_t)max_rank * 2;
    }
    return total;
}

static const po_module* find_module(const po_module* m, int n, int layer, const char* name) {
    for (int i = 0; i < n; i++)
        if (m[i].layer == layer && strcmp(m[i].module, name) == 0) return &m[i];
    return NULL;
}

/* src/lora.rs:307-411 */
long po_prepare(const po_site* sites, int n_sites, const po_module* modules, int n_modules, int max_rank,
                int base_gguf, int tiled_file, int hk, int hv, po_site_data* out, uint8_t* bytes, size_t cap,
                int* adapter_rank) {
    if (tiled_file && !base_gguf) return -5; /* :308-312 */
    max_rank = next_mult(max_rank, PO_RANK_STEP);
    int rank = 0;
    size_t len = 0;
    int placed = 0;
    for (int si = 0; si < n_sites; si++) { /* :320-355 layout */
        const po_site* site = &sites[si];
        po_site_data* sd = &out[si];
        memset(sd, 0, sizeof(*sd));
        int r_total = 0;
        for (int pi = 0; pi < site->n_parts; pi++) {
            const po_module* f = find_module(modules, n_modules, site->layer, site->module[pi]);
            if (!f) continue;
            placed++;
            /* shapes are implied by (r, cols, rows) here; callers pass lengths through r only, so the
             * mismatch branch (:325-330) is exercised by the product's own length-carrying API */
            int rp = next_mult(f->r, PO_RANK_STEP);
            if (rp > max_rank) return -2; /* :332-337 */
            if (f->r > rank) rank = f->r;
            sd->b_off[pi] = 0;
            sd->r_off[pi] = r_total;
            sd->r[pi] = rp;
            r_total += rp;
        }
        sd->rank = r_total;
        if (r_total > 0) {
            sd->a = len;
            len += (size_t)r_total * (size_t)site->cols * 2;
            for (int pi = 0; pi < site->n_parts; pi++)
                if (sd->r[pi] > 0) {
                    sd->b_off[pi] = len;
                    len += (size_t)site->rows[pi] * (size_t)sd->r[pi] * 2;
                }
        }
    }
    if (placed == 0 || placed < n_modules) return -3; /* :356-372 */
    if (adapter_rank) *adapter_rank = rank;
    if (!bytes) return (long)len;
    if (cap < len) return -4;
    memset(bytes, 0, len); /* :375 */
    int32_t* order = NULL;
    if (base_gguf && !tiled_file && hk != hv) { /* :315 */
        order = (int32_t*)malloc(sizeof(int32_t) * (size_t)hv);
        po_tiled_order(hk, hv, order);
    }
    for (int si = 0; si < n_sites; si++) { /* :376-403 fill */
        const po_site* site = &sites[si];
        const po_site_data* sd = &out[si];
        for (int pi = 0; pi < site->n_parts; pi++) {
            int rp = sd->r[pi];
            if (rp == 0) continue;
            const po_module* f = find_module(modules, n_modules, site->layer, site->module[pi]);
            size_t na = (size_t)f->r * (size_t)site->cols, nb = (size_t)site->rows[pi] * (size_t)f->r;
            float* a = (float*)malloc(sizeof(float) * na);
            float* b = (float*)malloc(sizeof(float) * nb);
            memcpy(a, f->a, sizeof(float) * na);
            memcpy(b, f->b, sizeof(float) * nb);
            if (order) { /* :115-135 Factors::permute, grouped -> tiled */
                if (site->heads_start[pi] >= 0)
                    po_permute_blocks(b, (size_t)site->heads_start[pi] * (size_t)f->r,
                                      (size_t)site->heads_block[pi] * (size_t)f->r, order, hv, 0);
                if (site->col_heads_start >= 0)
                    for (int row = 0; row < f->r; row++)
                        po_permute_blocks(a + (size_t)row * (size_t)site->cols, (size_t)site->col_heads_start,
                                          (size_t)site->col_heads_block, order, hv, 0);
            }
            /* A rows r_off .. r_off + r of the stacked A; padding rows stay zero (:388-393) */
            uint16_t* adst = (uint16_t*)(bytes + sd->a + (size_t)sd->r_off[pi] * (size_t)site->cols * 2);
            po_bf16_from_f32_n(a, adst, na);
            /* B [rows, rp], last rp - r columns zero (:394-401) */
            for (int row = 0; row < site->rows[pi]; row++) {
                uint16_t* bdst = (uint16_t*)(bytes + sd->b_off[pi] + (size_t)row * (size_t)rp * 2);
                po_bf16_from_f32_n(b + (size_t)row * (size_t)f->r, bdst, (size_t)f->r);
            }
            free(a);
            free(b);
        }
    }
    free(order);
    return (long)len;
}

/* src/lora.rs:597-615 */
void po_desc_for(const po_site* site, const po_site_data* sd, uint64_t base, po_desc* d) {
    memset(d, 0, sizeof(*d));
    if (sd->rank == 0) return; /* :611-613 */
    d->a = base + sd->a;
    d->rank = sd->rank;
    for (int pi = 0; pi < site->n_parts; pi++) {
        d->b[pi] = base + sd->b_off[pi];
        d->r[pi] = sd->r[pi];
        d->r_off[pi] = sd->r_off[pi];
        d->off[pi] = site->off[pi];
        d->rows[pi] = site->rows[pi];
    }
}

/* --------------------------------------------------------------- arithmetic */

/* S row of one token in fp64: s[n] = sum_k x[k] A[n,k], n < rank (lora.cuh:40-53 names the elements). */
static void shrink_row_f64(const uint16_t* x, int K, const po_desc* d, double* s) {
    const uint16_t* A = (const uint16_t*)(uintptr_t)d->a;
    for (int n = 0; n < d->rank; n++) {
        const uint16_t* an = A + (size_t)n * (size_t)K;
        double acc = 0.0;
        for (int k = 0; k < K; k++) acc += (double)po_bf16_to_f32(x[k]) * (double)po_bf16_to_f32(an[k]);
        s[n] = acc;
    }
}

enum { MODE_F64 = 0, MODE_EMUL = 1, MODE_F32S = 2 };

static void site_apply(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, void* Y,
                       int ldy, int mode, int f32_out) {
    int count = tiles[0];
    double* s = (double*)malloc(sizeof(double) * 4096);
    for (int ti = 0; ti < count; ti++) {
        int t0 = tiles[1 + 3 * ti], len = tiles[2 + 3 * ti], slot = tiles[3 + 3 * ti];
        const po_desc* d = &table[slot];
        if (d->rank == 0) continue;
        for (int row = 0; row < len; row++) {
            size_t t = (size_t)(t0 + row);
            shrink_row_f64(X + t * (size_t)ldx, K, d, s);
            if (mode == MODE_EMUL) /* S lives in f32, then bf2() rounds it (lora.cuh:96-102) */
                for (int n = 0; n < d->rank; n++) s[n] = (double)po_bf16_to_f32(po_bf16_from_f32((float)s[n]));
            else if (mode == MODE_F32S)
                for (int n = 0; n < d->rank; n++) s[n] = (double)(float)s[n];
            for (int p = 0; p < PO_MAX_PARTS; p++) {
                int r = d->r[p];
                if (r == 0) continue;
                const uint16_t* B = (const uint16_t*)(uintptr_t)d->b[p];
                const double* sp = s + d->r_off[p];
                for (int n = 0; n < d->rows[p]; n++) {
                    const uint16_t* bn = B + (size_t)n * (size_t)r;
                    double acc = 0.0;
                    for (int j = 0; j < r; j++) acc += sp[j] * (double)po_bf16_to_f32(bn[j]);
                    size_t at = t * (size_t)ldy + (size_t)d->off[p] + (size_t)n;
                    if (mode == MODE_F64) ((double*)Y)[at] += acc;
                    else if (f32_out) ((float*)Y)[at] += (float)acc; /* lora.cuh:122 */
                    else { /* lora.cuh:123 */
                        uint16_t* y = (uint16_t*)Y;
                        y[at] = po_bf16_from_f32(po_bf16_to_f32(y[at]) + (float)acc);
                    }
                }
            }
        }
    }
    free(s);
}

void po_site_f64(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, double* Y64,
                 int ldy) {
    site_apply(X, ldx, K, tiles, table, Y64, ldy, MODE_F64, 0);
}

void po_site_emul(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, void* Y, int ldy,
                  int f32_out) {
    site_apply(X, ldx, K, tiles, table, Y, ldy, MODE_EMUL, f32_out);
}

void po_site_f32s(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, void* Y, int ldy,
                  int f32_out) {
    site_apply(X, ldx, K, tiles, table, Y, ldy, MODE_F32S, f32_out);
}

/* ---- multithreaded f32 implementation: the timed CPU baseline ----
 * Same math as lora_shrink / lora_expand (src/kernels/lora.cuh:23-126) with f32 accumulation, laid out for a CPU:
 * the tokens are grouped by slot first, so a row of A or of B is read once per slot and applied to all of the
 * slot's tokens while it sits in the core's cache; the work units (slot x row of A for the shrink, slot x part x
 * 64-column block for the expand) are dealt to a pool of threads that lives across calls; the two phases of a
 * call are separated by a barrier. */

typedef struct {
    const uint16_t* X;
    int ldx, K;
    const po_desc* table;
    float* S;
    int lds;
    void* Y;
    int ldy, f32_out;
    /* tokens grouped by slot: group g holds tok[goff[g] .. goff[g + 1]) of slot gslot[g] */
    const int32_t *tok, *goff, *gslot;
    int n_groups;
    /* work units: prefix sums over the groups */
    const int32_t *shrink_units, *expand_units;
} mt_job;

static struct {
    pthread_t th[256];
    int n; /* threads including the caller */
    pthread_barrier_t go, phase, done;
    const mt_job* job;
    int quit;
} g_pool;

#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
/* 8 bf16 -> 8 f32: a bf16 is the upper half of an f32 */
static inline __m256 widen8(const uint16_t* p) {
    return _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(_mm_loadu_si128((const __m128i*)p)), 16));
}
static float dot_bf16(const uint16_t* a, const uint16_t* b, int n) {
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    int k = 0;
    for (; k + 16 <= n; k += 16) {
        acc0 = _mm256_fmadd_ps(widen8(a + k), widen8(b + k), acc0);
        acc1 = _mm256_fmadd_ps(widen8(a + k + 8), widen8(b + k + 8), acc1);
    }
    for (; k + 8 <= n; k += 8) acc0 = _mm256_fmadd_ps(widen8(a + k), widen8(b + k), acc0);
    float v[8];
    _mm256_storeu_ps(v, _mm256_add_ps(acc0, acc1));
    float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    for (; k < n; k++) s += po_bf16_to_f32(a[k]) * po_bf16_to_f32(b[k]);
    return s;
}
#else
static float dot_bf16(const uint16_t* a, const uint16_t* b, int n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int k = 0;
    for (; k + 8 <= n; k += 8)
        for (int e = 0; e < 8; e++) acc[e] += po_bf16_to_f32(a[k + e]) * po_bf16_to_f32(b[k + e]);
    float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    for (; k < n; k++) s += po_bf16_to_f32(a[k]) * po_bf16_to_f32(b[k]);
    return s;
}
#endif

static int find_group(const int32_t* prefix, int n_groups, int unit) {
    int lo = 0, hi = n_groups; /* last g with prefix[g] <= unit */
    while (hi - lo > 1) {
        int mid = (lo + hi) / 2;
        if (prefix[mid] <= unit) lo = mid;
        else hi = mid;
    }
    return lo;
}

static void mt_shrink(const mt_job* j, int tid, int nthreads) {
    const int total = j->shrink_units[j->n_groups];
    for (int u = tid; u < total; u += nthreads) {
        const int g = find_group(j->shrink_units, j->n_groups, u), n = u - j->shrink_units[g];
        const po_desc* d = &j->table[j->gslot[g]];
        const uint16_t* arow = (const uint16_t*)(uintptr_t)d->a + (size_t)n * (size_t)j->K;
        for (int i = j->goff[g]; i < j->goff[g + 1]; i++) {
            const size_t t = (size_t)j->tok[i];
            j->S[t * (size_t)j->lds + n] = dot_bf16(j->X + t * (size_t)j->ldx, arow, j->K);
        }
    }
}

static void mt_expand(const mt_job* j, int tid, int nthreads) {
    const int total = j->expand_units[j->n_groups];
    for (int u = tid; u < total; u += nthreads) {
        const int g = find_group(j->expand_units, j->n_groups, u);
        int blk = u - j->expand_units[g];
        const po_desc* d = &j->table[j->gslot[g]];
        int p = 0;
        for (; p < PO_MAX_PARTS; p++) {
            const int nb = d->r[p] ? (d->rows[p] + 63) / 64 : 0;
            if (blk < nb) break;
            blk -= nb;
        }
        if (p == PO_MAX_PARTS) continue;
        const int r = d->r[p], n1 = (blk + 1) * 64 < d->rows[p] ? (blk + 1) * 64 : d->rows[p];
        const uint16_t* B = (const uint16_t*)(uintptr_t)d->b[p];
        for (int n = blk * 64; n < n1; n++) {
            float bf[512]; /* one row of B, widened once for all of the slot's tokens */
            const uint16_t* bn = B + (size_t)n * (size_t)r;
            for (int q = 0; q < r; q++) bf[q] = po_bf16_to_f32(bn[q]);
            for (int i = j->goff[g]; i < j->goff[g + 1]; i++) {
                const size_t t = (size_t)j->tok[i];
                const float* sp = j->S + t * (size_t)j->lds + d->r_off[p];
                float acc = 0.f;
                for (int q = 0; q < r; q++) acc += sp[q] * bf[q];
                const size_t at = t * (size_t)j->ldy + (size_t)d->off[p] + (size_t)n;
                if (j->f32_out) ((float*)j->Y)[at] += acc;
                else {
                    uint16_t* y = (uint16_t*)j->Y;
                    y[at] = po_bf16_from_f32(po_bf16_to_f32(y[at]) + acc);
                }
            }
        }
    }
}

static void mt_both(const mt_job* j, int tid, int nthreads) {
    mt_shrink(j, tid, nthreads);
    pthread_barrier_wait(&g_pool.phase);
    mt_expand(j, tid, nthreads);
}

static void* pool_worker(void* arg) {
    const int tid = (int)(intptr_t)arg;
    for (;;) {
        pthread_barrier_wait(&g_pool.go);
        if (g_pool.quit) return NULL;
        mt_both(g_pool.job, tid, g_pool.n);
        pthread_barrier_wait(&g_pool.done);
    }
}

static void pool_stop(void) {
    if (g_pool.n <= 1) {
        g_pool.n = 0;
        return;
    }
    g_pool.quit = 1;
    pthread_barrier_wait(&g_pool.go);
    for (int i = 1; i < g_pool.n; i++) pthread_join(g_pool.th[i], NULL);
    pthread_barrier_destroy(&g_pool.go);
    pthread_barrier_destroy(&g_pool.phase);
    pthread_barrier_destroy(&g_pool.done);
    g_pool.n = 0;
    g_pool.quit = 0;
}

static void pool_start(int n) {
    if (g_pool.n == n) return;
    pool_stop();
    g_pool.n = n;
    if (n <= 1) return;
    pthread_barrier_init(&g_pool.go, NULL, (unsigned)n);
    pthread_barrier_init(&g_pool.phase, NULL, (unsigned)n);
    pthread_barrier_init(&g_pool.done, NULL, (unsigned)n);
    for (int i = 1; i < n; i++) pthread_create(&g_pool.th[i], NULL, pool_worker, (void*)(intptr_t)i);
}

int po_site_mt(const uint16_t* X, int ldx, int K, const int32_t* tiles, const po_desc* table, float* S, int lds,
               void* Y, int ldy, int f32_out, int n_threads) {
    if (n_threads <= 0) n_threads = po_hw_threads();
    if (n_threads > 256) n_threads = 256;
    /* tokens of the step grouped by slot (stable): count, prefix, fill */
    const int count = tiles[0];
    int max_slot = 0, n_tok = 0;
    for (int i = 0; i < count; i++) {
        if (tiles[3 + 3 * i] > max_slot) max_slot = tiles[3 + 3 * i];
        n_tok += tiles[2 + 3 * i];
    }
    int32_t* per = (int32_t*)calloc((size_t)max_slot + 2, sizeof(int32_t));
    for (int i = 0; i < count; i++) per[tiles[3 + 3 * i] + 1] += tiles[2 + 3 * i];
    int32_t* tok = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_tok + 1));
    int32_t* goff = (int32_t*)malloc(sizeof(int32_t) * (size_t)(max_slot + 2));
    int32_t* gslot = (int32_t*)malloc(sizeof(int32_t) * (size_t)(max_slot + 2));
    int32_t* su = (int32_t*)malloc(sizeof(int32_t) * (size_t)(max_slot + 2));
    int32_t* eu = (int32_t*)malloc(sizeof(int32_t) * (size_t)(max_slot + 2));
    int32_t* fill = (int32_t*)malloc(sizeof(int32_t) * (size_t)(max_slot + 2));
    int ng = 0, at = 0;
    su[0] = eu[0] = 0;
    for (int s = 1; s <= max_slot; s++) {
        fill[s] = -1;
        if (per[s + 1] == 0 || table[s].rank == 0) continue;
        const po_desc* d = &table[s];
        int blocks = 0;
        for (int p = 0; p < PO_MAX_PARTS; p++)
            if (d->r[p]) blocks += (d->rows[p] + 63) / 64;
        gslot[ng] = s;
        goff[ng] = at;
        fill[s] = at;
        at += per[s + 1];
        su[ng + 1] = su[ng] + d->rank;
        eu[ng + 1] = eu[ng] + blocks;
        ng++;
    }
    goff[ng] = at;
    for (int i = 0; i < count; i++) {
        const int s = tiles[3 + 3 * i];
        if (s < 1 || fill[s] < 0) continue;
        for (int r = 0; r < tiles[2 + 3 * i]; r++) tok[fill[s]++] = tiles[1 + 3 * i] + r;
    }
    mt_job job = {X, ldx, K, table, S, lds, Y, ldy, f32_out, tok, goff, gslot, ng, su, eu};
    pool_start(n_threads);
    if (n_threads <= 1) {
        mt_shrink(&job, 0, 1);
        mt_expand(&job, 0, 1);
    } else {
        g_pool.job = &job;
        pthread_barrier_wait(&g_pool.go);
        mt_both(&job, 0, n_threads);
        pthread_barrier_wait(&g_pool.done);
    }
    free(per);
    free(tok);
    free(goff);
    free(gslot);
    free(su);
    free(eu);
    free(fill);
    return n_threads;
}

/* ---- FP8 base layer ---- */

void po_fp8_quant_rows(const uint16_t* X, int ldx, int T, int K, uint8_t* Xq, float* st) {
    for (int t = 0; t < T; t++) {
        const uint16_t* x = X + (size_t)t * (size_t)ldx;
        float amax = 0.f;
        for (int k = 0; k < K; k++) {
            float v = fabsf(po_bf16_to_f32(x[k]));
            if (v > amax) amax = v;
        }
        float s = amax > 0.f ? amax / 448.0f : 1.0f;
        st[t] = s;
        for (int k = 0; k < K; k++) Xq[(size_t)t * (size_t)K + k] = po_e4m3_from_f32(po_bf16_to_f32(x[k]) / s);
    }
}

typedef struct {
    const uint8_t *Xq, *Wq;
    const float *st, *sn;
    int T, K, N;
    double* Y;
    int ldy, tid, nthreads;
    const float* lut;
} fp8_job;

static void* fp8_run(void* arg) {
    fp8_job* j = (fp8_job*)arg;
    float* xr = (float*)malloc(sizeof(float) * (size_t)j->K);
    for (int t = 0; t < j->T; t++) {
        for (int k = 0; k < j->K; k++) xr[k] = j->lut[j->Xq[(size_t)t * (size_t)j->K + k]];
        for (int n = j->tid; n < j->N; n += j->nthreads) {
            const uint8_t* w = j->Wq + (size_t)n * (size_t)j->K;
            double acc = 0.0;
            for (int k = 0; k < j->K; k++) acc += (double)xr[k] * (double)j->lut[w[k]];
            j->Y[(size_t)t * (size_t)j->ldy + n] = (double)j->st[t] * (double)j->sn[n] * acc;
        }
    }
    free(xr);
    return NULL;
}

void po_fp8_base_f64(const uint8_t* Xq, const float* st, const uint8_t* Wq, const float* sn, int T, int K, int N,
                     double* Y64, int ldy, int n_threads) {
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = po_e4m3_to_f32((uint8_t)i);
    if (n_threads <= 0) n_threads = po_hw_threads();
    if (n_threads > 256) n_threads = 256;
    pthread_t th[256];
    fp8_job jobs[256];
    for (int i = 0; i < n_threads; i++) {
        fp8_job j = {Xq, Wq, st, sn, T, K, N, Y64, ldy, i, n_threads, lut};
        jobs[i] = j;
        if (i > 0) pthread_create(&th[i], NULL, fp8_run, &jobs[i]);
    }
    fp8_run(&jobs[0]);
    for (int i = 1; i < n_threads; i++) pthread_join(th[i], NULL);
}
