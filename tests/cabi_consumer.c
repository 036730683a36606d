/* A plain C consumer of include/plora.h, the way a foreign-function binding sees the library: struct layouts as
 * the header declares them, a layout-only handle (device -1: no GPU needed), the registry, the descriptor of
 * src/lora.rs:597-615, the slot policy of src/sched.rs:410-449 and the tile rule of src/sched.rs:1096-1104.
 * Built and run by tests/test_host.py; exits 0 when every check holds, otherwise prints the failed line. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "plora.h"

#define CHECK(c)                                                        \
    do {                                                                \
        if (!(c)) {                                                     \
            fprintf(stderr, "line %d: %s\n", __LINE__, #c);             \
            return 1;                                                   \
        }                                                               \
    } while (0)

int main(void) {
    CHECK(plora_abi_version() == PLORA_ABI_VERSION);
    CHECK(sizeof(plora_desc) == 112); /* src/lora.rs:59-70 */
    CHECK(sizeof(plora_hook) == 32);
    CHECK(sizeof(plora_step) == 48);

    /* one layer: fused q/k/v (64 -> 32, 16, 16) and o (32 -> 64) */
    plora_site sites[2];
    memset(sites, 0, sizeof sites);
    sites[0].layer = 0;
    sites[0].cols = 64;
    sites[0].n_parts = 3;
    sites[0].col_heads_start = -1;
    const char* names[3] = {"self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"};
    const int rows[3] = {32, 16, 16};
    int off = 0;
    for (int p = 0; p < 3; p++) {
        sites[0].parts[p].module = names[p];
        sites[0].parts[p].rows = rows[p];
        sites[0].parts[p].off = off;
        sites[0].parts[p].heads_start = -1;
        off += rows[p];
    }
    sites[1].layer = 0;
    sites[1].cols = 32;
    sites[1].n_parts = 1;
    sites[1].col_heads_start = -1;
    sites[1].parts[0].module = "self_attn.o_proj";
    sites[1].parts[0].rows = 64;
    sites[1].parts[0].heads_start = -1;

    plora_t* h = NULL;
    CHECK(plora_create(sites, 2, 0, 0, 0, /*max_slots*/ 2, /*max_rank*/ 16, /*max_tokens*/ 32, /*max_seqs*/ 8, -1, &h) == PLORA_OK);
    CHECK(h != NULL);
    /* slot_bytes = sum over sites of parts * max_rank * cols * 2 + sum rows * max_rank * 2 (src/lora.rs:482-488) */
    CHECK(plora_slot_bytes(h) == (uint64_t)(3 * 16 * 64 * 2 + 64 * 16 * 2) + (uint64_t)(1 * 16 * 32 * 2 + 64 * 16 * 2));

    /* a rank-8 adapter on q and v only: the slab pads to 16, k stays untargeted */
    static float aq[8 * 64], bq[32 * 8], av[8 * 64], bv[16 * 8];
    for (int i = 0; i < 8 * 64; i++) aq[i] = av[i] = 0.5f;
    for (int i = 0; i < 32 * 8; i++) bq[i] = 1.0f;
    for (int i = 0; i < 16 * 8; i++) bv[i] = -2.0f;
    plora_module mods[2];
    memset(mods, 0, sizeof mods);
    mods[0].layer = 0;
    mods[0].r = 8;
    mods[0].module = "self_attn.q_proj";
    mods[0].a = aq;
    mods[0].b = bq;
    mods[0].a_len = 8 * 64;
    mods[0].b_len = 32 * 8;
    mods[1] = mods[0];
    mods[1].module = "self_attn.v_proj";
    mods[1].a = av;
    mods[1].b = bv;
    mods[1].b_len = 16 * 8;
    plora_adapter_t* ad = NULL;
    CHECK(plora_adapter_prepare(h, "first", mods, 2, 0, &ad) == PLORA_OK);
    CHECK(plora_adapter_rank(ad) == 8);
    /* stacked A [32, 64] then B_q [32, 16] and B_v [16, 16], bf16 */
    CHECK(plora_adapter_len(ad) == (uint64_t)(32 * 64 + 32 * 16 + 16 * 16) * 2);
    const uint16_t* slab = (const uint16_t*)plora_adapter_data(ad);
    CHECK(slab[0] == 0x3f00);                              /* bf16(0.5): row 0 of q's A */
    CHECK(slab[8 * 64] == 0);                              /* rows 8..15 of q's block are padding */
    CHECK(slab[16 * 64] == 0x3f00);                        /* v's block starts at stacked row 16 */
    CHECK(slab[32 * 64] == 0x3f80 && slab[32 * 64 + 8] == 0); /* B_q row 0: 8 values of 1.0, then padding */
    CHECK(slab[32 * 64 + 32 * 16] == 0xc000);              /* B_v: bf16(-2.0) */

    plora_desc d;
    CHECK(plora_adapter_desc(h, ad, 0, 0x1000, &d) == PLORA_OK);
    CHECK(d.a == 0x1000 && d.rank == 32);
    CHECK(d.r[0] == 16 && d.r[1] == 0 && d.r[2] == 16);
    CHECK(d.r_off[0] == 0 && d.r_off[2] == 16);
    /* an untargeted part keeps offset 0, so its pointer is the slab's base and its rank 0 (src/lora.rs:603-606) */
    CHECK(d.b[0] == 0x1000 + 32 * 64 * 2 && d.b[1] == 0x1000 && d.b[2] == d.b[0] + 32 * 16 * 2);
    CHECK(d.off[0] == 0 && d.off[2] == 48 && d.rows[0] == 32 && d.rows[2] == 16);
    CHECK(plora_adapter_desc(h, ad, 1, 0x1000, &d) == PLORA_OK);
    CHECK(d.rank == 0); /* the adapter skips the o projection (src/lora.rs:611-613) */

    uint32_t id = 0, again = 0;
    CHECK(plora_insert(h, ad, &id) == PLORA_OK && id == 1); /* ids from 1 (src/lora.rs:507) */
    CHECK(plora_adapter_of(h, 1) == ad && plora_adapter_of(h, 2) == NULL);
    CHECK(plora_id(h, "first", &again) == PLORA_OK && again == 1);
    CHECK(plora_id(h, "second", &again) == PLORA_ERR_UNKNOWN_ID);
    char buf[64];
    CHECK(plora_names(h, buf, sizeof buf) == 1 && strcmp(buf, "first") == 0);
    plora_adapter_t* dup = NULL;
    CHECK(plora_adapter_prepare(h, "first", mods, 2, 0, &dup) == PLORA_OK);
    CHECK(plora_insert(h, dup, &again) == PLORA_ERR_DUPLICATE);
    CHECK(strstr(plora_last_error(h), "already loaded") != NULL);
    plora_adapter_drop(dup);
    mods[0].r = 24; /* pads to 32 > max_rank 16 */
    mods[0].a_len = 24 * 64;
    mods[0].b_len = 32 * 24;
    CHECK(plora_adapter_prepare(h, "wide", mods, 1, 0, &dup) == PLORA_ERR_RANK && dup == NULL);
    CHECK(strstr(plora_adapter_error(), "rank 24") != NULL);
    CHECK(plora_upload(h, 1, 1, NULL) == PLORA_ERR_CUDA); /* a layout-only handle has no device: no fallback */

    /* slot policy: reuse the holder, else an empty slot first, else the least recently placed idle one */
    plora_slots_t* s = plora_slots_new(2);
    CHECK(s != NULL);
    CHECK(plora_slots_place(s, 7) == 1 && plora_slots_place(s, 9) == 2 && plora_slots_place(s, 7) == 1);
    CHECK(plora_slots_can_place(s, 11) == 0 && plora_slots_place(s, 11) == -1);
    plora_slots_release(s, 2);
    CHECK(plora_slots_place(s, 11) == 2 && plora_slots_holding(s, 9) == 0);
    int32_t ls[4];
    uint32_t li[4];
    CHECK(plora_slots_take_loads(s, ls, li, 4) == 3 && ls[2] == 2 && li[2] == 11);
    plora_slots_free(s);

    /* tile rule: rows in step order, 16 tokens per tile, never across sequences, base-only rows skipped */
    const int32_t row_n[4] = {1, 1, 33, 16}, row_slot[4] = {2, 0, 1, 2};
    int32_t words[1 + 3 * 8];
    CHECK(plora_plan_tiles(row_n, row_slot, 4) == 5);
    CHECK(plora_fill_tiles(row_n, row_slot, 4, words, 8) == 5 && words[0] == 5);
    const int32_t want[15] = {0, 1, 2, 2, 16, 1, 18, 16, 1, 34, 1, 1, 35, 16, 2};
    CHECK(memcmp(words + 1, want, sizeof want) == 0);
    CHECK(plora_fill_tiles(row_n, row_slot, 4, words, 4) == -1); /* over capacity */

    CHECK(plora_free(h, 1) == PLORA_OK && plora_adapter_of(h, 1) == NULL);
    plora_destroy(h);
    printf("ok\n");
    return 0;
}
