"""The CPU oracle against the reference's own known answers (src/lora.rs:640-659), against independent
numpy restatements, and against hand-computed layouts."""
import ctypes as C

import numpy as np
import pytest

import harness


def _i32(n):
    return (C.c_int32 * n)()


def test_tiled_order_matches_the_reference_known_answer(oracle):
    # src/lora.rs:641-648: 2 key heads, 6 value heads
    out = _i32(6)
    oracle.lib().po_tiled_order(2, 6, out)
    assert list(out) == [0, 3, 1, 4, 2, 5]
    for t, g in enumerate(out):
        assert g // 3 == t % 2


def test_permutation_round_trips_like_the_reference(oracle):
    # src/lora.rs:651-659
    order = _i32(4)
    oracle.lib().po_tiled_order(2, 4, order)
    orig = np.arange(8 * 3, dtype=np.float32)
    v = orig.copy()
    p = v.ctypes.data_as(C.POINTER(C.c_float))
    oracle.lib().po_permute_blocks(p, 0, 6, order, 4, 0)
    assert not np.array_equal(v, orig)
    oracle.lib().po_permute_blocks(p, 0, 6, order, 4, 1)
    assert np.array_equal(v, orig)


def test_bf16_round_to_nearest_even(oracle, pe):
    import torch
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 3,
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40, -1e-40], np.float32)])
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got_np = pe.bf16_bits(x)
    got_c = np.array([oracle.lib().po_bf16_from_f32(float(v)) for v in x[:2000]], np.uint16)
    assert np.array_equal(got_np, want)
    assert np.array_equal(got_c, want[:2000])
    out = np.zeros(x.size, np.uint16)
    oracle.lib().po_bf16_from_f32_n(x.ctypes.data_as(C.POINTER(C.c_float)), out.ctypes.data_as(C.POINTER(C.c_uint16)),
                                    x.size)
    assert np.array_equal(out, want)


def test_e4m3_saturating_round_to_nearest_even(oracle):
    import torch
    L = oracle.lib()
    # every code decodes to what torch decodes
    codes = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    got = np.array([L.po_e4m3_to_f32(int(c)) for c in codes], np.float32)
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok], want[ok]) and np.all(np.isnan(got[~ok]))
    # encoding agrees with torch inside the finite range, ties included
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(4000).astype(np.float32) * 100, rng.standard_normal(4000).astype(np.float32),
                        rng.standard_normal(2000).astype(np.float32) * 0.01,
                        np.array([0.0, 2 ** -10, 2 ** -9, 3 * 2 ** -10, 447.9, 448.0, 17.0, 18.0, 19.0, 0.0009765625 * 1.5],
                                 np.float32)])
    x = x[np.abs(x) <= 448]
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([L.po_e4m3_from_f32(float(v)) for v in x], np.uint8)
    # torch keeps the sign of values that round to zero; so does the saturating CUDA conversion
    assert np.array_equal(got, want)
    # saturation: anything above 448 clamps to +-448 (0x7e), NaN -> 0x7f
    assert L.po_e4m3_from_f32(1e9) == 0x7E and L.po_e4m3_from_f32(-500.0) == 0xFE
    assert L.po_e4m3_from_f32(float("inf")) == 0x7E and L.po_e4m3_from_f32(float("nan")) == 0x7F
    assert L.po_e4m3_from_f32(464.0) == 0x7E


@pytest.mark.parametrize("rows,slots,want", [
    ([1], [3], [1, 0, 1, 3]),
    ([15], [2], [1, 0, 15, 2]),
    ([16], [2], [1, 0, 16, 2]),
    ([17], [2], [2, 0, 16, 2, 16, 1, 2]),
    ([33], [1], [3, 0, 16, 1, 16, 16, 1, 32, 1, 1]),
    ([1, 1, 1], [0, 0, 0], [0]),
    ([1, 1, 5, 1], [2, 0, 2, 1], [3, 0, 1, 2, 2, 5, 2, 7, 1, 1]),
    ([], [], [0]),
])
def test_tile_rule_hand_cases(oracle, rows, slots, want):
    # src/sched.rs:1096-1104: per sequence in step order, chunks of 16, slot 0 skipped, never merged
    got = oracle.fill_tiles(rows, slots, 64)
    assert list(got) == want
    assert oracle.plan_tiles(rows, slots) == want[0]


def test_tile_rule_capacity(oracle):
    assert oracle.fill_tiles([64], [1], 3) is None
    assert list(oracle.fill_tiles([64], [1], 4))[0] == 4
    assert oracle.lib().po_max_lora_tiles(4096, 64) == 4096 // 16 + 64  # src/model.rs:1346-1348


def test_slot_policy_scenario(oracle):
    # src/sched.rs:430-448: holder first; else a free slot, empty before least recently used
    s = oracle.Slots(2)
    assert s.place(7) == 1 and s.place(9) == 2
    assert s.take_loads() == [(1, 7), (2, 9)]
    assert not s.can_place(11) and s.place(11) == -1
    assert s.place(7) == 1 and s.take_loads() == []
    s.release(1)
    assert not s.can_place(11)  # slot 1 still has one user
    s.release(1)
    s.release(2)
    # both free and both holding: least recently placed wins -> slot 2 (placed at clock 2, slot 1 at 3)
    assert s.place(11) == 2 and s.take_loads() == [(2, 11)]
    assert s.holding(9) is None and s.holding(7) == 1
    s.forget(7)
    assert s.holding(7) is None
    s.release(2)
    # slot 1 is empty now: empty beats least recently used
    assert s.place(13) == 1


def test_slab_layout_hand_computed(oracle, pe):
    # a 3-part site where the adapter skips the middle part, rank 8 padded to 16; a 1-part site it skips;
    # a 2-part site with rank 24 padded to 32 on the second part only
    sites = [pe.Site.fused(0, 64, [("q", 32), ("k", 16), ("v", 16)]),
             pe.Site.fused(0, 64, [("o", 64)]),
             pe.Site.fused(1, 128, [("gate", 48), ("up", 48)])]
    rng = np.random.default_rng(3)

    def fac(layer, mod, r, cols, rows):
        return pe.Factors(layer, mod, rng.standard_normal((r, cols)).astype(np.float32),
                          rng.standard_normal((rows, r)).astype(np.float32))
    mods = [fac(0, "q", 8, 64, 32), fac(0, "v", 8, 64, 16), fac(1, "up", 24, 128, 48)]
    a = oracle.OracleAdapter(sites, mods, 32)
    assert a.rank == 24
    # site 0: stacked A [32, 64] (q rows 0..16, v rows 16..32), then B_q [32,16], B_v [16,16]
    sd = a.sd[0]
    assert (sd.a, sd.rank) == (0, 32)
    assert list(sd.r) == [16, 0, 16, 0] and list(sd.r_off) == [0, 0, 16, 0]
    assert sd.b_off[0] == 32 * 64 * 2 and sd.b_off[2] == 32 * 64 * 2 + 32 * 16 * 2
    end0 = 32 * 64 * 2 + 32 * 16 * 2 + 16 * 16 * 2
    assert a.sd[1].rank == 0
    sd2 = a.sd[2]
    assert (sd2.a, sd2.rank) == (end0, 32) and list(sd2.r) == [0, 32, 0, 0] and list(sd2.r_off) == [0, 0, 0, 0]
    assert sd2.b_off[1] == end0 + 32 * 128 * 2
    assert a.len == end0 + 32 * 128 * 2 + 48 * 32 * 2
    words = a.data[:a.len].view(np.uint16)
    A0 = words[:32 * 64].reshape(32, 64)
    assert np.array_equal(A0[:8], pe.bf16_bits(mods[0].a)) and not A0[8:16].any()
    assert np.array_equal(A0[16:24], pe.bf16_bits(mods[1].a)) and not A0[24:].any()
    Bq = words[32 * 64:32 * 64 + 32 * 16].reshape(32, 16)
    assert np.array_equal(Bq[:, :8], pe.bf16_bits(mods[0].b)) and not Bq[:, 8:].any()
    Bup = a.data[sd2.b_off[1]:a.len].view(np.uint16).reshape(48, 32)
    assert np.array_equal(Bup[:, :24], pe.bf16_bits(mods[2].b)) and not Bup[:, 24:].any()
    # descriptors: src/lora.rs:597-615
    d = a.desc(0, 1 << 20)
    assert d.a == 1 << 20 and d.rank == 32 and list(d.r) == [16, 0, 16, 0] and list(d.off) == [0, 32, 48, 0]
    assert list(d.rows) == [32, 16, 16, 0] and d.b[2] == (1 << 20) + sd.b_off[2]
    z = a.desc(1, 1 << 20)
    assert bytes(z) == bytes(112)
    # slot size: src/lora.rs:482-488
    want = sum(len(s.parts) * 32 * s.cols * 2 + sum(p.rows * 32 * 2 for p in s.parts) for s in sites)
    assert oracle.lib().po_slot_bytes(oracle.c_sites(sites), 3, 32) == want


def test_prepare_rejections(oracle, pe):
    sites = [pe.Site.fused(0, 64, [("q", 32)])]
    z = np.zeros
    with pytest.raises(ValueError, match="-2"):  # rank over max (src/lora.rs:332-337)
        oracle.OracleAdapter(sites, [pe.Factors(0, "q", z((40, 64)), z((32, 40)))], 32)
    with pytest.raises(ValueError, match="-3"):  # a module that matches no site (src/lora.rs:356-372)
        oracle.OracleAdapter(sites, [pe.Factors(0, "q", z((8, 64)), z((32, 8))),
                                     pe.Factors(5, "q", z((8, 64)), z((32, 8)))], 32)
    with pytest.raises(ValueError, match="-3"):
        oracle.OracleAdapter(sites, [], 32)
    with pytest.raises(ValueError, match="-5"):  # GGUF adapter on a non-GGUF base (src/lora.rs:308-312)
        oracle.OracleAdapter(sites, [pe.Factors(0, "q", z((8, 64)), z((32, 8)))], 32, tiled_file=True)


def test_gguf_base_permutes_value_heads(oracle, pe):
    # src/lora.rs:115-135,313-315: a PEFT adapter on a GGUF base moves value heads to tiled order
    hk, hv, blk = 2, 4, 3
    part = pe.SitePart("z", hv * blk, 0, heads=pe.Heads(0, blk))
    site_rows = pe.Site(0, 16, [part])
    site_cols = pe.Site(0, hv * blk, [pe.SitePart("out", 8, 0)], col_heads=pe.Heads(0, blk))
    rng = np.random.default_rng(5)
    f0 = pe.Factors(0, "z", rng.standard_normal((8, 16)).astype(np.float32),
                    rng.standard_normal((hv * blk, 8)).astype(np.float32))
    f1 = pe.Factors(0, "out", rng.standard_normal((8, hv * blk)).astype(np.float32),
                    rng.standard_normal((8, 8)).astype(np.float32))
    a = oracle.OracleAdapter([site_rows, site_cols], [f0, f1], 16, base_gguf=True, heads=(hk, hv))
    order = [(t % hk) * (hv // hk) + t // hk for t in range(hv)]
    B = a.data[a.sd[0].b_off[0]:a.sd[0].b_off[0] + hv * blk * 16 * 2].view(np.uint16).reshape(hv, blk, 16)
    want = pe.bf16_bits(f0.b).reshape(hv, blk, 8)[order]
    assert np.array_equal(B[:, :, :8], want)
    A = a.data[a.sd[1].a:a.sd[1].a + 16 * hv * blk * 2].view(np.uint16).reshape(16, hv, blk)
    wantA = pe.bf16_bits(f1.a).reshape(8, hv, blk)[:, order]
    assert np.array_equal(A[:8], wantA)


def _numpy_reference(pe, wl, si, tiles):
    """y64 = y_base + (x A^T)(scale B)^T in numpy fp64 over the bf16-rounded operands."""
    site = wl.sites[si]
    x = pe.bf16_to_f32(wl.x_bits(si)).reshape(wl.tokens, site.cols).astype(np.float64)
    y = wl.y_base(si).astype(np.float64)
    tslot = wl.token_slot()
    for t in range(wl.tokens):
        s = tslot[t]
        if s == 0:
            continue
        mods = {f.module: f for f in wl.factors(s - 1)}
        for part in site.parts:
            f = mods[part.module]
            a = pe.bf16_to_f32(pe.bf16_bits(f.a)).reshape(f.a.shape).astype(np.float64)
            b = pe.bf16_to_f32(pe.bf16_bits(f.b)).reshape(f.b.shape).astype(np.float64)
            y[t, part.off:part.off + part.rows] += b @ (a @ x[t])
    return y


def test_fp64_oracle_matches_numpy_on_the_plumbing_config(oracle, pe):
    from pocket_engine_b200 import workloads
    wl = workloads.config1()
    table, _ = harness.oracle_registry(wl)
    tiles = oracle.fill_tiles(wl.row_n, wl.row_slot, 32)
    assert tiles[0] == 13  # 16 tokens, every fifth is base only
    y64 = harness.oracle_f64(wl, table, tiles)[0]
    want = _numpy_reference(pe, wl, 0, tiles)
    assert np.allclose(y64, want, rtol=0, atol=1e-12)
    # base-only rows are untouched
    base = wl.y_base(0).astype(np.float64)
    for t in range(16):
        assert (t % 5 == 4) == np.array_equal(y64[t], base[t])


def test_rounded_modes_and_threaded_port_stay_within_tolerance(oracle, pe):
    from pocket_engine_b200 import workloads
    wl = workloads.config1()
    table, _ = harness.oracle_registry(wl)
    tiles = oracle.fill_tiles(wl.row_n, wl.row_slot, 32)
    y64 = harness.oracle_f64(wl, table, tiles)[0]
    for mode in ("f32s", "emul"):
        y = harness.oracle_rounded(wl, table, tiles, True, pe, mode=mode)[0]
        mx, mn = harness.tolerance(y, y64)
        # rounding S to bf16 (the reference kernels' choice) costs about 2^-9 of the adapter's share
        lim = (1e-4, 1e-5) if mode == "f32s" else (2e-3, 2e-4)
        assert mx < lim[0] and mn < lim[1], (mode, mx, mn)
    site = wl.sites[0]
    y = wl.y_base(0).copy()
    s = np.zeros((wl.tokens, 64), np.float32)
    used = oracle.site_mt(wl.x_bits(0), site.cols, tiles, table.tables[0], s, y, True, 4)
    assert used == 4
    mx, mn = harness.tolerance(y, y64)
    assert mx < 1e-4 and mn < 1e-5
    # bf16 output of the threaded port: within one bf16 step of the rounded oracle
    yb = pe.bf16_bits(wl.y_base(0)).reshape(16, 1024).copy()
    oracle.site_mt(wl.x_bits(0), site.cols, tiles, table.tables[0], s, yb, False, 3)
    want = harness.oracle_rounded(wl, table, tiles, False, pe)[0]
    assert harness.bf16_ulp_diff(pe.bf16_to_f32(yb).reshape(16, 1024), want, pe).max() <= 1


def test_zero_b_adapter_leaves_the_base_bit_identical(oracle, pe):
    # the property tests/gpu.rs:1055-1078 checks through whole-model logits
    from pocket_engine_b200 import workloads
    wl = workloads.config1()
    wl.scale = 0.0
    table, _ = harness.oracle_registry(wl)
    tiles = oracle.fill_tiles(wl.row_n, wl.row_slot, 32)
    yb = pe.bf16_bits(wl.y_base(0)).reshape(16, 1024)
    for mode in ("f32s", "emul"):
        y = yb.copy()
        fn = oracle.site_f32s if mode == "f32s" else oracle.site_emul
        fn(wl.x_bits(0), 1024, tiles, table.tables[0], y, False)
        assert np.array_equal(y, yb)
