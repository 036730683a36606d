"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle, the reference's own
kernels, and the properties the reference tests through whole-model logits (tests/gpu.rs:1055-1132)."""
import numpy as np
import pytest

import harness

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def wls():
    from pocket_engine_b200 import workloads
    return workloads


@pytest.mark.parametrize("meta", ["host", "device"])
@pytest.mark.parametrize("f32_out", [True, False])
def test_plumbing_config_matches_the_oracle(pe, wls, meta, f32_out):
    harness.run_and_check(pe, wls.config1(), f32_out=f32_out, meta=meta)


@pytest.mark.parametrize("fused,early_x", [(False, False), ("early", False), ("cluster", False), ("early", True), ("cluster", True)],
                         ids=["bracket", "apply-pair", "apply-cluster", "apply-pair-early-x", "apply-cluster-early-x"])
@pytest.mark.parametrize("f32_out", [True, False])
def test_decode_block_matches_the_oracle(pe, wls, f32_out, fused, early_x):
    res = harness.run_and_check(pe, wls.config2(), f32_out=f32_out, meta="device", fused=fused, early_x=early_x)
    assert len(res) == 4


def test_device_tiles_are_bit_exact_with_the_host_rule(pe, oracle):
    import torch
    rng = np.random.default_rng(21)
    sites = [pe.Site.fused(0, 64, [("q", 32)])]
    loras = pe.Loras(sites, 7, 16, 4096, 2100, device=0)
    cases = [([], []), ([1], [0]), ([1], [3]), ([15, 16, 17, 33], [1, 2, 0, 3]), ([2048] * 2, [5, 6])]
    for trial in range(30):
        n = int(rng.integers(1, 2100 if trial % 10 == 0 else 80))
        rows = rng.choice([1, 1, 1, 2, 15, 16, 17, 33], n).astype(np.int32)
        if rows.sum() > 4096:
            rows = np.ones(n, np.int32)
        cases.append((rows, rng.choice([0, 0, 1, 2, 3, 7], n).astype(np.int32)))
    for rows, slots in cases:
        rows, slots = np.asarray(rows, np.int32), np.asarray(slots, np.int32)
        cu = torch.from_numpy(np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)).cuda()
        ss = torch.from_numpy(np.concatenate([slots, [0]]).astype(np.int32)).cuda()
        loras.meta_build(cu.data_ptr(), ss.data_ptr(), len(rows))
        got = harness.read_tiles(loras)
        want = oracle.fill_tiles(rows, slots, loras.max_lora_tiles())
        assert np.array_equal(got, want), (rows[:10], slots[:10])
        assert np.array_equal(got, pe.fill_tiles(rows, slots, loras.max_lora_tiles()))
    loras.device_status()
    loras.close()


def test_grouping_is_a_stable_sort_by_slot(pe):
    rng = np.random.default_rng(22)
    sites = [pe.Site.fused(0, 64, [("q", 32)])]
    loras = pe.Loras(sites, 9, 16, 4096, 1500, device=0)
    loras.set_run_min(1 << 30)  # everything through the gather grouping
    for trial in range(25):
        n = int(rng.integers(1, 1400 if trial % 8 == 0 else 70))
        rows = rng.choice([1, 1, 1, 3, 16, 17, 40], n).astype(np.int32)
        if rows.sum() > 4096:
            rows = np.ones(n, np.int32)
        slots = rng.choice([0, 1, 2, 5, 9], n).astype(np.int32)
        loras.meta_upload(pe.fill_tiles(rows, slots, loras.max_lora_tiles()))
        step = loras.lora_step(loras.max_lora_tiles())
        seg = harness.SegView(loras, step)
        tslot = np.repeat(slots, rows)
        tok = np.nonzero(tslot)[0]
        order = tok[np.argsort(tslot[tok], kind="stable")]
        assert seg.status == 0 and seg.n_mma == 0
        assert np.array_equal(seg.perm, order)
        present = np.unique(tslot[tok])
        assert np.array_equal(seg.act, present)
        counts = np.array([(tslot == s).sum() for s in present])
        assert np.array_equal(seg.seg_off, np.concatenate([[0], np.cumsum(counts)]))
        # work items: each slot's segment cut into pieces of at most 16 tokens, in order
        want = [(s, o + k, min(16, c - k)) for s, o, c in zip(present, seg.seg_off, counts) for k in range(0, c, 16)]
        assert [tuple(w) for w in seg.work] == want
        assert seg.work_tokens == [list(order[o:o + c]) for _, o, c in want]
    loras.device_status()
    loras.close()


def test_long_runs_become_tensor_core_tiles(pe):
    sites = [pe.Site.fused(0, 64, [("q", 32)])]
    loras = pe.Loras(sites, 4, 16, 1024, 16, device=0)
    loras.set_run_min(64)
    rows, slots = [1, 200, 3, 64, 130, 63], [1, 2, 2, 0, 3, 3]
    # tokens: [0] s1, [1..201) s2, [201..204) s2 (contiguous with the previous: one run of 203), 64 base,
    # [268..398) s3 then [398..461) s3: one run of 193
    loras.meta_upload(pe.fill_tiles(rows, slots, loras.max_lora_tiles()))
    seg = harness.SegView(loras, loras.lora_step(loras.max_lora_tiles()))
    assert [tuple(m) for m in seg.mma] == [(1, 128, 2), (129, 75, 2), (268, 128, 3), (396, 65, 3)]
    assert list(seg.perm) == [0] and list(seg.act) == [1]
    loras.close()


def test_zero_b_adapter_leaves_the_base_bit_identical(pe, wls):
    # tests/gpu.rs:1055-1078, at the layer boundary
    wl = wls.config1()
    wl.scale = 0.0
    loras = harness.product_registry(pe, wl)
    for f32_out in (True, False):
        y = harness.run_gpu(pe, loras, wl, f32_out)[0]
        base = wl.y_base(0)
        if not f32_out:
            base = pe.bf16_to_f32(pe.bf16_bits(base)).reshape(base.shape)
        assert np.array_equal(y, base)
    loras.close()


def test_mixed_batch_equals_each_adapter_alone_bitwise(pe, wls):
    # tests/gpu.rs:1083-1132, at the layer boundary and exact: the kernels are deterministic and a token's
    # arithmetic does not depend on what else is in the batch
    wl = wls.config2(tokens=48, adapters=6)
    loras = harness.product_registry(pe, wl, max_tokens=64, max_seqs=64)
    xs = [wl.x_bits(si) for si in range(4)]
    yb = [wl.y_base(si) for si in range(4)]
    for fused in (False, "early", "cluster"):
        _mixed_equals_alone(pe, wls, wl, loras, xs, yb, fused=fused)
    loras.close()


def _mixed_equals_alone(pe, wls, wl, loras, xs, yb, fused):
    mixed = harness.run_gpu(pe, loras, wl, False, xs=xs, y_base=yb, fused=fused)
    tslot = wl.token_slot()
    for s in range(1, 7):
        idx = np.nonzero(tslot == s)[0]
        if len(idx) == 0:
            continue
        alone = wls.Workload("alone", wl.sites, wl.ranks, wl.scale, [1] * len(idx), [s] * len(idx), wl.seed)
        ya = harness.run_gpu(pe, loras, alone, False, xs=[x[idx] for x in xs], y_base=[y[idx] for y in yb], fused=fused)
        for si in range(4):
            assert np.array_equal(ya[si], mixed[si][idx]), (s, si, fused)
    # base-only tokens are untouched
    idx = np.nonzero(tslot == 0)[0]
    for si in range(4):
        want = pe.bf16_to_f32(pe.bf16_bits(yb[si][idx])).reshape(len(idx), -1)
        assert np.array_equal(mixed[si][idx], want)


RAGGED = [
    ("ragged-rows", [1, 15, 16, 17, 33, 2], [1, 2, 0, 3, 1, 2], [16, 16, 16], 256, [("a", 64), ("b", 32)]),
    ("all-base", [3, 4], [0, 0], [16], 128, [("a", 64)]),
    ("one-slot", [40], [1], [24], 512, [("a", 96), ("b", 32), ("c", 32), ("d", 64)]),
    ("odd-k", [5, 1, 1], [2, 1, 2], [8, 40], 1096, [("a", 130)]),
    ("one-token", [1], [1], [1], 64, [("a", 2)]),
    # 9 to 12 tokens of a slot: the cluster kernel takes a work item's tokens 8 at a time (second passes of 1 to 4)
    ("second-passes", [9, 10, 12, 8], [1, 2, 3, 2], [16, 32, 16], 512, [("a", 256), ("b", 64)]),
]


@pytest.mark.parametrize("case", RAGGED, ids=[c[0] for c in RAGGED])
def test_ragged_and_edge_shapes(pe, wls, case):
    name, rows, slots, ranks, K, mods = case
    sites = [pe.Site.fused(0, K, mods), pe.Site.fused(0, K, [("z", 48)])]
    wl = wls.Workload(name, sites, ranks, 1.5, rows, slots, 3)
    for f32_out in (True, False):
        for meta in ("host", "device"):
            harness.run_and_check(pe, wl, f32_out=f32_out, meta=meta)
        harness.run_and_check(pe, wl, f32_out=f32_out, fused="early")
        harness.run_and_check(pe, wl, f32_out=f32_out, fused="cluster")  # one cluster kernel per layer


def test_untargeted_parts_and_sites_are_skipped(pe, wls, oracle):
    sites = [pe.Site.fused(0, 256, [("q", 64), ("k", 32), ("v", 32)]), pe.Site.fused(0, 256, [("o", 64)])]
    wl = wls.Workload("partial", sites, [16, 8], 1.0, [3, 2, 4], [1, 2, 1], 5)
    full = wl.factors
    wl.factors = lambda i: [f for f in full(i) if (f.module in ("q", "v") if i == 0 else f.module == "o")]
    res = harness.run_and_check(pe, wl, f32_out=True)
    assert set(res) == {0, 1}
    res = harness.run_and_check(pe, wl, f32_out=False)
    for fused in ("early", "cluster"):
        harness.run_and_check(pe, wl, f32_out=True, fused=fused)
        harness.run_and_check(pe, wl, f32_out=False, fused=fused)


def test_reference_kernels_agree(pe, wls, oracle):
    """pocket-engine's own lora_shrink / lora_expand on the same descriptor tables and tile words: they
    must sit within the stated tolerance of the fp64 oracle, within rounding of the oracle's emulation
    of their rounding points, and within tolerance of the new kernels."""
    for wl in (wls.config1(), wls.config2()):
        loras = harness.product_registry(pe, wl)
        table, _ = harness.oracle_registry(wl)
        tiles = harness.tiles_of(pe, wl)
        ref = harness.run_reference_kernels(pe, loras, wl, True)
        if ref is None:
            pytest.skip("oracle/_ref fatbin is not built")
        ours = harness.run_gpu(pe, loras, wl, True)
        y64 = harness.oracle_f64(wl, table, tiles)
        emul = harness.oracle_rounded(wl, table, tiles, True, pe, mode="emul")
        for si in range(len(wl.sites)):
            mx, mn = harness.tolerance(ref[si], y64[si])
            assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL, ("ref vs f64", wl.name, si, mx, mn)
            mx, mn = harness.tolerance(ref[si], emul[si].astype(np.float64))
            assert mx <= 1e-3 and mn <= 5e-5, ("ref vs emul", wl.name, si, mx, mn)
            mx, mn = harness.tolerance(ours[si], ref[si].astype(np.float64))
            assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL, ("ours vs ref", wl.name, si, mx, mn)
        # bf16 output: the reference against its emulation, at most one bf16 step apart
        refb = harness.run_reference_kernels(pe, loras, wl, False)
        emb = harness.oracle_rounded(wl, table, tiles, False, pe, mode="emul")
        for si in range(len(wl.sites)):
            # the reference's float atomics can round an S value to the other bf16 neighbour than the oracle's
            # fp64 sum does; that moves y by up to ~5e-4 (of RMS 1), many bf16 steps when y is next to zero
            ulp = harness.bf16_ulp_diff(refb[si], emb[si], pe, floor=5e-4)
            assert ulp.max() <= 1 and (ulp > 0).mean() < 5e-3, (wl.name, si, int(ulp.max()), float((ulp > 0).mean()))
        loras.close()


def test_drop_in_kernel_image_under_the_engine_grids(pe, wls):
    """plora_compat.fatbin exports lora_shrink / lora_expand with the reference's names, signatures and
    two-buffer S contract; here it is driven exactly as the engine drives its own kernels
    (src/linear.rs:853-921) and checked against the fp64 oracle."""
    import os
    image = os.path.join(os.path.dirname(pe.LIB_PATH), "plora_compat.fatbin")
    assert os.path.exists(image)
    ragged = wls.Workload("compat-ragged", [pe.Site.fused(0, 1024, [("a", 320), ("b", 130), ("c", 64)]),
                                            pe.Site.fused(0, 1024, [("o", 200)])],
                          [8, 40, 16], 1.5, [1, 15, 16, 17, 33, 2, 1], [1, 2, 0, 3, 1, 2, 3], 3)
    for wl in (wls.config1(), wls.config2(), ragged):
        loras = harness.product_registry(pe, wl)
        table, _ = harness.oracle_registry(wl)
        tiles = harness.tiles_of(pe, wl)
        y64 = harness.oracle_f64(wl, table, tiles)
        got = harness.run_reference_kernels(pe, loras, wl, True, image=image)
        for si in range(len(wl.sites)):
            mx, mn = harness.tolerance(got[si], y64[si])
            assert mx <= 1e-5 and mn <= 1e-6, (wl.name, si, mx, mn)  # f32 S: far inside the stated tolerance
        gotb = harness.run_reference_kernels(pe, loras, wl, False, image=image)
        want = harness.oracle_rounded(wl, table, tiles, False, pe)
        for si in range(len(wl.sites)):
            ulp = harness.bf16_ulp_diff(gotb[si], want[si], pe)
            assert ulp.max() <= 1 and (ulp > 0).mean() < 2e-3, (wl.name, si, int(ulp.max()))
        loras.close()


def test_prefill_segments_reduced(pe, wls):
    wl = wls.config3(seqs=3, seq_len=160, rank=64)
    for run_min in (64, 1 << 30):  # through the tensor-core tile kernels, and through the gather kernels alone
        harness.run_and_check(pe, wl, f32_out=True, meta="device", run_min=run_min)
        harness.run_and_check(pe, wl, f32_out=False, meta="device", run_min=run_min)


TILE_CASES = [
    # name, rows per sequence, slot per sequence, ranks, K, parts
    ("three-prompts-r64", [160, 160, 160], [1, 2, 3], [64, 64, 64], 4096, [("a", 1024), ("b", 256)]),
    ("ragged-lengths-r16", [64, 65, 127, 129, 300, 5, 1], [1, 2, 1, 3, 2, 3, 1], [16, 16, 16], 512, [("a", 384)]),
    ("decode-then-prompts-r32", [1] * 20 + [128, 128], list(range(1, 5)) * 5 + [2, 3], [32] * 4, 5120,
     [("q", 768)]),
    ("odd-k-odd-width-r128", [200, 70], [1, 2], [128, 8], 1096, [("a", 1000), ("b", 130), ("c", 2)]),
    ("wide-rank-total", [256], [1], [128], 256, [("a", 128), ("b", 128), ("c", 128), ("d", 128)]),
]


@pytest.mark.parametrize("case", TILE_CASES, ids=[c[0] for c in TILE_CASES])
def test_tensor_core_tile_path(pe, wls, case):
    """Runs of 64 or more contiguous tokens of one slot go through the tcgen05 kernels; everything else in the
    same step through the gather kernels."""
    name, rows, slots, ranks, K, mods = case
    sites = [pe.Site.fused(0, K, mods)]
    wl = wls.Workload(name, sites, ranks, 1.0, rows, slots, 7)
    for f32_out in (True, False):
        harness.run_and_check(pe, wl, f32_out=f32_out, meta="device", run_min=64)
        harness.run_and_check(pe, wl, f32_out=f32_out, meta="device", run_min=64, fused="early")
        harness.run_and_check(pe, wl, f32_out=f32_out, meta="device", run_min=64, fused="cluster")


def test_tile_split_never_changes_a_bit(pe, wls):
    """However many thread blocks share a tile's K ranges, and whether the prompt runs alone or inside a larger
    batch, the tile path gives the same bits: the K ranges and the order they are added in depend on the layer
    and the adapter only."""
    mods = [("gate", 640), ("up", 640)]
    sites = [pe.Site.fused(0, 8192, mods), pe.Site.fused(0, 5120, [("q", 384)])]
    ranks = [16, 32, 64]
    mixed = wls.Workload("prompts-in-decode", sites, ranks, 1.0, [1] * 40 + [128, 200], [1, 2, 3, 0] * 10 + [1, 2], 31)
    for f32_out in (True, False):
        outs = []
        for blocks in (0, 1, 2, 4, 8):
            loras = harness.product_registry(pe, mixed)
            loras.set_run_min(64)
            loras.set_tile_split(blocks)
            outs.append(harness.run_gpu(pe, loras, mixed, f32_out, meta="device"))
            loras.close()
        for o in outs[1:]:
            for a, b in zip(outs[0], o):
                assert np.array_equal(a, b)
        # the 200-token prompt alone, in a step of its own (another automatic split): same bits for its rows
        alone = wls.Workload("prompt-alone", sites, ranks, 1.0, [200], [2], 31)
        first = mixed.tokens - 200
        xs = [mixed.x_bits(si)[first:] for si in range(2)]
        yb = [mixed.y_base(si)[first:] for si in range(2)]
        loras = harness.product_registry(pe, alone)
        loras.set_run_min(64)
        loras.set_tile_split(1)
        got = harness.run_gpu(pe, loras, alone, f32_out, meta="device", xs=xs, y_base=yb)
        loras.close()
        for si in range(2):
            assert np.array_equal(got[si], outs[0][si][first:])
    harness.run_and_check(pe, mixed, f32_out=True, meta="device", run_min=64)


def test_heterogeneous_ranks_reduced(pe, wls):
    wl = wls.config4(tokens=96, adapters=20)
    harness.run_and_check(pe, wl, f32_out=True, meta="device")
    harness.run_and_check(pe, wl, f32_out=False, meta="host")


def test_capacity_errors_are_reported_not_faulted(pe):
    import torch
    sites = [pe.Site.fused(0, 64, [("q", 32)])]
    loras = pe.Loras(sites, 2, 16, 64, 4, device=0)
    with pytest.raises(pe.PloraError) as e:  # more sequences than max_seqs
        loras.meta_build(1 << 20, 1 << 20, 5)
    assert e.value.code == pe.ERR_CAPACITY
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    step = loras.lora_step(8)
    with pytest.raises(pe.PloraError) as e:  # more rows than max_tokens
        loras.shrink(loras.hook(0), step, x.data_ptr(), 100)
    assert e.value.code == pe.ERR_CAPACITY
    with pytest.raises(pe.PloraError) as e:  # misaligned x
        loras.shrink(loras.hook(0), step, x.data_ptr() + 2, 4)
    assert e.value.code == pe.ERR_ARG
    with pytest.raises(pe.PloraError) as e:  # upload of an unknown id (src/lora.rs:590-593)
        loras.upload(1, 42)
    assert e.value.code == pe.ERR_UNKNOWN_ID
    # device side: more tiles than the region holds -> status word, count clamped to zero
    cu = torch.tensor([0, 16, 32, 48, 64], dtype=torch.int32, device="cuda")
    # cap = 64/16 + 4 = 8 tiles; 4 sequences of 16 -> 4 tiles: fits
    ss = torch.tensor([1, 1, 2, 2, 0], dtype=torch.int32, device="cuda")
    loras.meta_build(cu.data_ptr(), ss.data_ptr(), 4)
    loras.device_status()
    # a tile word list that names a slot out of range is flagged by the grouping kernel
    loras.meta_upload(np.array([1, 0, 1, 9], np.int32))
    loras.lora_step(8)
    with pytest.raises(pe.PloraError) as e:
        loras.device_status()
    assert e.value.code == pe.ERR_ARG
    # tiles that overlap one another: each is fine by itself, together they name more rows than the step has
    loras.meta_upload(np.array([8] + [0, 16, 1] * 4 + [16, 16, 2] * 4, np.int32))
    loras.lora_step(8)
    with pytest.raises(pe.PloraError) as e:
        loras.device_status()
    assert e.value.code == pe.ERR_ARG
    loras.meta_upload(np.array([2, 0, 16, 1, 16, 16, 2], np.int32))  # the same rows once: accepted
    loras.lora_step(8)
    loras.device_status()
    loras.close()


def test_kernel_profile_names_the_launches(pe, wls):
    """plora_profile_begin / _end (the engine's POCKET_PROFILE, src/gpu.rs:1741-1791): launches counted per kernel."""
    import torch
    wl = wls.config2(tokens=32, adapters=4)
    loras = harness.product_registry(pe, wl)
    loras.profile_begin()
    harness.run_gpu(pe, loras, wl, False, meta="device", fused="cluster")
    harness.run_gpu(pe, loras, wl, False, meta="device")
    prof = loras.profile_end()
    assert prof["site kernel"][0] == 4 and prof["shrink"][0] == 4 and prof["expand"][0] == 4
    assert prof["meta_group"][0] == 2 and prof["meta_tiles"][0] == 2
    assert all(us > 0 for _, us in prof.values())
    assert loras.profile_end() == {}  # closed: nothing is collected any more
    harness.run_gpu(pe, loras, wl, False)
    assert loras.profile_end() == {}
    loras.close()


def test_random_steps_match_the_oracle(pe, wls):
    """Seeded random steps: run lengths on both sides of the tile threshold and of the 128-token tile size, base-only
    sequences, ranks from 8 to 64, one to three parts, input widths that are and are not multiples of
    64, output widths that do and do not meet the alignment of tensor copies; both output types, both paths."""
    rng = np.random.default_rng(2024)
    for trial in range(8):
        K = int(rng.choice([256, 520, 1024, 2048 + 64, 4096]))
        nparts = int(rng.integers(1, 4))
        widths = [int(rng.choice([64, 130, 256, 384, 1000, 1024])) for _ in range(nparts)]
        sites = [pe.Site.fused(0, K, [(f"m{p}", w) for p, w in enumerate(widths)])]
        n_ad = int(rng.integers(2, 6))
        ranks = [int(rng.choice([8, 16, 32, 48, 64])) for _ in range(n_ad)]
        n_seq = int(rng.integers(3, 14))
        rows = [int(rng.choice([1, 1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 200, 300])) for _ in range(n_seq)]
        slots = [int(rng.integers(0, n_ad + 1)) for _ in range(n_seq)]
        wl = wls.Workload(f"random-{trial}", sites, ranks, 1.0, rows, slots, 100 + trial, max_rank=64)
        for f32_out in (True, False):
            harness.run_and_check(pe, wl, f32_out=f32_out, meta="device", run_min=64)
            harness.run_and_check(pe, wl, f32_out=f32_out, meta="device", run_min=64, fused="early")
