"""CPU tests of the C-ABI library: it loads, exports every symbol include/plora.h declares, and its
host-side registry / scheduler logic agrees bit for bit with the oracle. No compute call runs here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import harness

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(pe):
    text = open(os.path.join(ROOT, "include", "plora.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(plora_[a-z0-9_]+)\s*\(", text))
    assert declared, "no declarations parsed"
    assert declared == set(pe.SYMBOLS), declared ^ set(pe.SYMBOLS)
    lib = C.CDLL(pe.LIB_PATH)
    for name in declared:
        assert getattr(lib, name) is not None


def test_null_arguments_are_refused_not_dereferenced(pe):
    """Every entry point called with null pointers and zero sizes returns (an error status, 0 or null): a
    binding that passes a handle it failed to create must get a status back, not a crash."""
    ints = (C.c_int, C.c_uint32, C.c_uint64, C.c_size_t)
    for name, (res, args) in sorted(pe.SYMBOLS.items()):
        if name == "plora_create":
            continue
        out = getattr(pe.lib, name)(*[0 if a in ints else None for a in args])
        handle_first = args and args[0] is C.c_void_p and name not in ("plora_adapter_drop",)
        if res is C.c_int and handle_first and name.startswith(("plora_shrink", "plora_expand", "plora_apply", "plora_upload",
                                                                "plora_insert", "plora_meta", "plora_step_begin",
                                                                "plora_linear", "plora_s_", "plora_exchange")):
            assert out != 0, name


def test_compute_fails_loudly_without_a_device(pe):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    sites = [pe.Site.fused(0, 64, [("q", 32)])]
    with pytest.raises(pe.PloraError) as e:
        pe.Loras(sites, 2, 16, 16, device=0)
    assert e.value.code == pe.ERR_CUDA
    lay = pe.Loras(sites, 2, 16, 16, device=-1)  # layout-only handle
    hook = lay.hook(0)
    step = pe.StepLora()
    for call in (lambda: lay.upload(1, 1), lambda: lay.lora_step(4), lambda: lay.shrink(hook, step, 256, 1),
                 lambda: lay.expand(hook, step, 1, 256, 32), lambda: lay.meta_upload(np.zeros(1, np.int32))):
        with pytest.raises(pe.PloraError) as e:
            call()
        assert e.value.code in (pe.ERR_CUDA, pe.ERR_UNKNOWN_ID)


def _random_sites(pe, rng):
    sites = []
    for layer in range(2):
        cols = int(rng.choice([64, 128, 256]))
        nparts = int(rng.integers(1, 5))
        sites.append(pe.Site.fused(layer, cols, [(f"m{p}", int(rng.choice([16, 32, 48]))) for p in range(nparts)]))
        sites.append(pe.Site.fused(layer, int(rng.choice([64, 192])), [("out", 64)]))
    return sites


def test_prepared_slab_and_descriptors_match_the_oracle(pe, oracle):
    rng = np.random.default_rng(11)
    for trial in range(6):
        sites = _random_sites(pe, rng)
        max_rank = 48
        mods = []
        for s in sites:
            for p in s.parts:
                if rng.random() < 0.7:
                    r = int(rng.choice([1, 8, 16, 24, 40]))
                    mods.append(pe.Factors(s.layer, p.module, rng.standard_normal((r, s.cols)).astype(np.float32),
                                           rng.standard_normal((p.rows, r)).astype(np.float32)))
        # module names repeat across sites of one layer only where they are distinct parts
        seen = set()
        mods = [m for m in mods if (m.layer, m.module) not in seen and not seen.add((m.layer, m.module))]
        # "out" appears in two sites of the same layer? no: one "out" per layer
        if not mods:
            continue
        lay = pe.Loras(sites, 3, max_rank, 64, device=-1)
        want = oracle.OracleAdapter(sites, mods, max_rank)
        got = lay.prep().prepare("a", mods)
        assert got.len == want.len and got.rank == want.rank
        assert np.array_equal(got.bytes(), want.data[:want.len])
        for si in range(len(sites)):
            d, w = lay.adapter_desc(got, si, 0x7000000), want.desc(si, 0x7000000)
            assert bytes(d) == bytes(w)
        assert lay.slot_bytes == oracle.lib().po_slot_bytes(oracle.c_sites(sites), len(sites), max_rank)
        hook = lay.hook(1)
        assert (hook.parts, hook.max_rows, hook.parity, hook.cols) == (1, 64, 1, sites[1].cols)
        got.drop()
        lay.close()


def test_registry_semantics(pe):
    sites = [pe.Site.fused(0, 64, [("q", 32), ("k", 16)])]
    lay = pe.Loras(sites, 2, 16, 32, device=-1)
    prep = lay.prep()
    z = np.zeros

    def adapter(name, r=8):
        return prep.prepare(name, [pe.Factors(0, "q", z((r, 64)), z((32, r)))])
    a, b = adapter("alpha"), adapter("beta")
    assert lay.insert(a) == 1 and lay.insert(b) == 2  # ids from 1 (src/lora.rs:507,569-570)
    assert lay.names() == ["alpha", "beta"] and lay.id("beta") == 2 and lay.id("gamma") is None
    got = lay.adapter(2)  # src/lora.rs:625-627
    assert got.rank == 8 and got.len == (16 * 64 + 32 * 16) * 2 and lay.adapter(9) is None
    got.drop()  # a borrowed view: dropping it leaves the registry's adapter alone
    assert lay.adapter(2).rank == 8
    with pytest.raises(pe.PloraError) as e:  # src/lora.rs:563-568
        lay.insert(adapter("alpha"))
    assert e.value.code == pe.ERR_DUPLICATE
    assert lay.retire("alpha") == 1 and lay.retire("alpha") is None  # src/lora.rs:578-580
    assert lay.names() == ["beta"]
    lay.free(1)
    lay.free(1)  # dropping twice is harmless (src/lora.rs:583-585)
    assert lay.insert(adapter("alpha")) == 3
    # rejections of Prep::prepare
    with pytest.raises(pe.PloraError) as e:  # rank over max (src/lora.rs:332-337)
        adapter("big", 17)
    assert e.value.code == pe.ERR_RANK and "rank 17" in e.value.text
    with pytest.raises(pe.PloraError) as e:  # shapes (src/lora.rs:325-330)
        prep.prepare("bad", [pe.Factors(0, "q", z((8, 32)), z((32, 8)))])
    assert e.value.code == pe.ERR_CONFIG and "shapes" in e.value.text
    with pytest.raises(pe.PloraError) as e:  # unplaced modules (src/lora.rs:356-372)
        prep.prepare("bad", [pe.Factors(0, "q", z((8, 64)), z((32, 8))), pe.Factors(3, "q", z((8, 64)), z((32, 8)))])
    assert e.value.code == pe.ERR_CONFIG and "1 of its 2 modules" in e.value.text
    with pytest.raises(pe.PloraError) as e:
        prep.prepare("none", [])
    assert e.value.code == pe.ERR_CONFIG
    with pytest.raises(pe.PloraError) as e:  # src/lora.rs:308-312
        prep.prepare("gg", [pe.Factors(0, "q", z((8, 64)), z((32, 8)))], tiled_file=True)
    assert e.value.code == pe.ERR_CONFIG and "GGUF" in e.value.text
    lay.close()


def test_site_validation(pe):
    with pytest.raises(pe.PloraError):
        pe.Loras([pe.Site.fused(0, 60, [("q", 32)])], 2, 16, 32, device=-1)  # cols not a multiple of 8
    with pytest.raises(pe.PloraError):
        pe.Loras([pe.Site.fused(0, 64, [("q", 31)])], 2, 16, 32, device=-1)  # odd rows
    with pytest.raises(pe.PloraError):
        pe.Loras([pe.Site.fused(0, 64, [("q", 32)])], 2000, 16, 32, device=-1)  # slots over the limit
    one = pe.Loras([pe.Site.fused(0, 64, [("q", 32)])], 2, 9, 32, device=-1)  # odd site count is accepted
    assert one.max_rank == 16 and one.lds == 64  # src/lora.rs:481,491
    assert one.max_lora_tiles() == 32 // 16 + 32
    one.close()


def test_tile_rule_matches_the_oracle_bit_for_bit(pe, oracle):
    rng = np.random.default_rng(5)
    for trial in range(200):
        n = int(rng.integers(0, 40))
        rows = rng.choice([1, 1, 1, 2, 15, 16, 17, 33, 100], n).astype(np.int32)
        slots = rng.choice([0, 0, 1, 2, 3, 7], n).astype(np.int32)
        if trial % 3 == 0:
            # decode rows first, then prompt chunks (src/sched.rs:911)
            order = np.argsort(rows > 1, kind="stable")
            rows, slots = rows[order], slots[order]
        cap = int(rows.sum()) // 16 + n + 1
        want = oracle.fill_tiles(rows, slots, cap)
        got = pe.fill_tiles(rows, slots, cap)
        assert np.array_equal(got, want)
        assert pe.plan_tiles(rows, slots) == oracle.plan_tiles(rows, slots) == want[0]
    with pytest.raises(pe.PloraError) as e:
        pe.fill_tiles([64], [1], 3)
    assert e.value.code == pe.ERR_CAPACITY


def test_slot_policy_matches_the_oracle(pe, oracle):
    rng = np.random.default_rng(9)
    for trial in range(20):
        n = int(rng.integers(1, 6))
        a, b = pe.LoraSlots(n), oracle.Slots(n)
        live = []
        for step in range(300):
            op = rng.random()
            ad = int(rng.integers(1, 9))
            if op < 0.5:
                assert a.can_place(ad) == b.can_place(ad)
                if a.can_place(ad):
                    sa, sb = a.place(ad), b.place(ad)
                    assert sa == sb
                    live.append(sa)
                else:
                    with pytest.raises(pe.PloraError) as e:
                        a.place(ad)
                    assert e.value.code == pe.ERR_NO_SLOT and b.place(ad) == -1
            elif op < 0.85 and live:
                s = live.pop(int(rng.integers(0, len(live))))
                a.release(s)
                b.release(s)
            elif op < 0.92:
                a.forget(ad)
                b.forget(ad)
            else:
                assert a.take_loads() == b.take_loads()
            assert a.holding(ad) == b.holding(ad)
        assert a.take_loads() == b.take_loads()


def test_workload_accounting(pe):
    from pocket_engine_b200 import workloads
    w = workloads.config2().work()
    # 16 distinct slots present: slabs 38.80 MB, x 2.36 MB, y 7.47 MB (bf16 read + write)
    assert w["slots_present"] == 16 and w["lora_tokens"] == 48 and w["tiles"] == 48
    assert w["parts"]["slabs"] == 16 * 2 * 16 * (36864 + 38912)
    assert w["parts"]["x"] == 2 * 48 * (3 * 4096 + 12288)
    assert w["parts"]["y"] == 48 * 38912 * 4
    assert abs(w["bytes"] / 1e6 - 48.67) < 0.05
    w3 = workloads.config3().work()
    assert abs(w3["bytes"] / 1e6 - 3491.7) < 1.0 and abs(w3["flops"] / 1e9 - 158.9) < 0.2


def test_a_plain_c_program_can_use_the_library(pe, tmp_path):
    """include/plora.h compiles as C99 and a C program linked against libplora.so sees the struct layouts, the
    registry, descriptors, slot policy and tile rule the header promises (tests/cabi_consumer.c)."""
    import subprocess
    exe = tmp_path / "cabi_consumer"
    lib_dir = os.path.dirname(pe.LIB_PATH)
    build = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                            os.path.join(ROOT, "tests", "cabi_consumer.c"), "-o", str(exe), "-L", lib_dir,
                            "-l:" + os.path.basename(pe.LIB_PATH), "-Wl,-rpath," + lib_dir],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and run.stdout.strip() == "ok", run.stderr
