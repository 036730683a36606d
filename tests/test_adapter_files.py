"""CPU tests of the adapter readers (PEFT directories, llama.cpp GGUF adapters: src/lora.rs:148-306) and of the
adapter lifecycle around the registry (src/engine.rs:490-655). Files are synthesised the way the engine's own
integration tests do (tests/gpu.rs:947-1024): a safetensors file written by hand plus adapter_config.json."""
import json
import os
import struct

import numpy as np
import pytest


def write_safetensors(path, tensors):
    """tensors: {name: (dtype 'F32'|'BF16'|'I32', numpy array)}; the published layout: u64 header size, JSON, data."""
    header, blobs, at = {}, [], 0
    for name, (dtype, arr) in tensors.items():
        raw = arr.tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    header["__metadata__"] = {"format": "pt"}
    h = json.dumps(header).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def block_sites(pe, layers=2):
    sites = []
    for layer in range(layers):
        sites += [pe.Site.fused(layer, 64, [("self_attn.q_proj", 64), ("self_attn.k_proj", 32), ("self_attn.v_proj", 32)]),
                  pe.Site.fused(layer, 64, [("self_attn.o_proj", 64)]),
                  pe.Site.fused(layer, 64, [("mlp.gate_proj", 96), ("mlp.up_proj", 96)]),
                  pe.Site.fused(layer, 96, [("mlp.down_proj", 64)])]
    return sites


def random_modules(pe, sites, r, rng, skip=()):
    mods = {}
    for s in sites:
        for p in s.parts:
            if (s.layer, p.module) in skip:
                continue
            a = rng.standard_normal((r, s.cols), dtype=np.float32) / np.float32(np.sqrt(s.cols))
            b = rng.standard_normal((p.rows, r), dtype=np.float32) * np.float32(0.05)
            mods[(s.layer, p.module)] = (a, b)
    return mods


def write_peft(pe, out_dir, mods, r, cfg=None, bf16=False, prefix="base_model.model.model.language_model.layers"):
    os.makedirs(out_dir, exist_ok=True)
    tensors = {}
    for (layer, module), (a, b) in mods.items():
        k = f"{prefix}.{layer}.{module}"
        if bf16:
            tensors[f"{k}.lora_A.weight"] = ("BF16", pe.bf16_bits(a).reshape(a.shape))
            tensors[f"{k}.lora_B.weight"] = ("BF16", pe.bf16_bits(b).reshape(b.shape))
        else:
            tensors[f"{k}.lora_A.weight"] = ("F32", a)
            tensors[f"{k}.lora_B.weight"] = ("F32", b)
    write_safetensors(os.path.join(out_dir, "adapter_model.safetensors"), tensors)
    config = {"r": r, "lora_alpha": r, "peft_type": "LORA", "bias": "none"}
    config.update(cfg or {})
    with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
        json.dump(config, f)


def expected(pe, loras, name, mods, scale):
    fac = [pe.Factors.scaled(layer, module, a, b, scale) for (layer, module), (a, b) in mods.items()]
    return loras.prep().prepare(name, fac)


def test_peft_directory_gives_the_same_slab_as_in_memory_factors(pe, tmp_path):
    rng = np.random.default_rng(3)
    sites = block_sites(pe)
    loras = pe.Loras(sites, 2, 32, 64, device=-1)
    for case, (r, cfg, scale, bf16) in enumerate([
            (8, {}, 1.0, False),                                     # alpha = r
            (16, {"lora_alpha": 32}, 2.0, False),                    # alpha / r
            (16, {"lora_alpha": 32, "use_rslora": True}, 8.0, False),  # alpha / sqrt(r)
            (4, {"lora_alpha": None}, 2.0, True)]):                  # alpha defaults to 8; bf16 tensors
        mods = random_modules(pe, sites, r, rng, skip={(1, "mlp.up_proj"), (0, "self_attn.o_proj")})
        if bf16:  # what the file can hold
            mods = {k: (pe.bf16_to_f32(pe.bf16_bits(a)).reshape(a.shape), pe.bf16_to_f32(pe.bf16_bits(b)).reshape(b.shape))
                    for k, (a, b) in mods.items()}
        d = tmp_path / f"peft{case}"
        write_peft(pe, str(d), mods, r, cfg, bf16=bf16)
        got = loras.prep().read(f"a{case}", d)
        want = expected(pe, loras, f"a{case}", mods, scale)
        assert got.rank == want.rank and got.len == want.len
        assert np.array_equal(got.bytes(), want.bytes())
        got.drop()
        want.drop()
    loras.close()


def test_peft_reader_skips_and_rejects_like_the_engine(pe, tmp_path):
    rng = np.random.default_rng(4)
    sites = block_sites(pe, layers=1)
    loras = pe.Loras(sites, 2, 16, 64, device=-1)
    mods = random_modules(pe, sites, 8, rng)

    def read(cfg=None, extra=None, name="x"):
        d = tmp_path / f"case{read.n}"
        read.n += 1
        write_peft(pe, str(d), mods, 8, cfg)
        if extra:
            extra(d)
        return loras.prep().read(name, d)
    read.n = 0

    for cfg, text in [({"use_dora": True}, "DoRA"), ({"modules_to_save": ["lm_head"]}, "modules_to_save"),
                      ({"bias": "all"}, "biases"), ({"alpha_pattern": {"q_proj": 4}}, "alpha_pattern")]:
        with pytest.raises(pe.PloraError) as e:
            read(cfg)
        assert e.value.code == pe.ERR_CONFIG and text in e.value.text
    # tolerated: empty / null variants of the same keys
    read({"modules_to_save": None, "alpha_pattern": {}, "use_dora": False, "modules_to_save_": []}).drop()
    read({"modules_to_save": []}).drop()

    # .mtp. modules are skipped, vision modules are refused, names outside decoder layers are errors
    def add(names):
        def go(d):
            t = {}
            for (layer, module), (a, b) in mods.items():
                k = f"base_model.model.model.layers.{layer}.{module}"
                t[f"{k}.lora_A.weight"], t[f"{k}.lora_B.weight"] = ("F32", a), ("F32", b)
            for n in names:
                t[f"{n}.lora_A.weight"] = ("F32", np.zeros((8, 64), np.float32))
                t[f"{n}.lora_B.weight"] = ("F32", np.zeros((64, 8), np.float32))
            write_safetensors(os.path.join(d, "adapter_model.safetensors"), t)
        return go
    want = expected(pe, loras, "x", mods, 1.0)
    got = read(extra=add(["base_model.model.mtp.layers.0.self_attn.q_proj"]))
    assert np.array_equal(got.bytes(), want.bytes())
    with pytest.raises(pe.PloraError) as e:
        read(extra=add(["base_model.model.visual.blocks.layers.0.attn.qkv"]))
    assert "vision" in e.value.text
    with pytest.raises(pe.PloraError) as e:
        read(extra=add(["base_model.model.lm_head"]))
    assert "not a decoder layer" in e.value.text
    with pytest.raises(pe.PloraError) as e:  # a module the model does not have
        read(extra=add(["base_model.model.model.layers.0.mlp.router"]))
    assert e.value.code == pe.ERR_CONFIG
    # rank over max_rank, B of another rank, missing B, no safetensors at all, broken JSON
    big = random_modules(pe, sites, 32, rng)
    d = tmp_path / "big"
    write_peft(pe, str(d), big, 32)
    with pytest.raises(pe.PloraError) as e:
        loras.prep().read("big", d)
    assert e.value.code == pe.ERR_RANK

    def bad_b(d):
        t = {"base_model.model.model.layers.0.mlp.down_proj.lora_A.weight": ("F32", np.zeros((8, 96), np.float32)),
             "base_model.model.model.layers.0.mlp.down_proj.lora_B.weight": ("F32", np.zeros((64, 4), np.float32))}
        write_safetensors(os.path.join(d, "adapter_model.safetensors"), t)
    with pytest.raises(pe.PloraError) as e:
        read(extra=bad_b)
    assert "A is rank 8" in e.value.text

    def no_b(d):
        t = {"base_model.model.model.layers.0.mlp.down_proj.lora_A.weight": ("F32", np.zeros((8, 96), np.float32))}
        write_safetensors(os.path.join(d, "adapter_model.safetensors"), t)
    with pytest.raises(pe.PloraError) as e:
        read(extra=no_b)
    assert "missing tensor" in e.value.text
    with pytest.raises(pe.PloraError) as e:
        read(extra=lambda d: os.remove(os.path.join(d, "adapter_model.safetensors")))
    assert "no safetensors" in e.value.text
    with pytest.raises(pe.PloraError) as e:
        read(extra=lambda d: open(os.path.join(d, "adapter_config.json"), "w").write("{ not json"))
    assert "adapter_config.json" in e.value.text
    with pytest.raises(pe.PloraError):
        loras.prep().read("nowhere", tmp_path / "does-not-exist")
    want.drop()
    loras.close()


# ---------------------------------------------------------------- GGUF adapters

GGUF_NAMES = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
              "self_attn.o_proj": "attn_output", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
              "mlp.down_proj": "ffn_down", "linear_attn.in_proj_qkv": "attn_qkv", "linear_attn.in_proj_z": "attn_gate",
              "linear_attn.out_proj": "ssm_out"}


def f16_bits(a):
    return a.astype(np.float16).view(np.uint16)


def write_gguf(path, kv, tensors, align=32, version=3):
    """The published GGUF container: magic, version, counts, key-values, tensor infos, aligned data.
    tensors: [(name, dims innermost first, ggml type, raw bytes)]."""
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    out = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv))
    for k, (t, v) in kv.items():
        out += s(k) + struct.pack("<I", t)
        if t == 8:
            out += s(v)
        elif t == 6:
            out += struct.pack("<f", v)
        elif t == 4:
            out += struct.pack("<I", v)
        elif t == 9:  # an array of strings, to be skipped by readers that do not need it
            out += struct.pack("<IQ", 8, len(v)) + b"".join(s(x) for x in v)
        else:
            raise ValueError(t)
    at, infos, blobs = 0, b"", b""
    for name, dims, ty, raw in tensors:
        infos += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", ty, at)
        pad = (align - len(raw) % align) % align
        blobs += raw + b"\0" * pad
        at += len(raw) + pad
    out += infos
    out += b"\0" * ((align - len(out) % align) % align)
    with open(path, "wb") as f:
        f.write(out + blobs)


def gguf_tensors(pe, mods, kind):
    ts = []
    for (layer, module), (a, b) in mods.items():
        base = f"blk.{layer}.{GGUF_NAMES[module]}.weight"
        for suffix, m in ((".lora_a", a), (".lora_b", b)):
            dims = [m.shape[1], m.shape[0]]  # innermost first
            if kind == "f32":
                ts.append((base + suffix, dims, 0, m.astype(np.float32).tobytes()))
            elif kind == "f16":
                ts.append((base + suffix, dims, 1, f16_bits(m).tobytes()))
            else:
                ts.append((base + suffix, dims, 30, pe.bf16_bits(m).tobytes()))
    return ts


@pytest.mark.parametrize("kind", ["f32", "f16", "bf16"])
def test_gguf_adapter_gives_the_same_slab(pe, tmp_path, kind):
    rng = np.random.default_rng(5)
    sites = block_sites(pe)
    loras = pe.Loras(sites, 2, 16, 64, base_gguf=True, device=-1)
    mods = random_modules(pe, sites, 8, rng, skip={(0, "mlp.gate_proj")})
    if kind == "f16":
        mods = {k: (a.astype(np.float16).astype(np.float32), b.astype(np.float16).astype(np.float32)) for k, (a, b) in mods.items()}
    if kind == "bf16":
        mods = {k: (pe.bf16_to_f32(pe.bf16_bits(a)).reshape(a.shape), pe.bf16_to_f32(pe.bf16_bits(b)).reshape(b.shape))
                for k, (a, b) in mods.items()}
    path = tmp_path / "adapter.gguf"
    kv = {"general.architecture": (8, "qwen35"), "general.type": (8, "adapter"), "adapter.type": (8, "lora"),
          "tokenizer.list": (9, ["a", "bc"]), "adapter.lora.alpha": (6, 16.0)}
    write_gguf(str(path), kv, gguf_tensors(pe, mods, kind))
    got = loras.prep().read("g", path)
    fac = [pe.Factors.scaled(layer, module, a, b, 2.0) for (layer, module), (a, b) in mods.items()]  # alpha / r = 16 / 8
    want = loras.prep().prepare("g", fac, tiled_file=True)
    assert np.array_equal(got.bytes(), want.bytes())
    got.drop()
    want.drop()
    # no alpha: scale 1
    del kv["adapter.lora.alpha"]
    write_gguf(str(path), kv, gguf_tensors(pe, mods, kind), align=64, version=2)
    kv["general.alignment"] = (4, 64)
    write_gguf(str(path), kv, gguf_tensors(pe, mods, kind), align=64, version=2)
    got = loras.prep().read("g", path)
    want = loras.prep().prepare("g", [pe.Factors.scaled(layer, module, a, b, 1.0) for (layer, module), (a, b) in mods.items()],
                                tiled_file=True)
    assert np.array_equal(got.bytes(), want.bytes())
    got.drop()
    want.drop()
    loras.close()


def test_value_head_order_follows_the_file_kind(pe, tmp_path):
    """A llama.cpp adapter keeps value heads tiled like its GGUF base, a PEFT directory keeps them grouped
    (src/lora.rs:98-136, 307-315): on a GGUF base the GGUF adapter goes in as it is and the PEFT one is reordered;
    on a safetensors base a GGUF adapter is refused. A GDN-style layer with 2 key / 6 value heads."""
    rng = np.random.default_rng(6)
    hk, hv, dim = 2, 6, 8
    part = pe.SitePart("linear_attn.in_proj_z", hv * dim, 0, heads=pe.Heads(0, dim))
    out = pe.Site(0, hv * dim, [pe.SitePart("linear_attn.out_proj", 32, 0)], col_heads=pe.Heads(0, dim))
    sites = [pe.Site(0, 32, [part]), out]
    mods = random_modules(pe, sites, 8, rng)
    fac = [pe.Factors.scaled(l, m, a, b, 1.0) for (l, m), (a, b) in mods.items()]
    gguf = tmp_path / "heads.gguf"
    write_gguf(str(gguf), {"general.type": (8, "adapter")}, gguf_tensors(pe, mods, "f32"))
    peft = tmp_path / "heads-peft"
    write_peft(pe, str(peft), mods, 8)
    on_gguf = pe.Loras(sites, 2, 16, 64, base_gguf=True, heads=(hk, hv), device=-1)
    tiled = on_gguf.prep().prepare("h", fac, tiled_file=True)
    grouped = on_gguf.prep().prepare("h", fac, tiled_file=False)
    assert not np.array_equal(tiled.bytes(), grouped.bytes())  # the reordering does something here
    got = on_gguf.prep().read("h", gguf)
    assert np.array_equal(got.bytes(), tiled.bytes())
    got.drop()
    got = on_gguf.prep().read("h", peft)
    assert np.array_equal(got.bytes(), grouped.bytes())
    got.drop()
    on_st = pe.Loras(sites, 2, 16, 64, base_gguf=False, heads=(hk, hv), device=-1)
    with pytest.raises(pe.PloraError) as e:
        on_st.prep().read("h", gguf)
    assert "need a GGUF base" in e.value.text
    for x in (tiled, grouped):
        x.drop()
    on_gguf.close()
    on_st.close()


def test_gguf_reader_rejections(pe, tmp_path):
    rng = np.random.default_rng(7)
    sites = block_sites(pe, layers=1)
    loras = pe.Loras(sites, 2, 16, 64, base_gguf=True, device=-1)
    mods = random_modules(pe, sites, 8, rng)
    path = tmp_path / "x.gguf"
    write_gguf(str(path), {"general.type": (8, "model")}, gguf_tensors(pe, mods, "f32"))
    with pytest.raises(pe.PloraError) as e:
        loras.prep().read("x", path)
    assert "is not a LoRA adapter" in e.value.text
    write_gguf(str(path), {"general.type": (8, "adapter")}, [])
    with pytest.raises(pe.PloraError) as e:
        loras.prep().read("x", path)
    assert "no LoRA tensors" in e.value.text
    bad = dict(mods)
    a, b = bad[(0, "mlp.down_proj")]
    bad[(0, "mlp.down_proj")] = (a[:, :64], b)  # wrong input width
    write_gguf(str(path), {"general.type": (8, "adapter")}, gguf_tensors(pe, bad, "f32"))
    with pytest.raises(pe.PloraError) as e:
        loras.prep().read("x", path)
    assert "unexpected LoRA shapes" in e.value.text
    ts = gguf_tensors(pe, mods, "f32")
    ts[0] = (ts[0][0], ts[0][1], 8, ts[0][3])  # a quantised type
    write_gguf(str(path), {"general.type": (8, "adapter")}, ts)
    with pytest.raises(pe.PloraError) as e:
        loras.prep().read("x", path)
    assert "F32, F16 or BF16" in e.value.text
    open(path, "wb").write(b"GGML" + b"\0" * 64)
    with pytest.raises(pe.PloraError) as e:
        loras.prep().read("x", path)
    assert "not a GGUF file" in e.value.text
    loras.close()


# ---------------------------------------------------------------- lifecycle

def make_dirs(pe, tmp_path, sites, names, r=8):
    rng = np.random.default_rng(9)
    for n in names:
        write_peft(pe, str(tmp_path / n), random_modules(pe, sites, r, rng), r)


def test_adapter_lifecycle_loads_answers_and_evicts(pe, tmp_path):
    sites = block_sites(pe, layers=1)
    loras = pe.Loras(sites, 2, 16, 64, device=-1)
    slots = pe.LoraSlots(2)
    mgr = pe.AdapterManager(loras, slots, max_cpu_loras=2)
    make_dirs(pe, tmp_path, sites, ["a", "b", "c", "d"])
    # an explicit load, a duplicate of it while it is still being read, and on-demand waiters that join it
    t1 = mgr.load("a", tmp_path / "a")
    t_dup = mgr.load("a", tmp_path / "a")
    t_wait = mgr.load("a", tmp_path / "a", on_demand=True)
    assert mgr.loading()
    done, status, text = mgr.poll(t_dup)
    assert done and status == pe.ERR_DUPLICATE and "already loading" in text
    assert mgr.settle(t1) == (pe.OK, "")
    assert mgr.settle(t_wait) == (pe.OK, "")
    assert loras.id("a") == 1 and not mgr.loading()
    # already loaded: an error for an explicit load, fine on demand
    assert mgr.settle(mgr.load("a", tmp_path / "a"))[0] == pe.ERR_DUPLICATE
    assert mgr.settle(mgr.load("a", tmp_path / "a", on_demand=True))[0] == pe.OK
    # a broken adapter answers its ticket with the reader's text and registers nothing
    status, text = mgr.settle(mgr.load("nope", tmp_path / "nope"))
    assert status == pe.ERR_CONFIG and "nope" in text and loras.id("nope") is None
    # on demand: at most two stay resident; the least recently used idle one goes; explicit loads do not count
    for n in ("b", "c"):
        assert mgr.settle(mgr.load(n, tmp_path / n, on_demand=True))[0] == pe.OK
    assert mgr.resident_on_demand() == 2
    b_id, c_id = loras.id("b"), loras.id("c")
    mgr.submit(b_id)  # touches b and marks it in use
    assert mgr.settle(mgr.load("d", tmp_path / "d", on_demand=True))[0] == pe.OK
    assert loras.id("c") is None and loras.id("b") == b_id and loras.id("a") == 1  # c was idle and oldest
    assert mgr.resident_on_demand() == 2
    with pytest.raises(pe.PloraError) as e:
        mgr.submit(c_id)
    assert "unloaded" in e.value.text
    mgr.release(b_id)
    mgr.close()
    loras.close()


def test_unload_waits_for_the_requests_that_use_the_adapter(pe, tmp_path):
    sites = block_sites(pe, layers=1)
    loras = pe.Loras(sites, 2, 16, 64, device=-1)
    slots = pe.LoraSlots(2)
    mgr = pe.AdapterManager(loras, slots)
    make_dirs(pe, tmp_path, sites, ["a", "b"])
    for n in ("a", "b"):
        assert mgr.settle(mgr.load(n, tmp_path / n))[0] == pe.OK
    a = loras.id("a")
    mgr.submit(a)
    slot = slots.place(a)
    assert slot == 1 and slots.holding(a) == 1
    mgr.unload("a")
    assert loras.id("a") is None          # new requests can no longer name it
    assert mgr.loading()                  # draining
    mgr.submit(a)                         # the adapter itself is still resident: another request of the same
    mgr.release(a)                        # conversation could still be counted against it
    mgr.finish_loads()
    assert mgr.loading()
    slots.release(slot)
    mgr.release(a)
    mgr.finish_loads()
    assert not mgr.loading()
    with pytest.raises(pe.PloraError):
        mgr.submit(a)                     # freed now
    assert slots.holding(a) is None       # and its GPU slot was forgotten
    with pytest.raises(pe.PloraError):
        mgr.unload("a")
    mgr.unload("b")                       # idle: freed at once
    assert not mgr.loading() and loras.names() == []
    mgr.close()
    loras.close()


def test_readers_survive_damaged_files(pe, tmp_path):
    """Damaged adapter files (bytes flipped in the headers, truncation, absurd 64-bit sizes and offsets, characters
    dropped from the JSON) end in an error or in an adapter, never in an out-of-bounds read: both readers check
    every length and offset against the file before using it."""
    rng = np.random.default_rng(11)
    sites = block_sites(pe)
    loras = pe.Loras(sites, 2, 16, 64, base_gguf=True, device=-1)
    mods = random_modules(pe, sites, 8, rng)
    write_peft(pe, tmp_path / "peft", mods, 8)
    kv = {"general.architecture": (8, "qwen35"), "general.type": (8, "adapter"), "adapter.type": (8, "lora"),
          "tokenizer.list": (9, ["a", "bc"]), "adapter.lora.alpha": (6, 16.0)}
    write_gguf(str(tmp_path / "a.gguf"), kv, gguf_tensors(pe, mods, "f16"))
    good = [(tmp_path / "peft" / "adapter_model.safetensors").read_bytes(), (tmp_path / "a.gguf").read_bytes(),
            (tmp_path / "peft" / "adapter_config.json").read_bytes()]
    huge = [2 ** 63, 2 ** 64 - 1, 2 ** 40, 2 ** 32 + 5, 0]
    read = failed = 0
    for i in range(400):
        kind = int(rng.integers(0, 3))
        b = bytearray(good[kind])
        head = min(len(b), 4096)
        mode = int(rng.integers(0, 4))
        if mode == 0:
            for _ in range(int(rng.integers(1, 8))):
                b[int(rng.integers(0, head))] = int(rng.integers(0, 256))
        elif mode == 1:
            b = b[:int(rng.integers(0, len(b)))]
        elif mode == 2:
            at = int(rng.integers(0, max(1, head - 8)))
            b[at:at + 8] = struct.pack("<Q", huge[int(rng.integers(0, 5))])
        else:
            at = int(rng.integers(0, head))
            del b[at:at + int(rng.integers(1, 4))]
        if kind == 1:
            path = tmp_path / f"c{i}.gguf"
            path.write_bytes(bytes(b))
        else:
            path = tmp_path / f"c{i}"
            path.mkdir()
            (path / "adapter_model.safetensors").write_bytes(bytes(b) if kind == 0 else good[0])
            (path / "adapter_config.json").write_bytes(bytes(b) if kind == 2 else good[2])
        try:
            loras.prep().read("x", path).drop()
            read += 1
        except Exception as e:
            assert str(e)  # a message, not an empty error
            failed += 1
    assert failed > 200 and read + failed == 400
    loras.close()


def test_many_loads_in_flight_at_once(pe, tmp_path):
    """Twelve adapters started back to back (one worker thread each, two of them unreadable) while the engine
    thread keeps calling finish_loads: every ticket gets its own answer, every good adapter is registered exactly
    once with the slab a direct read gives, and closing the manager leaves no thread behind."""
    sites = block_sites(pe, layers=2)
    loras = pe.Loras(sites, 4, 16, 64, device=-1)
    mgr = pe.AdapterManager(loras)
    names = [f"ad{i}" for i in range(10)]
    make_dirs(pe, tmp_path, sites, names)
    (tmp_path / "broken").mkdir()
    (tmp_path / "broken" / "adapter_config.json").write_text("{")
    tickets = {n: mgr.load(n, tmp_path / n) for n in names}
    tickets["broken"] = mgr.load("broken", tmp_path / "broken")
    tickets["missing"] = mgr.load("missing", tmp_path / "missing")
    joined = {n: mgr.load(n, tmp_path / n, on_demand=True) for n in names[:3]}  # wait for the loads in flight
    answers = {n: mgr.settle(t) for n, t in tickets.items()}
    for n in names:
        assert answers[n] == (pe.OK, ""), (n, answers[n])
        want = loras.prep().read(n, tmp_path / n)
        assert np.array_equal(loras.adapter(loras.id(n)).bytes(), want.bytes())
        want.drop()
    for n in names[:3]:
        assert mgr.settle(joined[n]) == (pe.OK, "")
    assert answers["broken"][0] == pe.ERR_CONFIG and answers["missing"][0] == pe.ERR_CONFIG
    assert sorted(loras.names()) == sorted(names) and not mgr.loading()
    assert sorted(loras.id(n) for n in names) == list(range(1, 11))
    mgr.close()
    loras.close()
