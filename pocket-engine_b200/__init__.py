"""Host-side mirror of pocket-engine's adapter interface over the plora C ABI.

The names follow the engine (src/lora.rs, src/sched.rs, src/linear.rs): ``Site``/``SitePart``,
``Loras`` (the registry), ``Prep`` (off-thread preparation), ``Hook``, ``StepLora``, ``LoraSlots``
(the scheduler's slot policy), ``fill_tiles`` (the tile rule of ``Scheduler::fill``) and ``Linear``
(the bracket ``Linear::forward`` puts around a layer's own matrix multiply).

Everything that computes goes through ``libplora.so``; importing this package without the built
library raises, and there is no CPU fallback.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# PLORA_LIB points at another build of the same library (a debug or instrumented one)
LIB_PATH = os.environ.get("PLORA_LIB") or os.path.join(_HERE, "libplora.so")

MAX_PARTS = 4   # src/lora.rs:14
RANK_STEP = 16  # src/lora.rs:16
TILE = 16       # src/lora.rs:18

OK, ERR_CUDA, ERR_CONFIG, ERR_RANK, ERR_UNKNOWN_ID, ERR_DUPLICATE, ERR_NO_SLOT, ERR_TIMEOUT, ERR_ARG, \
    ERR_CAPACITY = range(10)
_CODE_NAMES = ["ok", "cuda", "config", "rank", "unknown id", "duplicate", "no slot", "timeout", "argument",
               "capacity"]


class PloraError(RuntimeError):
    """Error::Cuda / Error::Config of the engine (src/gpu.rs:19-35)."""

    def __init__(self, code, text):
        super().__init__(f"plora [{_CODE_NAMES[code] if 0 <= code < len(_CODE_NAMES) else code}]: {text}")
        self.code = code
        self.text = text


class CSitePart(C.Structure):
    _fields_ = [("module", C.c_char_p), ("rows", C.c_int32), ("off", C.c_int32), ("heads_start", C.c_int32),
                ("heads_block", C.c_int32)]


class CSite(C.Structure):
    _fields_ = [("layer", C.c_int32), ("cols", C.c_int32), ("n_parts", C.c_int32), ("col_heads_start", C.c_int32),
                ("col_heads_block", C.c_int32), ("parts", CSitePart * MAX_PARTS)]


class CModule(C.Structure):
    _fields_ = [("layer", C.c_int32), ("r", C.c_int32), ("module", C.c_char_p), ("a", C.POINTER(C.c_float)),
                ("b", C.POINTER(C.c_float)), ("a_len", C.c_uint64), ("b_len", C.c_uint64)]


class Desc(C.Structure):
    """src/lora.rs:59-70"""
    _fields_ = [("a", C.c_uint64), ("b", C.c_uint64 * MAX_PARTS), ("rank", C.c_int32), ("r", C.c_int32 * MAX_PARTS),
                ("r_off", C.c_int32 * MAX_PARTS), ("off", C.c_int32 * MAX_PARTS), ("rows", C.c_int32 * MAX_PARTS),
                ("pad_", C.c_int32)]


class Hook(C.Structure):
    """src/lora.rs:445-452"""
    _fields_ = [("table", C.c_uint64), ("parts", C.c_int32), ("max_rows", C.c_int32), ("parity", C.c_int32),
                ("cols", C.c_int32), ("site", C.c_int32), ("pad_", C.c_int32)]


class StepLora(C.Structure):
    """src/lora.rs:455-467"""
    _fields_ = [("tiles", C.c_uint64), ("s", C.c_uint64), ("s_stride", C.c_uint64), ("segs", C.c_uint64),
                ("max_tiles", C.c_int32), ("lds", C.c_int32), ("run_min", C.c_int32), ("pad_", C.c_int32)]


assert C.sizeof(Desc) == 112

# name -> (restype, argtypes); also the list of every symbol include/plora.h declares
_P = C.c_void_p
_I = C.c_int
_U64 = C.c_uint64
_I32P = C.POINTER(C.c_int32)
_U32P = C.POINTER(C.c_uint32)
SYMBOLS = {
    "plora_create": (_I, [C.POINTER(CSite), _I, _I, _I, _I, _I, _I, _I, _I, _I, C.POINTER(_P)]),
    "plora_destroy": (None, [_P]),
    "plora_last_error": (C.c_char_p, [_P]),
    "plora_bytes": (_U64, [_P]),
    "plora_slot_bytes": (_U64, [_P]),
    "plora_pool_ptr": (_U64, [_P]),
    "plora_tables_ptr": (_U64, [_P]),
    "plora_s_ptr": (_U64, [_P]),
    "plora_max_lora_tiles": (_I, [_P]),
    "plora_site_splits": (_I, [_P, _I]),
    "plora_adapter_prepare": (_I, [_P, C.c_char_p, C.POINTER(CModule), _I, _I, C.POINTER(_P)]),
    "plora_adapter_drop": (None, [_P]),
    "plora_adapter_rank": (_I, [_P]),
    "plora_adapter_len": (_U64, [_P]),
    "plora_adapter_data": (C.POINTER(C.c_uint8), [_P]),
    "plora_adapter_error": (C.c_char_p, []),
    "plora_adapter_desc": (_I, [_P, _P, _I, _U64, C.POINTER(Desc)]),
    "plora_adapter_read": (_I, [_P, C.c_char_p, C.c_char_p, C.POINTER(_P)]),
    "plora_manager_new": (_P, [_P, _P, _I]),
    "plora_manager_free": (None, [_P]),
    "plora_manager_error": (C.c_char_p, [_P]),
    "plora_manager_load": (_I, [_P, C.c_char_p, C.c_char_p, _I, C.POINTER(C.c_uint64)]),
    "plora_manager_finish_loads": (_I, [_P]),
    "plora_manager_wait": (_I, [_P, _I]),
    "plora_manager_poll": (_I, [_P, C.c_uint64, C.POINTER(_I), C.POINTER(_I), C.c_char_p, _I]),
    "plora_manager_loading": (_I, [_P]),
    "plora_manager_unload": (_I, [_P, C.c_char_p]),
    "plora_manager_submit": (_I, [_P, C.c_uint32]),
    "plora_manager_release": (None, [_P, C.c_uint32]),
    "plora_manager_resident_on_demand": (_I, [_P]),
    "plora_insert": (_I, [_P, _P, _U32P]),
    "plora_retire": (_I, [_P, C.c_char_p, _U32P]),
    "plora_free": (_I, [_P, C.c_uint32]),
    "plora_id": (_I, [_P, C.c_char_p, _U32P]),
    "plora_abi_version": (_I, []),
    "plora_bounds_build": (_I, []),
    "plora_names": (_I, [_P, C.c_char_p, C.c_size_t]),
    "plora_adapter_of": (_P, [_P, C.c_uint32]),
    "plora_upload": (_I, [_P, _I, C.c_uint32, _P]),
    "plora_hook_of": (_I, [_P, _I, C.POINTER(Hook)]),
    "plora_desc_of": (_I, [_P, _I, _I, C.POINTER(Desc)]),
    "plora_slots_new": (_P, [_I]),
    "plora_slots_free": (None, [_P]),
    "plora_slots_holding": (_I, [_P, C.c_uint32]),
    "plora_slots_can_place": (_I, [_P, C.c_uint32]),
    "plora_slots_place": (_I, [_P, C.c_uint32]),
    "plora_slots_release": (None, [_P, _I]),
    "plora_slots_forget": (None, [_P, C.c_uint32]),
    "plora_slots_take_loads": (_I, [_P, _I32P, _U32P, _I]),
    "plora_plan_tiles": (_I, [_I32P, _I32P, _I]),
    "plora_fill_tiles": (_I, [_I32P, _I32P, _I, _I32P, _I]),
    "plora_meta_build": (_I, [_P, _U64, _U64, _I, _P]),
    "plora_meta_upload": (_I, [_P, _I32P, _P]),
    "plora_step_begin": (_I, [_P, _I, _I, _P, C.POINTER(StepLora)]),
    "plora_tiles_ptr": (_U64, [_P]),
    "plora_shrink": (_I, [_P, C.POINTER(Hook), C.POINTER(StepLora), _U64, _I, _P]),
    "plora_expand": (_I, [_P, C.POINTER(Hook), C.POINTER(StepLora), _I, _U64, _I, _I, _P]),
    "plora_fp8_quant_rows": (_I, [_P, _U64, _I, _I, _U64, _U64, _P]),
    "plora_linear_fp8_fused": (_I, [_P, C.POINTER(Hook), C.POINTER(StepLora), _U64, _U64, _U64, _U64, _I, _U64, _I, _I,
                                    _P]),
    "plora_linear_bf16_fused": (_I, [_P, C.POINTER(Hook), C.POINTER(StepLora), _U64, _U64, _I, _U64, _I, _I, _P]),
    "plora_set_fused_tile_rows": (_I, [_P, _I]),
    "plora_apply": (_I, [_P, C.POINTER(Hook), C.POINTER(StepLora), _U64, _I, _U64, _I, _I, _P]),
    "plora_set_apply_mode": (_I, [_P, _I]),
    "plora_set_early_x": (_I, [_P, _I]),
    "plora_s_reduce": (_I, [_P, C.POINTER(Hook), C.POINTER(StepLora), _I, _P]),
    "plora_expand_reduced": (_I, [_P, C.POINTER(Hook), C.POINTER(StepLora), _I, _U64, _I, _I, _P]),
    "plora_exchange_create": (_I, [_P, _I, _I, _I]),
    "plora_exchange_reset": (_I, [_P, _P]),
    "plora_exchange_export": (_I, [_P, _P]),
    "plora_exchange_import": (_I, [_P, _I, _P]),
    "plora_exchange_import_local": (_I, [_P, _I, _P]),
    "plora_s_exchange": (_I, [_P, C.POINTER(Hook), C.POINTER(StepLora), _I, _P]),
    "plora_s_exchange_all_ranks": (_I, [C.POINTER(_P), C.POINTER(C.POINTER(Hook)), C.POINTER(C.POINTER(StepLora)), _I, _I,
                                        _P]),
    "plora_fork": (_I, [_P, _P, _P]),
    "plora_join": (_I, [_P, _P, _P]),
    "plora_set_run_min": (_I, [_P, _I]),
    "plora_set_tile_split": (_I, [_P, _I]),
    "plora_device_status": (_I, [_P]),
    "plora_profile_begin": (_I, [_P]),
    "plora_profile_end": (_I, [_P, C.c_char_p, C.c_size_t]),
    "plora_site_apply_static": (_I, [_U64, _I, _I, _U64, _I, _U64, _I, _I, _I, _U64, _I, _I, _P]),
    "plora_static_scratch_bytes": (_U64, []),
    "plora_static_splits": (_I, [_I]),
    "plora_static_bad_tiles": (C.c_longlong, []),
    "plora_recs_ptr": (_U64, [_P]),
    "plora_static_error": (C.c_char_p, []),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python pocket-engine_b200/build.py` "
                          "(there is no fallback path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()
ABI_VERSION = 2  # include/plora.h PLORA_ABI_VERSION
if lib.plora_abi_version() != ABI_VERSION:
    raise ImportError(f"{LIB_PATH} has ABI version {lib.plora_abi_version()}, this binding was written for {ABI_VERSION}: "
                      "rebuild it with `python pocket-engine_b200/build.py --force`")


from .sites import Factors, Heads, Site, SitePart, bf16_bits, bf16_to_f32  # noqa: E402,F401


def _c_site(site):
    """A Site as the C ABI's plora_site."""
    c = CSite()
    c.layer, c.cols, c.n_parts = site.layer, site.cols, len(site.parts)
    c.col_heads_start = site.col_heads.start if site.col_heads else -1
    c.col_heads_block = site.col_heads.block if site.col_heads else 0
    for i, p in enumerate(site.parts):
        c.parts[i].module = p.module.encode()
        c.parts[i].rows, c.parts[i].off = p.rows, p.off
        c.parts[i].heads_start = p.heads.start if p.heads else -1
        c.parts[i].heads_block = p.heads.block if p.heads else 0
    return c


class Adapter:
    """src/lora.rs:82-88. Owns the prepared host image until it is inserted into a registry."""

    def __init__(self, ptr, name):
        self._ptr, self.name = ptr, name

    @property
    def rank(self):
        return lib.plora_adapter_rank(self._ptr)

    @property
    def len(self):
        return lib.plora_adapter_len(self._ptr)

    def bytes(self):
        n = self.len
        if n == 0:
            return np.zeros(0, np.uint8)
        return np.ctypeslib.as_array(lib.plora_adapter_data(self._ptr), shape=(n,)).copy()

    def drop(self):
        if self._ptr and not getattr(self, "_borrowed", False):
            lib.plora_adapter_drop(self._ptr)
        self._ptr = None


class Prep:
    """src/lora.rs:286-293: what preparing an adapter needs; usable from a worker thread."""

    def __init__(self, loras):
        self._loras = loras

    def prepare(self, name, modules, tiled_file=False):
        """Prep::prepare (src/lora.rs:307-411) over in-memory factors."""
        arr = (CModule * max(1, len(modules)))()
        keep = []
        for i, f in enumerate(modules):
            arr[i].layer, arr[i].r = f.layer, f.r
            arr[i].module = f.module.encode()
            arr[i].a = f.a.ctypes.data_as(C.POINTER(C.c_float))
            arr[i].b = f.b.ctypes.data_as(C.POINTER(C.c_float))
            arr[i].a_len, arr[i].b_len = f.a.size, f.b.size
            keep.append(f)
        out = _P()
        rc = lib.plora_adapter_prepare(self._loras._h, name.encode(), arr, len(modules), int(tiled_file),
                                       C.byref(out))
        if rc != OK:
            raise PloraError(rc, lib.plora_adapter_error().decode())
        return Adapter(out.value, name)

    def read(self, name, path):
        """Prep::read (src/lora.rs:298-306): a PEFT directory or a llama.cpp GGUF adapter file."""
        out = _P()
        rc = lib.plora_adapter_read(self._loras._h, name.encode(), str(path).encode(), C.byref(out))
        if rc != OK:
            raise PloraError(rc, lib.plora_adapter_error().decode())
        return Adapter(out.value, name)


class AdapterManager:
    """The adapter lifecycle of src/engine.rs:490-655 around a registry: loads on worker threads, tickets for
    the answers, least-recently-used drop of on-demand adapters, unload that drains."""

    def __init__(self, loras, slots=None, max_cpu_loras=0):
        self._loras = loras
        self._m = lib.plora_manager_new(loras._h, slots._s if slots is not None else None, max_cpu_loras)
        if not self._m:
            raise PloraError(ERR_ARG, "could not create the adapter manager")

    def close(self):
        if self._m:
            lib.plora_manager_free(self._m)
            self._m = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load(self, name, path, on_demand=False):
        """Engine::start_load: returns a ticket; poll() it after finish_loads()."""
        t = C.c_uint64()
        rc = lib.plora_manager_load(self._m, name.encode(), str(path).encode(), int(on_demand), C.byref(t))
        if rc != OK:
            raise PloraError(rc, "plora_manager_load")
        return t.value

    def finish_loads(self):
        return lib.plora_manager_finish_loads(self._m)

    def wait(self, timeout_ms=1000):
        return lib.plora_manager_wait(self._m, timeout_ms)

    def poll(self, ticket):
        """(done, status, text) of a load."""
        done, status = _I(), _I()
        buf = C.create_string_buffer(512)
        rc = lib.plora_manager_poll(self._m, ticket, C.byref(done), C.byref(status), buf, 512)
        if rc != OK:
            raise PloraError(rc, "unknown ticket")
        return bool(done.value), status.value, buf.value.decode()

    def settle(self, ticket, timeout_s=30.0):
        """Runs finish_loads until the ticket is answered; returns (status, text)."""
        import time
        end = time.time() + timeout_s
        while True:
            self.finish_loads()
            done, status, text = self.poll(ticket)
            if done:
                return status, text
            if time.time() > end:
                raise TimeoutError("adapter load did not finish")
            self.wait(100)

    def loading(self):
        return bool(lib.plora_manager_loading(self._m))

    def unload(self, name):
        rc = lib.plora_manager_unload(self._m, name.encode())
        if rc != OK:
            raise PloraError(rc, lib.plora_manager_error(self._m).decode())

    def submit(self, adapter_id):
        rc = lib.plora_manager_submit(self._m, adapter_id)
        if rc != OK:
            raise PloraError(rc, lib.plora_manager_error(self._m).decode())

    def release(self, adapter_id):
        lib.plora_manager_release(self._m, adapter_id)

    def resident_on_demand(self):
        return lib.plora_manager_resident_on_demand(self._m)


class Loras:
    """src/lora.rs:416-442: adapters by id, the GPU slots and their per-layer descriptor tables."""

    def __init__(self, sites, max_slots, max_rank, max_tokens, max_seqs=None, base_gguf=False, heads=(0, 0),
                 device=0):
        self.sites = list(sites)
        self.max_slots = max_slots
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs if max_seqs is not None else max_tokens
        self.device = device
        csites = (CSite * len(self.sites))(*[_c_site(s) for s in self.sites])
        h = _P()
        rc = lib.plora_create(csites, len(self.sites), int(base_gguf), heads[0], heads[1], max_slots, max_rank,
                              max_tokens, self.max_seqs, device, C.byref(h))
        if rc != OK:
            raise PloraError(rc, lib.plora_last_error(None).decode())
        self._h = h.value
        self.max_rank = (max_rank + RANK_STEP - 1) // RANK_STEP * RANK_STEP
        self.lds = MAX_PARTS * self.max_rank

    def _check(self, rc):
        if rc != OK:
            raise PloraError(rc, lib.plora_last_error(self._h).decode())

    def close(self):
        if self._h:
            lib.plora_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def bytes(self):  # src/lora.rs:526-528
        return lib.plora_bytes(self._h)

    @property
    def slot_bytes(self):
        return lib.plora_slot_bytes(self._h)

    @property
    def pool(self):
        return lib.plora_pool_ptr(self._h)

    @property
    def s(self):
        return lib.plora_s_ptr(self._h)

    @property
    def tiles(self):
        return lib.plora_tiles_ptr(self._h)

    def max_lora_tiles(self):  # src/model.rs:1346-1348
        return lib.plora_max_lora_tiles(self._h)

    def site_splits(self, site):
        return lib.plora_site_splits(self._h, site)

    def prep(self):  # src/lora.rs:551-559
        return Prep(self)

    def hook(self, site):  # src/lora.rs:530-538
        hk = Hook()
        self._check(lib.plora_hook_of(self._h, site, C.byref(hk)))
        return hk

    def id(self, name):  # src/lora.rs:540-542
        v = C.c_uint32()
        rc = lib.plora_id(self._h, name.encode(), C.byref(v))
        return v.value if rc == OK else None

    def names(self):  # src/lora.rs:544-548
        buf = C.create_string_buffer(1 << 16)
        n = lib.plora_names(self._h, buf, len(buf))
        return buf.value.decode().split("\n") if n else []

    def adapter(self, id):  # src/lora.rs:625-627
        """The registered adapter (owned by the registry: valid until free(id)), or None."""
        ptr = lib.plora_adapter_of(self._h, id)
        if not ptr:
            return None
        a = Adapter(ptr, None)
        a._borrowed = True
        return a

    def insert(self, adapter):  # src/lora.rs:562-574
        v = C.c_uint32()
        self._check(lib.plora_insert(self._h, adapter._ptr, C.byref(v)))
        adapter._ptr = None  # the registry owns it now
        return v.value

    def retire(self, name):  # src/lora.rs:578-580
        v = C.c_uint32()
        rc = lib.plora_retire(self._h, name.encode(), C.byref(v))
        return v.value if rc == OK else None

    def free(self, id):  # src/lora.rs:583-585
        self._check(lib.plora_free(self._h, id))

    def upload(self, slot, id, stream=0):  # src/lora.rs:589-623
        self._check(lib.plora_upload(self._h, slot, id, _P(stream)))

    def desc(self, site, slot):
        d = Desc()
        self._check(lib.plora_desc_of(self._h, site, slot, C.byref(d)))
        return d

    def adapter_desc(self, adapter, site, base):
        d = Desc()
        self._check(lib.plora_adapter_desc(self._h, adapter._ptr, site, base, C.byref(d)))
        return d

    # ---- the step (src/model.rs:1603-1618, src/sched.rs:1096-1104) ----

    def meta_build(self, cu_dev, seq_slot_dev, n_seqs, stream=0):
        """Tile words from cu[n_seqs+1] / seq_slot[n_seqs] already on the device; no host round trip."""
        self._check(lib.plora_meta_build(self._h, cu_dev, seq_slot_dev, n_seqs, _P(stream)))

    def meta_upload(self, words, stream=0):
        """The engine's own route: tile words written by the scheduler on the host."""
        w = np.ascontiguousarray(words, dtype=np.int32)
        self._check(lib.plora_meta_upload(self._h, w.ctypes.data_as(_I32P), _P(stream)))
        return w

    def lora_step(self, max_tiles, stream=0, decode=False):
        """Act::lora_step(l, max_tiles, decode): groups the step's tiles by slot on the device and returns the
        StepLora. ``decode`` marks a step of few-token tiles only (no tensor-core tile kernels)."""
        st = StepLora()
        self._check(lib.plora_step_begin(self._h, max_tiles, int(decode), _P(stream), C.byref(st)))
        return st

    def set_run_min(self, tokens):
        self._check(lib.plora_set_run_min(self._h, tokens))

    def set_tile_split(self, blocks):
        """How many thread blocks share one 128-token tile's K ranges (0 = automatic); never changes a bit."""
        self._check(lib.plora_set_tile_split(self._h, blocks))

    def device_status(self):
        self._check(lib.plora_device_status(self._h))

    def profile_begin(self):
        """Starts timing every kernel launch of this registry (src/gpu.rs:1741-1791, POCKET_PROFILE)."""
        self._check(lib.plora_profile_begin(self._h))

    def profile_end(self):
        """{kernel name: (launches, microseconds)} since profile_begin."""
        buf = C.create_string_buffer(1 << 16)
        n = lib.plora_profile_end(self._h, buf, len(buf))
        if n < 0:
            self._check(-n)
        out = {}
        for line in buf.value.decode().splitlines():
            name, calls, us = line.split("\t")
            out[name] = (int(calls), float(us))
        return out

    # ---- Linear::forward's bracket ----

    def shrink(self, hook, step, x, rows, stream=0):  # src/linear.rs:853-885
        self._check(lib.plora_shrink(self._h, C.byref(hook), C.byref(step), x, rows, _P(stream)))

    def expand(self, hook, step, rows, y, ldy, f32_out=False, stream=0):  # src/linear.rs:889-921
        self._check(lib.plora_expand(self._h, C.byref(hook), C.byref(step), rows, y, ldy, int(f32_out), _P(stream)))

    def fp8_quant_rows(self, x, rows, cols, xq, st, stream=0):
        """Per-token e4m3 quantisation of bf16 activations: st[t] = amax_t / 448, xq = e4m3(x / st)."""
        self._check(lib.plora_fp8_quant_rows(self._h, x, rows, cols, xq, st, _P(stream)))

    def linear_fp8_fused(self, hook, step, xq, st, wq, sn, rows, y, ldy, f32_out=False, stream=0):
        """FP8 base layer + adapter expand in one kernel; plora_shrink on the bf16 activations goes first."""
        self._check(lib.plora_linear_fp8_fused(self._h, C.byref(hook), C.byref(step), xq, st, wq, sn, rows, y, ldy,
                                               int(f32_out), _P(stream)))

    def apply(self, hook, step, x, rows, y, ldy, f32_out=False, stream=0):
        """Shrink + expand of one layer in one call (x and y both ready): one cluster kernel per layer where the
        shapes fit, else the shrink / expand pair."""
        self._check(lib.plora_apply(self._h, C.byref(hook), C.byref(step), x, rows, y, ldy, int(f32_out), _P(stream)))

    def set_apply_mode(self, mode):
        """1 (default): apply() = one cluster kernel per layer where the shapes fit; 0: the shrink / expand pair."""
        self._check(lib.plora_set_apply_mode(self._h, mode))

    def set_early_x(self, on):
        """The caller vouches that x is complete before the kernel right before apply() starts: apply() then reads
        x ahead of its dependency wait. y is never read early."""
        self._check(lib.plora_set_early_x(self._h, int(on)))

    def linear_bf16_fused(self, hook, step, x, w, rows, y, ldy, f32_out=False, stream=0):
        """y = x w^T + adapter term in one tensor-core kernel (bf16 x [rows, cols] and w [width, cols]); shrink first."""
        self._check(lib.plora_linear_bf16_fused(self._h, C.byref(hook), C.byref(step), x, w, rows, y, ldy, int(f32_out),
                                                _P(stream)))

    def set_fused_tile_rows(self, rows):
        self._check(lib.plora_set_fused_tile_rows(self._h, rows))

    def s_reduce(self, hook, step, rows, stream=0):
        """Adds the shrink's K-split partials into plane 0 of S (before a tensor-parallel all-reduce)."""
        self._check(lib.plora_s_reduce(self._h, C.byref(hook), C.byref(step), rows, _P(stream)))

    def expand_reduced(self, hook, step, rows, y, ldy, f32_out=False, stream=0):
        """expand() from plane 0 of S alone (after s_reduce and the all-reduce)."""
        self._check(lib.plora_expand_reduced(self._h, C.byref(hook), C.byref(step), rows, y, ldy, int(f32_out),
                                             _P(stream)))

    # ---- tensor-parallel exchange of the shrink partials in one kernel per GPU ----
    def exchange_create(self, world, rank, timeout_ms=2000):
        self._check(lib.plora_exchange_create(self._h, world, rank, timeout_ms))

    def exchange_reset(self, stream=0):
        """After a timed-out exchange: flags and call counters back to zero (every rank, then a barrier)."""
        self._check(lib.plora_exchange_reset(self._h, _P(stream)))

    def exchange_export(self):
        """The 64-byte handle another process passes to exchange_import."""
        buf = C.create_string_buffer(64)
        self._check(lib.plora_exchange_export(self._h, buf))
        return buf.raw

    def exchange_import(self, peer, handle):
        self._check(lib.plora_exchange_import(self._h, peer, C.c_char_p(bytes(handle))))

    def exchange_import_local(self, peer, other):
        self._check(lib.plora_exchange_import_local(self._h, peer, other._h))

    def s_exchange(self, hook, step, rows, stream=0):
        """Sums the shrink partials of all ranks into plane 0 of S (all ranks must call it in the same order)."""
        self._check(lib.plora_s_exchange(self._h, C.byref(hook), C.byref(step), rows, _P(stream)))

    def fork(self, main=0, side=0):  # src/gpu.rs:849-858
        self._check(lib.plora_fork(self._h, _P(main), _P(side)))

    def join(self, main=0, side=0):  # src/gpu.rs:861-870
        self._check(lib.plora_join(self._h, _P(main), _P(side)))


class Linear:
    """The adapter bracket of Linear::forward (src/linear.rs:428-443,844-849): shrink forked to the side
    stream before the layer's own matrix multiply, expand after the join. ``base`` is whatever computes
    y = x W^T on the main stream (it is an input to this path, not part of it)."""

    def __init__(self, loras, site, base=None):
        self.loras, self.site, self.base = loras, site, base
        self.lora = loras.hook(site)  # Linear.lora, src/linear.rs:48-49
        self.cols = loras.sites[site].cols

    def forward(self, x, rows, y, ldy, f32_out=False, lora=None, main=0, side=None, fused=False):
        L = self.loras
        if fused:
            # the whole adapter application after the layer's own matrix multiply, one kernel per layer
            if self.base is not None:
                self.base(x, rows, y, ldy, f32_out)
            if lora is not None:
                L.apply(self.lora, lora, x, rows, y, ldy, f32_out, main)
            return
        if lora is not None:
            if side is not None and side != main:
                L.fork(main, side)
                L.shrink(self.lora, lora, x, rows, side)
            else:
                L.shrink(self.lora, lora, x, rows, main)
        if self.base is not None:
            self.base(x, rows, y, ldy, f32_out)
        if lora is not None:
            if side is not None and side != main:
                L.join(main, side)
            L.expand(self.lora, lora, rows, y, ldy, f32_out, main)


def s_exchange_all_ranks(ranks, hooks, steps, rows, stream=0):
    """plora_s_exchange for every rank of one process on one device in a single cooperative launch; ranks[r] is
    the Loras of rank r."""
    n = len(ranks)
    hs = (_P * n)(*[r._h for r in ranks])
    hk = (C.POINTER(Hook) * n)(*[C.pointer(h) for h in hooks])
    st = (C.POINTER(StepLora) * n)(*[C.pointer(s) for s in steps])
    rc = lib.plora_s_exchange_all_ranks(hs, hk, st, n, rows, _P(stream))
    if rc != 0:
        ranks[0]._check(rc)


def site_apply_static(x, rows, cols, tiles, max_tiles, hook, lds, y, ldy, f32_out=False, stream=0):
    """One layer's shrink + expand for callers that cannot allocate device memory (an engine whose memory is
    fully claimed at start-up, a plugin host that forbids allocation): the f32 intermediate sits in a fixed
    8 MiB array inside the library. Calls on one device must not overlap on the GPU; sizes over the array raise
    a capacity error. ``hook`` supplies the layer's descriptor table, part count and widest part."""
    rc = lib.plora_site_apply_static(x, rows, cols, tiles, max_tiles, hook.table, hook.parts, hook.max_rows, lds, y,
                                     ldy, int(f32_out), _P(stream))
    if rc != OK:
        raise PloraError(rc, lib.plora_static_error().decode())


# ----------------------------------------------------------------------------- scheduler side

class LoraSlots:
    """src/sched.rs:410-449"""

    def __init__(self, slots):
        self._s = lib.plora_slots_new(slots)
        self.slots = slots

    def __del__(self):
        try:
            if self._s:
                lib.plora_slots_free(self._s)
                self._s = None
        except Exception:
            pass

    def holding(self, a):
        v = lib.plora_slots_holding(self._s, a)
        return v if v else None

    def can_place(self, a):
        return bool(lib.plora_slots_can_place(self._s, a))

    def place(self, a):
        v = lib.plora_slots_place(self._s, a)
        if v < 0:
            raise PloraError(ERR_NO_SLOT, f"no slot for adapter {a}")
        return v

    def release(self, slot):
        lib.plora_slots_release(self._s, slot)

    def forget(self, a):
        lib.plora_slots_forget(self._s, a)

    def take_loads(self):
        cap = self.slots + 1
        sl = (C.c_int32 * cap)()
        ids = (C.c_uint32 * cap)()
        out = []
        while True:
            n = lib.plora_slots_take_loads(self._s, sl, ids, cap)
            out += [(sl[i], ids[i]) for i in range(n)]
            if n < cap:
                break
        return out


def plan_tiles(row_n, row_slot):
    """src/sched.rs:1019-1025"""
    n = np.ascontiguousarray(row_n, dtype=np.int32)
    s = np.ascontiguousarray(row_slot, dtype=np.int32)
    return lib.plora_plan_tiles(n.ctypes.data_as(_I32P), s.ctypes.data_as(_I32P), len(n))


def fill_tiles(row_n, row_slot, cap_tiles):
    """src/sched.rs:1096-1104,1189: the step's tile words [count, (start, len, slot) x count]."""
    n = np.ascontiguousarray(row_n, dtype=np.int32)
    s = np.ascontiguousarray(row_slot, dtype=np.int32)
    words = np.zeros(1 + 3 * cap_tiles, np.int32)
    c = lib.plora_fill_tiles(n.ctypes.data_as(_I32P), s.ctypes.data_as(_I32P), len(n), words.ctypes.data_as(_I32P),
                             cap_tiles)
    if c < 0:
        raise PloraError(ERR_CAPACITY, "more tiles than the metadata holds")
    return words[:1 + 3 * c]
