"""TEST INFRASTRUCTURE: ctypes front end of oracle/libplora_oracle.so (plora_oracle.c), the CPU
restatement of pocket-engine's adapter path. Imported only by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline / reference arm. The product package never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libplora_oracle.so")
REF_FATBIN = os.path.join(_HERE, "_ref", "qwen35_sm100a.fatbin")
MAX_PARTS = 4


def build(force=False):
    src = os.path.join(_HERE, "plora_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libplora_oracle.so"], check=True, capture_output=True)
    return LIB_PATH


class PoDesc(C.Structure):
    _fields_ = [("a", C.c_uint64), ("b", C.c_uint64 * MAX_PARTS), ("rank", C.c_int32), ("r", C.c_int32 * MAX_PARTS),
                ("r_off", C.c_int32 * MAX_PARTS), ("off", C.c_int32 * MAX_PARTS), ("rows", C.c_int32 * MAX_PARTS),
                ("pad_", C.c_int32)]


class PoSite(C.Structure):
    _fields_ = [("layer", C.c_int32), ("cols", C.c_int32), ("n_parts", C.c_int32), ("rows", C.c_int32 * MAX_PARTS),
                ("off", C.c_int32 * MAX_PARTS), ("heads_start", C.c_int32 * MAX_PARTS),
                ("heads_block", C.c_int32 * MAX_PARTS), ("col_heads_start", C.c_int32),
                ("col_heads_block", C.c_int32), ("module", C.c_char_p * MAX_PARTS)]


class PoModule(C.Structure):
    _fields_ = [("layer", C.c_int32), ("r", C.c_int32), ("module", C.c_char_p), ("a", C.POINTER(C.c_float)),
                ("b", C.POINTER(C.c_float))]


class PoSiteData(C.Structure):
    _fields_ = [("a", C.c_uint64), ("rank", C.c_int32), ("b_off", C.c_uint64 * MAX_PARTS),
                ("r_off", C.c_int32 * MAX_PARTS), ("r", C.c_int32 * MAX_PARTS)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        I32P, U16P, U8P, F32P, F64P = (C.POINTER(t) for t in (C.c_int32, C.c_uint16, C.c_uint8, C.c_float, C.c_double))
        L.po_bf16_from_f32.restype = C.c_uint16
        L.po_bf16_from_f32.argtypes = [C.c_float]
        L.po_bf16_to_f32.restype = C.c_float
        L.po_bf16_to_f32.argtypes = [C.c_uint16]
        L.po_e4m3_from_f32.restype = C.c_uint8
        L.po_e4m3_from_f32.argtypes = [C.c_float]
        L.po_e4m3_to_f32.restype = C.c_float
        L.po_e4m3_to_f32.argtypes = [C.c_uint8]
        L.po_bf16_from_f32_n.argtypes = [F32P, U16P, C.c_size_t]
        L.po_tiled_order.argtypes = [C.c_int, C.c_int, I32P]
        L.po_permute_blocks.argtypes = [F32P, C.c_size_t, C.c_size_t, I32P, C.c_int, C.c_int]
        L.po_plan_tiles.argtypes = [I32P, I32P, C.c_int]
        L.po_fill_tiles.argtypes = [I32P, I32P, C.c_int, I32P, C.c_int]
        L.po_max_lora_tiles.argtypes = [C.c_int, C.c_int]
        L.po_slots_new.restype = C.c_void_p
        L.po_slots_new.argtypes = [C.c_int]
        L.po_slots_free.argtypes = [C.c_void_p]
        for n in ("po_slots_holding", "po_slots_can_place", "po_slots_place"):
            getattr(L, n).argtypes = [C.c_void_p, C.c_uint32]
        L.po_slots_release.argtypes = [C.c_void_p, C.c_int]
        L.po_slots_forget.argtypes = [C.c_void_p, C.c_uint32]
        L.po_slots_take_loads.argtypes = [C.c_void_p, I32P, C.POINTER(C.c_uint32), C.c_int]
        L.po_slot_bytes.restype = C.c_size_t
        L.po_slot_bytes.argtypes = [C.POINTER(PoSite), C.c_int, C.c_int]
        L.po_prepare.restype = C.c_long
        L.po_prepare.argtypes = [C.POINTER(PoSite), C.c_int, C.POINTER(PoModule), C.c_int, C.c_int, C.c_int, C.c_int,
                                 C.c_int, C.c_int, C.POINTER(PoSiteData), U8P, C.c_size_t, C.POINTER(C.c_int)]
        L.po_desc_for.argtypes = [C.POINTER(PoSite), C.POINTER(PoSiteData), C.c_uint64, C.POINTER(PoDesc)]
        L.po_site_f64.argtypes = [U16P, C.c_int, C.c_int, I32P, C.POINTER(PoDesc), F64P, C.c_int]
        for n in ("po_site_emul", "po_site_f32s"):
            getattr(L, n).argtypes = [U16P, C.c_int, C.c_int, I32P, C.POINTER(PoDesc), C.c_void_p, C.c_int, C.c_int]
        L.po_site_mt.argtypes = [U16P, C.c_int, C.c_int, I32P, C.POINTER(PoDesc), F32P, C.c_int, C.c_void_p, C.c_int,
                                 C.c_int, C.c_int]
        L.po_fp8_base_f64.argtypes = [U8P, F32P, U8P, F32P, C.c_int, C.c_int, C.c_int, F64P, C.c_int, C.c_int]
        L.po_fp8_quant_rows.argtypes = [U16P, C.c_int, C.c_int, C.c_int, U8P, F32P]
        _lib = L
    return _lib


def _p(arr, ty):
    return arr.ctypes.data_as(C.POINTER(ty))


def c_sites(sites):
    """``sites``: objects with layer, cols, parts[(module, rows, off, heads)], col_heads (the package's Site)."""
    arr = (PoSite * len(sites))()
    for i, s in enumerate(sites):
        arr[i].layer, arr[i].cols, arr[i].n_parts = s.layer, s.cols, len(s.parts)
        arr[i].col_heads_start = s.col_heads.start if s.col_heads else -1
        arr[i].col_heads_block = s.col_heads.block if s.col_heads else 0
        for p, part in enumerate(s.parts):
            arr[i].rows[p], arr[i].off[p] = part.rows, part.off
            arr[i].heads_start[p] = part.heads.start if part.heads else -1
            arr[i].heads_block[p] = part.heads.block if part.heads else 0
            arr[i].module[p] = part.module.encode()
    return arr


class OracleAdapter:
    """Host slab of one adapter (src/lora.rs:307-411) and its per-site layout."""

    def __init__(self, sites, modules, max_rank, base_gguf=False, tiled_file=False, heads=(0, 0)):
        L = lib()
        self.sites = sites
        self._cs = c_sites(sites)
        mods = (PoModule * max(1, len(modules)))()
        self._keep = []
        for i, f in enumerate(modules):
            mods[i].layer, mods[i].r = f.layer, f.r
            mods[i].module = f.module.encode()
            mods[i].a = _p(f.a, C.c_float)
            mods[i].b = _p(f.b, C.c_float)
            self._keep.append(f)
        self.sd = (PoSiteData * len(sites))()
        rank = C.c_int(0)
        args = (self._cs, len(sites), mods, len(modules), max_rank, int(base_gguf), int(tiled_file), heads[0], heads[1],
                self.sd)
        n = L.po_prepare(*args, None, 0, C.byref(rank))
        if n < 0:
            raise ValueError(f"po_prepare: {n}")
        self.len = n
        self.rank = rank.value
        self.data = np.zeros(max(n, 1), np.uint8)
        n2 = L.po_prepare(*args, _p(self.data, C.c_uint8), self.data.size, C.byref(rank))
        assert n2 == n

    def desc(self, site, base):
        d = PoDesc()
        lib().po_desc_for(C.byref(self._cs[site]), C.byref(self.sd[site]), base, C.byref(d))
        return d


class OracleTable:
    """Per-site descriptor tables over HOST slabs: table[site][slot], slot 0 all-zero (src/lora.rs:489-494)."""

    def __init__(self, sites, max_slots):
        self.sites, self.max_slots = sites, max_slots
        self.tables = [(PoDesc * (max_slots + 1))() for _ in sites]
        self._slabs = {}

    def upload(self, slot, adapter):
        self._slabs[slot] = adapter  # keeps the host bytes alive
        for si in range(len(self.sites)):
            self.tables[si][slot] = adapter.desc(si, adapter.data.ctypes.data)


def fill_tiles(row_n, row_slot, cap_tiles):
    n = np.ascontiguousarray(row_n, dtype=np.int32)
    s = np.ascontiguousarray(row_slot, dtype=np.int32)
    words = np.zeros(1 + 3 * cap_tiles, np.int32)
    c = lib().po_fill_tiles(_p(n, C.c_int32), _p(s, C.c_int32), len(n), _p(words, C.c_int32), cap_tiles)
    if c < 0:
        return None
    return words[:1 + 3 * c]


def plan_tiles(row_n, row_slot):
    n = np.ascontiguousarray(row_n, dtype=np.int32)
    s = np.ascontiguousarray(row_slot, dtype=np.int32)
    return lib().po_plan_tiles(_p(n, C.c_int32), _p(s, C.c_int32), len(n))


def site_f64(x_bits, K, tiles, table, y64):
    """y64 [T, ldy] float64, updated in place."""
    lib().po_site_f64(_p(x_bits, C.c_uint16), x_bits.shape[1], K, _p(tiles, C.c_int32), table, _p(y64, C.c_double),
                      y64.shape[1])


def site_emul(x_bits, K, tiles, table, y, f32_out):
    lib().po_site_emul(_p(x_bits, C.c_uint16), x_bits.shape[1], K, _p(tiles, C.c_int32), table,
                       C.c_void_p(y.ctypes.data), y.shape[1], int(f32_out))


def site_f32s(x_bits, K, tiles, table, y, f32_out):
    lib().po_site_f32s(_p(x_bits, C.c_uint16), x_bits.shape[1], K, _p(tiles, C.c_int32), table,
                       C.c_void_p(y.ctypes.data), y.shape[1], int(f32_out))


def site_mt(x_bits, K, tiles, table, s_scratch, y, f32_out, threads=0):
    return lib().po_site_mt(_p(x_bits, C.c_uint16), x_bits.shape[1], K, _p(tiles, C.c_int32), table,
                            _p(s_scratch, C.c_float), s_scratch.shape[1], C.c_void_p(y.ctypes.data), y.shape[1],
                            int(f32_out), threads)


def hw_threads():
    return lib().po_hw_threads()


class Slots:
    def __init__(self, n):
        self._s = lib().po_slots_new(n)
        self.n = n

    def __del__(self):
        if self._s:
            lib().po_slots_free(self._s)
            self._s = None

    def holding(self, a):
        return lib().po_slots_holding(self._s, a) or None

    def can_place(self, a):
        return bool(lib().po_slots_can_place(self._s, a))

    def place(self, a):
        return lib().po_slots_place(self._s, a)

    def release(self, s):
        lib().po_slots_release(self._s, s)

    def forget(self, a):
        lib().po_slots_forget(self._s, a)

    def take_loads(self):
        cap = 4096
        sl = (C.c_int32 * cap)()
        ids = (C.c_uint32 * cap)()
        n = lib().po_slots_take_loads(self._s, sl, ids, cap)
        return [(sl[i], ids[i]) for i in range(n)]


def fp8_quant_rows(x_bits):
    """Per-token quantisation: returns (xq uint8 [T, K], st float32 [T])."""
    T, K = x_bits.shape
    xq = np.zeros((T, K), np.uint8)
    st = np.zeros(T, np.float32)
    lib().po_fp8_quant_rows(_p(x_bits, C.c_uint16), K, T, K, _p(xq, C.c_uint8), _p(st, C.c_float))
    return xq, st


def fp8_base_f64(xq, st, wq, sn, threads=0):
    """Y64[t, n] = st[t] * sn[n] * sum_k e4m3(xq[t,k]) * e4m3(wq[n,k])."""
    T, K = xq.shape
    N = wq.shape[0]
    y = np.zeros((T, N), np.float64)
    lib().po_fp8_base_f64(_p(xq, C.c_uint8), _p(st, C.c_float), _p(wq, C.c_uint8), _p(sn, C.c_float), T, K, N,
                          _p(y, C.c_double), N, threads)
    return y
