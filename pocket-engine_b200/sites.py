"""Plain-Python pieces of the host-side mirror that need no shared library: the bf16 helpers and the layout types
of src/lora.rs (Site, SitePart, Heads, Factors). The synthetic workloads build on these alone, so that a process
which only wants the inputs (the benchmark's CPU arm) never loads libplora.so."""
import numpy as np

MAX_PARTS = 4   # src/lora.rs:14
RANK_STEP = 16  # src/lora.rs:16
TILE = 16       # src/lora.rs:18


def bf16_bits(x):
    """f32 array -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_to_f32(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------------------------- sites

class Heads:
    """src/lora.rs:23-31; ``None`` in a field stands for Heads::None."""

    def __init__(self, start, block):
        self.start, self.block = start, block


class SitePart:
    """src/lora.rs:33-41"""

    def __init__(self, module, rows, off, heads=None):
        self.module, self.rows, self.off, self.heads = module, rows, off, heads


class Site:
    """src/lora.rs:43-50"""

    def __init__(self, layer, cols, parts, col_heads=None):
        self.layer, self.cols, self.parts, self.col_heads = layer, cols, list(parts), col_heads

    @staticmethod
    def fused(layer, cols, modules):
        """A site whose parts are laid out back to back: ``modules`` is [(module path, rows), ...]."""
        parts, off = [], 0
        for m, rows in modules:
            parts.append(SitePart(m, rows, off))
            off += rows
        return Site(layer, cols, parts)

    def max_rows(self):  # src/lora.rs:52-56
        return max((p.rows for p in self.parts), default=0)

    def width(self):
        return max(p.off + p.rows for p in self.parts)


class Factors:
    """src/lora.rs:91-95: one module's A [r, cols] and B [rows, r] in f32, scale folded into B."""

    def __init__(self, layer, module, a, b):
        self.layer, self.module = layer, module
        self.a = np.ascontiguousarray(a, dtype=np.float32)
        self.b = np.ascontiguousarray(b, dtype=np.float32)
        self.r = self.a.shape[0]

    @staticmethod
    def scaled(layer, module, a, b, scale):
        """Folds ``scale`` into B in f32 as read_peft does (src/lora.rs:225-228)."""
        b = np.asarray(b, dtype=np.float32) * np.float32(scale)
        return Factors(layer, module, a, b)
