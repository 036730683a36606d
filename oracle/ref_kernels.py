"""TEST INFRASTRUCTURE: drives pocket-engine's own lora_shrink / lora_expand, compiled from the
reference sources into oracle/_ref/qwen35_sm100a.fatbin (make -C oracle ref), through the CUDA driver
API with the grids the engine uses (src/linear.rs:862-884,900-920). Used by GPU parity tests, by the
golden-fixture generator and by the reference arm of bench.py; never by the product path.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
FATBIN = os.path.join(_HERE, "_ref", "qwen35_sm100a.fatbin")


def available():
    return os.path.exists(FATBIN)


class RefKernels:
    def __init__(self, path=None):
        """path: another kernel image exporting lora_shrink / lora_expand with the reference's signatures."""
        from cuda.bindings import driver as drv
        self.drv = drv
        with open(path or FATBIN, "rb") as f:
            self._image = f.read()
        err, self.module = drv.cuModuleLoadData(self._image)
        self._ok(err, "cuModuleLoadData")
        err, self.shrink = drv.cuModuleGetFunction(self.module, b"lora_shrink")
        self._ok(err, "lora_shrink")
        err, self.expand = drv.cuModuleGetFunction(self.module, b"lora_expand")
        self._ok(err, "lora_expand")

    def _ok(self, err, what):
        if int(err) != 0:
            raise RuntimeError(f"{what}: CUDA driver error {err}")

    def launch_shrink(self, x, ldx, K, tiles, table, s, lds, max_tiles, rows, parts, stream=0):
        """src/linear.rs:853-885: grid (min(max_tiles, rows), ceil(parts*max_rank/32), ceil(K/256)), 128 threads."""
        n_tiles = min(max_tiles, rows)
        rank = parts * (lds // 4)
        args = ((x, ldx, K, tiles, table, s, lds),
                (C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int))
        err, = self.drv.cuLaunchKernel(self.shrink, n_tiles, (rank + 31) // 32, (K + 255) // 256, 128, 1, 1, 0, stream,
                                       args, 0)
        self._ok(err, "launch lora_shrink")

    def launch_expand(self, s, lds, nxt, tiles, table, y, ldy, f32_out, max_tiles, rows, max_rows, parts, stream=0):
        """src/linear.rs:889-921: grid (min(max_tiles, rows), ceil(max_rows/128), parts), 128 threads."""
        n_tiles = min(max_tiles, rows)
        args = ((s, lds, nxt, tiles, table, y, ldy, int(f32_out)),
                (C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int))
        err, = self.drv.cuLaunchKernel(self.expand, n_tiles, (max_rows + 127) // 128, parts, 128, 1, 1, 0, stream,
                                       args, 0)
        self._ok(err, "launch lora_expand")
