"""Generates tests/golden/reference_kernels.npz by running pocket-engine's OWN lora_shrink / lora_expand
(compiled from the reference sources into oracle/_ref/ by `make -C oracle ref`) on a B200:

    python tests/golden/make_golden.py [output.npz]

The fixture holds, for two small seeded workloads, the reference kernels' outputs in f32-out and bf16-out
mode. tests/test_golden.py checks the CPU oracle against them without a GPU. Inputs are not stored: they are
re-drawn from the same seeds (pocket-engine_b200/workloads.py)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def cases(pe, workloads):
    ragged = workloads.Workload(
        "golden-ragged", [pe.Site.fused(0, 256, [("a", 64), ("b", 32), ("c", 32)]), pe.Site.fused(0, 256, [("o", 48)])],
        [8, 24, 16], 1.5, [1, 15, 16, 17, 33, 2, 1], [1, 2, 0, 3, 1, 2, 3], 3)
    return {"plumbing": workloads.config1(), "ragged": ragged}


def main():
    import __graft_entry__ as entry
    import harness
    pe = entry.load_package()
    from pocket_engine_b200 import workloads
    out = {}
    for name, wl in cases(pe, workloads).items():
        loras = harness.product_registry(pe, wl)
        for f32_out in (True, False):
            ys = harness.run_reference_kernels(pe, loras, wl, f32_out)
            if ys is None:
                raise SystemExit("oracle/_ref fatbin is missing: make -C oracle ref")
            for si, y in enumerate(ys):
                key = f"{name}.site{si}.{'f32' if f32_out else 'bf16'}"
                out[key] = y.astype(np.float32) if f32_out else pe.bf16_bits(y).reshape(y.shape)
        loras.close()
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_kernels.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
