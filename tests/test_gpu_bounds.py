"""The range-checked build of the library (-DPLORA_BOUNDS), the stand-in on this path for running the suite under
a memory checker: the few-token kernels validate every launch record against what the launch may touch and skip
what does not fit, recording an error instead of reading or writing through it. Run in a process of its own
because the library a process loads is chosen once (PLORA_LIB)."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_the_range_checked_build_passes_the_suite_and_refuses_out_of_range_records(pe):
    lib = os.path.join(os.path.dirname(pe.LIB_PATH), "libplora_bounds.so")
    assert os.path.exists(lib), "built by pocket-engine_b200/build.py beside libplora.so"
    env = dict(os.environ, PLORA_LIB=lib)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "bounds_worker.py")], capture_output=True, text=True,
                       timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert res["bounds_check"] == "ok" and "decode block" in res["cases"] and len(res["cases"]) >= 7
    for form, got in res["refused"].items():
        assert got["code"] == pe.ERR_ARG, (form, got)          # the status word says a record was refused
        assert got["rows_changed_past_8"] == 0, (form, got)    # nothing past the named rows was touched
