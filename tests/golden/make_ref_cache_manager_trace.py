"""Writes tests/golden/ref_cache_manager_trace.npz: the outcomes of the REFERENCE's own LlamaCacheManager
(src/turbomind/models/llama/LlamaCacheManager.cc, compiled unmodified into oracle/_ref/libtm_ref.so by oracle/build_ref.py)
for the seeded operation streams of tests/cache_trace.py.  Needs a GPU (the reference zero-fills slabs with
cudaMemsetAsync).  tests/test_cache_manager.py replays the file on the CPU against oracle/cache_manager.py and against
tm_cache_* in host mode.

    python tests/golden/make_ref_cache_manager_trace.py [output.npz]
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import cache_trace as ct  # noqa: E402


def main():
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libtm_ref.so"))
    out = {}
    for seed, max_entries, chunk in ct.CASES:
        ops = ct.gen_ops(seed, max_entries)
        a = ct.RefAdapter(lib, max_entries, chunk)
        out[f"rows_{seed}"] = ct.run(a, ops, 2 * max_entries + 2)
        a.close()
    path = sys.argv[1] if len(sys.argv) > 1 else ct.GOLDEN
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
