"""Generate ``awq_reference_vectors.npz`` from the reference's own torch code.

Run where a checkout of lmdeploy v0.0.9 is available:

    python tests/golden/make_awq_reference_vectors.py /path/to/lmdeploy

The three files that hold the arithmetic are loaded BY FILE PATH (``import
lmdeploy.lite`` itself needs fire / accelerate / mmengine, which are not required for
the arithmetic):

    lmdeploy/lite/utils/cal_qparams.py
    lmdeploy/lite/utils/global_avail.py
    lmdeploy/lite/quantization/weight/quantizer.py
    lmdeploy/pytorch/modules/linear.py

For each seeded fp16 weight the script stores the input and the reference's outputs:
scales, zero points, the un-clamped integer weight (``quant(real=True)``), the
pseudo-quant weight (``quant(real=False)``), and — for the cases where no element
leaves 0..15 — the packed ``qweight`` / ``qzeros`` / ``scales`` of
``WeightOnlyQLinear.from_linear``; plus ``Y = (X.float() @ Wq.float().T).half()``.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch
from torch import nn


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_reference(root):
    for pkg in ("lmdeploy", "lmdeploy.lite", "lmdeploy.lite.utils"):
        if pkg not in sys.modules:
            m = types.ModuleType(pkg)
            m.__path__ = []
            sys.modules[pkg] = m
    cal = _load("lmdeploy.lite.utils.cal_qparams", os.path.join(root, "lmdeploy/lite/utils/cal_qparams.py"))
    utils = sys.modules["lmdeploy.lite.utils"]
    for k in dir(cal):
        if k.startswith("cal_qparams") or k == "QParams":
            setattr(utils, k, getattr(cal, k))
    _load("lmdeploy.lite.utils.global_avail", os.path.join(root, "lmdeploy/lite/utils/global_avail.py"))
    quantizer = _load("ref_quantizer", os.path.join(root, "lmdeploy/lite/quantization/weight/quantizer.py"))
    linear = _load("ref_linear", os.path.join(root, "lmdeploy/pytorch/modules/linear.py"))
    return quantizer.WeightQuantizer, linear.WeightOnlyQLinear


# (name, N, K, seed, std)  — small enough that from_linear's Python loop takes < 1 s
CASES = [
    ("a", 64, 256, 0, 0.02),
    ("b", 96, 384, 1, 0.02),
    ("c", 32, 128, 2, 1.0),
    ("d", 256, 512, 3, 0.02),
]


def main(root):
    WeightQuantizer, WeightOnlyQLinear = load_reference(root)
    out = {}
    for name, n, k, seed, std in CASES:
        g = torch.Generator().manual_seed(seed)
        w = (torch.randn(n, k, generator=g) * std).half()
        x = torch.randn(16, k, generator=g).half()
        quant = WeightQuantizer(4, False, "per_group", 128)
        qp = quant.calculate_qparams(w)
        real = quant.quant(w, qp, real=True)
        fake = quant.quant(w, qp, real=False)
        out[f"{name}_w"] = w.numpy()
        out[f"{name}_x"] = x.numpy()
        out[f"{name}_scales"] = qp.scales.squeeze(-1).numpy()
        out[f"{name}_zeros"] = qp.zero_points.squeeze(-1).numpy()
        out[f"{name}_real"] = real.numpy().astype(np.int32)
        out[f"{name}_fake"] = fake.numpy()
        out[f"{name}_y"] = (x.float() @ fake.float().T).half().numpy()
        overflow = int(((real < 0) | (real > 15)).sum()) + int(((qp.zero_points < 0) | (qp.zero_points > 15)).sum())
        out[f"{name}_overflow"] = np.array(overflow)
        if overflow == 0:
            lin = nn.Linear(k, n, bias=False)
            lin.weight.data = w
            ql = WeightOnlyQLinear.from_linear(lin, quant)
            out[f"{name}_qweight"] = ql.qweight.numpy().astype(np.int32)
            out[f"{name}_qzeros"] = ql.qzeros.numpy().astype(np.int32)
            out[f"{name}_qscales"] = ql.scales.numpy()
        print(name, n, k, "overflow", overflow)
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "awq_reference_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
