"""Golden vectors from the REFERENCE's own CUDA kernels (lmdeploy v0.0.9) for the prefill-side writers around the KV
cache and for its unfused context-attention route: invokeAddFusedQKVBiasTranspose, invokeExtendKVCache,
invokeTransposeKVCache, invokeCreateCausalMasks + invokeMaskedSoftmax (the two batched GEMMs between them by cuBLAS
through torch.matmul, as the reference calls cuBLAS).  Run on a machine with a GPU and oracle/_ref/libtm_ref.so built
(python oracle/build_ref.py):

    python tests/golden/make_ref_prefill_vectors.py [out.npz]

The committed tests/golden/ref_prefill_vectors.npz was made this way on a B200; tests/test_oracle_prefill_vectors.py
checks the CPU oracle against it.  Inputs are seeded random data."""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import test_gpu_prefill as tp  # noqa: E402

D = 128


def main(out_path):
    ref = tp.load_ref()
    assert ref is not None, "build oracle/_ref/libtm_ref.so first"
    out = {}
    # ---- QKV bias + RoPE + transpose: ragged batch with history, padded rows, bias
    case = tp.qkv_case([12, 5, 9], [0, 7, 300], 12, 4, 2, 201)
    q, k, v = tp.run_qkv(case, "reference", ref)
    out.update(qkv_in=case["qkv"], qkv_bias=case["bias"], qkv_pad=case["pad"], qkv_history=case["history"],
               qkv_input=case["input"], qkv_q=q, qkv_k=k, qkv_v=v)
    # ---- cache extend / transpose, fp16 and int8
    for int8 in (False, True):
        tag = "s8" if int8 else "f16"
        c = tp.cache_case(B=2, Hkv=2, layers=2, layer=1, S_max=24, max_q=10, q_len=[10, 3], hist=[0, 21], seed=203, int8=int8)
        kc, vc = tp.run_extend(c, "reference", ref)
        out.update({f"ext_{tag}_k_src": c["k_src"], f"ext_{tag}_v_src": c["v_src"], f"ext_{tag}_k_in": np.stack(c["kc"]),
                    f"ext_{tag}_v_in": np.stack(c["vc"]), f"ext_{tag}_k_out": np.stack(kc), f"ext_{tag}_v_out": np.stack(vc)})
        kt, vt = tp.run_transpose(c, [24, 6], 24, 2, "reference", ref)
        out.update({f"tr_{tag}_k": kt, f"tr_{tag}_v": vt})
        if int8:
            out["kv_scale"] = c["scale"]
    # ---- context attention by the unfused route, GQA 4/2, history
    for int8 in (False, True):
        tag = "s8" if int8 else "f16"
        q_lens, hist, H, Hkv, S_max = [40, 9], [0, 30], 4, 2, 48
        c = tp.attention_case(q_lens, hist, H, Hkv, S_max, layers=1, layer=0, seed=205, int8=int8)
        B, max_q, max_k = c["B"], c["max_q"], int(c["ctx"].max())
        kd, vd, kp, vp = tp._cache_tensors(c)
        kt = torch.zeros((B, H, max_k, D), dtype=torch.float16, device="cuda")
        vt = torch.zeros_like(kt)
        ctx_d, ql_d = tp.dev(c["ctx"]), tp.dev(np.asarray(q_lens, np.int32))
        sc = None if c["scale"] is None else (C.c_float * 4)(*[float(x) for x in c["scale"]])
        assert ref.ref_transpose_kv_cache(tp._p(kt), tp._p(vt), tp._p(kp), tp._p(vp), 0, B, tp._p(ctx_d), max_k, S_max, D, H, H // Hkv,
                                          None, 4 if int8 else 0, sc) == 0
        qk = torch.matmul(tp.dev(c["q"]), kt.transpose(2, 3)).contiguous()
        mask = torch.zeros((B, max_q, max_k), dtype=torch.float16, device="cuda")
        assert ref.ref_create_causal_masks(tp._p(mask), tp._p(ql_d), tp._p(ctx_d), max_q, max_k, B, None) == 0
        assert ref.ref_masked_softmax(tp._p(qk), tp._p(qk), tp._p(mask), B, max_q, max_k, H, 1.0 / np.sqrt(D), None) == 0
        o = torch.matmul(qk, vt)
        packed = np.concatenate([o[b, :, :n].transpose(0, 1).reshape(n, H * D).cpu().numpy() for b, n in enumerate(q_lens)])
        out.update({f"attn_{tag}_q": c["q"], f"attn_{tag}_k": np.stack(c["kc"]), f"attn_{tag}_v": np.stack(c["vc"]),
                    f"attn_{tag}_cu": c["cu"], f"attn_{tag}_ctx": c["ctx"], f"attn_{tag}_out": packed,
                    f"attn_{tag}_mask": mask.cpu().numpy()})
        if int8:
            out["attn_kv_scale"] = c["scale"]
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_prefill_vectors.npz"))
