"""Golden vectors from the REFERENCE's own CUDA kernels (lmdeploy v0.0.9) for the CUDA-only parts of
the path: int4 format converters, GemmS4F16, decode attention (fp16 and int8 cache) and the fused
residual-add RMSNorm.  Run on a machine with a GPU and with oracle/_ref/libtm_ref.so built
(python oracle/build_ref.py, which compiles the reference sources where they lie):

    python tests/golden/make_ref_kernel_vectors.py [out.npz]

The committed tests/golden/ref_kernel_vectors.npz was made this way on a B200; the CPU test
tests/test_oracle_ref_vectors.py checks the oracle against it.  Inputs are seeded random data."""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import attention as oa  # noqa: E402
from tests.helpers import make_linear  # noqa: E402


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p()


def _words(shape, seed):
    return np.random.default_rng(seed).integers(0, 2 ** 32, size=shape, dtype=np.uint64).astype(np.uint32)


def _cuda(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        t = t.view(dtype)
    return t.cuda()


def main(out_path):
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libtm_ref.so"))
    vp, i, f32 = C.c_void_p, C.c_int, C.c_float
    lib.ref_convert_s4_k_m8.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, vp]
    lib.ref_transpose_qk_s4_k_m8_hf.argtypes = [vp, vp, i, i, i, vp]
    lib.ref_fuse_w1_w3_s4_k_m8.argtypes = [vp, vp, i, i, vp]
    lib.ref_dequantize_s4.argtypes = [vp, vp, C.c_size_t, vp]
    lib.ref_gemm_s4_f16.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp]
    lib.ref_add_residual_rmsnorm.argtypes = [vp, vp, vp, vp, f32, i, i, vp]
    lib.ref_mmha_decode.argtypes = [vp] * 7 + [i] * 5 + [i, f32, i, vp, vp, vp, vp, vp, C.c_size_t, i, f32, f32, f32, f32, i, i, i,
                                                          vp]
    out = {}

    # ---- format
    n, k = 256, 256
    a_src, qz = _words((k, n // 8), 1), _words((k // 128, n // 8), 2)
    scales = np.random.default_rng(3).standard_normal((k // 128, n)).astype(np.float16)
    A = torch.zeros((k, n // 8), dtype=torch.int32, device="cuda")
    Q = torch.zeros((k // 128, n, 2), dtype=torch.float16, device="cuda")
    ws = torch.zeros(k // 128 * n, dtype=torch.float16, device="cuda")
    ins = (_cuda(a_src, torch.int32), _cuda(scales), _cuda(qz, torch.int32))
    assert lib.ref_convert_s4_k_m8(_p(A), _p(Q), _p(ws), _p(ins[0]), _p(ins[1]), _p(ins[2]), n, k, 128, None) == 0
    out.update(convert_a_src=a_src, convert_qzeros=qz, convert_scales=scales, convert_A=A.cpu().numpy().view(np.uint32),
               convert_Q=Q.cpu().numpy().view(np.uint16))
    m, kk = 256, 32
    src = _words((kk, m // 8), 4)
    d, s = torch.zeros((kk, m // 8), dtype=torch.int32, device="cuda"), _cuda(src, torch.int32)
    assert lib.ref_transpose_qk_s4_k_m8_hf(_p(d), _p(s), m, kk, 128, None) == 0
    out.update(transpose_src=src, transpose_dst=d.cpu().numpy().view(np.uint32))
    m, kk = 128, 16
    src = _words((2, kk, m // 8), 5)
    d, s = torch.zeros((kk, m // 4), dtype=torch.int32, device="cuda"), _cuda(src, torch.int32)
    assert lib.ref_fuse_w1_w3_s4_k_m8(_p(d), _p(s), m, kk, None) == 0
    out.update(fuse_src=src, fuse_dst=d.cpu().numpy().view(np.uint32))
    src = _words((64,), 6)
    d, s = torch.zeros(8 * 64, dtype=torch.float16, device="cuda"), _cuda(src, torch.int32)
    assert lib.ref_dequantize_s4(_p(d), _p(s), 64, None) == 0
    out.update(dequant_src=src, dequant_dst=d.cpu().numpy().view(np.uint16))

    # ---- GEMM (plain and fused SiLU), small shapes the reference's kernels accept (m % 256 == 0, k % 512 == 0)
    for name, n, k, t, fused in (("gemm_plain", 256, 512, 5, False), ("gemm_silu", 512, 512, 8, True)):
        lin = make_linear(n, k, 40 + int(fused))
        x = np.random.default_rng(7).standard_normal((t, k)).astype(np.float16)
        Ad, Qd, Xd = _cuda(lin["A"], torch.int32), _cuda(lin["Q"]), _cuda(x)
        y = torch.zeros((t, n // 2 if fused else n), dtype=torch.float16, device="cuda")
        assert lib.ref_gemm_s4_f16(_p(y), _p(Ad), _p(Xd), _p(Qd), n, t, k, 128, int(fused), None) == 0
        out.update({f"{name}_A": lin["A"], f"{name}_Q": np.asarray(lin["Q"]).view(np.uint16), f"{name}_x": x,
                    f"{name}_y": y.cpu().numpy()})

    # ---- attention: 3 sequences, GQA 4/2, fp16 and int8 cache
    from tests.test_gpu_attention import make_case
    H, Hkv, D, S_max = 4, 2, 128, 64
    lengths = [1, 17, 40]
    for int8 in (False, True):
        case = make_case(3, H, Hkv, S_max, lengths, 51, int8, bias=True)
        tag = "attn_int8" if int8 else "attn_fp16"
        kd = [torch.from_numpy(c).reshape(-1).cuda() for c in case["kc"]]
        vd = [torch.from_numpy(c).reshape(-1).cuda() for c in case["vc"]]
        kp = torch.tensor([t.data_ptr() for t in kd], dtype=torch.int64, device="cuda")
        vpp = torch.tensor([t.data_ptr() for t in vd], dtype=torch.int64, device="cuda")
        qkv, b = _cuda(case["qkv"]), _cuda(case["bias"])
        o = torch.zeros((3, H * D), dtype=torch.float16, device="cuda")
        ld = _cuda(case["lengths"])
        ts = int(max(lengths))
        pad = _cuda((ts - case["lengths"]).astype(np.int32))
        kq = case["kq"]
        sc = (kq.k_scale, kq.k_zp, kq.v_scale, kq.v_zp) if int8 else (0.0, 0.0, 0.0, 0.0)
        assert lib.ref_mmha_decode(_p(o), _p(qkv), _p(qkv[:, H * D:]), _p(qkv[:, (H + Hkv) * D:]), _p(b), _p(b[H * D:]),
                                   _p(b[(H + Hkv) * D:]), (H + 2 * Hkv) * D, 3, S_max, H, Hkv, D, 10000.0, ts, _p(pad), None, _p(ld),
                                   _p(kp), _p(vpp), 0, 4 if int8 else 0, *sc, 2048, 0, 0, None) == 0
        out.update({f"{tag}_qkv": case["qkv"], f"{tag}_bias": case["bias"], f"{tag}_lengths": case["lengths"],
                    f"{tag}_k_in": np.stack(case["kc"]), f"{tag}_v_in": np.stack(case["vc"]),
                    f"{tag}_out": o.cpu().numpy(), f"{tag}_scales": np.asarray(sc, np.float32)})
        # the cache after the call: only the appended row of every sequence is kept (the rest must be untouched)
        for kv, bufs, before in (("k", kd, case["kc"]), ("v", vd, case["vc"])):
            after = [t.cpu().numpy().reshape(Hkv, S_max, D) for t in bufs]
            rows = []
            for bidx, L in enumerate(lengths):
                keep = np.ones(S_max, bool)
                keep[L % S_max] = False
                assert np.array_equal(after[bidx][:, keep], before[bidx][:, keep])
                rows.append(after[bidx][:, L % S_max])
            out[f"{tag}_{kv}_new"] = np.stack(rows)

    # ---- fused residual add + RMSNorm
    rng = np.random.default_rng(9)
    m, n = 3, 1024
    res, x = rng.standard_normal((m, n)).astype(np.float16), rng.standard_normal((m, n)).astype(np.float16)
    bias, w = (rng.standard_normal(n) * 0.1).astype(np.float16), (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    r, io, bd, wd = _cuda(res), _cuda(x), _cuda(bias), _cuda(w)
    assert lib.ref_add_residual_rmsnorm(_p(r), _p(io), _p(bd), _p(wd), 1e-5, m, n, None) == 0
    out.update(norm_res=res, norm_x=x, norm_bias=bias, norm_w=w, norm_res_out=r.cpu().numpy(), norm_out=io.cpu().numpy())

    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_kernel_vectors.npz"))
