"""CPU: the oracle against golden vectors produced by the REFERENCE's own CUDA kernels
(tests/golden/ref_kernel_vectors.npz, written by tests/golden/make_ref_kernel_vectors.py on a B200
from the reference sources compiled as they are).  Format converters bit for bit; GEMM, attention
and the fused norm within the fp16 tolerances of the GPU parity tests."""
import os

import numpy as np

from oracle import attention as oa, gemm as og, norm as on, s4_format as f
from tests.helpers import assert_close

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernel_vectors.npz"))


def test_format_converters_bit_exact():
    a, q = f.convert_s4_k_m8(G["convert_a_src"], G["convert_scales"], G["convert_qzeros"], 256, 256, 128)
    assert np.array_equal(a, G["convert_A"])
    assert np.array_equal(np.asarray(q).view(np.uint16).reshape(G["convert_Q"].shape), G["convert_Q"])
    assert np.array_equal(f.transpose_qk_s4_k_m8_hf(G["transpose_src"], 256, 32, 128), G["transpose_dst"])
    assert np.array_equal(f.fuse_w1_w3_s4_k_m8(G["fuse_src"], 128, 16), G["fuse_dst"])
    assert np.array_equal(f.dequantize_s4(G["dequant_src"]).view(np.uint16).reshape(-1), G["dequant_dst"])


def test_gemm_plain_and_fused_silu():
    for name, n, k, fused in (("gemm_plain", 256, 512, False), ("gemm_silu", 512, 512, True)):
        q = G[f"{name}_Q"].view(np.float16)
        w_kn = f.dequantize_runtime_weight(G[f"{name}_A"], q, n, k, 128)      # the fp16 weight the kernels see
        y = og.gemm_s4_f16(G[f"{name}_x"], w_kn, fused)
        assert_close(y, G[f"{name}_y"], f"oracle vs reference kernel ({name})", rel_slack=2.0 ** -9 if fused else 0.0)


def test_attention_fp16_and_int8_cache():
    H, Hkv, D, S_max = 4, 2, 128, 64
    for tag, int8 in (("attn_fp16", False), ("attn_int8", True)):
        lengths = G[f"{tag}_lengths"]
        kc = [k.copy() for k in G[f"{tag}_k_in"]]
        vc = [v.copy() for v in G[f"{tag}_v_in"]]
        sc = G[f"{tag}_scales"]
        kq = oa.KvQuant(float(sc[0]), float(sc[1]), float(sc[2]), float(sc[3])) if int8 else None
        out = oa.mmha_decode(G[f"{tag}_qkv"], kc, vc, lengths, H, Hkv, D, S_max, qkv_bias=G[f"{tag}_bias"], kv_quant=kq)
        assert_close(out, G[f"{tag}_out"], f"oracle vs reference kernel ({tag})")
        for b, L in enumerate(lengths):
            for new, cache in ((G[f"{tag}_k_new"][b], kc[b]), (G[f"{tag}_v_new"][b], vc[b])):
                row = cache[:, int(L) % S_max]
                if int8:
                    d = np.abs(row.astype(np.int32) - new.astype(np.int32))
                    assert d.max() <= 1 and (d != 0).mean() < 0.02
                else:
                    d = np.abs(row.astype(np.float32) - new.astype(np.float32))
                    assert (d <= 2.0 ** -9 * np.abs(new.astype(np.float32)) + 2e-3).all()


def test_fused_add_rmsnorm():
    r, o = on.add_residual_rmsnorm(G["norm_res"], G["norm_x"], G["norm_bias"], G["norm_w"], 1e-5)
    assert np.array_equal(np.asarray(r).view(np.uint16), G["norm_res_out"].view(np.uint16))
    assert_close(o, G["norm_out"], "oracle vs reference kernel (fused add + RMSNorm)", max_abs=4e-3)
