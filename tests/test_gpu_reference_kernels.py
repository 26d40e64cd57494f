"""The reference's own CUDA kernels (built from its sources into oracle/_ref/libtm_ref.so by
oracle/build_ref.py) run on the same inputs as this library and as the CPU oracle.

This is what pins the restated oracles of the CUDA-only parts of the path (int4 format converters,
GemmS4F16, decode attention) to the reference itself: format results must agree bit for bit, GEMM
and attention outputs within the fp16 tolerances of the other parity tests.  Skipped when the
reference build is not present."""
import ctypes as C
import math
import os

import numpy as np
import pytest
import torch

from oracle import attention as oa, gemm as og, s4_format as f
from tests.helpers import assert_close, dev, make_linear

pytestmark = pytest.mark.gpu

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libtm_ref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(_REF):
        pytest.skip("oracle/_ref/libtm_ref.so not built (python oracle/build_ref.py needs the reference tree)")
    lib = C.CDLL(_REF)
    vp, i, f32 = C.c_void_p, C.c_int, C.c_float
    lib.ref_reformat_s4_k_m8.argtypes = [vp, vp, i, i, vp]
    lib.ref_convert_s4_k_m8.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, vp]
    lib.ref_transpose_qk_s4_k_m8_hf.argtypes = [vp, vp, i, i, i, vp]
    lib.ref_fuse_w1_w3_s4_k_m8.argtypes = [vp, vp, i, i, vp]
    lib.ref_dequantize_s4.argtypes = [vp, vp, C.c_size_t, vp]
    lib.ref_gemm_s4_f16.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp]
    lib.ref_gemm_s4_f16_algo.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, vp]
    lib.ref_mmha_decode.argtypes = [vp] * 7 + [i] * 5 + [i, f32, i, vp, vp, vp, vp, vp, C.c_size_t, i, f32, f32, f32, f32, i, i,
                                                          i, vp]
    lib.ref_add_residual_rmsnorm.argtypes = [vp, vp, vp, vp, f32, i, i, vp]
    lib.ref_rmsnorm.argtypes = [vp, vp, vp, f32, i, i, vp]
    lib.ref_rmsnorm.restype = i
    for name in ("ref_reformat_s4_k_m8", "ref_convert_s4_k_m8", "ref_transpose_qk_s4_k_m8_hf", "ref_fuse_w1_w3_s4_k_m8",
                 "ref_dequantize_s4", "ref_gemm_s4_f16", "ref_mmha_decode", "ref_add_residual_rmsnorm"):
        getattr(lib, name).restype = i
    return lib


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p()


def _words(shape, seed):
    return np.random.default_rng(seed).integers(0, 2 ** 32, size=shape, dtype=np.uint64).astype(np.uint32)


# ---------------------------------------------------------------------------------------- format

@pytest.mark.parametrize("n,k", [(512, 128), (4096, 256), (11008, 128)])
def test_convert_matches_reference_bit_for_bit(ref, n, k):
    from lmdeploy_b200 import turbomind as tm
    a_src, qz = _words((k, n // 8), 1), _words((k // 128, n // 8), 2)
    scales = np.random.default_rng(3).standard_normal((k // 128, n)).astype(np.float16)
    outs = []
    for which in ("reference", "ours"):
        A = torch.zeros((k, n // 8), dtype=torch.int32, device="cuda")
        Q = torch.zeros((k // 128, n, 2), dtype=torch.float16, device="cuda")
        ws = torch.zeros(k // 128 * n, dtype=torch.float16, device="cuda")
        args = (dev(a_src, torch.int32), dev(scales), dev(qz, torch.int32))
        if which == "reference":
            assert ref.ref_convert_s4_k_m8(_p(A), _p(Q), _p(ws), _p(args[0]), _p(args[1]), _p(args[2]), n, k, 128, None) == 0
        else:
            tm.convert_s4_k_m8(A, Q, ws, *args, n, k, 128)
            torch.cuda.synchronize()
        outs.append((A.cpu().numpy().view(np.uint32), Q.cpu().numpy().view(np.uint16)))
    a_cpu, q_cpu = f.convert_s4_k_m8(a_src, scales, qz, n, k, 128)
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1]), "library != reference"
    assert np.array_equal(outs[0][0], a_cpu) and np.array_equal(outs[0][1], q_cpu.view(np.uint16)), "CPU oracle != reference"


def test_transpose_fuse_dequantize_match_reference_bit_for_bit(ref):
    from lmdeploy_b200 import turbomind as tm
    # q/k head-dim permutation
    m, k = 4 * 128, 64
    src = _words((k, m // 8), 4)
    a = torch.zeros((k, m // 8), dtype=torch.int32, device="cuda")
    b = torch.zeros_like(a)
    sd = dev(src, torch.int32)
    assert ref.ref_transpose_qk_s4_k_m8_hf(_p(a), _p(sd), m, k, 128, None) == 0
    tm.transpose_qk_s4_k_m8(sd, b, m, k, 128)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    assert np.array_equal(a.cpu().numpy().view(np.uint32), f.transpose_qk_s4_k_m8_hf(src, m, k, 128))
    # w1 | w3 interleave
    m, k = 11008, 16
    src = _words((2, k, m // 8), 5)
    a = torch.zeros((k, m // 4), dtype=torch.int32, device="cuda")
    b = torch.zeros_like(a)
    sd = dev(src, torch.int32)
    assert ref.ref_fuse_w1_w3_s4_k_m8(_p(a), _p(sd), m, k, None) == 0
    tm.fuse_w1_w3_s4_k_m8(sd, b, m, k)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    assert np.array_equal(a.cpu().numpy().view(np.uint32), f.fuse_w1_w3_s4_k_m8(src, m, k))
    # plain nibble -> half
    src = _words((4096,), 6)
    a = torch.zeros(8 * 4096, dtype=torch.float16, device="cuda")
    b = torch.zeros_like(a)
    sd = dev(src, torch.int32)
    assert ref.ref_dequantize_s4(_p(a), _p(sd), 4096, None) == 0
    tm.dequantize_s4(sd, b)
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert np.array_equal(a.cpu().numpy().view(np.uint16), f.dequantize_s4(src).view(np.uint16))


# ------------------------------------------------------------------------------------------ GEMM

def _gemm_three_ways(ref, n, k, tokens, fused, seed):
    from lmdeploy_b200 import turbomind as tm
    lin = make_linear(n, k, seed)
    x = (np.random.default_rng(5).standard_normal((tokens, k)) * 1.0).astype(np.float16)
    A, Q, X = dev(lin["A"], torch.int32), dev(lin["Q"]), dev(x)
    n_out = n // 2 if fused else n
    y_ref = torch.zeros((tokens, n_out), dtype=torch.float16, device="cuda")
    y_lib = torch.zeros_like(y_ref)
    assert ref.ref_gemm_s4_f16(_p(y_ref), _p(A), _p(X), _p(Q), n, tokens, k, 128, int(fused), None) == 0
    w = tm.LlamaDenseWeight(k, n, A, tm.WeightType.kINT4, None, Q, 128)
    op = tm.LlamaLinear(0)
    op.forward(y_lib, X, tokens, w, op.kFusedSiluFfn if fused else op.kGemm)
    torch.cuda.synchronize()
    return y_lib.cpu().numpy(), y_ref.cpu().numpy(), og.gemm_s4_f16(x, lin["w_kn"], fused)


@pytest.mark.parametrize("n,k,fused,tokens", [
    (4096, 4096, False, 1), (4096, 4096, False, 5), (4096, 4096, False, 8), (4096, 4096, False, 17), (4096, 4096, False, 33),
    (4096, 4096, False, 64), (4096, 4096, False, 128), (4096, 4096, False, 200), (1536, 2048, False, 1), (1536, 2048, False, 8),
    (2816, 1024, True, 1), (2816, 1024, True, 8), (2816, 1024, True, 16), (2816, 1024, True, 17), (2816, 1024, True, 64),
    (2816, 1024, True, 128), (2816, 1024, True, 200)])
def test_gemm_matches_reference_kernel(ref, n, k, fused, tokens):
    """GemmS4F16::Run of the reference (its own mma.sync kernels, its own kernel choice) against
    tm_gemm_s4_f16 and against the CPU oracle, same packed weight and activations."""
    y_lib, y_ref, y_cpu = _gemm_three_ways(ref, n, k, tokens, fused, 21 + int(fused))
    slack = 2.0 ** -9 if fused else 0.0
    assert_close(y_lib, y_ref, f"library vs reference kernel {n}x{k} T={tokens} fused={fused}", rel_slack=slack)
    assert_close(y_ref, y_cpu, f"reference kernel vs CPU oracle {n}x{k} T={tokens} fused={fused}", rel_slack=slack)
    assert_close(y_lib, y_cpu, f"library vs CPU oracle {n}x{k} T={tokens} fused={fused}", rel_slack=slack)


@pytest.mark.parametrize("n,k,tokens,algo", [(4096, 4096, 12, 15), (4096, 4096, 16, 15), (4096, 4096, 12, 13), (1536, 2048, 24, 15),
                                             (1536, 2048, 24, 13), (4096, 4096, 8, 16)])
def test_gemm_matches_reference_kernel_with_a_named_tile(ref, n, k, tokens, algo):
    """Where the reference's own estimate picks its 64 x 8 x 256 tile (index 16 of gemm_s4_f16.cu:72-93) for more than
    8 tokens (on 148 SMs: 9..16 tokens on 4096 x 4096 and 4096 x 11008, every count above 8 on 1536 x 2048), that kernel
    returns wrong rows.  Its activation iterator (cta_iterator.h:452-457) deals the tile's rows to
    kWarpN = WARPS / kWarpK = 2 warps although one warp's footprint (8 rows) already covers the tile (kIterN is clamped
    to 1), and masks a row only by the global token count (`is_valid_n_`, :547,591,611; the copy is predicated on it, :616-617).  With at most 8 tokens the
    second warp's rows 8..15 are masked; with more they are real tokens, and their copies land 8 rows further down in
    shared memory, which is rows 0..7 of the next pipeline stage, racing with that stage's own copies.  The same
    arithmetic gives the 256 x 8 x 256 tile (index 5) twice as many warps as rows.  The other tiles deal the rows
    exactly, so the comparison names one of them: 15 = 64 x 16 x 256, 13 = 128 x 8 x 512; 16 itself up to 8 tokens."""
    from lmdeploy_b200 import turbomind as tm
    lin = make_linear(n, k, 21)
    x = (np.random.default_rng(5).standard_normal((tokens, k)) * 1.0).astype(np.float16)
    A, Q, X = dev(lin["A"], torch.int32), dev(lin["Q"]), dev(x)
    y_ref = torch.zeros((tokens, n), dtype=torch.float16, device="cuda")
    y_lib = torch.zeros_like(y_ref)
    assert ref.ref_gemm_s4_f16_algo(_p(y_ref), _p(A), _p(X), _p(Q), n, tokens, k, 128, 0, algo, None) == 0
    w = tm.LlamaDenseWeight(k, n, A, tm.WeightType.kINT4, None, Q, 128)
    op = tm.LlamaLinear(0)
    op.forward(y_lib, X, tokens, w, op.kGemm)
    torch.cuda.synchronize()
    y_lib, y_ref, y_cpu = y_lib.cpu().numpy(), y_ref.cpu().numpy(), og.gemm_s4_f16(x, lin["w_kn"], False)
    assert_close(y_lib, y_ref, f"library vs reference tile {algo}, {n}x{k} T={tokens}")
    assert_close(y_ref, y_cpu, f"reference tile {algo} vs CPU oracle {n}x{k} T={tokens}")
    assert_close(y_lib, y_cpu, f"library vs CPU oracle {n}x{k} T={tokens}")


@pytest.mark.parametrize("n,k,tokens", [(4096, 4096, 12), (4096, 4096, 16), (1536, 2048, 24)])
def test_library_follows_the_definition_where_the_reference_estimate_picks_the_broken_tile(ref, n, k, tokens):
    """The cases above through GemmS4F16::Run's own choice (algo_id = -1): the library must agree with the CPU
    definition; how far the reference's pick is from it is printed, not asserted (a race decides it)."""
    y_lib, y_ref, y_cpu = _gemm_three_ways(ref, n, k, tokens, False, 21)
    assert_close(y_lib, y_cpu, f"library vs CPU oracle {n}x{k} T={tokens}")
    err = float(np.abs(y_ref.astype(np.float32) - y_cpu.astype(np.float32)).max())
    print(f"reference's own pick vs its CPU definition, {n}x{k} T={tokens}: max abs difference {err:.3f}")


# ------------------------------------------------------------------------------------------ norm

@pytest.mark.parametrize("m,n,bias", [(1, 4096, False), (64, 4096, False), (5, 8192, True)])
def test_fused_add_rmsnorm_matches_reference_kernel(ref, m, n, bias):
    """invokeFusedAddBiasResidualRMSNorm of the reference against tm_add_residual_rmsnorm and the CPU oracle."""
    from lmdeploy_b200 import turbomind as tm
    from oracle import norm as on
    rng = np.random.default_rng(9)
    res = rng.standard_normal((m, n)).astype(np.float16)
    x = rng.standard_normal((m, n)).astype(np.float16)
    b = (rng.standard_normal(n) * 0.1).astype(np.float16) if bias else None
    w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    outs = []
    bd, wd = (dev(b) if bias else None), dev(w)   # kept alive across the calls
    for which in ("reference", "ours"):
        r, io = dev(res), dev(x)
        if which == "reference":
            assert ref.ref_add_residual_rmsnorm(_p(r), _p(io), _p(bd), _p(wd), 1e-5, m, n, None) == 0
        else:
            tm.invokeFusedAddBiasResidualRMSNorm(r, io, bd, wd, 1e-5, m, n)
            torch.cuda.synchronize()
        outs.append((r.cpu().numpy(), io.cpu().numpy()))
    r_cpu, o_cpu = on.add_residual_rmsnorm(res, x, b, w, 1e-5)
    assert np.array_equal(outs[0][0].view(np.uint16), outs[1][0].view(np.uint16)), "residual: library != reference"
    assert np.array_equal(outs[0][0].view(np.uint16), np.asarray(r_cpu).view(np.uint16)), "residual: CPU oracle != reference"
    assert_close(outs[1][1], outs[0][1], "norm output: library vs reference kernel", max_abs=4e-3)
    assert_close(outs[0][1], o_cpu, "norm output: reference kernel vs CPU oracle", max_abs=4e-3)


@pytest.mark.parametrize("m,n", [(1, 4096), (64, 4096), (3, 8192)])
def test_rmsnorm_matches_reference_kernel(ref, m, n):
    """invokeRootMeanSquareNorm of the reference against tm_rmsnorm and the CPU oracle."""
    from lmdeploy_b200 import turbomind as tm
    from oracle import norm as on
    rng = np.random.default_rng(19)
    x = (rng.standard_normal((m, n)) * 1.5).astype(np.float16)
    w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    xd, wd = dev(x), dev(w)
    o_ref = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    o_lib = torch.zeros_like(o_ref)
    assert ref.ref_rmsnorm(_p(o_ref), _p(xd), _p(wd), 1e-6, m, n, None) == 0
    tm.invokeRootMeanSquareNorm(o_lib, xd, wd, 1e-6, m, n)
    torch.cuda.synchronize()
    assert_close(o_lib.cpu().numpy(), o_ref.cpu().numpy(), "rmsnorm: library vs reference kernel", max_abs=4e-3)
    assert_close(on.rmsnorm(x, w, 1e-6), o_ref.cpu().numpy(), "rmsnorm: CPU oracle vs reference kernel", max_abs=4e-3)


# ------------------------------------------------------------------------------------- attention

def _attention_case(B, H, Hkv, S_max, lengths, seed, int8, bias):
    from tests.test_gpu_attention import make_case
    return make_case(B, H, Hkv, S_max, lengths, seed, int8, bias=bias)


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("H,Hkv,bias", [(8, 8, False), (16, 2, True)])
def test_attention_matches_reference_kernel(ref, int8, H, Hkv, bias):
    """masked_multihead_attention of the reference against tm_mmha_decode and the CPU oracle:
    outputs and the appended cache rows."""
    from tests.test_gpu_attention import check_cache, run_gpu, run_oracle
    D, S_max = 128, 640
    lengths = [1, 15, 16, 17, 63, 64, 65, 200, 257, 511, 600]
    B = len(lengths)
    case = _attention_case(B, H, Hkv, S_max, lengths, 31, int8, bias)
    out_lib, kc_lib, vc_lib = run_gpu(case)
    out_cpu, kc_cpu, vc_cpu = run_oracle(case)

    kd = [torch.from_numpy(k).reshape(-1).cuda() for k in case["kc"]]
    vd = [torch.from_numpy(v).reshape(-1).cuda() for v in case["vc"]]
    kp = torch.tensor([t.data_ptr() for t in kd], dtype=torch.int64, device="cuda")
    vp = torch.tensor([t.data_ptr() for t in vd], dtype=torch.int64, device="cuda")
    qkv = dev(case["qkv"])
    out = torch.full((B, H * D), 555.0, dtype=torch.float16, device="cuda")
    ld = dev(case["lengths"])
    timestep = int(case["lengths"].max())
    padding = dev((timestep - case["lengths"]).astype(np.int32))
    b = dev(case["bias"]) if bias else None
    kq = case["kq"]
    scales = (kq.k_scale, kq.k_zp, kq.v_scale, kq.v_zp) if int8 else (0.0, 0.0, 0.0, 0.0)
    rc = ref.ref_mmha_decode(
        _p(out), _p(qkv), _p(qkv[:, H * D:]), _p(qkv[:, (H + Hkv) * D:]), _p(b), _p(b[H * D:]) if bias else None,
        _p(b[(H + Hkv) * D:]) if bias else None, (H + 2 * Hkv) * D, B, S_max, H, Hkv, D, 10000.0, timestep, _p(padding), None,
        _p(ld), _p(kp), _p(vp), 0, 4 if int8 else 0, *scales, 2048, 0, 0, None)
    assert rc == 0
    out_ref = out.cpu().numpy()
    kc_ref = [t.cpu().numpy().reshape(Hkv, S_max, D) for t in kd]
    vc_ref = [t.cpu().numpy().reshape(Hkv, S_max, D) for t in vd]
    assert_close(out_lib, out_ref, f"library vs reference attention int8={int8} H={H}/{Hkv}")
    assert_close(out_ref, out_cpu, f"reference attention vs CPU oracle int8={int8} H={H}/{Hkv}")
    check_cache(kc_lib, kc_ref, int8, case["lengths"], S_max)
    check_cache(vc_lib, vc_ref, int8, case["lengths"], S_max)
    check_cache(kc_ref, kc_cpu, int8, case["lengths"], S_max)
    check_cache(vc_ref, vc_cpu, int8, case["lengths"], S_max)
