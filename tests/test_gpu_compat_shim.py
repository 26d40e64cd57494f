"""GPU: calls made through the header shims of include/compat reach the same kernels as direct C-ABI calls.

A small shared object is compiled from this file's C++ text against include/compat and linked with the
library: it drives turbomind::GemmS4F16::Run, turbomind::dequantize_s4 and masked_multihead_attention()
with the reference's signatures.  Results must be bit-identical to the direct calls on the same inputs.
"""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

from tests.helpers import dev, make_linear

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"

SOURCE = r'''
#include "src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.h"
#include "src/turbomind/kernels/gemm_s_f16/format.h"
#include "src/turbomind/kernels/decoder_masked_multihead_attention.h"
#include <cstring>
extern "C" int shim_gemm(void* c, const void* a, const void* b, const void* q, int m, int n, int k, int fused, void* st)
{
    try {
        turbomind::GemmS4F16 g;
        g.Run((half*)c, (const unsigned int*)a, (const half*)b, (const half2*)q, m, n, k, 128,
              fused ? turbomind::GemmS4F16::kFusedSiluFfn : turbomind::GemmS4F16::kGemm, -1, (cudaStream_t)st);
    } catch (const std::exception&) { return 1; }
    return 0;
}
extern "C" int shim_dequant(void* dst, const void* src, size_t count, void* st)
{
    try { turbomind::dequantize_s4((uint4*)dst, (const uint32_t*)src, count, (cudaStream_t)st); } catch (const std::exception&) { return 1; }
    return 0;
}
// the way fusedQKV_masked_attention_dispatch fills the struct (LlamaDecoderSelfAttentionLayer.cc:88-160)
extern "C" int shim_mmha(void* out, const void* qkv, void** kc, void** vc, const int* len, int batch, int heads, int kv_heads,
                         int max_len, int step, int beam, void* st)
{
    Masked_multihead_attention_params<uint16_t> p;
    memset(&p, 0, sizeof(p));
    p.out = (uint16_t*)out;
    p.q = (const uint16_t*)qkv;
    p.k = p.q + heads * 128;
    p.v = p.q + (heads + kv_heads) * 128;
    p.stride = (heads + 2 * kv_heads) * 128;
    p.k_cache_per_sample = (uint16_t**)kc;
    p.v_cache_per_sample = (uint16_t**)vc;
    p.batch_size = batch;
    p.beam_width = beam;
    p.memory_max_len = max_len;
    p.length_per_sample = len;
    p.timestep = step;
    p.num_heads = heads;
    p.num_kv_heads = kv_heads;
    p.hidden_size_per_head = 128;
    p.rotary_embedding_dim = 128;
    p.rotary_embedding_base = 10000.f;
    p.max_position_embeddings = 2048;
    p.inv_sqrt_dh = 0.08838834764831845f;
    try { masked_multihead_attention(p, (cudaStream_t)st); } catch (const std::exception&) { return 1; }
    return 0;
}
'''


@pytest.fixture(scope="module")
def shim(tmp_path_factory):
    if not os.path.exists(NVCC):
        pytest.skip("nvcc not found")
    from lmdeploy_b200 import build
    lib = build.build()
    d = tmp_path_factory.mktemp("shim")
    src = d / "shim.cu"
    src.write_text(SOURCE)
    so = str(d / "libshim.so")
    r = subprocess.run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-w", "-shared", "-Xcompiler", "-fPIC",
                        str(src), "-o", so, "-I", os.path.join(ROOT, "include", "compat"), "-I", os.path.join(ROOT, "include"),
                        "-L", os.path.dirname(lib), "-ltm_b200", "-Xlinker", "-rpath," + os.path.dirname(lib)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    from lmdeploy_b200 import lib as _l   # the library is loaded before the shim resolves against it
    assert _l.lib is not None
    return C.CDLL(so)


@pytest.mark.parametrize("t,fused", [(1, False), (16, True), (64, False)])
def test_gemm_through_the_shim_is_the_same_launch(shim, t, fused):
    from lmdeploy_b200 import lib as l
    n, k = 4096, 4096
    lin = make_linear(n, k, 11)
    A, Q = dev(lin["A"], torch.int32), dev(lin["Q"])
    x = torch.randn(t, k, generator=torch.Generator().manual_seed(t)).half().cuda()
    n_out = n // 2 if fused else n
    ref = torch.empty(t, n_out, dtype=torch.float16, device="cuda")
    out = torch.full((t, n_out), 7.0, dtype=torch.float16, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    h = l.default_handle(torch.cuda.current_device())
    assert l.lib.tm_gemm_s4_f16(h.ptr, ref.data_ptr(), A.data_ptr(), x.data_ptr(), Q.data_ptr(), n, t, k, 128, int(fused), None, 0,
                                st) == l.TM_OK
    shim.shim_gemm.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_void_p]
    assert shim.shim_gemm(out.data_ptr(), A.data_ptr(), x.data_ptr(), Q.data_ptr(), n, t, k, int(fused), st) == 0
    torch.cuda.synchronize()
    assert torch.equal(out, ref)


def test_dequantize_through_the_shim(shim):
    from lmdeploy_b200 import lib as l
    src = torch.randint(-2 ** 31, 2 ** 31 - 1, (4096,), dtype=torch.int32, device="cuda")
    a = torch.empty(4096 * 8, dtype=torch.float16, device="cuda")
    b = torch.empty_like(a)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert l.lib.tm_dequantize_s4(a.data_ptr(), src.data_ptr(), 4096, st) == l.TM_OK
    shim.shim_dequant.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    assert shim.shim_dequant(b.data_ptr(), src.data_ptr(), 4096, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_mmha_through_the_shim_matches_the_direct_call_and_refuses_beams(shim):
    from lmdeploy_b200 import lib as l
    B, H, KV, L = 5, 8, 8, 256
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B, (H + 2 * KV) * 128, device="cuda", generator=g).half()
    lens = torch.tensor([3, 100, 0, 255, 17], dtype=torch.int32, device="cuda")
    step = 255
    outs = []
    for which in range(2):
        kc = (torch.randn(B, KV, L, 128, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9))).half()
        vc = (torch.randn(B, KV, L, 128, device="cuda", generator=torch.Generator(device="cuda").manual_seed(10))).half()
        kp = torch.tensor([kc[b].data_ptr() for b in range(B)], dtype=torch.int64, device="cuda")
        vp = torch.tensor([vc[b].data_ptr() for b in range(B)], dtype=torch.int64, device="cuda")
        out = torch.zeros(B, H * 128, dtype=torch.float16, device="cuda")
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        if which == 0:
            p = l.TmMmhaParams()
            p.out, p.q = out.data_ptr(), qkv.data_ptr()
            p.k, p.v = qkv.data_ptr() + H * 128 * 2, qkv.data_ptr() + (H + KV) * 128 * 2
            p.stride, p.batch_size, p.memory_max_len, p.num_heads, p.num_kv_heads = (H + 2 * KV) * 128, B, L, H, KV
            p.hidden_size_per_head, p.rotary_embedding_dim, p.timestep = 128, 128, step
            p.inv_sqrt_dh, p.rotary_embedding_base, p.max_position_embeddings = 0.08838834764831845, 10000.0, 2048
            p.length_per_sample, p.k_cache_per_sample, p.v_cache_per_sample = lens.data_ptr(), kp.data_ptr(), vp.data_ptr()
            h = l.default_handle(torch.cuda.current_device())
            assert l.lib.tm_mmha_decode(h.ptr, C.byref(p), st) == l.TM_OK
        else:
            shim.shim_mmha.argtypes = [C.c_void_p] * 5 + [C.c_int] * 6 + [C.c_void_p]
            assert shim.shim_mmha(out.data_ptr(), qkv.data_ptr(), kp.data_ptr(), vp.data_ptr(), lens.data_ptr(), B, H, KV, L, step, 1,
                                  st) == 0
        torch.cuda.synchronize()
        outs.append((out.clone(), kc.clone(), vc.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1]) and torch.equal(outs[0][2], outs[1][2])
    assert np.isfinite(outs[1][0].float().cpu().numpy()).all() and float(outs[1][0].abs().max()) > 0
    # a beam search request is outside the LLaMA path: refused, not computed wrongly
    assert shim.shim_mmha(out.data_ptr(), qkv.data_ptr(), kp.data_ptr(), vp.data_ptr(), lens.data_ptr(), B, H, KV, L, step, 4, st) == 1
