"""CPU: the header shims under include/compat let the reference's own call sites compile unchanged.

The shims shadow three headers of lmdeploy v0.0.9 by path (`-I include/compat` ahead of the TurboMind source
root).  Compiled here, with nvcc and no GPU, and with every symbol left undefined in the object being one the
library exports:
  * a translation unit that includes the reference's src/turbomind/models/llama/LlamaLinear.h as it is and
    instantiates LlamaLinear<half> (forwardInt4, LlamaLinear.h:62-81, calls GemmS4F16::Run);
  * the reference's src/turbomind/models/llama/LlamaDecoderSelfAttentionLayer.cc as it is
    (fusedQKV_masked_attention_dispatch, :44-166, fills Masked_multihead_attention_params<uint16_t>);
  * a translation unit of this test that calls every converter of format.h (needs no reference tree).
The first two are skipped where the reference tree is absent.
"""
import os
import re
import shutil
import subprocess

import pytest

from oracle.build_ref import DEFAULT_REFERENCE

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
INCLUDES = ["-I", os.path.join(ROOT, "include", "compat"), "-I", os.path.join(ROOT, "include")]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-w", "-x", "cu", "-c"]

pytestmark = pytest.mark.skipif(not os.path.exists(NVCC), reason="nvcc not found")


def undefined_tm_symbols(obj):
    out = subprocess.run(["nm", "-C", obj], capture_output=True, text=True, check=True).stdout
    return sorted(set(re.findall(r"^\s+U (tm_\w+)", out, flags=re.M)))


def exported_symbols():
    from lmdeploy_b200.build import build
    lib = build()
    out = subprocess.run(["nm", "-D", "--defined-only", lib], capture_output=True, text=True, check=True).stdout
    return set(re.findall(r" T (tm_\w+)", out))


def compile_tu(tmp_path, name, source_path, extra=()):
    obj = str(tmp_path / (name + ".o"))
    r = subprocess.run([NVCC] + FLAGS + [source_path, "-o", obj] + INCLUDES + list(extra), capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return obj


def need_reference():
    probe = os.path.join(DEFAULT_REFERENCE, "src", "turbomind", "models", "llama", "LlamaLinear.h")
    if not os.path.exists(probe):
        pytest.skip("reference tree not present")
    return DEFAULT_REFERENCE


def test_reference_llama_linear_compiles_against_the_gemm_shim(tmp_path):
    ref = need_reference()
    src = tmp_path / "tu_linear.cu"
    src.write_text('#include "src/turbomind/models/llama/LlamaLinear.h"\n'
                   "template class turbomind::LlamaLinear<half>;\n")
    obj = compile_tu(tmp_path, "tu_linear", str(src), ["-I", ref])
    und = undefined_tm_symbols(obj)
    assert "tm_gemm_s4_f16" in und and "tm_handle_of_current_device" in und
    assert set(und) <= exported_symbols()
    # the shim was the header that got used: the reference's class has an Impl and an out-of-line constructor
    syms = subprocess.run(["nm", "-C", obj], capture_output=True, text=True).stdout
    assert "GemmS4F16::Impl" not in syms and "U turbomind::GemmS4F16::GemmS4F16" not in syms


def test_reference_decoder_self_attention_layer_compiles_against_the_shims(tmp_path):
    ref = need_reference()
    src = os.path.join(ref, "src", "turbomind", "models", "llama", "LlamaDecoderSelfAttentionLayer.cc")
    obj = compile_tu(tmp_path, "tu_attn", src, ["-I", ref])
    und = undefined_tm_symbols(obj)
    assert {"tm_mmha_decode", "tm_gemm_s4_f16", "tm_handle_of_current_device"} <= set(und)
    assert set(und) <= exported_symbols()
    syms = subprocess.run(["nm", "-C", obj], capture_output=True, text=True).stdout
    # no call into the reference's own kernels is left in the object
    assert not re.search(r"U .*masked_multihead_attention", syms)


def test_format_shim_compiles_standalone(tmp_path):
    src = tmp_path / "tu_format.cu"
    src.write_text(
        '#include "src/turbomind/kernels/gemm_s_f16/format.h"\n'
        "void use_all(uint32_t* a, const uint32_t* b, half2* q, half* w, const half* s, uint4* d, cudaStream_t st)\n"
        "{\n"
        "    turbomind::reformat_s4_k_m8(a, b, 4096, 4096, st);\n"
        "    turbomind::convert_s4_k_m8(a, q, w, b, s, b, 4096, 4096, 128, st);\n"
        "    turbomind::transpose_qk_s4_k_m8_hf(a, b, 4096, 4096, 128);\n"
        "    turbomind::fuse_w1_w3_s4_k_m8(a, b, 22016, 4096);\n"
        "    turbomind::dequantize_s4(d, b, 1024, st);\n"
        "}\n")
    obj = compile_tu(tmp_path, "tu_format", str(src))
    und = undefined_tm_symbols(obj)
    assert {"tm_reformat_s4_k_m8", "tm_convert_s4_k_m8", "tm_transpose_qk_s4_k_m8_hf", "tm_fuse_w1_w3_s4_k_m8",
            "tm_dequantize_s4"} <= set(und)
    assert set(und) <= exported_symbols()
