"""Build oracle/_ref/libtm_ref.so: the REFERENCE's own CUDA kernels for this path, compiled from the
sources where they lie (never copied), plus the flat C entry layer in ref_kernels.cu.

    python oracle/build_ref.py [--reference /path/to/lmdeploy]

Test infrastructure only.  The output directory is git-ignored; the built library travels with the
working tree to a GPU machine, where the reference sources are not needed any more.  Without the
reference tree (or nvcc) this does nothing and returns None; tests that need the library skip.
"""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libtm_ref.so")
# the reference tree: TM_REFERENCE_ROOT, else a checkout named "reference" beside this repository
DEFAULT_REFERENCE = os.environ.get("TM_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))

REFERENCE_SOURCES = [
    "src/turbomind/kernels/gemm_s_f16/format.cu",
    "src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.cu",
    "src/turbomind/kernels/decoder_masked_multihead_attention.cu",
    "src/turbomind/kernels/decoder_masked_multihead_attention/decoder_masked_multihead_attention_128.cu",
    "src/turbomind/models/llama/llama_decoder_kernels.cu",
    "src/turbomind/models/llama/llama_kernels.cu",
    "src/turbomind/kernels/unfused_attention_kernels.cu",
    "src/turbomind/models/llama/LlamaCacheManager.cc",
    "src/turbomind/kernels/sampling_penalty_kernels.cu",
    "src/turbomind/kernels/sampling_topk_kernels.cu",
    "src/turbomind/kernels/sampling_topp_kernels.cu",
    "src/turbomind/kernels/ban_bad_words.cu",
    "src/turbomind/kernels/stop_criteria_kernels.cu",
    "src/turbomind/utils/logger.cc",
    "src/turbomind/utils/Tensor.cc",
]


def build(reference: str = DEFAULT_REFERENCE, force: bool = False):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    srcs = [os.path.join(reference, s) for s in REFERENCE_SOURCES]
    if not os.path.exists(nvcc) or not all(os.path.exists(s) for s in srcs):
        return LIB if os.path.exists(LIB) else None
    wrapper = os.path.join(HERE, "ref_kernels.cu")
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= max(os.path.getmtime(f) for f in srcs + [wrapper]):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-w", "-I", reference]
    objs = []
    for src in srcs + [wrapper]:
        obj = os.path.join(OUT_DIR, os.path.basename(src) + ".o")
        r = subprocess.run([nvcc] + flags + ["-c", src, "-o", obj], capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError(f"nvcc failed on {src}")
        objs.append(obj)
    r = subprocess.run([nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"],
                       capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    for o in objs:
        os.remove(o)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.force))
