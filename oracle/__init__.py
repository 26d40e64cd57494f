"""CPU oracle for the W4A16 decode hot path (TEST INFRASTRUCTURE, not product code).

Every function here restates, on the CPU with numpy / torch, the arithmetic of one
piece of the reference lmdeploy v0.0.9 TurboMind decode path and cites the reference
file:line it follows.  Nothing under ``lmdeploy_b200/`` imports this package: only
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` do,
and only as the checker or as the timed CPU baseline.

Pin status
----------
* ``oracle.awq`` (quantiser, AWQ nibble packing) is pinned against outputs of the
  reference's own torch code (``lmdeploy/lite/utils/cal_qparams.py``,
  ``lmdeploy/lite/quantization/weight/quantizer.py``,
  ``lmdeploy/pytorch/modules/linear.py``) imported by file path; the vectors live in
  ``tests/golden/awq_reference_vectors.npz`` next to the script that wrote them.
* ``oracle.s4_format`` (layout conversion), ``oracle.gemm``, ``oracle.attention`` and the fused
  residual-add of ``oracle.norm`` restate CUDA code for which the reference holds no CPU
  implementation, golden vector or test of its own.  They are pinned against the reference's
  CUDA kernels themselves: ``oracle/build_ref.py`` compiles the reference sources, unmodified and
  where they lie, into ``oracle/_ref/libtm_ref.so`` (``ref_kernels.cu`` is the flat C entry layer);
  ``tests/golden/make_ref_kernel_vectors.py`` ran them on a B200 and wrote
  ``tests/golden/ref_kernel_vectors.npz``, which ``tests/test_oracle_ref_vectors.py`` checks on the
  CPU (format bit for bit, the rest within the fp16 tolerances), and
  ``tests/test_gpu_reference_kernels.py`` runs reference kernel, library and oracle side by side
  on a GPU.  The plain ``rmsnorm`` of ``oracle.norm`` is pinned the same way (``llama_kernels.cu`` is part
  of that build; the flash-attention entry it references is an empty stub in ``ref_kernels.cu``).
  Not pinned: ``oracle.decoder`` (the sequencing of the pinned parts).
* ``oracle.cache_manager`` is pinned against the reference's own ``LlamaCacheManager.cc`` compiled into
  ``oracle/_ref`` (side by side on a GPU, and through the committed trace ``tests/golden/ref_cache_manager_trace.npz``
  on the CPU); ``oracle.sampling`` against the reference's penalty, top-k and top-p sampling kernels in the same library
  (``tests/test_gpu_sampling.py``), with known answers on the CPU (``tests/test_oracle_sampling.py``).
"""
