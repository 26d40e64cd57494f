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
* ``oracle.s4_format`` (layout conversion), ``oracle.gemm`` , ``oracle.attention`` and
  ``oracle.norm`` restate CUDA code for which the reference holds no CPU
  implementation, golden vector or known-answer test: **parity unpinned** by the
  reference's own tests.  They are cross-checked on a GPU against the reference's CUDA
  sources compiled unmodified into ``oracle/_ref`` (see ``oracle/build_ref.py``).
"""
