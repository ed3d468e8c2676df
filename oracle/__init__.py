"""CPU oracle for the quantized single-token decode hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; the only callers are the test-suite, the GPU smoke check and the
CPU-baseline leg of the benchmark.  The shipped operators raise when the CUDA
library is missing instead of falling back to this code.

What it is
----------
A torch-CPU restatement, cast point by cast point, of the pure-MLX
``backend="reference"`` functions of manishklach/mlx-metal-kernels:

* ``quant_ops``                -> ops/quant_ops.py:166-212, 256-276, 336-342, 509-526, 574-588
* ``elementwise_ops``          -> ops/activation_ops.py:83-88, ops/norm_ops.py:47-52,
                                  ops/fused_ops.py:149-152, 194-209
* ``mlp_block_ops``            -> ops/mlp_block_ops.py:77-101, 128-166, 236-364
* ``paged_kv_ops``             -> ops/paged_kv_ops.py:138-152, ops/kv_cache_ops.py:37-61,
                                  ops/gqa_ops.py:42-66
* ``paged_quantized_kv_ops``   -> ops/paged_quantized_kv_ops.py:38-186, 194-341, 375-515
                                  (ragged-length semantics from
                                  kernels/q4_paged_gqa_decode_attention.metal:37-93)

The arithmetic that defines those functions lives in MLX (``mx.matmul`` in
fp32, ``astype`` round-to-nearest-even, ``mx.round`` = rint, ``mx.softmax``),
an un-vendored and unpinned dependency of the reference (pyproject.toml:15,
``dependencies = ["mlx", "numpy"]``) that cannot be installed here.

Pinning status
--------------
* dequantisation, q4 packing and the symmetric weight quantiser are pinned
  against the numpy code the reference ships (models/quantize_weights.py)
  through the committed fixtures in tests/golden/.
* dequantisation, the serial matvec, the paged q4/q8 decode attention, the
  block-table lookup and SwiGLU are additionally pinned against the
  reference's own Metal kernel bodies compiled as C++ (``oracle/_ref``,
  built by ``oracle/Makefile`` from the sources where they lie).
* the MLX ``reference_*`` functions themselves could not be executed:
  at the MLX boundary **parity is unpinned** by bytes and rests on the
  formulas restated here.
"""
