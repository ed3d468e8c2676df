"""B200-native quantized single-token decode hot path.

Drop-in CUDA (sm_100a) backend for the q4/q8 group-wise matvec family, the fused
gate/up + SwiGLU MLP block and the q4/q8 paged-KV GQA decode attention of
manishklach/mlx-metal-kernels, behind that project's Python entry points
(``ops.quant_ops``, ``ops.mlp_block_ops``, ``ops.paged_quantized_kv_ops``).

The directory name is not a Python identifier; load it with
``importlib`` (see ``__graft_entry__.load_package``) under the alias
``mlx_metal_kernels_b200``.
"""
__version__ = "0.1.0"
