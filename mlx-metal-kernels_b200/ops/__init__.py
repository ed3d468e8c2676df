"""Operator modules mirroring the reference's ``ops`` package for the quantized decode path.

``quant_ops``, ``mlp_block_ops``, ``paged_quantized_kv_ops`` and ``quantized_kv_cache_ops`` keep the reference's function
names, argument order, defaults and error messages; ``activation_ops``, ``norm_ops``,
``fused_ops``, ``paged_kv_ops`` and ``gqa_ops`` carry the small pieces those three call.
Tensors are ``torch.Tensor`` on a CUDA device; every compute call goes through the C ABI of
``libb200q.so`` (``_cabi``).
"""
