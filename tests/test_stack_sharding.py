"""Host-side logic of the tensor-parallel decode stack on CPU: two (and four) gloo ranks shard one layer with
``shard_layer``, run the layer with the oracle's per-op functions on their shards, re-assemble the
activations with the stack's own ``_all_gather_rows`` and must reproduce the unsharded oracle layer."""
import importlib
import os
import socket
import sys
import types

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tiny(stack_mod):
    cfg = stack_mod.StackConfig(hidden=512, intermediate=1024, n_layers=1, n_heads=8, n_kv_heads=4, head_dim=64,
                                vocab=31, bits=4, group_size=64, kv_bits=8, kv_group_size=32)
    layer = stack_mod.random_layer(cfg, 7, "cpu")
    gen = torch.Generator().manual_seed(5)
    layer["input_norm"] = (torch.rand(cfg.hidden, generator=gen) + 0.5).to(torch.float16)
    layer["post_norm"] = (torch.rand(cfg.hidden, generator=gen) + 0.5).to(torch.float16)
    return cfg, layer


def _kv_case(cfg, batch, context):
    from oracle import paged_quantized_kv_ops as opq
    P = cfg.page_size
    blocks = (context + 1 + P - 1) // P
    gen = torch.Generator().manual_seed(11)
    shape = (batch * blocks, P, cfg.n_kv_heads, cfg.head_dim)
    k = torch.randn(shape, generator=gen)
    v = torch.randn(shape, generator=gen)
    cache = opq.quantize_kv_pages(k, v, torch.arange(batch * blocks, dtype=torch.int32).reshape(batch, blocks),
                                  torch.full((batch,), context, dtype=torch.int32), bits=cfg.kv_bits,
                                  group_size=cfg.kv_group_size)
    return cache


def _slice_heads(cache, lo, hi):
    """The kv heads [lo, hi) of an oracle cache as a cache of their own."""
    from oracle import paged_quantized_kv_ops as opq
    n, P, _, D = cache.original_page_shape
    return opq.OraclePagedKV(k_pages_q=cache.k_pages_q[:, :, lo:hi].clone(), v_pages_q=cache.v_pages_q[:, :, lo:hi].clone(),
                             k_scales=cache.k_scales[:, :, lo:hi].clone(), v_scales=cache.v_scales[:, :, lo:hi].clone(),
                             block_table=cache.block_table, lengths=cache.lengths, bits=cache.bits,
                             group_size=cache.group_size, original_page_shape=(n, P, hi - lo, D))


def _rank_main(rank, WORLD, port, result_path, B=3):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        import __graft_entry__ as entry
        entry.load_package()
        stack_mod = importlib.import_module("mlx_metal_kernels_b200.stack")
        from oracle import stack as ostack
        from oracle.elementwise_ops import reference_residual_add, reference_rms_norm, reference_swiglu
        from oracle.mlp_block_ops import reference_quantized_linear
        from oracle.paged_quantized_kv_ops import reference_paged_quantized_kv_gqa_decode_attention

        torch.manual_seed(0)
        cfg, layer = _tiny(stack_mod)
        context = 21
        D, bits, G = cfg.head_dim, cfg.bits, cfg.group_size
        h = (torch.randn(B, 1, cfg.hidden, generator=torch.Generator().manual_seed(3)) * 0.5).to(torch.float16)
        positions = torch.full((B,), context, dtype=torch.int32)
        if B > 3:                                           # ragged batch: every length from 1 to the full context
            positions = (torch.arange(B, dtype=torch.int32) * 5) % (context + 1)
        cos, sin = ostack.rope_tables(D, cfg.rope_theta, 64)

        # unsharded answer
        full_cache = _kv_case(cfg, B, context)
        want = ostack.layer_decode_step(h, layer, full_cache, cos, sin, positions, cfg.oracle_dict())

        # this rank's share, with the stack's own sharding and gather helpers
        w = stack_mod.shard_layer(layer, cfg, rank, WORLD)
        hq, hkv = cfg.n_heads // WORLD, cfg.n_kv_heads // WORLD
        fake = types.SimpleNamespace(pg=None)
        gather = lambda local: stack_mod.DecodeStack._all_gather_rows(           # noqa: E731
            fake, local.contiguous(), torch.empty((WORLD, *local.shape), dtype=local.dtype))
        lin = lambda x, triple: reference_quantized_linear(x, *triple, bits=bits, group_size=G)  # noqa: E731

        x_norm = reference_rms_norm(h, layer["input_norm"], eps=cfg.eps)
        qkv = lin(x_norm, w["qkv"]).reshape(B, hq + 2 * hkv, D)
        q = ostack.apply_rope_rows(qkv[:, :hq], cos, sin, positions)
        k = ostack.apply_rope_rows(qkv[:, hq:hq + hkv], cos, sin, positions)
        cache = _slice_heads(_kv_case(cfg, B, context), rank * hkv, (rank + 1) * hkv)
        ostack.append_kv(cache, k, qkv[:, hq + hkv:], positions)
        cache.lengths = positions + 1
        attn = reference_paged_quantized_kv_gqa_decode_attention(q.reshape(B, 1, hq, D), cache).reshape(B, hq * D)
        attn_full = gather(attn)
        o_full = gather(lin(attn_full.unsqueeze(1), w["o"]).squeeze(1))
        h2 = reference_residual_add(h.squeeze(1), o_full)
        normed = reference_rms_norm(h2.unsqueeze(1), layer["post_norm"], eps=cfg.eps)
        act = reference_swiglu(lin(normed, w["gate"]), lin(normed, w["up"])).squeeze(1)
        act_full = gather(act)
        d_full = gather(lin(act_full.unsqueeze(1), w["down"]).squeeze(1))
        got = reference_residual_add(h2, d_full)

        # every rank holds the whole answer after the last gather
        err = (got.float() - want.squeeze(1).float()).abs().max().item()
        ref = want.float().abs().max().item()
        ok_shapes = got.shape == (B, cfg.hidden) and attn_full.shape == (B, cfg.n_heads * D)
        all_err = [None] * WORLD
        dist.all_gather_object(all_err, (err, ref, bool(ok_shapes)))
        if rank == 0:
            torch.save(all_err, result_path)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("WORLD,B", [(2, 3), (4, 3), (2, 32)])
def test_sharded_layer_matches_unsharded(tmp_path, WORLD, B):
    result = str(tmp_path / "result.pt")
    mp.spawn(_rank_main, args=(WORLD, _free_port(), result, B), nprocs=WORLD, join=True)
    rows = torch.load(result)
    assert len(rows) == WORLD
    for err, ref, ok_shapes in rows:
        assert ok_shapes
        # same dot products on both sides; only the host BLAS blocking may differ between row subsets
        assert err <= 2.0 ** -10 * max(ref, 1.0), (err, ref)


def _desync_rank(rank, WORLD, port, result_path):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        import __graft_entry__ as entry
        entry.load_package()
        stack_mod = importlib.import_module("mlx_metal_kernels_b200.stack")
        counts = [0, 0, 0]                       # exchanges issued per buffer (attention rows, hidden rows, MLP rows)
        report = {}
        for step in range(3):
            for which in (0, 1, 2, 1):           # the four exchanges of a layer
                if step == 1 and rank == WORLD - 1 and which == 2:
                    continue                     # this rank skips one exchange of the second step
                counts[which] += 1
            try:
                report[step] = ("ok", stack_mod.verify_exchange_counts(counts))
            except stack_mod.ExchangeDesync as exc:
                report[step] = ("desync", str(exc))
                break                            # every rank stops before its next launch
        rows = [None] * WORLD
        dist.all_gather_object(rows, report)
        if rank == 0:
            torch.save(rows, result_path)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("WORLD", [2, 3])
def test_skipped_exchange_is_reported_on_every_rank(tmp_path, WORLD):
    """A rank that skips an exchange is found by the host-side count check before the next step on ALL ranks
    (the device-side symptom would be the peers' bounded wait running out one step later)."""
    result = str(tmp_path / "result.pt")
    mp.spawn(_desync_rank, args=(WORLD, _free_port(), result), nprocs=WORLD, join=True)
    rows = torch.load(result)
    assert len(rows) == WORLD
    for report in rows:
        assert report[0] == ("ok", [1, 2, 1])
        kind, text = report[1]
        assert kind == "desync" and f"lagging ranks {{{WORLD - 1}: [2, 4, 1]}}" in text and "[2, 4, 2]" in text
        assert 2 not in report


def test_shard_rows_and_qkv_layout():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    stack_mod = importlib.import_module("mlx_metal_kernels_b200.stack")
    cfg, layer = _tiny(stack_mod)
    assert stack_mod.shard_rows(8, 1, 2) == (4, 8)
    with pytest.raises(ValueError):
        stack_mod.shard_rows(7, 0, 2)
    D = cfg.head_dim
    codes = layer["qkv"][0]
    parts = [stack_mod.shard_layer(layer, cfg, r, 2)["qkv"][0] for r in range(2)]
    hq, hkv = cfg.n_heads // 2, cfg.n_kv_heads // 2
    for r, part in enumerate(parts):
        assert part.shape[0] == (hq + 2 * hkv) * D
        assert torch.equal(part[:hq * D], codes[r * hq * D:(r + 1) * hq * D])
        k0 = cfg.n_heads * D + r * hkv * D
        assert torch.equal(part[hq * D:(hq + hkv) * D], codes[k0:k0 + hkv * D])
        v0 = (cfg.n_heads + cfg.n_kv_heads) * D + r * hkv * D
        assert torch.equal(part[(hq + hkv) * D:], codes[v0:v0 + hkv * D])
    for key, n in (("o", cfg.hidden), ("gate", cfg.intermediate), ("up", cfg.intermediate), ("down", cfg.hidden)):
        whole = torch.cat([stack_mod.shard_layer(layer, cfg, r, 2)[key][0] for r in range(2)])
        assert torch.equal(whole, layer[key][0]) and whole.shape[0] == n
    assert stack_mod.shard_layer(layer, cfg, 0, 1) is layer
