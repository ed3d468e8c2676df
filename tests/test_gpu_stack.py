"""GPU parity of the decode-layer glue and of the whole decode stack against the CPU oracle."""
import dataclasses
import importlib

import pytest
import torch

import __graft_entry__ as entry
from helpers import cabi, pq_ops, rel_l2, synth
from oracle import paged_quantized_kv_ops as opq, stack as ostack
from oracle.elementwise_ops import reference_rms_norm
from oracle.mlp_block_ops import reference_quantized_linear

pytestmark = pytest.mark.gpu
entry.load_package()
layer_ops = importlib.import_module("mlx_metal_kernels_b200.ops.decode_layer_ops")
stack_mod = importlib.import_module("mlx_metal_kernels_b200.stack")


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("K,N,B", [(512, 768, 1), (1024, 300, 5), (96, 50, 2)])
def test_norm_quantized_linear(cuda, bits, K, N, B):
    G = 32 if K % 128 else 64
    w, s, z = synth.quantized_weight(N, K, bits, G, seed=K + N)
    x = synth.activations((B, K), 3)
    nw = (torch.rand(K) + 0.5).to(torch.float16)
    normed = reference_rms_norm(x.unsqueeze(1), nw, eps=1e-5)
    want = reference_quantized_linear(normed, w, s, z, bits=bits, group_size=G).squeeze(1)
    got, gn = layer_ops.norm_quantized_linear(x.to(cuda), nw.to(cuda), w.to(cuda), s.to(cuda), z.to(cuda), bits=bits,
                                              group_size=G, return_normed=True)
    assert rel_l2(got, want) <= 1e-3
    if K % 128 == 0:
        pass                                  # the fused path does not materialise the normalised rows
    else:
        assert rel_l2(gn, normed.squeeze(1)) <= 5e-4


@pytest.mark.parametrize("bits,G", [(8, 32), (4, 32), (8, 64)])
def test_rope_kv_append_exact(cuda, bits, G):
    B, Hq, Hkv, D, P = 3, 4, 2, 128, 16
    positions = torch.tensor([0, 17, 40], dtype=torch.int32)
    case = synth.paged_kv_case(B, Hkv, D, P, num_pages=16, min_len=48, max_len=48, bits=bits, group_size=G, seed=9)
    qkv = synth.activations((B, (Hq + 2 * Hkv) * D), 10)
    cos, sin = ostack.rope_tables(D, 500000.0, 64)
    ocache = opq.OraclePagedKV(**{k: (v.clone() if torch.is_tensor(v) else v) for k, v in case.items()})
    x3 = qkv.reshape(B, Hq + 2 * Hkv, D)
    want_q = ostack.apply_rope_rows(x3[:, :Hq], cos, sin, positions)
    ostack.append_kv(ocache, ostack.apply_rope_rows(x3[:, Hq:Hq + Hkv], cos, sin, positions), x3[:, Hq + Hkv:], positions)
    dcache = pq_ops.PagedQuantizedKVCache(**{k: (v.to(cuda) if torch.is_tensor(v) else v) for k, v in case.items()})
    got_q = layer_ops.rope_kv_append(qkv.to(cuda), cos.to(cuda), sin.to(cuda), positions.to(cuda), dcache, Hq)
    assert torch.equal(got_q.cpu(), want_q)
    for name in ("k_pages_q", "v_pages_q", "k_scales", "v_scales"):
        assert torch.equal(getattr(dcache, name).cpu(), getattr(ocache, name)), name


def test_rope_kv_append_reports_bad_positions_and_unassigned_pages(cuda):
    """A position outside the rotary table, or one whose block-table entry is -1, is recorded in the status word
    (events 6 and 7) instead of being dropped silently; the other sequences are appended as usual."""
    B, Hq, Hkv, D, P = 3, 4, 2, 128, 16
    case = synth.paged_kv_case(B, Hkv, D, P, num_pages=16, min_len=48, max_len=48, bits=8, group_size=32, seed=9)
    qkv = synth.activations((B, (Hq + 2 * Hkv) * D), 10)
    cos, sin = ostack.rope_tables(D, 500000.0, 64)
    assert cabi.device_status() == 0

    def run(positions, block_table=None, table=64):
        c = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in case.items()}
        if block_table is not None:
            c["block_table"] = block_table
        dcache = pq_ops.PagedQuantizedKVCache(**{k: (v.to(cuda) if torch.is_tensor(v) else v) for k, v in c.items()})
        layer_ops.rope_kv_append(qkv.to(cuda), cos[:table].to(cuda), sin[:table].to(cuda), positions.to(cuda), dcache, Hq)
        return dcache

    run(torch.tensor([0, 17, 40], dtype=torch.int32))
    assert cabi.device_status() == 0
    run(torch.tensor([0, 17, 40], dtype=torch.int32), table=32)   # position 40 is outside a 32-entry rotary table
    assert cabi.device_status() == 6
    bt = case["block_table"].clone()
    bt[1, 1] = -1                                                  # position 17 of sequence 1 has no page
    before = case["k_pages_q"].clone()
    dcache = run(torch.tensor([0, 17, 40], dtype=torch.int32), bt)
    assert cabi.device_status() == 7
    assert cabi.device_status() == 0                               # reading with reset cleared it
    # sequences 0 and 2 were appended, nothing else changed
    changed = (dcache.k_pages_q.cpu() != before).flatten(1).any(dim=1).nonzero().flatten().tolist()
    assert changed == sorted({int(case["block_table"][0, 0]), int(case["block_table"][2, 2])})


def _tiny_stack(cuda, kv_bits, batch, positions):
    cfg = stack_mod.StackConfig(hidden=512, intermediate=1024, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128,
                                vocab=97, bits=4, group_size=64, kv_bits=kv_bits, kv_group_size=32)
    layers = [stack_mod.random_layer(cfg, 100 + i, "cpu") for i in range(cfg.n_layers)]
    for i, l in enumerate(layers):      # non-trivial norm weights
        g = torch.Generator().manual_seed(i)
        l["input_norm"] = (torch.rand(cfg.hidden, generator=g) + 0.5).to(torch.float16)
        l["post_norm"] = (torch.rand(cfg.hidden, generator=g) + 0.5).to(torch.float16)
    emb = synth.activations((cfg.vocab, cfg.hidden), 5)
    final_norm = torch.ones(cfg.hidden, dtype=torch.float16)
    to = lambda t: t.to(cuda) if torch.is_tensor(t) else tuple(u.to(cuda) for u in t)
    dlayers = [{k: to(v) for k, v in l.items()} for l in layers]
    stack = stack_mod.DecodeStack(cfg, dlayers, final_norm.to(cuda), emb.to(cuda), batch, 96, cuda)
    stack.set_context(0, seed=7)
    stack.positions.copy_(positions.to(cuda))
    stack.lengths.copy_((positions + 1).to(cuda))
    return cfg, layers, emb, final_norm, stack


@pytest.mark.parametrize("kv_bits", [8, 4])
def test_decode_stack_matches_oracle(cuda, kv_bits):
    batch = 3
    positions = torch.tensor([33, 5, 64], dtype=torch.int32)
    cfg, layers, emb, final_norm, stack = _tiny_stack(cuda, kv_bits, batch, positions)
    # oracle caches = copies of the device caches before the step
    ocaches = []
    for c in stack.caches:
        ocaches.append(opq.OraclePagedKV(
            k_pages_q=c.k_codes.cpu().clone(), v_pages_q=c.v_codes.cpu().clone(), k_scales=c.k_scales.cpu().clone(),
            v_scales=c.v_scales.cpu().clone(), block_table=stack.block_table.cpu(), lengths=(positions + 1),
            bits=kv_bits, page_size=cfg.page_size, group_size=cfg.kv_group_size,
            original_page_shape=(stack.num_pages, cfg.page_size, cfg.n_kv_heads, cfg.head_dim)))
    tokens = torch.tensor([3, 50, 96])
    cos, sin = ostack.rope_tables(cfg.head_dim, cfg.rope_theta, 96)
    want = ostack.stack_decode_step(tokens, emb, layers, ocaches, final_norm, cos, sin, positions, cfg.oracle_dict())
    got = stack.step(tokens.to(cuda))
    assert rel_l2(got, want.squeeze(1)) <= 3e-3          # two layers of 1e-3-class operators
    assert torch.equal(stack.positions.cpu(), positions + 1)
    # a captured graph replays the same step bit for bit
    stack.positions.copy_(positions.to(cuda))
    stack.lengths.copy_((positions + 1).to(cuda))
    stack.capture()
    again = stack.step(tokens.to(cuda)).clone()
    assert torch.equal(again, got)
    assert cabi.device_status() == 0


@pytest.mark.parametrize("batch", [1, 32])
def test_full_shape_layer_matches_oracle(cuda, batch):
    """One layer at the shapes the headline number is measured on (hidden 4096, 32 query / 8 kv heads of 128, MLP 14336,
    q4 group-64 weights, q8 group-32 paged KV at context 4096) against the oracle's layer_decode_step: layer output
    within 1e-3 rel-L2; the appended K/V codes and scales are exactly the oracle's quantisation of the rows the device
    computed (they are a rounding of the QKV matvec output, which itself is held to 1e-3, so against the oracle's own
    QKV rows a code may differ by one step)."""
    cfg = stack_mod.StackConfig(n_layers=1, vocab=128)
    assert (cfg.hidden, cfg.intermediate, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim) == (4096, 14336, 32, 8, 128)
    assert (cfg.bits, cfg.group_size, cfg.kv_bits, cfg.kv_group_size) == (4, 64, 8, 32)
    layer = stack_mod.random_layer(cfg, 321, "cpu")
    g = torch.Generator().manual_seed(1)
    layer["input_norm"] = (torch.rand(cfg.hidden, generator=g) + 0.5).to(torch.float16)
    layer["post_norm"] = (torch.rand(cfg.hidden, generator=g) + 0.5).to(torch.float16)
    emb = synth.activations((cfg.vocab, cfg.hidden), 5)
    final_norm = (torch.rand(cfg.hidden, generator=g) + 0.5).to(torch.float16)
    to = lambda t: t.to(cuda) if torch.is_tensor(t) else tuple(u.to(cuda) for u in t)
    context = 4096
    stack = stack_mod.DecodeStack(cfg, [{k: to(v) for k, v in layer.items()}], final_norm.to(cuda), emb.to(cuda), batch,
                                  context + 16, cuda)
    stack.set_context(context, seed=11)
    if batch == 1:
        positions = torch.tensor([context], dtype=torch.int32)
    else:       # ragged: the full context, the first token, page edges, and random lengths
        positions = torch.randint(0, context + 1, (batch,), generator=g, dtype=torch.int32)
        positions[:4] = torch.tensor([context, 0, 15, 16], dtype=torch.int32)
    stack.positions.copy_(positions.to(cuda))
    stack.lengths.copy_((positions + 1).to(cuda))
    c = stack.caches[0]
    ocache = opq.OraclePagedKV(
        k_pages_q=c.k_codes.cpu().clone(), v_pages_q=c.v_codes.cpu().clone(), k_scales=c.k_scales.cpu().clone(),
        v_scales=c.v_scales.cpu().clone(), block_table=stack.block_table.cpu(), lengths=(positions + 1),
        bits=cfg.kv_bits, page_size=cfg.page_size, group_size=cfg.kv_group_size,
        original_page_shape=(stack.num_pages, cfg.page_size, cfg.n_kv_heads, cfg.head_dim))
    before = {n: getattr(ocache, n).clone() for n in ("k_pages_q", "v_pages_q", "k_scales", "v_scales")}
    tokens = torch.randint(0, cfg.vocab, (batch,), generator=g)
    cos, sin = stack.cos.cpu(), stack.sin.cpu()        # the stack's own rotary table: the oracle's formula, host-built
    assert torch.equal(cos, ostack.rope_tables(cfg.head_dim, cfg.rope_theta, cos.shape[0])[0])
    h0 = emb[tokens].unsqueeze(1)
    want_h = ostack.layer_decode_step(h0, layer, ocache, cos, sin, positions, cfg.oracle_dict())
    want_out = reference_rms_norm(want_h, final_norm, eps=cfg.eps)
    got_out = stack.step(tokens.to(cuda))
    torch.cuda.synchronize()
    assert cabi.device_status() == 0
    assert rel_l2(stack.h, want_h.squeeze(1)) <= 1e-3            # the layer's output rows
    assert rel_l2(got_out, want_out.squeeze(1)) <= 1e-3
    # the QKV rows the device produced, and the append of exactly those rows
    Hq, Hkv, D = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    want_qkv = reference_quantized_linear(reference_rms_norm(h0, layer["input_norm"], eps=cfg.eps), *layer["qkv"],
                                          bits=cfg.bits, group_size=cfg.group_size).squeeze(1)
    dev_qkv = stack.qkv.cpu()
    assert rel_l2(dev_qkv, want_qkv) <= 1e-3
    exact = opq.OraclePagedKV(**{**ocache.__dict__, **{n: v.clone() for n, v in before.items()}})
    x3 = dev_qkv.reshape(batch, Hq + 2 * Hkv, D)
    ostack.append_kv(exact, ostack.apply_rope_rows(x3[:, Hq:Hq + Hkv], cos, sin, positions), x3[:, Hq + Hkv:], positions)
    for name, dev in (("k_pages_q", c.k_codes), ("v_pages_q", c.v_codes), ("k_scales", c.k_scales), ("v_scales", c.v_scales)):
        assert torch.equal(dev.cpu(), getattr(exact, name)), name
    # against the oracle's own rows: only the appended slots changed, codes within one step
    for name, dev in (("k_pages_q", c.k_codes), ("v_pages_q", c.v_codes)):
        diff = (dev.cpu().to(torch.int16) - getattr(ocache, name).to(torch.int16)).abs()
        assert int(diff.max()) <= 1, name
        assert float((diff != 0).float().sum()) <= 0.02 * batch * Hkv * D, name
    stack.close()


@pytest.mark.parametrize("bits,B,Hq,Hkv,poss", [(8, 1, 32, 8, [4096]), (4, 2, 32, 8, [16, 700]), (8, 3, 8, 2, [0, 31, 95]),
                                               (8, 1, 4, 4, [47]), (4, 5, 16, 8, [3, 200, 15, 16, 1023])])
@pytest.mark.parametrize("cluster", [1, -1])
def test_rope_append_attention_one_call(cuda, bits, B, Hq, Hkv, poss, cluster):
    """b200q_rope_append_paged_gqa_decode (one cluster kernel at small batch, else append + split-KV attention) against
    the oracle's RoPE, append and attention: appended codes / scales exact, attention rows within 2e-3."""
    P, D = 16, 128
    maxpos = max(poss) + 1
    case = synth.paged_kv_case(B, Hkv, D, P, num_pages=B * ((maxpos + 15) // 16) + 5, min_len=maxpos, max_len=maxpos,
                               bits=bits, group_size=32, seed=9)
    case["lengths"] = torch.tensor([p + 1 for p in poss], dtype=torch.int32)
    qkv = synth.activations((B, (Hq + 2 * Hkv) * D), 10)
    cos, sin = ostack.rope_tables(D, 500000.0, maxpos + 1)
    positions = torch.tensor(poss, dtype=torch.int32)
    ocache = opq.OraclePagedKV(**{k: (v.clone() if torch.is_tensor(v) else v) for k, v in case.items()})
    x3 = qkv.reshape(B, Hq + 2 * Hkv, D)
    want_q = ostack.apply_rope_rows(x3[:, :Hq], cos, sin, positions)
    ostack.append_kv(ocache, ostack.apply_rope_rows(x3[:, Hq:Hq + Hkv], cos, sin, positions), x3[:, Hq + Hkv:], positions)
    want = opq.reference_paged_quantized_kv_gqa_decode_attention(want_q.reshape(B, 1, Hq, D), ocache).reshape(B, Hq, D)
    dcache = pq_ops.PagedQuantizedKVCache(**{k: (v.to(cuda) if torch.is_tensor(v) else v) for k, v in case.items()})
    cabi.set_tuning("attn.cluster", cluster)
    try:
        got = layer_ops.rope_append_attention(qkv.to(cuda), cos.to(cuda), sin.to(cuda), positions.to(cuda), dcache, Hq)
        again_cache = pq_ops.PagedQuantizedKVCache(**{k: (v.to(cuda) if torch.is_tensor(v) else v) for k, v in case.items()})
        again = layer_ops.rope_append_attention(qkv.to(cuda), cos.to(cuda), sin.to(cuda), positions.to(cuda), again_cache, Hq)
    finally:
        cabi.set_tuning("attn.cluster", 0)
    for name in ("k_pages_q", "v_pages_q", "k_scales", "v_scales"):
        assert torch.equal(getattr(dcache, name).cpu(), getattr(ocache, name)), name
    assert float((got.cpu().float() - want.float()).abs().max()) <= 2e-3
    assert torch.equal(again, got)                 # fixed merge order: bitwise repeatable
    assert cabi.device_status() == 0
