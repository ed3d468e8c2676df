"""Two-GPU checks of the NVLink peer all-gather and of the tensor-parallel stack built on it (skipped on a
single GPU): the gathered rows equal torch's all_gather, repeated calls and CUDA-graph replays keep working,
and the sharded stack, over peer gathers as over NCCL gathers, reproduces the unsharded one bit for bit (the
matvec sums a row's k-spans in k order whatever CTA holds the row, and the attention cuts the page list
independently of the number of heads)."""
import importlib
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, result_path):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    ok = {}
    try:
        import __graft_entry__ as entry
        entry.load_package()
        stack_mod = importlib.import_module("mlx_metal_kernels_b200.stack")
        cabi = importlib.import_module("mlx_metal_kernels_b200.ops._cabi")
        cfg = stack_mod.StackConfig(hidden=512, intermediate=1024, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128,
                                    vocab=97, bits=4, group_size=64, kv_bits=8, kv_group_size=32)
        layers = [stack_mod.random_layer(cfg, 100 + i, device) for i in range(cfg.n_layers)]
        gen = torch.Generator(device=device).manual_seed(5)
        emb = torch.randn((cfg.vocab, cfg.hidden), generator=gen, device=device).to(torch.float16)
        fnorm = torch.ones(cfg.hidden, dtype=torch.float16, device=device)
        B = 3

        def make(tp_rank, tp_size, peer, fused=False):
            st = stack_mod.DecodeStack(cfg, layers, fnorm, emb, B, 96, device, tp_rank=tp_rank, tp_size=tp_size,
                                       process_group=None, use_peer_gather=peer, fuse_exchange=fused)
            for i, c in enumerate(st.caches):          # same context on every rank: fill the full cache, keep own heads
                full = stack_mod.PagedKV(cfg, cfg.n_kv_heads, st.num_pages, device)
                full.fill_random(cfg, 900 + i)
                lo = tp_rank * st.hkv
                for name in ("k_codes", "v_codes", "k_scales", "v_scales"):
                    getattr(c, name).copy_(getattr(full, name)[:, :, lo:lo + st.hkv])
            st.positions.fill_(40)
            st.lengths.fill_(41)
            return st

        single = make(0, 1, False)
        nccl = make(rank, world, False)
        peer = make(rank, world, True)
        fused = make(rank, world, True, fused=True)
        ok["peer_enabled"] = bool(peer.peer_gather)
        ok["fused_enabled"] = bool(fused.peer_fused)
        ok["peer_error"] = getattr(peer, "peer_gather_error", "")
        # the gather by itself, several calls in a row
        if peer.peer_gather:
            for it in range(5):
                local = torch.randn((B, cfg.hidden // world), device=device).to(torch.float16) + rank
                got = peer._gather(1, local).clone()
                parts = [torch.empty_like(local) for _ in range(world)]
                dist.all_gather(parts, local)
                ok[f"gather_{it}"] = bool(torch.equal(got, torch.cat(parts, dim=1)))
        toks = torch.randint(0, cfg.vocab, (4, B), device=device)
        dist.broadcast(toks, 0)
        outs = {}
        for name, st in (("single", single), ("nccl", nccl), ("peer", peer), ("fused", fused)):
            st.capture()
            outs[name] = [st.step(toks[i]).clone() for i in range(4)]
        torch.cuda.synchronize()
        ok["nccl_equals_single"] = all(torch.equal(a, b) for a, b in zip(outs["nccl"], outs["single"]))
        ok["peer_equals_single"] = all(torch.equal(a, b) for a, b in zip(outs["peer"], outs["single"]))
        ok["fused_equals_single"] = all(torch.equal(a, b) for a, b in zip(outs["fused"], outs["single"]))
        ok["status"] = int(cabi.device_status())
        gathered = [None] * world
        dist.all_gather_object(gathered, ok)
        if rank == 0:
            torch.save(gathered, result_path)
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        sys.stdout.flush()
        os._exit(0)          # captured graphs hold NCCL kernels: leave without the library teardown


def test_peer_gather_and_sharded_stack(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    result = str(tmp_path / "result.pt")
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    rows = torch.load(result)
    for ok in rows:
        assert ok["status"] == 0, ok
        assert ok["nccl_equals_single"], ok
        if ok["peer_enabled"]:
            assert ok["peer_equals_single"], ok
        if ok["fused_enabled"]:
            assert ok["fused_equals_single"], ok
            assert all(v for k, v in ok.items() if k.startswith("gather_")), ok
    print("peer gather enabled:", rows[0]["peer_enabled"], "fused exchange enabled:", rows[0]["fused_enabled"],
          rows[0]["peer_error"])
