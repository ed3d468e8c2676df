"""Checks on 2, 4 and 8 GPUs of the NVLink peer all-gather and of the tensor-parallel stack built on it (each world
size is skipped when fewer GPUs are visible): the gathered rows equal torch's all_gather, repeated calls and CUDA-graph replays keep working,
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


def _rank_main(rank, world, port, result_path, batch):
    import traceback
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    code = 1
    try:
        torch.cuda.set_device(rank)
        device = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        ok = {}
        import __graft_entry__ as entry
        entry.load_package()
        stack_mod = importlib.import_module("mlx_metal_kernels_b200.stack")
        cabi = importlib.import_module("mlx_metal_kernels_b200.ops._cabi")
        n_kv = max(2, world)
        cfg = stack_mod.StackConfig(hidden=512, intermediate=1024, n_layers=2, n_heads=2 * n_kv, n_kv_heads=n_kv,
                                    head_dim=128, vocab=97, bits=4, group_size=64, kv_bits=8, kv_group_size=32)
        layers = [stack_mod.random_layer(cfg, 100 + i, device) for i in range(cfg.n_layers)]
        gen = torch.Generator(device=device).manual_seed(5)
        emb = torch.randn((cfg.vocab, cfg.hidden), generator=gen, device=device).to(torch.float16)
        fnorm = torch.ones(cfg.hidden, dtype=torch.float16, device=device)
        B = batch

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
        plain = stack_mod.DecodeStack(cfg, layers, fnorm, emb, B, 96, device, tp_rank=rank, tp_size=world, process_group=None,
                                      use_peer_gather=True, fuse_exchange=True, exchange_packets=False)
        for src, dst in zip(fused.caches, plain.caches):
            for name in ("k_codes", "v_codes", "k_scales", "v_scales"):
                getattr(dst, name).copy_(getattr(src, name))
        plain.positions.fill_(40)
        plain.lengths.fill_(41)
        ok["peer_enabled"] = bool(peer.peer_gather)
        ok["fused_enabled"] = bool(fused.peer_fused)
        ok["fused_expected"] = bool(fused.fuse_exchange)       # the stack fuses the exchange at small batches only
        ok["transports"] = (nccl.transport, peer.transport, fused.transport)
        ok["peer_error"] = getattr(peer, "peer_gather_error", "") or getattr(fused, "peer_gather_error", "")
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
        for name, st in (("single", single), ("nccl", nccl), ("peer", peer), ("fused", fused), ("plain", plain)):
            st.capture()
            outs[name] = [st.step(toks[i]).clone() for i in range(4)]
        torch.cuda.synchronize()
        ok["nccl_equals_single"] = all(torch.equal(a, b) for a, b in zip(outs["nccl"], outs["single"]))
        ok["peer_equals_single"] = all(torch.equal(a, b) for a, b in zip(outs["peer"], outs["single"]))
        ok["fused_equals_single"] = all(torch.equal(a, b) for a, b in zip(outs["fused"], outs["single"]))
        ok["plain_fused_equals_single"] = all(torch.equal(a, b) for a, b in zip(outs["plain"], outs["single"]))
        ok["exchange_counts"] = [fused.verify_exchanges(), plain.verify_exchanges()]
        ok["status"] = int(cabi.device_status())
        gathered = [None] * world
        dist.all_gather_object(gathered, ok)
        if rank == 0:
            torch.save(gathered, result_path)
        torch.cuda.synchronize()
        dist.barrier()                     # no rank leaves while a peer still runs kernels on the shared buffers
        code = 0
    except BaseException:                  # noqa: BLE001 - reported through the exit code and the error file
        with open(f"{result_path}.rank{rank}.err", "w") as fh:
            fh.write(traceback.format_exc())
    finally:
        sys.stdout.flush()
        sys.stderr.flush()
        # captured graphs hold NCCL kernels, so the library teardown is skipped; a rank that failed leaves with a
        # non-zero code and the parent ends the others
        os._exit(code)


def _run_world(world, batch, tmp_path):
    import time
    import torch.multiprocessing as mp
    result = str(tmp_path / "result.pt")
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, result, batch)) for r in range(world)]
    for p in procs:
        p.start()
    deadline = time.time() + 300
    while time.time() < deadline and any(p.is_alive() for p in procs):
        if any(p.exitcode not in (None, 0) for p in procs):
            break                          # a rank failed: its peers may be waiting for it
        time.sleep(0.2)
    stragglers = [p for p in procs if p.is_alive()]
    if stragglers and all(p.exitcode in (None, 0) for p in procs) and time.time() < deadline:
        for p in stragglers:
            p.join(timeout=10)
        stragglers = [p for p in procs if p.is_alive()]
    for p in stragglers:
        p.terminate()
    for p in stragglers:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
            p.join(timeout=20)
    errors = []
    for r in range(world):
        path = f"{result}.rank{r}.err"
        if os.path.exists(path):
            errors.append(f"rank {r}:\n" + open(path).read())
    assert not errors, "\n".join(errors)
    assert not stragglers, f"{len(stragglers)} rank(s) had to be terminated"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return torch.load(result)


@pytest.mark.parametrize("world,batch", [(2, 3), (2, 20), (4, 3), (4, 32), (8, 3), (8, 32)])
def test_peer_gather_and_sharded_stack(tmp_path, world, batch):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    rows = _run_world(world, batch, tmp_path)
    assert all(ok["nccl_equals_single"] and ok["status"] == 0 for ok in rows), rows
    if not rows[0]["peer_enabled"]:
        pytest.skip(f"symmetric memory unavailable, NCCL transport only: {rows[0]['peer_error']}")
    for ok in rows:
        assert ok["status"] == 0, ok
        assert ok["nccl_equals_single"], ok
        assert ok["peer_enabled"], ok
        assert ok["peer_equals_single"], ok
        assert all(v for k, v in ok.items() if k.startswith("gather_")), ok
        assert ok["fused_enabled"] == ok["fused_expected"], ok
        assert ok["fused_equals_single"], ok          # at large batches this stack runs the stand-alone exchange
        assert ok["transports"] == ("nccl", "peer_kernel", "fused_packets" if ok["fused_expected"] else "peer_kernel"), ok
        assert ok["plain_fused_equals_single"], ok      # the fused exchange with flag words instead of packets
