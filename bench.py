#!/usr/bin/env python
"""Benchmark of the quantized single-token decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch B]

One "step" is one decode step of the 32-layer Llama-3-8B-shaped q4 stack (hidden 4096, 32 q / 8 kv
heads, head_dim 128, MLP 14336, q4 group-64 weights ~N(0,0.02), q8 paged KV cache at context 4096)
for a batch of random token ids: the composition of the hot-path operators (fused RMSNorm+QKV
matvec, RoPE + quantised KV append, paged GQA decode attention, O matvec + residual, fused
RMSNorm + gate/up + SwiGLU, down matvec + residual).  Each step streams about 4.2 GB of weights and
KV from HBM (far more than L2), so no cache flush is needed between steps.

Rank 0 prints ONE JSON line.  With N > 1 the stack is tensor-parallel over the N GPUs of the node
(weights sharded by output rows, KV by kv heads, NCCL all-gather at the layer boundaries): total work
is fixed, so ``scaling`` is "strong".
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

CONTEXT = 4096
ROTATE_BYTES = 512 * 1024 * 1024          # distinct operand bytes per rotation of a kernel micro-benchmark (> 2x L2)
METRIC = "decode tokens/s"
WORKLOAD = "c5_llama3_8b_shaped_q4_stack_32_layers_q8_paged_kv_ctx4096"


# dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of one batch-1 matvec launch, per shape of the
# stack, from the ncu captures summarised in profiles/qgemv_kernel_c5_stack_shapes_b1.md (one kernel, two launches
# each, `bench.py --profile-case <shape>_q4_b1`); the kernels read every weight byte once.
DRAM_TRAFFIC_RATIO = {"qkv": 1.0040, "o": 1.0064, "gate": 1.0075, "down": 1.0018}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# clocks sampled during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.rows = gpu_index, []
        self._stop, self._thread = threading.Event(), None

    def _loop(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.gpu_index)], capture_output=True, text=True, timeout=5).stdout
                self.rows += [[c.strip() for c in line.split(",")] for line in out.strip().splitlines()]
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                reasons |= {n for n, v in zip(names, r[5:9]) if v.lower().startswith("active")}
            except (ValueError, IndexError):
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# kernel micro-benchmarks (cold cache through rotating operand copies), reported beside the headline
# ------------------------------------------------------------------------------------------------
def _time_graph(fn, iters, stream):
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            graph.replay()
        e1.record(stream)
        e1.synchronize()
    return e0.elapsed_time(e1) / 1e3 / iters


def _cpu_time(fn, budget_s=8.0):
    """Mean seconds of ``fn`` on the host cores: one warm-up, then runs until ``budget_s`` is spent (at most 5)."""
    fn()
    t0 = time.perf_counter()
    n = 0
    while n < 5 and (n == 0 or time.perf_counter() - t0 < budget_s):
        fn()
        n += 1
    return (time.perf_counter() - t0) / n, n


def kernel_microbenchmarks(device, peak, all_configs=False, cpu=False):
    """BASELINE configs C1 (q4 matvec 4096x4096, batch 1) and C4 (q4 paged GQA decode attention, batch 16,
    lengths U[1024, 8192]); with ``all_configs`` also C2 (q8 matvec 4096->14336, batch 1 / 8) and C3 (q4 MLP
    block, batch 1 / 8 / 32).  achieved = algorithmic bytes / average launch time, operands rotated through
    copies totalling more than ROTATE_BYTES so that every launch reads cold data.  With ``cpu`` the same
    call is timed through the oracle on the host cores."""
    q = importlib.import_module(f"{entry.PKG_ALIAS}.ops.quant_ops")
    mlp = importlib.import_module(f"{entry.PKG_ALIAS}.ops.mlp_block_ops")
    pq = importlib.import_module(f"{entry.PKG_ALIAS}.ops.paged_quantized_kv_ops")
    synth = importlib.import_module(f"{entry.PKG_ALIAS}.synth")
    stream = torch.cuda.Stream(device)
    out = {}
    cores = torch.get_num_threads()

    def record(name, sec, nbytes, R, extra=None, cpu_fn=None):
        row = {"us": round(sec * 1e6, 3), "algorithmic_bytes": nbytes, "gbs": round(nbytes / sec / 1e9, 1),
               "frac_of_peak": round(nbytes / sec / 1e9 / peak, 4), "rotating_copies": R}
        if extra:
            row.update(extra)
        if cpu and cpu_fn is not None:
            cs, n = _cpu_time(cpu_fn)
            row["cpu_oracle_us"] = round(cs * 1e6, 1)
            row["cpu_cores"] = cores
            row["cpu_runs"] = n
        out[name] = row

    def matvec_case(name, bits, B, N, K, seed):
        w, s, z = synth.quantized_weight(N, K, bits, 64, seed=seed)
        nbytes = w.numel() + (s.numel() + z.numel()) * 2 + B * K * 2 + B * N * 2
        R = -(-ROTATE_BYTES // nbytes)
        ws, ss, zs = ([t.to(device).clone() for _ in range(R)] for t in (w, s, z))
        x = synth.activations((B, K), seed + 500, device)
        fn = q.q4_matvec_decode if bits == 4 else q.q8_matvec_decode
        sec = _time_graph(lambda: [fn(x, ws[i], ss[i], zs[i], group_size=64, backend="cuda") for i in range(R)], 10, stream) / R
        cpu_fn = None
        if cpu:
            from oracle import quant_ops as oq
            ref = oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode
            xc = x.cpu()
            cpu_fn = lambda: ref(xc, w, s, z, group_size=64)
        record(name, sec, nbytes, R, cpu_fn=cpu_fn)

    matvec_case("c1_q4_matvec_b1_4096x4096_g64", 4, 1, 4096, 4096, 1001)
    if all_configs:
        matvec_case("c2_q8_matvec_b1_4096to14336_g64", 8, 1, 14336, 4096, 1002)
        matvec_case("c2_q8_matvec_b8_4096to14336_g64", 8, 8, 14336, 4096, 1002)
        gw, gs, gz = synth.quantized_weight(14336, 4096, 4, 64, seed=1003)
        uw, us, uz = synth.quantized_weight(14336, 4096, 4, 64, seed=1013)
        dw, ds, dz = synth.quantized_weight(4096, 14336, 4, 64, seed=1023)
        host = (gw, gs, gz, uw, us, uz, dw, ds, dz)
        wbytes = sum(t.numel() * t.element_size() for t in host)
        R = -(-ROTATE_BYTES // wbytes)
        devs = [[t.to(device).clone() for t in host] for _ in range(R)]
        nw = torch.ones(4096, dtype=torch.float16)
        nwd = nw.to(device)
        for B in (1, 8, 32):
            x = synth.activations((B, 1, 4096), 1503 + B, device)
            res = torch.zeros_like(x)
            nbytes = wbytes + B * (4096 * 2 * 3 + 14336 * 2 * 2)   # x, residual, out; the SwiGLU rows written and re-read
            call = lambda d: mlp.quantized_mlp_block(x, res, nwd, d[0], d[1], d[3], d[4], d[6], d[7], gate_zeros=d[2],
                                                     up_zeros=d[5], down_zeros=d[8], bits=4, group_size=64,
                                                     backend_preset="cuda")
            sec = _time_graph(lambda: [call(d) for d in devs], 10, stream) / R
            cpu_fn = None
            if cpu:
                from oracle import mlp_block_ops as om
                xc, rc = x.cpu(), res.cpu()
                cpu_fn = lambda: om.reference_quantized_mlp_block(xc, rc, nw, gw, gs, uw, us, dw, ds, gate_zeros=gz,
                                                                  up_zeros=uz, down_zeros=dz, bits=4, group_size=64)
            record(f"c3_q4_mlp_block_b{B}_4096_14336_g64", sec, nbytes, R, extra={"launches_per_block": 2 if B < 5 else 3},
                   cpu_fn=cpu_fn)
        del devs
        torch.cuda.empty_cache()
    # C4
    case = synth.paged_kv_case(16, 8, 128, 16, num_pages=9000, min_len=1024, max_len=8192, bits=4, group_size=32, seed=1004)
    total = int(case["lengths"].sum())
    nbytes = total * 8 * 144 + int(((case["lengths"] + 15) // 16).sum()) * 4 + 2 * 16 * 32 * 128 * 2
    R = -(-ROTATE_BYTES // nbytes)
    caches = [pq.PagedQuantizedKVCache(**{k: (v.to(device).clone() if torch.is_tensor(v) else v) for k, v in case.items()})
              for _ in range(R)]
    qq = synth.activations((16, 1, 32, 128), 1005, device)
    sec = _time_graph(lambda: [pq.paged_quantized_kv_gqa_decode_attention(qq, c, backend="cuda") for c in caches], 10, stream) / R
    cpu_fn = None
    if cpu:
        from oracle import paged_quantized_kv_ops as opq
        ocache = opq.OraclePagedKV(**case)
        qc = qq.cpu()
        cpu_fn = lambda: opq.reference_paged_quantized_kv_gqa_decode_attention(qc, ocache)
    record("c4_q4_paged_gqa_decode_b16_h32_kv8_d128_p16", sec, nbytes, R, extra={"sum_lengths": total}, cpu_fn=cpu_fn)
    if all_configs:
        # the same caches through the sliding-window entry point (4 sink tokens + the last 1024): the kernel walks
        # only the pages that hold an attended position, so bytes and time follow the window, not the context
        sparse = importlib.import_module(f"{entry.PKG_ALIAS}.ops.sparse_attention_ops")
        pattern = sparse.SparseAttentionPattern("sliding_window_sink", window_size=1024, sink_tokens=4)
        attended = int(torch.clamp(case["lengths"], max=1024 + 4).sum())
        wbytes = attended * 8 * 144 + 16 * 66 * 4 + 2 * 16 * 32 * 128 * 2
        sec = _time_graph(lambda: [pq.sparse_paged_quantized_kv_gqa_decode_attention(qq, c, pattern) for c in caches],
                          10, stream) / R
        record("c4_window1024_sink4_q4_paged_gqa_decode_b16", sec, wbytes, R, extra={"attended_tokens": attended})
    del caches
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------
# own arm
# ------------------------------------------------------------------------------------------------
def build_stack(device, batch, steps_total, rank, world, group):
    stack_mod = importlib.import_module(f"{entry.PKG_ALIAS}.stack")
    synth = importlib.import_module(f"{entry.PKG_ALIAS}.synth")
    cfg = stack_mod.StackConfig()
    layers = [stack_mod.random_layer(cfg, 1005 + i, device) for i in range(cfg.n_layers)]
    gen = torch.Generator(device=device).manual_seed(1005)
    emb = torch.randn((cfg.vocab, cfg.hidden), generator=gen, device=device, dtype=torch.float32).to(torch.float16)
    final_norm = torch.ones(cfg.hidden, dtype=torch.float16, device=device)
    stack = stack_mod.DecodeStack(cfg, layers, final_norm, emb, batch, CONTEXT + steps_total + 16, device,
                                  tp_rank=rank, tp_size=world, process_group=group)
    del layers
    torch.cuda.empty_cache()
    stack.set_context(CONTEXT, seed=2005)
    return cfg, stack


def gemv_only_graph(stack):
    """The matvec launches of one step (no attention, no glue) for the roofline of the dominant kernel."""
    cabi = importlib.import_module(f"{entry.PKG_ALIAS}.ops._cabi")
    lib, cfg, B = stack.lib, stack.cfg, stack.B
    F16 = cabi.F16
    D, G, bits = cfg.head_dim, cfg.group_size, cfg.bits

    def run():
        st = torch.cuda.current_stream().cuda_stream
        for w in stack.layers:
            qw, qs, qz = w["qkv"]
            ow, os_, oz = w["o"]
            gw, gs, gz = w["gate"]
            uw, us, uz = w["up"]
            dw, ds, dz = w["down"]
            cabi.check(lib.b200q_norm_qmatvec(bits, stack.h.data_ptr(), None, w["input_norm"].data_ptr(), F16, cfg.eps, None,
                                              None, qw.data_ptr(), qs.data_ptr(), qz.data_ptr(), None, stack.qkv.data_ptr(),
                                              B, qw.shape[0], cfg.hidden, G, F16, F16, st), "qkv")
            src = stack.attn if stack.tp_size == 1 else stack.attn_full
            dst = stack.h2 if stack.tp_size == 1 else stack.o_loc
            cabi.check(lib.b200q_qmatvec(bits, src.data_ptr(), ow.data_ptr(), os_.data_ptr(), oz.data_ptr(), None,
                                         dst.data_ptr(), B, ow.shape[0], cfg.n_heads * D, G, F16, F16, st), "o")
            cabi.check(lib.b200q_gate_up_swiglu(bits, stack.h2.data_ptr(), gw.data_ptr(), uw.data_ptr(), gs.data_ptr(),
                                                us.data_ptr(), gz.data_ptr(), uz.data_ptr(), None, None, stack.act.data_ptr(),
                                                None, w["post_norm"].data_ptr(), F16, cfg.eps, None, None, B, gw.shape[0],
                                                cfg.hidden, G, F16, F16, st), "gate_up")
            src = stack.act if stack.tp_size == 1 else stack.act_full
            dst = stack.h if stack.tp_size == 1 else stack.o_loc
            cabi.check(lib.b200q_qmatvec(bits, src.data_ptr(), dw.data_ptr(), ds.data_ptr(), dz.data_ptr(), None,
                                         dst.data_ptr(), B, dw.shape[0], cfg.intermediate, G, F16, F16, st), "down")
    return run, 4 * len(stack.layers)


STEPS_PER_ROUND = 128     # BASELINE config 5: 128 decode steps from context 4096; longer runs repeat the round


def time_steps(stack, tokens, steps, warmup, barrier, local, world, e2e=False, host_out=None, min_seconds=1.0):
    """Device time (or, with ``e2e``, host wall time with the token ids copied in from pinned memory and the hidden
    state copied out every step) of ``repeats`` x ``steps`` decode steps; every repeat restarts from context CONTEXT
    (and so does every STEPS_PER_ROUND-th step of a long repeat).  ``repeats`` is chosen so that the timed region
    lasts at least ``min_seconds``.  Returns (seconds per step as the max over ranks, repeats, clock summary)."""
    device = stack.device

    def reset():
        stack.positions.fill_(CONTEXT)
        stack.lengths.fill_(CONTEXT + 1)

    B = stack.B
    n_tok = tokens.shape[0]
    dev_tok = torch.empty(B, dtype=torch.int64, device=device)

    def one_step(i):
        if i and i % STEPS_PER_ROUND == 0:
            reset()
        if e2e:
            dev_tok.copy_(tokens[i % n_tok], non_blocking=True)
            host_out.copy_(stack.step(dev_tok), non_blocking=True)
            torch.cuda.current_stream().synchronize()          # the caller reads the result before the next token
        else:
            stack.step(tokens[i % n_tok])

    reset()
    for i in range(warmup):
        one_step(i)
    # estimate the step time to size the timed region (same count on every rank)
    reset()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(8):
        one_step(i)
    torch.cuda.synchronize()
    est = torch.tensor([(time.perf_counter() - t0) / 8], device=device, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(est, op=dist.ReduceOp.MAX)
    repeats = max(1, int(-(-min_seconds // (steps * float(est.item())))))
    reset()
    barrier()
    clocks = ClockSampler(local)
    with clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for r in range(repeats):
            reset()
            for i in range(steps):
                one_step(i)
        e1.record()
        e1.synchronize()
        sec = ((time.perf_counter() - t0) if e2e else e0.elapsed_time(e1) / 1e3) / (steps * repeats)
    barrier()
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([sec], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    return sec, repeats, clocks.summary()


def tp_parity_check(device, rank, world, group):
    """Two layers of the benchmark shapes at batch 3: the tensor-parallel stack against the single-GPU stack built on
    rank 0 from the same seeds.  Returns "bitwise" or the largest absolute difference."""
    stack_mod = importlib.import_module(f"{entry.PKG_ALIAS}.stack")
    cfg = stack_mod.StackConfig(n_layers=2)
    layers = [stack_mod.random_layer(cfg, 4005 + i, device) for i in range(cfg.n_layers)]
    gen = torch.Generator(device=device).manual_seed(4005)
    emb = torch.randn((512, cfg.hidden), generator=gen, device=device, dtype=torch.float32).to(torch.float16)
    fnorm = torch.ones(cfg.hidden, dtype=torch.float16, device=device)
    B, ctx = 3, 300
    toks = torch.randint(0, 512, (2, B), generator=gen, device=device)

    def make(tp_rank, tp_size, pg):
        st = stack_mod.DecodeStack(cfg, layers, fnorm, emb, B, ctx + 8, device, tp_rank=tp_rank, tp_size=tp_size, process_group=pg)
        for i, c in enumerate(st.caches):          # same context on every rank: fill the full cache, keep the own kv heads
            full = stack_mod.PagedKV(cfg, cfg.n_kv_heads, st.num_pages, device)
            full.fill_random(cfg, 4900 + i)
            lo = tp_rank * st.hkv
            for name in ("k_codes", "v_codes", "k_scales", "v_scales"):
                getattr(c, name).copy_(getattr(full, name)[:, :, lo:lo + st.hkv])
        st.positions.fill_(ctx)
        st.lengths.fill_(ctx + 1)
        return st

    sharded = make(rank, world, group)
    outs = [sharded.step(toks[i]).clone() for i in range(2)]
    torch.cuda.synchronize()
    result = None
    if rank == 0:
        cabi = importlib.import_module(f"{entry.PKG_ALIAS}.ops._cabi")
        cabi.set_tuning("ts.tp_world", world)          # the single-GPU stack below must not reset the shard count
        single = make(0, 1, None)
        cabi.set_tuning("ts.tp_world", world)
        ref = [single.step(toks[i]).clone() for i in range(2)]
        torch.cuda.synchronize()
        diff = max(float((a.float() - b.float()).abs().max()) for a, b in zip(outs, ref))
        result = "bitwise" if all(torch.equal(a, b) for a, b in zip(outs, ref)) else diff
    sharded.close()
    return result


def comm_breakdown(stack, device):
    """Exchanges per step and the device time of one stand-alone exchange of each of the three row widths
    (the same peer kernel / NCCL call the step uses, replayed alone in a CUDA graph)."""
    if stack.tp_size == 1:
        return None
    per_layer = 4
    out = {"transport": stack.transport, "exchanges_per_step": per_layer * stack.cfg.n_layers,
           "bytes_per_exchange": [stack.B * w * 2 for w in (stack.cfg.n_heads * stack.cfg.head_dim, stack.cfg.hidden,
                                                            stack.cfg.intermediate)]}
    if stack.peer_gather_error:
        out["note"] = stack.peer_gather_error
    locals_ = (stack.attn, stack.o_loc, stack.act)
    stream = torch.cuda.Stream(device)

    def run():
        for which, t in enumerate(locals_):
            for _ in range(8):
                stack._gather(which, t)
    try:
        sec = _time_graph(run, 10, stream) / 24
        out["us_per_exchange"] = round(sec * 1e6, 2)
        out["us_per_step"] = round(sec * 1e6 * out["exchanges_per_step"], 1)
        out["how"] = ("the stand-alone exchange kernel (payload, system fence, flag round trip) replayed alone in a CUDA graph; "
                      "transport fused_packets pays less inside the step: element and arrival mark travel in one 4-byte "
                      "peer store, without fence or flag")
    except Exception as exc:           # NCCL inside a private stream capture can be refused: report, do not fail the run
        out["note"] = f"exchange timing unavailable: {exc!r}"[:200]
    try:                               # host-side check: every rank issued the same exchanges
        out["exchange_counts_agree"] = stack.verify_exchanges() is not None or None
    except Exception as exc:
        out["exchange_counts_agree"] = False
        out["note"] = str(exc)[:200]
    return out


def run_own(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    group = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer stores only
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    entry.load_package()
    cabi = importlib.import_module(f"{entry.PKG_ALIAS}.ops._cabi")
    cabi.load()
    peak, peak_kind = measured_peaks()
    warmup = max(3, args.warmup)
    B = args.batch

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    cfg, stack = build_stack(device, B, STEPS_PER_ROUND + warmup + 16, rank, world, group)
    gen = torch.Generator(device=device).manual_seed(77)
    tokens = torch.randint(0, cfg.vocab, (STEPS_PER_ROUND, B), generator=gen, device=device)
    stack.capture()

    # ---- headline: K graph-replayed decode steps, device-timed ----
    sec_per_step, repeats, clocks = time_steps(stack, tokens, args.steps, warmup, barrier, local, world, min_seconds=args.min_seconds)
    tokens_per_s = B / sec_per_step

    # ---- end to end: host token ids in, host hidden state out, every step ----
    host_tokens = tokens.cpu().pin_memory()
    host_out = torch.empty((B, cfg.hidden), dtype=torch.float16).pin_memory()
    e2e_sec, e2e_repeats, _ = time_steps(stack, host_tokens, args.steps, 3, barrier, local, world, e2e=True, host_out=host_out,
                                         min_seconds=args.min_seconds)

    # ---- roofline of the dominant kernel: the matvec launches of one step, timed alone ----
    run_gemv, n_gemv = gemv_only_graph(stack)
    stream = torch.cuda.Stream(device)
    gemv_sec = _time_graph(run_gemv, 10, stream)
    weight_bytes = stack.weight_bytes_per_step()
    act_bytes = 0
    for w in stack.layers:
        for key, kdim in (("qkv", cfg.hidden), ("o", cfg.n_heads * cfg.head_dim), ("gate", cfg.hidden), ("down", cfg.intermediate)):
            act_bytes += B * kdim * 2 + B * w[key][0].shape[0] * 2 * (2 if key == "gate" else 1)
    gemv_bytes = weight_bytes + act_bytes
    gemv_traffic = 0.0
    for w in stack.layers:
        for key in ("qkv", "o", "gate", "down"):
            mats = (w["gate"], w["up"]) if key == "gate" else (w[key],)
            gemv_traffic += DRAM_TRAFFIC_RATIO[key] * sum(t.numel() * t.element_size() for m in mats for t in m if t is not None)
    gemv_traffic += act_bytes
    gemv_gbs = gemv_bytes / gemv_sec / 1e9
    step_bytes = weight_bytes + stack.kv_bytes_per_step(CONTEXT)
    comm = comm_breakdown(stack, device)
    launches_per_step = stack.launches_per_step
    transport = stack.transport

    status = cabi.device_status()
    line = {
        "metric": METRIC,
        "value": round(tokens_per_s, 2),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(sec_per_step * 1e3, 4),
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f16 activations, u4 weight codes, u8 KV codes, f32 accumulate",
        "data": "synthetic (random-init weights ~N(0,0.02) quantised q4 group 64; KV ~N(0,1) quantised q8 group 32; random token ids)",
        "config": {"workload": WORKLOAD, "batch": B, "context": CONTEXT, "parallelism": f"tp{world}", "transport": transport,
                   "decode_steps_per_round": STEPS_PER_ROUND,
                   "cache": "each step streams %.2f GB per GPU from HBM (> L2), no flush needed" % (step_bytes / 1e9),
                   "cuda_graph": True},
        "step_hbm": {"algorithmic_bytes_per_gpu": step_bytes, "achieved_gbs_per_gpu": round(step_bytes / sec_per_step / 1e9, 1),
                     "frac_of_peak": round(step_bytes / sec_per_step / 1e9 / peak, 4)},
        "roofline": {"bound": "hbm", "kernel": "qgemv_kernel (all q4 matvec launches of one step, timed alone)",
                     "achieved": round(gemv_gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gemv_gbs / peak, 4),
                     "traffic": round(gemv_traffic / n_gemv), "traffic_source": "per-shape ncu captures (profiles/qgemv_kernel_c5_stack_shapes_b1.md): dram bytes read+written / algorithmic bytes 1.002-1.008 for the QKV, O, gate/up and down shapes, applied to this launch mix",
                     "peak_kind": peak_kind, "launches": n_gemv,
                     "algorithmic_bytes_per_launch": round(gemv_bytes / n_gemv), "us_per_launch": round(gemv_sec / n_gemv * 1e6, 3)},
        "e2e": {"value": round(B / e2e_sec, 2), "unit": "tokens/s", "ms_per_step": round(e2e_sec * 1e3, 4),
                "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * cfg.hidden * 2, "repeats": e2e_repeats},
        "gpu_launches": launches_per_step * args.steps * repeats,
        "launches_per_step": launches_per_step,
        "repeats": repeats,
        "timed_seconds": round(sec_per_step * args.steps * repeats, 3),
        "timing": "the timed region is `repeats` x `steps` decode steps (at least one second); ms_per_step is its mean",
        "clocks": clocks,
        "device_status": status,
    }
    if comm is not None:
        line["comm"] = comm
    del stack
    torch.cuda.empty_cache()

    # ---- the same step at batch 32 (BASELINE config 5 names batch 1 and 32) ----
    if B != 32 and not args.no_batch32:
        cfg32, stack32 = build_stack(device, 32, STEPS_PER_ROUND + warmup + 16, rank, world, group)
        tok32 = torch.randint(0, cfg.vocab, (STEPS_PER_ROUND, 32), generator=gen, device=device)
        stack32.capture()
        steps32 = max(16, min(args.steps, 64))
        sec32, rep32, _ = time_steps(stack32, tok32, steps32, 3, barrier, local, world, min_seconds=0.5)
        bytes32 = stack32.weight_bytes_per_step() + stack32.kv_bytes_per_step(CONTEXT)
        line["batch32"] = {"ms_per_step": round(sec32 * 1e3, 4), "tokens_per_s": round(32 / sec32, 1), "steps": steps32, "repeats": rep32,
                           "algorithmic_bytes_per_gpu": bytes32, "achieved_gbs_per_gpu": round(bytes32 / sec32 / 1e9, 1),
                           "frac_of_peak": round(bytes32 / sec32 / 1e9 / peak, 4), "transport": stack32.transport,
                           "launches_per_step": stack32.launches_per_step, "device_status": cabi.device_status()}
        del stack32
        torch.cuda.empty_cache()
    if world > 1:
        line["tp_parity"] = tp_parity_check(device, rank, world, group)
    if rank == 0 and world == 1 and not args.step_only:
        line["kernels"] = kernel_microbenchmarks(device, peak, all_configs=True)
        line["cpu_baseline"] = cpu_baseline(B, budget_s=20.0)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # The captured graphs hold NCCL kernels; tearing the communicator down under them can block.  All
        # ranks are done once they pass this barrier, so leave without the library teardown.
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_kernels_only(cpu=False):
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(0)
    entry.load_package()
    importlib.import_module(f"{entry.PKG_ALIAS}.ops._cabi").load()
    peak, peak_kind = measured_peaks()
    print(json.dumps({"kernels": kernel_microbenchmarks(torch.device("cuda", 0), peak, all_configs=True, cpu=cpu),
                      "peak": peak, "peak_kind": peak_kind}), flush=True)


PROFILE_CASES = ("gate_up_q4_b1", "qkv_q4_b1", "o_q4_b1", "down_q4_b1", "gate_up_q4_b8", "gate_up_q4_b32", "down_q4_b8",
                 "matvec_q8_b8", "mlp_block_q4_b8", "mlp_block_q4_b32", "attn_cluster_q8_b1_ctx4096", "attn_splitkv_q8_b16",
                 "attn_fp16_b16")


def run_profile_case(name):
    """One kernel shape, a handful of eager launches over three rotating operand copies (more than L2 in all, a few
    hundred MB on the device): the small case an ``ncu -k ... -c 2`` capture is meant to be pointed at."""
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    entry.load_package()
    q = importlib.import_module(f"{entry.PKG_ALIAS}.ops.quant_ops")
    pq = importlib.import_module(f"{entry.PKG_ALIAS}.ops.paged_quantized_kv_ops")
    gqa = importlib.import_module(f"{entry.PKG_ALIAS}.ops.gqa_ops")
    synth = importlib.import_module(f"{entry.PKG_ALIAS}.synth")
    cabi = importlib.import_module(f"{entry.PKG_ALIAS}.ops._cabi")
    R, info = 3, {"case": name}
    if name.startswith("gate_up_q4"):
        B = int(name.rsplit("_b", 1)[1])
        sets = [[t.to(device) for t in synth.quantized_weight(14336, 4096, 4, 64, seed=11 + i) +
                 synth.quantized_weight(14336, 4096, 4, 64, seed=21 + i)] for i in range(R)]
        x = synth.activations((B, 4096), 5, device)
        call = lambda d: q.q4_gate_up_matvec_tiled(x, d[0], d[3], d[1], d[4], d[2], d[5], group_size=64)
        info["algorithmic_bytes"] = sum(t.numel() * t.element_size() for t in sets[0]) + B * (4096 + 2 * 14336) * 2
    elif name.startswith("mlp_block_q4"):
        mlp = importlib.import_module(f"{entry.PKG_ALIAS}.ops.mlp_block_ops")
        B = int(name.rsplit("_b", 1)[1])
        sets = [[t.to(device) for t in synth.quantized_weight(14336, 4096, 4, 64, seed=11 + i) +
                 synth.quantized_weight(14336, 4096, 4, 64, seed=21 + i) +
                 synth.quantized_weight(4096, 14336, 4, 64, seed=31 + i)] for i in range(R)]
        x = synth.activations((B, 1, 4096), 5, device)
        res = torch.zeros_like(x)
        nw = torch.ones(4096, dtype=torch.float16, device=device)
        call = lambda d: mlp.quantized_mlp_block(x, res, nw, d[0], d[1], d[3], d[4], d[6], d[7], gate_zeros=d[2],
                                                 up_zeros=d[5], down_zeros=d[8], bits=4, group_size=64,
                                                 backend_preset="cuda")
        info["algorithmic_bytes"] = sum(t.numel() * t.element_size() for t in sets[0]) + B * (4096 * 3 + 14336 * 2) * 2
    elif name in ("down_q4_b8", "matvec_q8_b8", "qkv_q4_b1", "o_q4_b1", "down_q4_b1"):
        bits, N, K = {"down": (4, 4096, 14336), "matvec": (8, 14336, 4096), "qkv": (4, 6144, 4096),
                      "o": (4, 4096, 4096)}[name.split("_")[0]]
        B = int(name.rsplit("_b", 1)[1])
        R = max(R, -(-200_000_000 // (N * K // (2 if bits == 4 else 1))))      # the copies together pass L2
        sets = [[t.to(device) for t in synth.quantized_weight(N, K, bits, 64, seed=31 + i)] for i in range(R)]
        x = synth.activations((B, K), 6, device)
        fn = q.q4_matvec_decode if bits == 4 else q.q8_matvec_decode
        call = lambda d: fn(x, d[0], d[1], d[2], group_size=64, backend="cuda")
        info["algorithmic_bytes"] = sum(t.numel() * t.element_size() for t in sets[0]) + B * (K + N) * 2
    elif name in ("attn_cluster_q8_b1_ctx4096", "attn_splitkv_q8_b16"):
        if name.startswith("attn_cluster"):
            B, lo, hi = 1, 4097, 4097
            R = 16                                                  # 9.5 MB per cache: 16 copies pass L2
        else:
            B, lo, hi = 16, 1024, 8192
        cases = [synth.paged_kv_case(B, 8, 128, 16, num_pages=B * 520, min_len=lo, max_len=hi, bits=8, group_size=32,
                                     seed=41 + i) for i in range(R)]
        sets = [pq.PagedQuantizedKVCache(**{k: (v.to(device) if torch.is_tensor(v) else v) for k, v in c.items()})
                for c in cases]
        qq = synth.activations((B, 1, 32, 128), 7, device)
        call = lambda c: pq.paged_quantized_kv_gqa_decode_attention(qq, c, backend="cuda")
        info["algorithmic_bytes"] = int(cases[0]["lengths"].sum()) * 8 * (2 * 128 + 2 * 4 * 2) + 2 * B * 32 * 128 * 2
    elif name == "attn_fp16_b16":
        B, ctx, P = 16, 4096, 16
        g = torch.Generator().manual_seed(3)
        sets = []
        for i in range(R):
            K = torch.randn((B * ctx // P, P, 8, 128), generator=g).to(torch.float16).to(device)
            V = torch.randn((B * ctx // P, P, 8, 128), generator=g).to(torch.float16).to(device)
            sets.append((K, V))
        bt = torch.arange(B * ctx // P, dtype=torch.int32, device=device).reshape(B, -1)
        ln = torch.full((B,), ctx, dtype=torch.int32, device=device)
        qq = synth.activations((B, 1, 32, 128), 7, device)
        call = lambda d: gqa.paged_gqa_decode_attention(qq, d[0], d[1], bt, ln)
        info["algorithmic_bytes"] = 2 * B * ctx * 8 * 128 * 2 + 2 * B * 32 * 128 * 2
    else:
        raise SystemExit(f"unknown --profile-case {name!r}; one of {PROFILE_CASES}")
    for _ in range(2):
        for d in sets:
            call(d)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for d in sets:
        call(d)
    end.record()
    torch.cuda.synchronize()
    info["eager_us_per_call"] = round(start.elapsed_time(end) * 1e3 / len(sets), 2)
    info["device_status"] = cabi.device_status()
    print(json.dumps(info), flush=True)


# ------------------------------------------------------------------------------------------------
# CPU arm: the torch-CPU restatement of the reference path on a bounded sample
# ------------------------------------------------------------------------------------------------
class CpuSample:
    """``n_layers`` layers of the stack at the benchmark shapes; a full step is 32 layers, so
    tokens/s = batch / (32 / n_layers * seconds per sample)."""

    def __init__(self, batch, n_layers):
        entry.load_package()
        stack_mod = importlib.import_module(f"{entry.PKG_ALIAS}.stack")
        synth = importlib.import_module(f"{entry.PKG_ALIAS}.synth")
        from oracle import paged_quantized_kv_ops as opq, stack as ostack
        self.ostack = ostack
        self.cfg = cfg = stack_mod.StackConfig()
        self.batch = batch
        self.n_layers = n_layers
        self.layers = [stack_mod.random_layer(cfg, 1005 + i, "cpu") for i in range(n_layers)]
        P = cfg.page_size
        blocks = (CONTEXT + 16 + P - 1) // P
        self.positions = torch.full((batch,), CONTEXT, dtype=torch.int32)
        self.caches = []
        for i in range(n_layers):
            case = synth.paged_kv_case(batch, cfg.n_kv_heads, cfg.head_dim, P, num_pages=batch * blocks, min_len=CONTEXT + 1,
                                       max_len=CONTEXT + 1, bits=cfg.kv_bits, group_size=cfg.kv_group_size, seed=2005 + i)
            self.caches.append(opq.OraclePagedKV(**case))
        self.cos, self.sin = ostack.rope_tables(cfg.head_dim, cfg.rope_theta, CONTEXT + 16)
        self.h = synth.activations((batch, 1, cfg.hidden), 3005)

    def run(self):
        h = self.h
        for w, cache in zip(self.layers, self.caches):
            h = self.ostack.layer_decode_step(h, w, cache, self.cos, self.sin, self.positions, self.cfg.oracle_dict())
        return h

    def tokens_per_s(self, sec_per_sample):
        return self.batch / (sec_per_sample * self.cfg.n_layers / self.n_layers)


def cpu_baseline(batch, budget_s):
    torch.set_num_threads(os.cpu_count() or 1)
    sample = CpuSample(batch, 1)
    sample.run()
    n, t0 = 0, time.perf_counter()
    while n < 2 or (time.perf_counter() - t0 < budget_s and n < 20):
        sample.run()
        n += 1
    sec = (time.perf_counter() - t0) / n
    return {"value": round(sample.tokens_per_s(sec), 4), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n} runs of 1 of the 32 layers (torch-CPU restatement of the reference path: dequantise W to "
                      f"fp16, fp32 matmul, paged q8 attention at context {CONTEXT}), {sec * 1e3:.0f} ms each, scaled to 32 layers"}


def run_reference(args):
    """The reference's CPU path for the same workload.  MLX cannot be installed here, so this is the torch-CPU
    restatement (kind "port").  One step = a bounded sample of the 32-layer step: up to 4 layers, fewer when the
    requested steps + warm-up would otherwise take more than about two minutes; the value is scaled to 32 layers."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    warmup = max(0, args.warmup)
    probe = CpuSample(args.batch, 1)
    probe.run()
    t0 = time.perf_counter()
    probe.run()
    per_layer = time.perf_counter() - t0
    n_layers = int(max(1, min(4, 120.0 / max(1e-3, (args.steps + warmup) * per_layer))))
    sample = probe if n_layers == 1 else CpuSample(args.batch, n_layers)
    for _ in range(warmup):
        sample.run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sample.run()
    sec = (time.perf_counter() - t0) / args.steps
    value = round(sample.tokens_per_s(sec), 4)
    desc = (f"each step = {n_layers} of the 32 layers of {WORKLOAD} at batch {args.batch} through the torch-CPU "
            f"restatement of the reference's pure-MLX path (MLX itself cannot be installed here); value scaled to 32 layers")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(sec * 1e3, 2), "ms_per_full_step_extrapolated": round(sec * 1e3 * 32 / n_layers, 2),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 activations, u4 weight codes, u8 KV codes, f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": args.batch, "context": CONTEXT, "parallelism": "cpu",
                   "extrapolated": f"{n_layers} of 32 layers timed per step; value = batch / (ms_per_step * 32 / {n_layers})"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128, help="decode steps per repeat (BASELINE config 5: 128 from context 4096)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--no-batch32", action="store_true", help="skip the secondary measurement of the step at batch 32")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="the timed region repeats the --steps block until it has lasted this long")
    ap.add_argument("--step-only", action="store_true",
                    help="only the decode step (no kernel table, no CPU baseline): the short run a launch list is taken from")
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--kernels-only", action="store_true",
                    help="run only the per-kernel micro-benchmarks of configs C1-C4 (the small cases used for profiler captures)")
    ap.add_argument("--profile-case", default=None, choices=PROFILE_CASES,
                    help="run one kernel shape a few times eagerly (the small case for an ncu capture) and exit")
    ap.add_argument("--cpu-baselines", action="store_true",
                    help="with --kernels-only: also time each config through the oracle on the host cores")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case)
        return
    if args.kernels_only:
        run_kernels_only(cpu=args.cpu_baselines)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
