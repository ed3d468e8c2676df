"""Llama-shaped q4/q8 decode stack on the hot-path kernels: the caller side of the matvec / MLP /
paged-attention operators for the layer-stack benchmark.

One decode step per layer is five calls through the C ABI:
  [RMSNorm + QKV matvec] -> [split + RoPE + quantised KV append + paged GQA decode attention: one kernel at
  small batch, three at large] -> [O matvec + residual] -> [RMSNorm + gate/up + SwiGLU] -> [down matvec + residual]
and the whole step is captured in a CUDA graph (positions and lengths live on the device and are
advanced inside the graph).

Tensor parallelism over ``tp_size`` GPUs of one node: every matrix is sharded by OUTPUT rows (QKV by
heads, so the KV cache is sharded by kv head) and the activations are re-assembled with an NCCL
all-gather after attention, O, SwiGLU and down (small kernels storing into NVLink peer memory, or NCCL
when symmetric memory is unavailable).  The kernels combine partial sums in an order that does not depend
on the sharding, so the sharded stack is bitwise identical to the single-GPU stack.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import synth
from .ops import _cabi


@dataclass
class StackConfig:
    hidden: int = 4096
    intermediate: int = 14336
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    rope_theta: float = 500000.0
    eps: float = 1e-5
    vocab: int = 128256
    bits: int = 4
    group_size: int = 64
    kv_bits: int = 8
    kv_group_size: int = 32
    page_size: int = 16

    def oracle_dict(self):
        return {"n_heads": self.n_heads, "n_kv_heads": self.n_kv_heads, "head_dim": self.head_dim,
                "bits": self.bits, "group_size": self.group_size, "eps": self.eps}


def rope_tables(head_dim: int, theta: float, length: int, device):
    """cos / sin [length, head_dim/2] fp32 (models/llama_config.py:107-124 of the reference).  Built on the host so that
    the table does not depend on the device's pow / cos implementation, then moved."""
    inv_freq = 1.0 / (float(theta) ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / float(head_dim)))
    freqs = torch.arange(length, dtype=torch.float32).reshape(length, 1) * inv_freq.reshape(1, -1)
    return torch.cos(freqs).contiguous().to(device), torch.sin(freqs).contiguous().to(device)


class ExchangeDesync(RuntimeError):
    """The ranks of a tensor-parallel group have not issued the same exchanges."""


def verify_exchange_counts(local_counts, group=None):
    """Host-side check between steps: every rank reports how many exchanges it has issued on each of its buffers
    (the sequence numbers its kernels publish); the counts must agree, because a rank that skipped an exchange, or
    stopped stepping, leaves its peers' next wait to run out.  Raises ``ExchangeDesync`` on every rank, naming the
    ranks that lag behind; works on any backend (the counts travel as Python objects)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    mine = [int(c) for c in local_counts]
    counts = [None] * world
    dist.all_gather_object(counts, mine, group=group)
    ahead = [max(c[i] for c in counts) for i in range(len(mine))]
    behind = {r: c for r, c in enumerate(counts) if c != ahead}
    if behind:
        raise ExchangeDesync(f"exchange counts differ: expected {ahead}, lagging ranks {behind}")
    return ahead


def shard_rows(n_rows: int, rank: int, world: int):
    """Row range [lo, hi) of an output dimension owned by ``rank`` (equal shards)."""
    if n_rows % world:
        raise ValueError(f"{n_rows} rows do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def shard_layer(full: dict, cfg: StackConfig, rank: int, world: int) -> dict:
    """Output-row shards of one layer's quantised matrices.  QKV is sharded by heads: the rank's
    q heads, then its k heads, then its v heads, so that its fused row keeps the [q | k | v] layout."""
    if world == 1:
        return full
    D = cfg.head_dim
    hq_lo, hq_hi = shard_rows(cfg.n_heads, rank, world)
    hk_lo, hk_hi = shard_rows(cfg.n_kv_heads, rank, world)
    q_rows = torch.arange(hq_lo * D, hq_hi * D)
    k_rows = cfg.n_heads * D + torch.arange(hk_lo * D, hk_hi * D)
    v_rows = (cfg.n_heads + cfg.n_kv_heads) * D + torch.arange(hk_lo * D, hk_hi * D)
    qkv_rows = torch.cat([q_rows, k_rows, v_rows])

    def take(triple, rows):
        return tuple(None if t is None else t[rows.to(t.device)].contiguous() for t in triple)

    def take_range(triple, n):
        lo, hi = shard_rows(n, rank, world)
        return tuple(None if t is None else t[lo:hi].contiguous() for t in triple)

    return {
        "input_norm": full["input_norm"], "post_norm": full["post_norm"],
        "qkv": take(full["qkv"], qkv_rows),
        "o": take_range(full["o"], cfg.hidden),
        "gate": take_range(full["gate"], cfg.intermediate),
        "up": take_range(full["up"], cfg.intermediate),
        "down": take_range(full["down"], cfg.hidden),
    }


def random_layer(cfg: StackConfig, seed: int, device) -> dict:
    """Random-init layer: W ~ N(0, 0.02) quantised affine group-wise, norm weights = 1."""
    gen = torch.Generator(device=device).manual_seed(seed)

    def qw(n, k):
        w = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02
        return synth.quantize_affine(w, cfg.bits, cfg.group_size)

    D = cfg.head_dim
    return {
        "input_norm": torch.ones(cfg.hidden, dtype=torch.float16, device=device),
        "post_norm": torch.ones(cfg.hidden, dtype=torch.float16, device=device),
        "qkv": qw((cfg.n_heads + 2 * cfg.n_kv_heads) * D, cfg.hidden),
        "o": qw(cfg.hidden, cfg.n_heads * D),
        "gate": qw(cfg.intermediate, cfg.hidden),
        "up": qw(cfg.intermediate, cfg.hidden),
        "down": qw(cfg.hidden, cfg.intermediate),
    }


class PagedKV:
    """Per-layer quantised page pool of the local kv heads plus the shared block table."""

    def __init__(self, cfg: StackConfig, n_kv_local: int, num_pages: int, device):
        D, P = cfg.head_dim, cfg.page_size
        dp = D // 2 if cfg.kv_bits == 4 else D
        gd = D // cfg.kv_group_size
        self.k_codes = torch.zeros((num_pages, P, n_kv_local, dp), dtype=torch.uint8, device=device)
        self.v_codes = torch.zeros_like(self.k_codes)
        self.k_scales = torch.zeros((num_pages, P, n_kv_local, gd), dtype=torch.float16, device=device)
        self.v_scales = torch.zeros_like(self.k_scales)

    def fill_random(self, cfg: StackConfig, seed: int):
        """Pre-fill with K/V ~ N(0,1) quantised by the cache rule (context that was 'already decoded')."""
        dev = self.k_codes.device
        gen = torch.Generator(device=dev).manual_seed(seed)
        shape = (*self.k_codes.shape[:3], cfg.head_dim)
        for codes, scales in ((self.k_codes, self.k_scales), (self.v_codes, self.v_scales)):
            vals = torch.randn(shape, generator=gen, device=dev, dtype=torch.float32)
            c, s = synth.quantize_kv_symmetric(vals, cfg.kv_bits, cfg.kv_group_size)
            codes.copy_(c)
            scales.copy_(s)


class DecodeStack:
    """Runs decode steps of ``cfg.n_layers`` layers on one GPU (or one tensor-parallel rank)."""

    _next_slot = 0      # exchange slots of the library handed out so far (process-wide)

    def __init__(self, cfg: StackConfig, layers, final_norm, embedding, batch: int, max_context: int, device,
                 tp_rank: int = 0, tp_size: int = 1, process_group=None, use_peer_gather: bool = True,
                 fuse_exchange: bool = True, exchange_packets: bool = True):
        self.cfg, self.B, self.device = cfg, batch, device
        self.tp_rank, self.tp_size, self.pg = tp_rank, tp_size, process_group
        self.lib = _cabi.load()
        self.layers = [shard_layer(l, cfg, tp_rank, tp_size) for l in layers]
        self.final_norm, self.embedding = final_norm, embedding
        self.hq = cfg.n_heads // tp_size
        self.hkv = cfg.n_kv_heads // tp_size
        if cfg.n_heads % tp_size or cfg.n_kv_heads % tp_size:
            raise ValueError("heads must split evenly over the tensor-parallel ranks")
        P = cfg.page_size
        self.max_blocks = (max_context + P - 1) // P
        self.num_pages = batch * self.max_blocks
        self.block_table = torch.arange(self.num_pages, dtype=torch.int32, device=device).reshape(batch, self.max_blocks)
        self.caches = [PagedKV(cfg, self.hkv, self.num_pages, device) for _ in range(cfg.n_layers)]
        self.positions = torch.zeros(batch, dtype=torch.int32, device=device)
        self.lengths = torch.zeros(batch, dtype=torch.int32, device=device)
        self.cos, self.sin = rope_tables(cfg.head_dim, cfg.rope_theta, max_context, device)
        f16 = dict(dtype=torch.float16, device=device)
        D = cfg.head_dim
        self.h = torch.zeros((batch, cfg.hidden), **f16)
        self.h2 = torch.zeros((batch, cfg.hidden), **f16)
        self.qkv = torch.zeros((batch, (self.hq + 2 * self.hkv) * D), **f16)
        self.q_rot = torch.zeros((batch, self.hq * D), **f16)
        self.attn = torch.zeros((batch, self.hq * D), **f16)
        self.act = torch.zeros((batch, cfg.intermediate // tp_size), **f16)
        self.out = torch.zeros((batch, cfg.hidden), **f16)
        # buffer for the normalised rows: the batches that run the tcgen05 matvec (5 rows and more) run the rmsnorm as a
        # launch of its own in front of it
        self.normed = torch.zeros((batch, cfg.hidden), **f16) if batch >= 5 else None
        self.peer_gather = False
        self.peer_fused = False
        # The exchange fused into the kernels exists in the mma.sync matvec kernel, which takes batches of up to 4
        # rows; larger batches run the tcgen05 kernel and exchange through the stand-alone peer kernel (or NCCL).
        self.fuse_exchange = fuse_exchange and batch <= 4
        # fused exchange in packet form: element and arrival mark in one 4-byte peer store (no fence, no flag round trip)
        self.exchange_packets = exchange_packets
        self.transport = "none"
        self.peer_gather_error = ""
        if tp_size > 1:
            self.transport = "nccl"
            self.o_loc = torch.zeros((batch, cfg.hidden // tp_size), **f16)
            self.gather_attn = torch.zeros((tp_size, batch, self.hq * D), **f16)
            self.gather_h = torch.zeros((tp_size, batch, cfg.hidden // tp_size), **f16)
            self.gather_act = torch.zeros((tp_size, batch, cfg.intermediate // tp_size), **f16)
            self.attn_full = torch.zeros((batch, cfg.n_heads * D), **f16)
            self.act_full = torch.zeros((batch, cfg.intermediate), **f16)
            if use_peer_gather:
                self._setup_peer_gather()
        ws_bytes = self.lib.b200q_paged_gqa_workspace_bytes(batch, self.hq, self.hkv, D)
        self.workspace = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
        self.token_ids = torch.zeros(batch, dtype=torch.int64, device=device)
        self.graph = None
        self.launches_per_step = 0

    # -- context management ------------------------------------------------------------------
    def set_context(self, context_len: int, seed: int = 0):
        """Pretend ``context_len`` tokens were already decoded: random quantised KV, positions = context_len."""
        for i, c in enumerate(self.caches):
            c.fill_random(self.cfg, seed + 131 * i + self.tp_rank)
        self.positions.fill_(context_len)
        self.lengths.fill_(context_len + 1)

    # -- one decode step -----------------------------------------------------------------------
    def _setup_peer_gather(self):
        """Maps one symmetric buffer (full attention rows, full hidden rows, full MLP rows, flag words) on all
        ranks so that the all-gathers of a step are single small kernels storing straight into peer memory.
        Falls back to NCCL all-gathers (``peer_gather = False``) when symmetric memory cannot be set up."""
        import ctypes
        import torch.distributed as dist
        cfg, B, W = self.cfg, self.B, self.tp_size
        widths = (cfg.n_heads * cfg.head_dim, cfg.hidden, cfg.intermediate)
        self.transport = "nccl"
        if any((w // W) * 2 % 16 for w in widths):
            self.peer_gather_error = "a shard row is not a multiple of 16 bytes"
            return
        try:
            import os
            # plain peer stores only: the buffer is never bound to an NVLink multicast object
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            group = self.pg if self.pg is not None else dist.group.WORLD
            sizes = [B * w * 2 for w in widths]
            offsets, off = [], 0
            for n in sizes:
                offsets.append(off)
                off += (n + 255) // 256 * 256
            flag_off = off
            off += 3 * 256                                    # one 256-byte line of flag words per buffer
            packet_offsets = []
            if self.fuse_exchange and self.exchange_packets:  # the same rows as 4-byte packets (fused exchange only)
                for n in sizes:
                    packet_offsets.append(off)
                    off += (2 * n + 255) // 256 * 256
            buf = symm.empty(off, dtype=torch.uint8, device=self.device)
            buf.zero_()
            handle = symm.rendezvous(buf, group)
            ptrs = [int(p) for p in handle.buffer_ptrs]
        except Exception as exc:                              # no fabric / unsupported build: keep NCCL
            self.peer_gather_error = repr(exc)
            return
        self._symm_buf, self._symm_handle = buf, handle
        self.peer_full, self.peer_ptrs, self.peer_flag_ptrs = [], [], []
        for i, (w, o) in enumerate(zip(widths, offsets)):
            self.peer_full.append(buf[o:o + B * w * 2].view(torch.float16).view(B, w))
            self.peer_ptrs.append((ctypes.c_void_p * W)(*[p + o for p in ptrs]))
            self.peer_flag_ptrs.append((ctypes.c_void_p * W)(*[p + flag_off + 256 * i for p in ptrs]))
        self.peer_epochs = torch.zeros(3, dtype=torch.int32, device=self.device)
        self.peer_counters = torch.zeros(3, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize()
        dist.barrier(group=self.pg)                            # every rank's buffer is zeroed before anyone stores
        self.peer_gather = True
        self.transport = "peer_kernel"
        # the same buffers as exchange slots of the kernels themselves (stores from the epilogue, waits in the
        # next prologue): three slots per stack instance
        base = DecodeStack._next_slot
        if self.fuse_exchange and base + 3 > 16:
            self.peer_gather_error = "the library's 16 exchange slots are in use"
        if self.fuse_exchange and base + 3 <= 16:
            DecodeStack._next_slot += 3
            self.slots = (base, base + 1, base + 2)
            self.fused_full = list(self.peer_full)            # what the consumer kernels are given as their input rows
            self.fused_epochs = self.peer_epochs
            fused_ptrs = self.peer_ptrs
            if packet_offsets:
                self.fused_full = [buf[o:o + B * w * 4].view(torch.int32).view(B, w) for w, o in zip(widths, packet_offsets)]
                fused_ptrs = [(ctypes.c_void_p * W)(*[p + o for p in ptrs]) for o in packet_offsets]
                self.fused_epochs = torch.zeros(3, dtype=torch.int32, device=self.device)
                self._fused_ptrs = fused_ptrs
            for i, slot in enumerate(self.slots):
                _cabi.check(self.lib.b200q_tp_register(slot, fused_ptrs[i], self.peer_flag_ptrs[i],
                                                       self.fused_epochs[i:].data_ptr(), self.peer_counters[i:].data_ptr(),
                                                       self.tp_rank, W), "tp_register")
                _cabi.check(self.lib.b200q_tp_set_packets(slot, 1 if packet_offsets else 0), "tp_set_packets")
            self.peer_fused = True
            self.transport = "fused_packets" if packet_offsets else "fused_peer"

    def verify_exchanges(self):
        """Compares this rank's exchange sequence numbers with its peers' (call between steps; synchronises)."""
        if not self.peer_gather:
            return None
        torch.cuda.synchronize(self.device)
        counts = self.peer_epochs.cpu().tolist()
        if self.peer_fused and self.fused_epochs is not self.peer_epochs:
            counts += self.fused_epochs.cpu().tolist()
        return verify_exchange_counts(counts, self.pg)

    def close(self):
        """Returns this stack's exchange slots to the process-wide pool (the last stack created is released first)."""
        if self.peer_fused and DecodeStack._next_slot == self.slots[2] + 1:
            DecodeStack._next_slot = self.slots[0]
        self.peer_fused = False

    def _gather(self, which: int, local):
        """All-gather of ``local`` [B, n_loc] into [B, tp * n_loc] (rank-major columns); ``which`` selects the
        full buffer: 0 attention rows, 1 hidden rows, 2 MLP rows."""
        if self.peer_gather:
            st = torch.cuda.current_stream().cuda_stream
            _cabi.check(self.lib.b200q_peer_allgather(local.data_ptr(), self.peer_ptrs[which], self.peer_flag_ptrs[which],
                                                      self.peer_epochs[which:].data_ptr(), self.tp_rank, self.tp_size,
                                                      self.B, local.shape[1] * 2, st), "peer_allgather")
            return self.peer_full[which]
        if which == 0:
            return self._all_gather_rows(local, self.gather_attn, self.attn_full)
        if which == 2:
            return self._all_gather_rows(local, self.gather_act, self.act_full)
        return self._all_gather_rows(local, self.gather_h)

    def _all_gather_rows(self, local, gathered, full=None):
        """[B, n_loc] on every rank -> [B, tp * n_loc] in rank-major column order."""
        import torch.distributed as dist
        dist.all_gather_into_tensor(gathered.view(-1, local.shape[-1]), local, group=self.pg)
        out = gathered.permute(1, 0, 2).reshape(local.shape[0], -1)
        if full is not None:
            full.copy_(out)
            return full
        return out

    def _launch_step(self):
        cfg, lib, B = self.cfg, self.lib, self.B
        st = torch.cuda.current_stream().cuda_stream
        D, G, bits = cfg.head_dim, cfg.group_size, cfg.bits
        F16, ck = _cabi.F16, _cabi.check
        n = 0
        # the tcgen05 matvec splits K as the unsharded launch would: sharded rows == unsharded rows, bit for bit
        _cabi.set_tuning("ts.tp_world", self.tp_size)
        attn_launches = lib.b200q_attention_stage_launches(B, self.hkv, 1)
        normed = None if self.normed is None else self.normed.data_ptr()
        norm_launch = 0 if normed is None else 1      # the library then runs the rmsnorm as a launch of its own
        torch.index_select(self.embedding, 0, self.token_ids, out=self.h)
        pending_slot = -1
        pending = None      # tensor-parallel path: gathered down-projection rows whose residual add (h2 + rows -> h)
                            # is folded into the next kernel's prologue instead of being a launch of its own
        for w, cache in zip(self.layers, self.caches):
            qw, qs, qz = w["qkv"]
            if pending is None:
                ck(lib.b200q_norm_qmatvec(bits, self.h.data_ptr(), None, w["input_norm"].data_ptr(), F16, cfg.eps, None,
                                          normed, qw.data_ptr(), qs.data_ptr(), qz.data_ptr(), None, self.qkv.data_ptr(), B,
                                          qw.shape[0], cfg.hidden, G, F16, F16, st), "norm_qmatvec")
            else:
                if pending_slot >= 0:
                    ck(lib.b200q_tp_next(pending_slot, -1), "tp_next")
                ck(lib.b200q_norm_qmatvec(bits, pending.data_ptr(), self.h2.data_ptr(), w["input_norm"].data_ptr(), F16,
                                          cfg.eps, self.h.data_ptr(), normed, qw.data_ptr(), qs.data_ptr(), qz.data_ptr(),
                                          None, self.qkv.data_ptr(), B, qw.shape[0], cfg.hidden, G, F16, F16, st),
                   "norm_qmatvec")
            if self.peer_fused:
                ck(lib.b200q_tp_next(-1, self.slots[0]), "tp_next")
            # split + RoPE + quantised KV append + attention: one kernel at small batch (a cluster per sequence and kv head)
            ck(lib.b200q_rope_append_paged_gqa_decode(self.qkv.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(),
                                                      self.positions.data_ptr(), self.cos.shape[0], cfg.kv_bits,
                                                      cache.k_codes.data_ptr(), cache.v_codes.data_ptr(),
                                                      cache.k_scales.data_ptr(), cache.v_scales.data_ptr(),
                                                      self.block_table.data_ptr(), self.lengths.data_ptr(),
                                                      None if self.peer_fused else self.attn.data_ptr(),
                                                      self.q_rot.data_ptr(), self.workspace.data_ptr(),
                                                      self.workspace.numel(), B, self.hq, self.hkv, D, cfg.page_size,
                                                      self.num_pages, self.max_blocks, cfg.kv_group_size,
                                                      1.0 / math.sqrt(D), st), "rope_append_attention")
            ow, os_, oz = w["o"]
            gw, gs, gz = w["gate"]
            uw, us, uz = w["up"]
            dw, ds, dz = w["down"]
            if self.tp_size == 1:
                ck(lib.b200q_qmatvec(bits, self.attn.data_ptr(), ow.data_ptr(), os_.data_ptr(), oz.data_ptr(),
                                     self.h.data_ptr(), self.h2.data_ptr(), B, cfg.hidden, cfg.n_heads * D, G, F16, F16, st),
                   "o_proj")
                ck(lib.b200q_gate_up_swiglu(bits, self.h2.data_ptr(), gw.data_ptr(), uw.data_ptr(), gs.data_ptr(),
                                            us.data_ptr(), gz.data_ptr(), uz.data_ptr(), None, None, self.act.data_ptr(),
                                            None, w["post_norm"].data_ptr(), F16, cfg.eps, None, normed, B,
                                            cfg.intermediate, cfg.hidden, G, F16, F16, st), "gate_up")
                ck(lib.b200q_qmatvec(bits, self.act.data_ptr(), dw.data_ptr(), ds.data_ptr(), dz.data_ptr(),
                                     self.h2.data_ptr(), self.h.data_ptr(), B, cfg.hidden, cfg.intermediate, G, F16, F16, st),
                   "down_proj")
                n += 4 + attn_launches + 2 * norm_launch
            elif not self.peer_fused:
                attn_full = self._gather(0, self.attn)
                ck(lib.b200q_qmatvec(bits, attn_full.data_ptr(), ow.data_ptr(), os_.data_ptr(), oz.data_ptr(), None,
                                     self.o_loc.data_ptr(), B, ow.shape[0], cfg.n_heads * D, G, F16, F16, st), "o_proj")
                o_full = self._gather(1, self.o_loc)
                # h2 = cast(h + o) (the layer's residual add) is formed in the prologue of the gate/up launch
                ck(lib.b200q_gate_up_swiglu(bits, o_full.data_ptr(), gw.data_ptr(), uw.data_ptr(), gs.data_ptr(),
                                            us.data_ptr(), gz.data_ptr(), uz.data_ptr(), None, None, self.act.data_ptr(),
                                            self.h.data_ptr(), w["post_norm"].data_ptr(), F16, cfg.eps, self.h2.data_ptr(),
                                            normed, B, gw.shape[0], cfg.hidden, G, F16, F16, st), "gate_up")
                act_full = self._gather(2, self.act)
                ck(lib.b200q_qmatvec(bits, act_full.data_ptr(), dw.data_ptr(), ds.data_ptr(), dz.data_ptr(), None,
                                     self.o_loc.data_ptr(), B, dw.shape[0], cfg.intermediate, G, F16, F16, st), "down_proj")
                pending = self._gather(1, self.o_loc)      # h = cast(h2 + down) happens in the next prologue
                n += 4 + attn_launches + (4 if self.peer_gather else 0) + 2 * norm_launch
            else:
                # exchanges fused into the kernels: the O, gate/up and down launches wait for the rows they read and
                # store the rows they produce straight into every rank's buffers (the attention rows were stored by
                # the merge kernel above)
                sa, sh, sm = self.slots
                last = w is self.layers[-1]
                ck(lib.b200q_tp_next(sa, sh), "tp_next")
                ck(lib.b200q_qmatvec(bits, self.fused_full[0].data_ptr(), ow.data_ptr(), os_.data_ptr(), oz.data_ptr(), None,
                                     None, B, ow.shape[0], cfg.n_heads * D, G, F16, F16, st), "o_proj")
                ck(lib.b200q_tp_next(sh, sm), "tp_next")
                ck(lib.b200q_gate_up_swiglu(bits, self.fused_full[1].data_ptr(), gw.data_ptr(), uw.data_ptr(), gs.data_ptr(),
                                            us.data_ptr(), gz.data_ptr(), uz.data_ptr(), None, None, None,
                                            self.h.data_ptr(), w["post_norm"].data_ptr(), F16, cfg.eps, self.h2.data_ptr(),
                                            None, B, gw.shape[0], cfg.hidden, G, F16, F16, st), "gate_up")
                if last:
                    # the final norm is not a kernel that can wait: close the step with the stand-alone exchange
                    ck(lib.b200q_tp_next(sm, -1), "tp_next")
                    ck(lib.b200q_qmatvec(bits, self.fused_full[2].data_ptr(), dw.data_ptr(), ds.data_ptr(), dz.data_ptr(),
                                         None, self.o_loc.data_ptr(), B, dw.shape[0], cfg.intermediate, G, F16, F16, st),
                       "down_proj")
                    pending = self._gather(1, self.o_loc)
                    pending_slot = -1
                    n += 5 + attn_launches
                else:
                    ck(lib.b200q_tp_next(sm, sh), "tp_next")
                    ck(lib.b200q_qmatvec(bits, self.fused_full[2].data_ptr(), dw.data_ptr(), ds.data_ptr(), dz.data_ptr(),
                                         None, None, B, dw.shape[0], cfg.intermediate, G, F16, F16, st), "down_proj")
                    pending = self.fused_full[1]
                    pending_slot = sh
                    n += 4 + attn_launches + 2 * norm_launch
        if pending is None:
            ck(lib.b200q_rmsnorm_residual(self.h.data_ptr(), None, self.final_norm.data_ptr(), self.out.data_ptr(), None,
                                          B, cfg.hidden, cfg.eps, F16, _cabi.dtype_code(self.final_norm.dtype), st),
               "final_norm")
        else:
            ck(lib.b200q_rmsnorm_residual(pending.data_ptr(), self.h2.data_ptr(), self.final_norm.data_ptr(),
                                          self.out.data_ptr(), self.h.data_ptr(), B, cfg.hidden, cfg.eps, F16,
                                          _cabi.dtype_code(self.final_norm.dtype), st), "final_norm")
        self.positions.add_(1)
        self.lengths.add_(1)
        self.launches_per_step = n + 1
        return self.out

    def capture(self):
        """Captures one decode step in a CUDA graph (after one eager warm-up step, whose effect on the
        positions is undone)."""
        pos, ln = self.positions.clone(), self.lengths.clone()
        self._launch_step()
        torch.cuda.synchronize()
        self.positions.copy_(pos)
        self.lengths.copy_(ln)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._launch_step()
        self.positions.copy_(pos)
        self.lengths.copy_(ln)
        return self.graph

    def step(self, token_ids: torch.Tensor) -> torch.Tensor:
        """token_ids [B] (device) -> final-normed hidden state [B, hidden]."""
        self.token_ids.copy_(token_ids)
        if self.graph is not None:
            self.graph.replay()
            return self.out
        return self._launch_step()

    def weight_bytes_per_step(self) -> int:
        total = 0
        for w in self.layers:
            for key in ("qkv", "o", "gate", "up", "down"):
                total += sum(t.numel() * t.element_size() for t in w[key] if t is not None)
        return total

    def kv_bytes_per_step(self, context_len: int) -> int:
        cfg = self.cfg
        dp = cfg.head_dim // 2 if cfg.kv_bits == 4 else cfg.head_dim
        per_tok = 2 * (dp + (cfg.head_dim // cfg.kv_group_size) * 2) * self.hkv
        return cfg.n_layers * self.B * context_len * per_tok
