"""The give-up branch of every bounded device wait, on one GPU and without a fault: a wait that nothing satisfies
runs out after a few thousand probes, the kernel returns, the host reads the event from the status word, and the
next ordinary call works.  The flags are simply never published; nothing here traps, faults or spins unbounded."""
import ctypes

import pytest
import torch

from helpers import cabi, quant_ops, rel_l2, synth
from oracle import quant_ops as oq

pytestmark = pytest.mark.gpu
EV_GEMV_FULL_WAIT, EV_PEER_WAIT = 1, 5


@pytest.fixture()
def short_waits():
    cabi.set_tuning("peer.spin_limit", 4096)
    cabi.set_tuning("tp.spin_limit", 4096)
    yield
    cabi.set_tuning("peer.spin_limit", 0)
    cabi.set_tuning("tp.spin_limit", 0)


def _matvec_ok(cuda):
    w, s, z = synth.quantized_weight(256, 512, 4, 64, seed=3)
    x = synth.activations((2, 512), 4)
    got = quant_ops.q4_matvec_decode(x.to(cuda), w.to(cuda), s.to(cuda), z.to(cuda), group_size=64, backend="cuda")
    want = oq.reference_q4_matvec_decode(x, w, s, z, group_size=64)
    return rel_l2(got, want) <= 1e-3


def test_expired_barrier_wait_reaches_the_host(cuda):
    lib = cabi.load()
    assert cabi.device_status() == 0
    probes = torch.zeros(1, dtype=torch.int32, device=cuda)
    cabi.check(lib.b200q_wait_expiry_selftest(4096, probes.data_ptr(), cabi.stream()), "selftest")
    assert cabi.device_status(reset=False) == EV_GEMV_FULL_WAIT        # stays until it is cleared
    assert cabi.device_status() == EV_GEMV_FULL_WAIT
    assert int(probes.item()) == 4096
    assert cabi.device_status() == 0
    assert _matvec_ok(cuda) and cabi.device_status() == 0
    assert lib.b200q_wait_expiry_selftest(0, None, cabi.stream()) != 0  # only short waits are accepted
    assert lib.b200q_wait_expiry_selftest(1 << 20, None, cabi.stream()) != 0


def test_peer_allgather_gives_up_on_a_silent_rank(cuda, short_waits):
    """Two ranks emulated on one GPU (their buffers are plain local allocations).  Rank 0 runs its exchange while rank 1
    never publishes: the wait runs out and event 5 is reported.  Rank 1's call afterwards finds rank 0's shard already
    there, so it completes at once and its full buffer holds both shards."""
    lib = cabi.load()
    rows, n_loc = 3, 64
    full = [torch.zeros((rows, 2 * n_loc), dtype=torch.float16, device=cuda) for _ in range(2)]
    flags = [torch.zeros(2, dtype=torch.int32, device=cuda) for _ in range(2)]
    epochs = [torch.zeros(1, dtype=torch.int32, device=cuda) for _ in range(2)]
    local = [torch.randn((rows, n_loc), device=cuda).to(torch.float16) for _ in range(2)]
    full_ptrs = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in full])
    flag_ptrs = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in flags])

    def call(rank):
        cabi.check(lib.b200q_peer_allgather(local[rank].data_ptr(), full_ptrs, flag_ptrs, epochs[rank].data_ptr(), rank,
                                            2, rows, n_loc * 2, cabi.stream()), "peer_allgather")

    assert cabi.device_status() == 0
    call(0)
    assert cabi.device_status() == EV_PEER_WAIT
    assert int(epochs[0].item()) == 1                              # the kernel ran to its end
    call(1)
    assert cabi.device_status() == 0
    want = torch.cat(local, dim=1)
    assert torch.equal(full[1], want) and torch.equal(full[0], want)


def test_fused_exchange_wait_gives_up_and_recovers(cuda, short_waits):
    """The wait in the prologue of a matvec whose input is an exchange buffer: with the second source's flag unset it
    runs out (event 5, the kernel still finishes); once the flag is there the same call is an ordinary matvec."""
    lib = cabi.load()
    B, K, N = 1, 512, 256
    w, s, z = synth.quantized_weight(N, K, 4, 64, seed=5)
    x = synth.activations((B, K), 6)
    want = oq.reference_q4_matvec_decode(x, w, s, z, group_size=64)
    dw, ds, dz = w.to(cuda), s.to(cuda), z.to(cuda)
    full = [x.to(cuda).clone() for _ in range(2)]                 # both ranks' views of the gathered rows
    flags = [torch.zeros(2, dtype=torch.int32, device=cuda) for _ in range(2)]
    epoch = torch.ones(1, dtype=torch.int32, device=cuda)         # this rank has published exchange number 1 ...
    counter = torch.zeros(1, dtype=torch.int32, device=cuda)
    flags[0][0] = 1                                               # ... and only its own flag has arrived
    full_ptrs = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in full])
    flag_ptrs = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in flags])
    slot = 15
    cabi.check(lib.b200q_tp_register(slot, full_ptrs, flag_ptrs, epoch.data_ptr(), counter.data_ptr(), 0, 2), "tp_register")
    y = torch.zeros((B, N), dtype=torch.float16, device=cuda)

    def call():
        cabi.check(lib.b200q_tp_next(slot, -1), "tp_next")
        cabi.check(lib.b200q_qmatvec(4, full[0].data_ptr(), dw.data_ptr(), ds.data_ptr(), dz.data_ptr(), None, y.data_ptr(),
                                     B, N, K, 64, cabi.F16, cabi.dtype_code(ds.dtype), cabi.stream()), "qmatvec")

    assert cabi.device_status() == 0
    call()
    assert cabi.device_status() == EV_PEER_WAIT
    flags[0][1] = 1                                               # the peer's shard "arrives"
    call()
    assert cabi.device_status() == 0
    assert rel_l2(y, want) <= 1e-3


def test_packet_exchange_wait_gives_up_and_recovers(cuda, short_waits):
    """The packet form of the fused exchange: the matvec's loads of its input rows poll the packets they need.  With
    the second rank's half of the row still carrying the previous sequence number the wait runs out (event 5, the
    kernel still finishes); once those packets are stamped the same call equals the oracle."""
    lib = cabi.load()
    B, K, N = 1, 512, 256
    w, s, z = synth.quantized_weight(N, K, 4, 64, seed=5)
    x = synth.activations((B, K), 6)
    want = oq.reference_q4_matvec_decode(x, w, s, z, group_size=64)
    dw, ds, dz = w.to(cuda), s.to(cuda), z.to(cuda)
    seq = 7                                                       # this rank's counter: exchange number 7 was issued
    stamp = (seq % 65535 + 1) << 16
    bits = x.view(torch.int16).to(torch.int32) & 0xFFFF          # the elements as the low halves of the packets
    packets = (bits | stamp).to(cuda)
    stale = packets.clone()
    stale[:, K // 2:] = bits[:, K // 2:].to(cuda) | (((seq - 1) % 65535 + 1) << 16)    # rank 1's half: previous exchange
    buffers = [stale.clone().contiguous(), torch.zeros_like(stale)]
    flags = [torch.zeros(2, dtype=torch.int32, device=cuda) for _ in range(2)]
    epoch = torch.full((1,), seq, dtype=torch.int32, device=cuda)
    counter = torch.zeros(1, dtype=torch.int32, device=cuda)
    full_ptrs = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in buffers])
    flag_ptrs = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in flags])
    slot = 14
    cabi.check(lib.b200q_tp_register(slot, full_ptrs, flag_ptrs, epoch.data_ptr(), counter.data_ptr(), 0, 2), "tp_register")
    cabi.check(lib.b200q_tp_set_packets(slot, 1), "tp_set_packets")
    assert lib.b200q_tp_set_packets(13, 1) != 0                   # a slot that was never registered
    y = torch.zeros((B, N), dtype=torch.float16, device=cuda)

    def call():
        cabi.check(lib.b200q_tp_next(slot, -1), "tp_next")
        cabi.check(lib.b200q_qmatvec(4, buffers[0].data_ptr(), dw.data_ptr(), ds.data_ptr(), dz.data_ptr(), None,
                                     y.data_ptr(), B, N, K, 64, cabi.F16, cabi.dtype_code(ds.dtype), cabi.stream()), "qmatvec")

    assert cabi.device_status() == 0
    call()
    assert cabi.device_status() == EV_PEER_WAIT
    buffers[0].copy_(packets)                                     # the peer's packets "arrive"
    call()
    assert cabi.device_status() == 0
    assert rel_l2(y, want) <= 1e-3
    cabi.check(lib.b200q_tp_set_packets(slot, 0), "tp_set_packets")
