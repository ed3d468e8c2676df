"""The allocation-free attention entry point (b200q_paged_gqa_decode_static) against the regular one.

Some callers of the library are not allowed to allocate device memory (a plugin inside another
runtime's memory budget, code running while a CUDA graph is being captured, a process whose memory
was all handed out at start-up).  For them the split-KV partial results live in an 8 MiB array that
is part of the library image instead of a caller-allocated workspace.  This file checks, through the
C ABI, that two calls in a row give exactly what the workspace variant gives, and that a problem
larger than the array is refused with its own error code.  It is collected last on purpose.
"""
import pytest
import torch

from helpers import cabi, synth

pytestmark = pytest.mark.gpu


def _call(lib, static, case, q, out, workspace=None):
    NUM_PAGES, P, Hkv, D = case["original_page_shape"]
    B, Hq = q.shape[0], q.shape[1]
    common_head = [case["bits"], q.data_ptr(), case["k_pages_q"].data_ptr(), case["v_pages_q"].data_ptr(),
                   case["k_scales"].data_ptr(), case["v_scales"].data_ptr(), case["block_table"].data_ptr(),
                   case["lengths"].data_ptr(), out.data_ptr()]
    common_tail = [B, Hq, Hkv, D, P, NUM_PAGES, case["block_table"].shape[1], case["group_size"], 1.0 / D ** 0.5,
                   cabi.F16, cabi.F16, cabi.stream()]
    if static:
        return lib.b200q_paged_gqa_decode_static(*common_head, *common_tail)
    return lib.b200q_paged_gqa_decode(*common_head, workspace.data_ptr(), workspace.numel(), *common_tail)


@pytest.mark.parametrize("bits", [4, 8])
def test_static_scratch_variant_matches_workspace_variant(cuda, bits):
    lib = cabi.load()
    assert lib.b200q_paged_gqa_static_scratch_bytes() == 8 << 20
    outs = []
    for seed in (11, 12):                     # two calls in a row, different inputs, same shared scratch
        case = synth.paged_kv_case(5, 8, 128, 16, num_pages=200, min_len=3, max_len=600, bits=bits, group_size=32, seed=seed)
        case = {k: (v.to(cuda) if torch.is_tensor(v) else v) for k, v in case.items()}
        q = synth.activations((5, 32, 128), seed + 100, cuda)
        ws = torch.empty(lib.b200q_paged_gqa_workspace_bytes(5, 32, 8, 128), dtype=torch.uint8, device=cuda)
        want = torch.full_like(q, float("nan"))
        got = torch.full_like(q, float("nan"))
        assert _call(lib, False, case, q, want, ws) == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(cuda)[0]
        assert _call(lib, True, case, q, got) == 0
        torch.cuda.synchronize()
        if seed != 11:                        # (the very first call on a device may load the kernel's module)
            # the call left device memory as it found it (a scratch allocation would show as 8 MiB or more)
            assert free_before - torch.cuda.mem_get_info(cuda)[0] < (4 << 20)
        assert not torch.isnan(got).any()
        assert torch.equal(got, want)          # same kernels, same partials: bit for bit
        outs.append(got)
    assert not torch.equal(outs[0], outs[1])
    assert cabi.device_status() == 0


def test_static_scratch_variant_refuses_oversized_problems(cuda):
    lib = cabi.load()
    B = 400                                    # workspace for 400 sequences x 32 heads exceeds 8 MiB
    assert lib.b200q_paged_gqa_workspace_bytes(B, 32, 8, 128) > lib.b200q_paged_gqa_static_scratch_bytes()
    case = synth.paged_kv_case(2, 8, 128, 16, num_pages=8, min_len=4, max_len=20, bits=4, group_size=32, seed=1)
    case = {k: (v.to(cuda) if torch.is_tensor(v) else v) for k, v in case.items()}
    q = torch.zeros((B, 32, 128), dtype=torch.float16, device=cuda)
    out = torch.zeros_like(q)
    rc = _call(lib, True, case, q, out)
    assert rc == -6
    assert b"built-in scratch" in lib.b200q_strerror(rc)
