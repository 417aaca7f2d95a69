"""The allocation-free attention entry point (kvq_int8_decode_attention_noalloc), called through the C ABI.

It serves callers that cannot allocate device memory (all HBM already given to the KV pool, code running under
someone else's allocator or graph capture), so it keeps its scratch in a fixed array inside the library. Here it
is compared with the regular entry point, which gets a workspace from the caller: same kernels, so the outputs
must agree (checked with the tolerance the other GPU tests use; bit-equal for single-token decode), and with the
CPU oracle directly: for multi-token queries the built-in scratch only fits the layout with one m tile per work
item, a mode of the kernel that no other caller reaches. Several calls in a row with different batches make sure
stale contents of the shared array do not leak into the next call.

This file sorts last on purpose: if it fails under `pytest -x`, every other test has already run.
"""
import ctypes

import numpy as np
import pytest
import torch
from gpu_util import assert_close, oracle_attention

from kvq_b200 import _native
from kvq_b200 import workloads
from oracle import kvq_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(lib, fn_name, case, out, workspace=None):
    """One attention call straight through the C ABI (no host-layer wrapper)."""
    q, kq, vq = case["q"], case["kq"], case["vq"]
    st = case["static"]
    args = [q.data_ptr(), kq.data_ptr(), vq.data_ptr(), out.data_ptr(), case["cu_seqlens_q"].data_ptr(),
            case["seq_lens"].data_ptr(), case["block_table"].data_ptr(), st["k_scale"].data_ptr(),
            st["v_scale"].data_ptr(), float(case["softmax_scale"]), case["cu_seqlens_q"].numel() - 1, q.size(1),
            kq.size(2), q.size(2), kq.size(1), kq.size(0), q.stride(0), q.stride(1), out.stride(0), out.stride(1),
            kq.stride(0), kq.stride(1), kq.stride(2), vq.stride(0), vq.stride(1), vq.stride(2),
            case["block_table"].stride(0), int(st["k_scale"].shape[-1] > 1), int(st["v_scale"].shape[-1] > 1),
            max(case["q_lens"]), 8]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel()]
    args.append(torch.cuda.current_stream().cuda_stream)
    _native.check(getattr(lib, fn_name)(*args))


def _to_device(case):
    dev = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in case.items() if k != "static"}
    dev["static"] = {k: v.to(DEV) for k, v in case["static"].items()}
    return dev


def test_noalloc_entry_point_matches_workspace_entry_point():
    lib = _native.lib()
    assert lib.kvq_static_workspace_bytes() == 10 << 20
    # two different batches back to back: a long single request cut over many CTAs (many partials left in the
    # scratch), then a ragged short-query batch that reuses the same array
    cases = [workloads.paged_case(61, 28, 4, 128, [1], [12000]),
             workloads.paged_case(62, 28, 4, 128, [1, 5, 8, 1, 3], [700, 90, 2500, 33, 1024], q_std=3.0),
             # verification batch in the shape of benchmark configuration 3: q_len 8, ragged contexts of 1k..8k
             workloads.paged_case(64, 28, 4, 128, [8] * 12, [1024, 8192, 3000, 5555, 2049, 7000, 1500, 4096, 6100, 2500,
                                                              7777, 1100])]
    for cpu_case in cases:
        case = _to_device(cpu_case)
        n = case["cu_seqlens_q"].numel() - 1
        ws = torch.empty(lib.kvq_decode_workspace_size(n, 128), dtype=torch.uint8, device=DEV)
        ref = torch.zeros_like(case["q"])
        out = torch.zeros_like(case["q"])
        _call(lib, "kvq_int8_decode_attention", case, ref, ws)
        _call(lib, "kvq_int8_decode_attention_noalloc", case, out)
        torch.cuda.synchronize()
        err = orc.compare(ref.float().cpu().numpy(), out.float().cpu().numpy())
        assert err["max_abs"] < 1e-2 and err["mean_abs"] < 1e-3, err     # the bar of the other GPU tests
        if max(case["q_lens"]) == 1:
            assert torch.equal(ref, out), err    # single-token decode takes the same code path: same bits
        # (multi-token queries: the workspace entry point lets warps share K/V streams across m tiles, the built-in
        #  scratch is too small for that mode's partials, so the summation order differs in the last fp32 bits)
        assert ref.abs().sum() > 0
        assert_close(oracle_attention(cpu_case), out.float().cpu().numpy(), "no-alloc entry point vs oracle")


def test_noalloc_rejects_batches_beyond_the_builtin_scratch():
    lib = _native.lib()
    case = _to_device(workloads.paged_case(63, 28, 4, 128, [1], [64]))
    huge = 400_000   # requests: the prefix-sum table alone no longer fits in 10 MiB
    assert lib.kvq_decode_workspace_size(huge, 128) > lib.kvq_static_workspace_bytes()
    q, kq, vq, st = case["q"], case["kq"], case["vq"], case["static"]
    rc = lib.kvq_int8_decode_attention_noalloc(
        q.data_ptr(), kq.data_ptr(), vq.data_ptr(), q.data_ptr(), case["cu_seqlens_q"].data_ptr(),
        case["seq_lens"].data_ptr(), case["block_table"].data_ptr(), st["k_scale"].data_ptr(), st["v_scale"].data_ptr(),
        0.1, huge, 28, 4, 128, 16, kq.size(0), q.stride(0), q.stride(1), q.stride(0), q.stride(1), kq.stride(0),
        kq.stride(1), kq.stride(2), vq.stride(0), vq.stride(1), vq.stride(2), case["block_table"].stride(0), 1, 1, 1, 8,
        torch.cuda.current_stream().cuda_stream)
    assert rc == 3 and b"built-in array" in lib.kvq_last_error()
    torch.cuda.synchronize()
