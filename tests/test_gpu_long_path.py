"""Mixed batches the way the backend runs them (the "next" row after the hot path): long queries have their
pages dequantized into temporary bf16 pages that vLLM's paged FlashAttention reads, short ones run the INT8
kernel afterwards. Needs vLLM's flash-attention build for this GPU; skipped (with the reason) where it is missing."""
import numpy as np
import pytest
import torch
from gpu_util import DEV, oracle_attention, short_row_mask, to_dev

from kvq_b200 import cuda_kernels as ck
from kvq_b200 import workloads
from oracle import kvq_oracle as orc

pytestmark = pytest.mark.gpu

MIXED = ([1, 1, 7, 40, 130, 1, 290, 9, 4], [590, 33, 7, 480, 130, 1400, 910, 1900, 70])
PREFILL = ([250, 97], [250, 1150])


def _flash_attention_or_skip():
    try:
        fa, version = ck._flash_attn_varlen()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM flash attention not importable: {e!r}")
    return fa, version


@pytest.mark.parametrize("name,lens", [("mixed", MIXED), ("prefill", PREFILL)])
@pytest.mark.parametrize("per_channel", [True, False])
def test_mixed_batch_matches_oracle(name, lens, per_channel, monkeypatch):
    _flash_attention_or_skip()
    monkeypatch.setenv("KVQ_LONG_PATH", "fa")   # this file covers the reference's route; test_gpu_prefill.py the other
    case = workloads.paged_case(90, 28, 4, 128, *lens, per_channel=per_channel, smooth=True, q_std=3.0)
    ref = oracle_attention(case)              # implementation B for short rows, A (dequantize) for long ones
    q = case["q"].to(DEV)
    out = torch.zeros_like(q)
    cu, sl, bt = case["cu_seqlens_q"].to(DEV), case["seq_lens"].to(DEV), case["block_table"].to(DEV)
    plan = ck.plan_long(case["cu_seqlens_q"], case["seq_lens"], 16)
    assert plan is not None and plan.has_short == (name == "mixed")
    try:
        ck.paged_attention(q, case["kq"].to(DEV), case["vq"].to(DEV), out, cu, sl, bt, max(case["q_lens"]),
                           case["softmax_scale"], to_dev(case["static"]), plan)
        torch.cuda.synchronize()
    except (RuntimeError, AssertionError, TypeError) as e:
        pytest.skip(f"paged FlashAttention unavailable on this GPU/build: {str(e)[:200]}")
    got = out.float().cpu().numpy()
    short = short_row_mask(case)
    # long rows: bf16 FlashAttention on dequantized bf16 K/V (the reference's own bound for them is rel_l2 < 1e-2)
    assert orc.compare(ref[~short], got[~short])["rel_l2"] < 1e-2
    if short.any():
        assert orc.compare(ref[short], got[short])["rel_l2"] < 5e-3
