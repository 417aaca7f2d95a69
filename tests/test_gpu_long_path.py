"""Mixed batches the way the backend runs them: long queries (more than SHORT_Q tokens) go to the long-query
path, short ones run the INT8 kernel afterwards. Both long-query routes are covered: the reference's (pages
dequantized into temporary bf16 pages that vLLM's paged FlashAttention reads; skipped where that library kernel
cannot be imported) and the INT8-page kernel. The cases follow the reference's own mixed-batch tests
(tests/test_cuda_kernels.py:100-133): mixed, prefill-only, a 256-request serving step, optimistic host lengths."""
import pytest
import torch
from gpu_util import DEV, oracle_attention, short_row_mask, to_dev

from kvq_b200 import cuda_kernels as ck
from kvq_b200 import workloads
from oracle import kvq_oracle as orc

pytestmark = pytest.mark.gpu

MIXED = ([1, 1, 7, 40, 130, 1, 290, 9, 4], [590, 33, 7, 480, 130, 1400, 910, 1900, 70])
PREFILL = ([250, 97], [250, 1150])
SERVING = workloads.serving_lengths(seed=0)
CASES = {"mixed": MIXED, "prefill": PREFILL, "serving": SERVING}


def _need_flash_attention():
    """Skip only when the third-party kernel is missing: probed by import, never by running the product path."""
    try:
        ck._flash_attn_varlen()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM flash attention not importable: {e!r}")


def _run(case, plan, route, monkeypatch, block_table=None):
    monkeypatch.setenv("KVQ_LONG_PATH", route)
    q = case["q"].to(DEV)
    out = torch.zeros_like(q)
    bt = (case["block_table"] if block_table is None else block_table).to(DEV)
    ck.paged_attention(q, case["kq"].to(DEV), case["vq"].to(DEV), out, case["cu_seqlens_q"].to(DEV),
                       case["seq_lens"].to(DEV), bt, max(case["q_lens"]), case["softmax_scale"], to_dev(case["static"]),
                       plan)
    torch.cuda.synchronize()
    assert ck.decode_status() == 0 and ck.prefill_status() == 0
    return out.float().cpu().numpy()


def _check(case, got, route):
    ref = oracle_attention(case)              # implementation B for short rows, A (dequantize) for long ones
    short = short_row_mask(case)
    # long rows: the reference's own bound for bf16 FlashAttention on dequantized K/V is rel_l2 < 1e-2
    assert orc.compare(ref[~short], got[~short])["rel_l2"] < 1e-2, route
    if short.any():
        assert orc.compare(ref[short], got[short])["rel_l2"] < 5e-3, route


@pytest.mark.parametrize("route", ["fa", "int8"])
@pytest.mark.parametrize("name", ["mixed", "prefill", "serving"])
@pytest.mark.parametrize("per_channel", [True, False])
def test_mixed_batch_matches_oracle(name, per_channel, route, monkeypatch):
    if route == "fa":
        _need_flash_attention()
    case = workloads.paged_case(90, 28, 4, 128, *CASES[name], per_channel=per_channel, smooth=True, q_std=3.0)
    plan = ck.plan_long(case["cu_seqlens_q"], case["seq_lens"], 16)
    assert plan is not None and plan.has_short == (name != "prefill")
    _check(case, _run(case, plan, route, monkeypatch), route)


@pytest.mark.parametrize("route", ["fa", "int8"])
def test_long_path_uses_gpu_lengths(route, monkeypatch):
    """Host-side lengths may be upper bounds (asynchronous speculative decoding counts every draft token as
    accepted): the plan may then copy extra pages, but attention must use the exact lengths held on the GPU.
    The block table is also wider than any request needs, as vLLM's are."""
    if route == "fa":
        _need_flash_attention()
    case = workloads.paged_case(91, 28, 4, 128, *MIXED, smooth=True, q_std=3.0)
    bt = case["block_table"]
    wide = torch.cat([bt, bt[:, :1].expand(-1, 2)], 1).contiguous()
    plan = ck.plan_long(case["cu_seqlens_q"], case["seq_lens"] + 5, 16)     # optimistic host lengths
    assert plan.max_seqlen_k == max(L for L, n in zip(MIXED[1], MIXED[0]) if n > ck.SHORT_Q) + 5
    _check(case, _run(case, plan, route, monkeypatch, block_table=wide), route)
