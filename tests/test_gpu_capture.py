"""Calibration capture (kvq_b200.capture, kernel kvq_calib_stats) against the reference's hook state machine
(fixture made by the reference's own kvq/capture.py) and against the CPU oracle on larger seeded inputs."""
import numpy as np
import pytest
import torch
from conftest import load_golden

from kvq_b200 import capture, scales
from oracle import kvq_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf16(bits):
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16)


def check(st, ref):
    assert st["tokens"] == int(ref["tokens"])
    for side in "kv":
        for f in ("absmax", "max", "min"):
            assert np.array_equal(st[f"{side}_{f}"].numpy(), ref[f"{side}_{f}"]), (side, f)   # exact
        assert np.allclose(st[f"{side}_sum"].numpy(), ref[f"{side}_sum"], rtol=1e-12, atol=1e-9)


def test_matches_reference_hook_on_its_fixture():
    fx = load_golden("calib_stats.npz")
    capture.reset()
    for i in (0, 1):
        capture.record("layer", bf16(fx[f"key{i}"]).to(DEV), bf16(fx[f"value{i}"]).to(DEV), torch.from_numpy(fx[f"slots{i}"]).to(DEV))
    st = capture.stats("layer")
    check(st, {k[5:]: fx[k] for k in fx if k.startswith("stat_")})
    # the scales derived from the captured statistics are the reference's
    got = scales.from_stats(st, None, "per_channel", "max", True)
    for f, v in got.items():
        assert np.allclose(v.numpy(), fx[f"scales_per_channel_max_1_{f}"], rtol=1e-6, atol=0)
    out = capture.collect(tp_rank=0, tp_size=1)
    assert out["tp_rank"] == 0 and out["samples"]["layer"]["k"].shape == (int(fx["stat_tokens"]), 4, 128)
    assert out["samples"]["layer"]["k"].dtype == torch.float16


@pytest.mark.parametrize("heads,dim,tokens", [(4, 128, 8192), (8, 128, 1000), (2, 64, 333), (1, 128, 1)])
def test_large_batches_and_strides_vs_oracle(heads, dim, tokens):
    gen = torch.Generator().manual_seed(heads * 1000 + tokens)
    batches = []
    capture.reset()
    for step in range(3):
        # fused qkv layout: K and V are slices of one [T, (q + 2 kv) heads, D] tensor
        qkv = (torch.randn(tokens, 3 * heads, dim, generator=gen) * (step + 1)).to(torch.bfloat16)
        key, value = qkv[:, heads:2 * heads], qkv[:, 2 * heads:]
        slots = None
        if step == 1:
            slots = torch.randperm(tokens * 2, generator=gen)[:max(1, tokens - 3)].long()
            slots[::7] = -1
        dk, dv = qkv.to(DEV)[:, heads:2 * heads], qkv.to(DEV)[:, 2 * heads:]
        capture.record("l", dk, dv, None if slots is None else slots.to(DEV))
        batches.append((key.float().numpy(), value.float().numpy(), None if slots is None else slots.numpy()))
    check(capture.stats("l"), orc.calib_stats(batches))


def test_sample_budget(monkeypatch):
    monkeypatch.setattr(capture, "MAX_SAMPLE_TOKENS", 64)
    capture.reset()
    x = torch.randn(40, 2, 64, device=DEV).to(torch.bfloat16)
    capture.record("s", x, x)                       # 40 rows kept
    capture.record("s", x, x)                       # past half the budget: a random eighth
    capture.record("s", x, x)
    n = capture.STATE["samples"]["s"]["n"]
    assert 40 < n <= 64 + 40 and capture.stats("s")["tokens"] == 120
    for _ in range(20):
        capture.record("s", x, x)
    assert capture.STATE["samples"]["s"]["n"] <= 64 + 5 and capture.stats("s")["tokens"] == 23 * 40


def test_rejects_wrong_inputs():
    capture.reset()
    x = torch.randn(4, 2, 64, device=DEV)
    with pytest.raises(RuntimeError):
        capture.record("e", x, x)                   # fp32
    with pytest.raises(RuntimeError):
        capture.record("e", x.bfloat16().cpu(), x.bfloat16().cpu())
