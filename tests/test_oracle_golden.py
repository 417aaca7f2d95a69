"""The CPU oracle against fixtures produced by the reference project's own code (tests/golden/make_golden.py).

Integer outputs (cache bytes, quantized q, dequantized bf16 bit patterns) must be identical; attention outputs
agree to float rounding (the oracle evaluates exp with numpy, the reference with torch)."""
import hashlib

import numpy as np
import pytest
import torch
from conftest import load_golden

from kvq_b200 import workloads
from oracle import kvq_oracle as orc

ATTN_TOL = dict(max_abs=2e-4, mean_abs=5e-6)   # oracle vs reference, both fp32 evaluations


def _attention_from_fixture(fx, q_group=None):
    q = orc.bf16_bits_to_f32(fx["q"])
    return orc.paged_static_attention(q, fx["kq"], fx["vq"], fx["cu_seqlens_q"], fx["seq_lens"], fx["block_table"],
                                      float(fx["softmax_scale"]), fx["k_scale"], fx["v_scale"], short_q=8, p_tile=32,
                                      q_group=q_group)


@pytest.mark.parametrize("name", ["attn_qgroup32.npz", "attn_qgroup32_per_head.npz"])
def test_group32_q_scales_match_reference(name):
    """One q scale per 32-channel slice (the reference's q_gran="group32", kvq/int8_ref.py:120-130 and
    CONFIGS["B_channel_smooth_qgroup32"]): fixtures made by the reference itself; and the option changes the result."""
    fx = load_golden(name)
    out = _attention_from_fixture(fx, q_group=32)
    err = orc.compare(fx["ref_out"], out)
    assert err["max_abs"] < ATTN_TOL["max_abs"] and err["mean_abs"] < ATTN_TOL["mean_abs"], err
    assert orc.compare(fx["ref_out"], _attention_from_fixture(fx))["max_abs"] > 10 * err["max_abs"]


@pytest.mark.parametrize("name", ["attn_short_smooth.npz", "attn_per_head_d64.npz", "attn_mixed_long.npz"])
def test_attention_matches_reference(name):
    fx = load_golden(name)
    err = orc.compare(fx["ref_out"], _attention_from_fixture(fx))
    assert err["max_abs"] < ATTN_TOL["max_abs"] and err["mean_abs"] < ATTN_TOL["mean_abs"], err


def test_config0_matches_reference_and_bf16_golden():
    """Benchmark configuration 0 (4 decode requests, contexts 128..512), inputs regenerated from the seed (checksummed), outputs from the reference."""
    fx = load_golden("attn_config0.npz")
    c = workloads.config0()
    h = hashlib.sha256()
    for t in (c["q"], c["kq"], c["vq"], c["block_table"]):
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    assert h.hexdigest() == str(fx["input_sha256"]), "seeded inputs differ from the ones the fixture was made from"
    st = c["static"]
    out = orc.paged_static_attention(c["q"].float().numpy(), c["kq"].numpy(), c["vq"].numpy(),
                                     c["cu_seqlens_q"].numpy(), c["seq_lens"].numpy(), c["block_table"].numpy(),
                                     c["softmax_scale"], st["k_scale"].numpy(), st["v_scale"].numpy())
    err = orc.compare(fx["ref_out"], out)
    assert err["max_abs"] < ATTN_TOL["max_abs"] and err["mean_abs"] < ATTN_TOL["mean_abs"], err
    # the oracle's own bf16 attention against the reference's bf16 golden (same unquantized inputs)
    gold = orc.paged_attention_bf16(c["q"].float().numpy(), c["k"].float().numpy(), c["v"].float().numpy(),
                                    c["cu_seqlens_q"].numpy(), c["seq_lens"].numpy(), c["block_table"].numpy(),
                                    c["softmax_scale"])
    assert orc.compare(fx["bf16_golden"], gold)["max_abs"] < 1e-4
    # implementation B against the bf16 golden: the reference's own quantization tolerance (rel_l2 < 0.05)
    assert orc.compare(fx["bf16_golden"], out)["rel_l2"] < 0.05


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("gran", ["channel", "head"])
def test_cache_write_and_dequant_bit_exact(d, gran):
    fx = load_golden(f"write_d{d}_{gran}.npz")
    key, value = orc.bf16_bits_to_f32(fx["key"]), orc.bf16_bits_to_f32(fx["value"])
    kc, vc = np.zeros_like(fx["k_cache"]), np.zeros_like(fx["v_cache"])
    orc.quant_cache_write(key, value, kc, vc, fx["slots"], fx["k_scale"], fx["v_scale"], fx["k_mu"])
    assert np.array_equal(kc, fx["k_cache"]) and np.array_equal(vc, fx["v_cache"])
    # dequantize every page through an identity page table
    nb = kc.shape[0]
    bt = np.arange(nb, dtype=np.int32)[None]
    ko, vo = orc.dequant_pages(kc, vc, bt, np.zeros(nb, np.int32), np.arange(nb, dtype=np.int32), fx["k_scale"],
                               fx["v_scale"])
    assert np.array_equal(orc.f32_to_bf16_bits(ko), fx["k_dequant"])
    assert np.array_equal(orc.f32_to_bf16_bits(vo), fx["v_dequant"])


def test_quant_q_bit_exact():
    fx = load_golden("quant_q.npz")
    q = orc.bf16_bits_to_f32(fx["q"])
    for group in (128, 32):
        qi, qs = orc.quant_q(q, fx["k_scale"], group)
        assert np.array_equal(qi, fx[f"q_i8_g{group}"]) and np.array_equal(qs, fx[f"q_scale_g{group}"])
    qi, qs = orc.quant_q(q, np.ones((4, 1), np.float32), 128)
    assert np.array_equal(qi, fx["q_i8_per_head"]) and np.array_equal(qs, fx["q_scale_per_head"])


def test_bf16_rounding_helpers_match_torch():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(100000, generator=g) * torch.exp(torch.randn(100000, generator=g) * 4)
    x[:4] = torch.tensor([0.0, -0.0, float("inf"), 1.00390625])   # the last one is a round-half-even tie
    want = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.f32_to_bf16_bits(x.numpy()), want)
    assert np.array_equal(orc.bf16_bits_to_f32(want), x.to(torch.bfloat16).float().numpy())


def test_round_trip_error_bound():
    """|x - dequant(quant(x))| <= s / 2 (+ fp32 rounding) inside the clamp range."""
    c = workloads.write_case(5, 512, 4, 128, num_blocks=64, smooth=False)
    st = c["static"]
    x = c["key"][:512].float().numpy()
    s = st["k_scale"].numpy()
    y = orc.dequantize(orc.quantize(x, s), s)
    assert (np.abs(x - y) <= s / 2 + 1e-6 * (1 + np.abs(x))).all()


def test_calibration_statistics_match_reference_hook():
    """oracle.calib_stats and kvq_b200.scales.from_stats against the reference's capture state machine and
    from_stats on the same two steps (fixture made by tests/golden/make_golden.py:save_calib)."""
    import torch

    from kvq_b200 import scales

    fx = load_golden("calib_stats.npz")
    batches = [(orc.bf16_bits_to_f32(fx[f"key{i}"]), orc.bf16_bits_to_f32(fx[f"value{i}"]), fx[f"slots{i}"]) for i in (0, 1)]
    st = orc.calib_stats(batches)
    assert st["tokens"] == int(fx["stat_tokens"])
    for side in "kv":
        for f in ("absmax", "max", "min"):
            assert np.array_equal(st[f"{side}_{f}"], fx[f"stat_{side}_{f}"]), (side, f)
        assert np.allclose(st[f"{side}_sum"], fx[f"stat_{side}_sum"], rtol=1e-12, atol=1e-9)
    tst = {k: (torch.from_numpy(np.asarray(v)) if isinstance(v, np.ndarray) else v) for k, v in st.items()}
    rows = [(b[0][:len(b[2])][b[2] >= 0], b[1][:len(b[2])][b[2] >= 0]) for b in batches]
    samples = {"k": torch.from_numpy(np.concatenate([r[0] for r in rows])).to(torch.float16),
               "v": torch.from_numpy(np.concatenate([r[1] for r in rows])).to(torch.float16)}
    for gran, method, smooth in (("per_channel", "max", False), ("per_channel", "max", True),
                                 ("per_channel", "q0.999", True), ("per_head", "max", True)):
        res = scales.from_stats(tst, samples, gran, method, smooth)
        for f, v in res.items():
            want = fx[f"scales_{gran}_{method}_{int(smooth)}_{f}"]
            assert np.allclose(v.numpy(), want, rtol=1e-6, atol=0), (gran, method, smooth, f)


def test_numpy_oracle_agrees_with_the_staged_reference_modules():
    """Where oracle/_ref holds the reference's own modules (byte-compiled by oracle/build_ref.py from a checkout), the
    numpy restatement is compared with them directly on fresh seeded cases, beyond the committed fixtures: decode,
    short multi-token queries and a long request (implementation A), per-channel and per-head scales."""
    import torch
    from oracle import build_ref
    from kvq_b200 import workloads

    mods = build_ref.load()
    if mods is None:
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    quant, ref_attn, int8_ref = mods
    for seed, per_channel in ((201, True), (202, False)):
        case = workloads.paged_case(seed, 12, 2, 128, [1, 5, 8, 1, 20], [300, 77, 1030, 16, 150], per_channel=per_channel,
                                    smooth=True, q_std=3.0)
        st = case["static"]
        gran = "per_channel" if per_channel else "per_head"
        fn = int8_ref.paged_static_attention(int8_ref.Cfg(smooth_k=True, p_tile=32, k_gran=gran, v_gran=gran), st,
                                             cache_is_int8=True, short_q=8)
        want = fn(case["q"].float(), case["kq"], case["vq"], case["cu_seqlens_q"], case["seq_lens"], case["block_table"],
                  case["softmax_scale"]).numpy()
        got = orc.paged_static_attention(case["q"].float().numpy(), case["kq"].numpy(), case["vq"].numpy(),
                                         case["cu_seqlens_q"].numpy(), case["seq_lens"].numpy(), case["block_table"].numpy(),
                                         case["softmax_scale"], st["k_scale"].numpy(), st["v_scale"].numpy())
        d = np.abs(want - got)
        assert d.max() < ATTN_TOL["max_abs"] and d.mean() < ATTN_TOL["mean_abs"]
        # cache bytes through the reference's quantize
        kq = quant.quantize(case["k"].float() - st["k_mu"], st["k_scale"]).numpy()
        assert np.array_equal(kq, case["kq"].numpy())
        assert np.array_equal(orc.quantize(case["k"].float().numpy() - st["k_mu"].numpy(), st["k_scale"].numpy()), kq)
