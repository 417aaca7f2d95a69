"""Helpers for the GPU parity tests: move seeded CPU cases to the device, call the kernels through the
C ABI (via the kvq_b200 host layer), run the CPU oracle on the same bytes."""
import numpy as np
import torch

from kvq_b200 import cuda_kernels as ck
from oracle import kvq_oracle as orc

DEV = "cuda"

MAX_ABS, MEAN_ABS, REL_L2 = 1e-2, 1e-3, 5e-3


def bf16_ulp(x):
    """Spacing of bf16 numbers at |x| (8 significand bits): 2^(floor(log2 |x|) - 7)."""
    ax = np.maximum(np.abs(np.asarray(x, np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(ax)) - 7)


def assert_close(ref, out, what=""):
    """The attention bar. ref: fp32 result of the oracle / the reference; out: the kernel's bf16 output as fp32.

    Where |ref| < 2: max-abs 1e-2 and mean-abs 1e-3 against the fp32 reference outright. Where |ref| >= 2 a
    correctly rounded bf16 store alone can be off by up to half an ulp = 2^-7 .. 2^-5, so there the kernel must
    hit the bf16 rounding of the reference or one of its two neighbours: |out - bf16(ref)| <= 1 bf16 ulp.
    Plus the reference's own bound for its CUDA kernel, rel_l2 < 5e-3, over everything."""
    ref, out = np.asarray(ref, np.float32), np.asarray(out, np.float32)
    err = orc.compare(ref, out)
    d = np.abs(ref.astype(np.float64) - out.astype(np.float64))
    small = np.abs(ref) < 2.0
    if small.any():
        err["max_abs_small"], err["mean_abs_small"] = float(d[small].max()), float(d[small].mean())
        assert err["max_abs_small"] <= MAX_ABS and err["mean_abs_small"] < MEAN_ABS, (what, err)
    if (~small).any():
        big = ~small
        steps = np.abs(orc.round_to_bf16(ref[big]).astype(np.float64) - out[big]) / bf16_ulp(ref[big])
        err["max_ulp_large"] = float(steps.max())
        assert err["max_ulp_large"] <= 1.0, (what, err)
    assert err["rel_l2"] < REL_L2, (what, err)
    return err


def to_dev(static):
    return {k: v.to(DEV) for k, v in static.items()}


def run_decode(case, max_query_len=None, out=None, interleaved=False, device_case=None, q_group=None):
    """decode_attention on the case's int8 cache; returns the bf16 output as a CPU float32 array.
    interleaved=True stores K and V in one [nb, bs, H, 2D] tensor (vLLM's layout) and passes strided views."""
    q = case["q"].to(DEV)
    if interleaved:
        kv = torch.cat([case["kq"], case["vq"]], dim=-1).to(DEV)
        kq, vq = kv.split(case["kq"].shape[-1], dim=-1)
    else:
        kq, vq = case["kq"].to(DEV), case["vq"].to(DEV)
    out = torch.zeros_like(q) if out is None else out
    mql = max_query_len if max_query_len is not None else max(case["q_lens"])
    ck.decode_attention(q, kq, vq, out, case["cu_seqlens_q"].to(DEV), case["seq_lens"].to(DEV),
                        case["block_table"].to(DEV), case["softmax_scale"], to_dev(case["static"]), max_query_len=mql,
                        q_group=q_group)
    torch.cuda.synchronize()
    assert ck.decode_status() == 0, "a bounded wait inside the attention kernel expired"
    return out.float().cpu().numpy()


def oracle_attention(case, requests=None, short_q=8, long_kv_bf16=True, q_group=None):
    st = case["static"]
    return orc.paged_static_attention(case["q"].float().numpy(), case["kq"].numpy(), case["vq"].numpy(),
                                      case["cu_seqlens_q"].numpy(), case["seq_lens"].numpy(),
                                      case["block_table"].numpy(), case["softmax_scale"], st["k_scale"].numpy(),
                                      st["v_scale"].numpy(), short_q=short_q, p_tile=32, requests=requests,
                                      long_kv_bf16=long_kv_bf16, q_group=q_group)


def short_row_mask(case, limit=8):
    """True for query rows of requests the INT8 kernel handles (1 <= q_len <= limit)."""
    q_lens = np.asarray(case["q_lens"])
    return np.repeat((q_lens >= 1) & (q_lens <= limit), q_lens)


def fixture_case(fx):
    """A golden .npz with stored inputs -> the dict layout workloads.paged_case returns."""
    cu = fx["cu_seqlens_q"]
    return {"q": torch.from_numpy(fx["q"].view(np.int16)).view(torch.bfloat16), "kq": torch.from_numpy(fx["kq"]),
            "vq": torch.from_numpy(fx["vq"]), "cu_seqlens_q": torch.from_numpy(cu),
            "seq_lens": torch.from_numpy(fx["seq_lens"]), "block_table": torch.from_numpy(fx["block_table"]),
            "static": {"k_scale": torch.from_numpy(fx["k_scale"]), "v_scale": torch.from_numpy(fx["v_scale"]),
                       "k_mu": torch.from_numpy(fx["k_mu"])},
            "softmax_scale": float(fx["softmax_scale"]), "q_lens": np.diff(cu).tolist()}
