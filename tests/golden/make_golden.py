"""Generate the golden fixtures in this folder by running the reference project's own Python code.

Run where the reference checkout is available (it is imported, never copied):

    KVQ_REF=/path/to/int8-kvcache python tests/golden/make_golden.py

The fixtures pin the CPU oracle (oracle/kvq_oracle.py) and, through it, the CUDA kernels. Each .npz holds
the inputs (small cases) or a checksum of the seeded inputs (config 0), and the outputs of:
  kvq.quant.quantize / dequantize            (cache bytes, dequantized pages)
  the fp32 q-quantization formula            (tests/test_cuda_kernels.py:46-55 of the reference)
  kvq.int8_ref.paged_static_attention        (implementation B / A, p_tile=32, short_q=8)
  kvq.ref_attn.paged_attention_ref           (bf16 golden on the unquantized cache)
  kvq.cuda_kernels.plan_long, kvq.scales.shard
  kvq.capture._record (calibration statistics), kvq.scales.from_stats
"""
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "int8-kvcache_b200"))
if "KVQ_REF" not in os.environ:
    raise SystemExit("set KVQ_REF to a checkout of the reference project (ischencheng/int8-kvcache)")
sys.path.insert(0, os.environ["KVQ_REF"])

from kvq import capture as ref_capture  # noqa: E402
from kvq import cuda_kernels as ref_ck  # noqa: E402
from kvq import quant as ref_quant  # noqa: E402
from kvq import scales as ref_scales  # noqa: E402
from kvq.int8_ref import Cfg, paged_static_attention  # noqa: E402
from kvq.ref_attn import paged_attention_ref  # noqa: E402

from kvq_b200 import workloads  # noqa: E402


def bits(t):
    """bf16 tensor -> uint16 bit patterns."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def ref_attention(case, per_channel=True, smooth=False, fp32=True, q_gran="token_head"):
    cfg = (Cfg(smooth_k=smooth, p_tile=32, q_gran=q_gran) if per_channel else
           Cfg(smooth_k=smooth, p_tile=32, k_gran="per_head", v_gran="per_head", q_gran=q_gran))
    fn = paged_static_attention(cfg, case["static"], cache_is_int8=True, short_q=8)
    q = case["q"].float() if fp32 else case["q"]
    return fn(q, case["kq"], case["vq"], case["cu_seqlens_q"], case["seq_lens"], case["block_table"],
              case["softmax_scale"])


def save_attention(name, case, per_channel, smooth, store_inputs=True, with_bf16_golden=False, q_gran="token_head"):
    # the workload generator's cache filler must agree with the reference's quantizer bit for bit
    st = case["static"]
    assert torch.equal(case["kq"], ref_quant.quantize(case["k"].float() - st["k_mu"], st["k_scale"]))
    assert torch.equal(case["vq"], ref_quant.quantize(case["v"], st["v_scale"]))
    out = {"ref_out": ref_attention(case, per_channel, smooth, q_gran=q_gran).numpy(),
           "ref_out_bf16": bits(ref_attention(case, per_channel, smooth, fp32=False, q_gran=q_gran)),
           "input_sha256": np.array(digest(case["q"], case["kq"], case["vq"], case["block_table"]))}
    if with_bf16_golden:
        out["bf16_golden"] = paged_attention_ref(case["q"].float(), case["k"], case["v"], case["cu_seqlens_q"],
                                                 case["seq_lens"], case["block_table"], case["softmax_scale"]).numpy()
    if store_inputs:
        out.update(q=bits(case["q"]), kq=case["kq"].numpy(), vq=case["vq"].numpy(),
                   cu_seqlens_q=case["cu_seqlens_q"].numpy(), seq_lens=case["seq_lens"].numpy(),
                   block_table=case["block_table"].numpy(), k_scale=st["k_scale"].numpy(),
                   v_scale=st["v_scale"].numpy(), k_mu=st["k_mu"].numpy(),
                   softmax_scale=np.float64(case["softmax_scale"]))
    np.savez_compressed(os.path.join(HERE, name), **out)
    print(name, {k: getattr(v, "shape", None) for k, v in out.items()})


def save_write(name, d, per_channel):
    c = workloads.write_case(7 + d + int(per_channel), 200, 4, d, num_blocks=64, per_channel=per_channel, smooth=True,
                             pad_rows=8, drop_every=17)
    st, slots, bs = c["static"], c["slots"], c["block_size"]
    ok = slots >= 0
    kc = torch.zeros(64, bs, 4, d, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    kc[slots[ok] // bs, slots[ok] % bs] = ref_quant.quantize(c["key"][:200][ok].float() - st["k_mu"], st["k_scale"])
    vc[slots[ok] // bs, slots[ok] % bs] = ref_quant.quantize(c["value"][:200][ok], st["v_scale"])
    # page dequantization of what was written (K stays k - mu)
    kd = ref_quant.dequantize(kc, st["k_scale"], torch.bfloat16)
    vd = ref_quant.dequantize(vc, st["v_scale"], torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, name), key=bits(c["key"]), value=bits(c["value"]), slots=slots.numpy(),
                        k_scale=st["k_scale"].numpy(), v_scale=st["v_scale"].numpy(), k_mu=st["k_mu"].numpy(),
                        k_cache=kc.numpy(), v_cache=vc.numpy(), k_dequant=bits(kd), v_dequant=bits(vd))
    print(name)


def save_quant_q():
    gen = torch.Generator().manual_seed(11)
    q = torch.randn(37, 28, 128, generator=gen).to(torch.bfloat16)
    ks = torch.rand(4, 128, generator=gen) + 0.01
    out = {"q": bits(q), "k_scale": ks.numpy()}
    for group in (128, 32):
        qf = (q.float().reshape(37, 4, 7, 128) * ks[None, :, None, :]).reshape(37, 28, 128 // group, group)
        s = ref_quant.scale_from_absmax(qf.abs().amax(-1, keepdim=True))
        out[f"q_i8_g{group}"] = ref_quant.quantize(qf, s).reshape(37, 28, 128).numpy()
        out[f"q_scale_g{group}"] = s[..., 0].numpy()
    # per-head K scale: nothing is folded into q
    s = ref_quant.scale_from_absmax(q.float().abs().amax(-1, keepdim=True))
    out["q_i8_per_head"] = ref_quant.quantize(q.float(), s).numpy()
    out["q_scale_per_head"] = s.numpy()
    np.savez_compressed(os.path.join(HERE, "quant_q.npz"), **out)
    print("quant_q.npz")


def save_plans():
    out = {}
    cases = {"a": ([0, 1, 13, 14, 314], [50, 40, 9, 330], 16), "b": ([0, 40, 41, 50, 51], [40, 77, 9, 1], 16),
             "c": ([0, 9, 20, 21], [100, 33, 5], 32), "none": ([0, 1, 9], [5, 8], 16)}
    for key, (cu, sl, bs) in cases.items():
        plan = ref_ck.plan_long(torch.tensor(cu, dtype=torch.int32), torch.tensor(sl, dtype=torch.int32), bs)
        out[f"{key}_cu"], out[f"{key}_sl"], out[f"{key}_bs"] = np.array(cu), np.array(sl), np.array(bs)
        out[f"{key}_is_none"] = np.array(plan is None)
        if plan is not None:
            out[f"{key}_src_req"], out[f"{key}_src_j"], out[f"{key}_bt"] = plan.src_req, plan.src_j, plan.block_table
            out[f"{key}_max_seqlen_k"], out[f"{key}_has_short"] = np.array(plan.max_seqlen_k), np.array(plan.has_short)
    np.savez_compressed(os.path.join(HERE, "plan_long.npz"), **out)
    print("plan_long.npz")


def save_shards():
    t = torch.arange(8 * 3, dtype=torch.float32).reshape(8, 3)
    out = {"t8": t.numpy(), "t2": t[:2].numpy()}
    for h, name in ((8, "t8"), (2, "t2")):
        for tp in (1, 2, 4, 8):
            for rank in range(tp):
                out[f"{name}_tp{tp}_r{rank}"] = ref_scales.shard(t[:h], rank, tp).numpy()
    np.savez_compressed(os.path.join(HERE, "scale_shards.npz"), **out)
    print("scale_shards.npz")


def save_calib():
    """Two steps of new K/V rows through the reference's capture hook state machine (kvq/capture.py:25-44; the
    hook masks rows by slot >= 0 before recording, kvq/capture.py:93-96) and the scales its from_stats derives."""
    gen = torch.Generator().manual_seed(13)
    out = {}
    ref_capture.STATE["stats"].clear(), ref_capture.STATE["samples"].clear()
    rows = []
    for i, (t, pad) in enumerate(((300, 0), (77, 5))):
        key = (torch.randn(t + pad, 4, 128, generator=gen) * 3 + torch.randn(4, 128, generator=gen)).to(torch.bfloat16)
        value = torch.randn(t + pad, 4, 128, generator=gen).to(torch.bfloat16)
        slots = torch.randperm(4096, generator=gen)[:t].long()
        slots[::11] = -1
        valid = slots >= 0
        ref_capture._record("layer", key[:t][valid], value[:t][valid])
        rows.append((key[:t][valid], value[:t][valid]))
        out[f"key{i}"], out[f"value{i}"], out[f"slots{i}"] = bits(key), bits(value), slots.numpy()
    st = ref_capture.STATE["stats"]["layer"]
    for f, v in st.items():
        out["stat_" + f] = v.numpy() if torch.is_tensor(v) else np.array(v)
    samples = {"k": torch.cat([r[0] for r in rows]).to(torch.float16), "v": torch.cat([r[1] for r in rows]).to(torch.float16)}
    for gran, method, smooth in (("per_channel", "max", False), ("per_channel", "max", True), ("per_channel", "q0.999", True),
                                 ("per_head", "max", True)):
        res = ref_scales.from_stats(st, samples, gran, method, smooth)
        for f, v in res.items():
            out[f"scales_{gran}_{method}_{int(smooth)}_{f}"] = v.numpy()
    np.savez_compressed(os.path.join(HERE, "calib_stats.npz"), **out)
    print("calib_stats.npz")


def main():
    torch.manual_seed(0)
    only = sys.argv[1:]   # fixture names to (re)generate; default: all
    if only:
        import builtins
        real_savez = np.savez_compressed

        def filtered(path, **kw):
            if os.path.basename(path) in only:
                real_savez(path, **kw)
            else:
                builtins.print("  (not rewritten)", end=" ")

        np.savez_compressed = filtered
    save_attention("attn_config0.npz", workloads.config0(), True, False, store_inputs=False, with_bf16_golden=True)
    save_attention("attn_short_smooth.npz",
                   workloads.paged_case(21, 12, 2, 128, [2, 8, 1, 5, 3], [40, 200, 129, 96, 8], num_blocks=40,
                                        smooth=True), True, True)
    save_attention("attn_per_head_d64.npz",
                   workloads.paged_case(22, 14, 2, 64, [1, 4, 7, 1, 0], [17, 300, 64, 333, 5], num_blocks=56,
                                        per_channel=False, smooth=True), False, True)
    save_attention("attn_mixed_long.npz",
                   workloads.paged_case(23, 12, 2, 128, [1, 33, 4, 9], [50, 100, 31, 70], num_blocks=24), True, False)
    # the reference's CONFIGS["B_channel_smooth_qgroup32"] (kvq/int8_ref.py:220) with the kernel's 32-key P tile, and the
    # same with per-head K/V scales
    save_attention("attn_qgroup32.npz",
                   workloads.paged_case(24, 12, 2, 128, [1, 8, 3, 1, 5], [300, 77, 1030, 16, 150], num_blocks=110,
                                        smooth=True, q_std=3.0), True, True, q_gran="group32")
    save_attention("attn_qgroup32_per_head.npz",
                   workloads.paged_case(25, 28, 4, 128, [1, 2, 7], [100, 513, 40], num_blocks=48, per_channel=False,
                                        smooth=True, q_std=3.0), False, True, q_gran="group32")
    for d in (128, 64):
        for pc in (True, False):
            save_write(f"write_d{d}_{'channel' if pc else 'head'}.npz", d, pc)
    save_quant_q()
    save_plans()
    save_shards()
    save_calib()


if __name__ == "__main__":
    main()
