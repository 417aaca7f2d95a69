"""Calibration capture: statistics of what a model writes into its KV cache, from which static scales are derived
(scales.from_stats). Mirrors the reference's kvq/capture.py: the same per-layer state, the same fields and the
same collect() result, so kvq/scales.py-style tooling and scripts/calibrate.py work unchanged on top of it.

Per attention layer: running |x| max, signed max / min and sum per (kv head, channel) of K and of V, the number of
tokens seen, and a bounded sample of raw rows for quantile scales. The statistics of a step are folded in by one
fused CUDA kernel (kvq_calib_stats) and stay on the GPU until collect(); the reference does eight torch reductions
per layer and step (kvq/capture.py:25-44). The one-call decode dump of the reference (KVQ_DUMP_AT_SEQLEN) is a
debugging aid of its golden tests and is not reproduced.
"""
import os

import torch

from . import _native

STATE = {"stats": {}, "samples": {}}
MAX_SAMPLE_TOKENS = int(os.environ.get("KVQ_CAPTURE_MAX_TOKENS", "16384"))

_FIELDS = ("k_absmax", "k_max", "k_min", "k_sum", "v_absmax", "v_max", "v_min", "v_sum")


def reset():
    STATE["stats"].clear()
    STATE["samples"].clear()


def _new_state(heads, dim, device):
    f32 = dict(dtype=torch.float32, device=device)
    st = {"k_absmax": torch.zeros(heads, dim, **f32), "v_absmax": torch.zeros(heads, dim, **f32),
          "k_max": torch.full((heads, dim), float("-inf"), **f32), "v_max": torch.full((heads, dim), float("-inf"), **f32),
          "k_min": torch.full((heads, dim), float("inf"), **f32), "v_min": torch.full((heads, dim), float("inf"), **f32),
          "k_sum": torch.zeros(heads, dim, dtype=torch.float64, device=device),
          "v_sum": torch.zeros(heads, dim, dtype=torch.float64, device=device),
          "_tokens": torch.zeros(1, dtype=torch.int64, device=device)}
    return st


def record(name, key, value, slot_mapping=None):
    """Fold one step's new K/V rows of layer `name` into its running statistics (kvq/capture.py:25-56).
    key, value: bf16 [T, Hkv, D] CUDA tensors (any token / head strides); with slot_mapping (int64 [n]) only its
    first n rows with a non-negative slot count, as in the reference's hook."""
    if not key.is_cuda or key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16 or key.stride(2) != 1 or value.stride(2) != 1:
        raise RuntimeError("kvq_b200: capture expects bf16 CUDA key/value with a contiguous last dim")
    n = key.shape[0] if slot_mapping is None else slot_mapping.shape[0]
    if n == 0:
        return
    heads, dim = key.shape[1], key.shape[2]
    st = STATE["stats"].get(name)
    if st is None:
        STATE["stats"][name] = st = _new_state(heads, dim, key.device)
    slots = 0
    if slot_mapping is not None:
        if slot_mapping.dtype != torch.int64 or not slot_mapping.is_contiguous():
            raise RuntimeError("kvq_b200: slot_mapping must be contiguous int64")
        slots = slot_mapping.data_ptr()
    _native.check(_native.lib().kvq_calib_stats(
        key.data_ptr(), value.data_ptr(), slots, n, heads, dim, key.stride(0), key.stride(1), value.stride(0),
        value.stride(1), st["k_absmax"].data_ptr(), st["k_max"].data_ptr(), st["k_min"].data_ptr(), st["k_sum"].data_ptr(),
        st["v_absmax"].data_ptr(), st["v_max"].data_ptr(), st["v_min"].data_ptr(), st["v_sum"].data_ptr(),
        st["_tokens"].data_ptr(), torch.cuda.current_stream().cuda_stream))
    _sample(name, key[:n], value[:n], slot_mapping)


def _sample(name, key, value, slot_mapping):
    """Bounded sample of raw rows (kvq/capture.py:45-56): every row until half the budget is used, then a random
    eighth of each batch, nothing once the budget is full. Rows go to the CPU as fp16."""
    smp = STATE["samples"].setdefault(name, {"k": [], "v": [], "n": 0})
    if smp["n"] >= MAX_SAMPLE_TOKENS:
        return
    if slot_mapping is not None:
        valid = slot_mapping >= 0
        key, value = key[valid], value[valid]
    if key.shape[0] == 0:
        return
    if smp["n"] > MAX_SAMPLE_TOKENS // 2:
        idx = torch.randperm(key.shape[0], device=key.device)[:max(1, key.shape[0] // 8)]
        key, value = key[idx], value[idx]
    smp["k"].append(key.to(torch.float16).cpu())
    smp["v"].append(value.to(torch.float16).cpu())
    smp["n"] += key.shape[0]


def stats(name):
    """One layer's statistics as CPU tensors in the reference's layout ("tokens" is an int)."""
    st = STATE["stats"][name]
    out = {f: st[f].cpu() for f in _FIELDS}
    out["tokens"] = int(st["_tokens"].item())
    return out


def install():
    """Hook vLLM's FlashAttention backend so that every KV-cache update is recorded (kvq/capture.py:87-106).
    Enabled by the plugin when KVQ_CAPTURE=1; the model then runs on its stock bf16 cache."""
    from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl

    if not hasattr(FlashAttentionImpl, "do_kv_cache_update"):
        raise RuntimeError("kvq_b200: this vLLM version has no FlashAttentionImpl.do_kv_cache_update to hook")
    orig_update = FlashAttentionImpl.do_kv_cache_update

    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
        record(layer.layer_name, key, value, slot_mapping)
        return orig_update(self, layer, key, value, kv_cache, slot_mapping)

    FlashAttentionImpl.do_kv_cache_update = do_kv_cache_update


def collect(worker=None, tp_rank=None, tp_size=None):
    """This rank's statistics and samples for scales.merge_tp / scales.from_stats (kvq/capture.py:109-118).
    Called through LLM.collective_rpc inside vLLM (rank and world size come from vLLM then)."""
    if tp_rank is None or tp_size is None:
        from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size
        tp_rank, tp_size = get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
    out = {"stats": {name: stats(name) for name in STATE["stats"]}, "samples": {}, "dumps": {}, "tp_rank": tp_rank,
           "tp_size": tp_size}
    for name, smp in STATE["samples"].items():
        if smp["k"]:
            out["samples"][name] = {"k": torch.cat(smp["k"]), "v": torch.cat(smp["v"])}
    return out
