"""Static KV scale files: load / save, tensor-parallel sharding, and derivation from calibration statistics.

Same on-disk format as the reference (kvq/scales.py:1-6): a safetensors file whose keys are
"<layer_name>|k_scale", "<layer_name>|v_scale" and optionally "<layer_name>|k_mu"; every tensor is fp32 and
shaped [num_kv_heads_total, head_dim] (per channel) or [num_kv_heads_total, 1] (per head). A scale is the
dequantization step: x ~= q * scale.
"""
import torch
from safetensors.torch import load_file, save_file

QMAX = 127.0
SEP = "|"


def save(path, scales):
    """scales: {layer_name: {"k_scale": t, "v_scale": t[, "k_mu": t]}} (kvq/scales.py:37-38)."""
    flat = {}
    for layer, fields in scales.items():
        for field, t in fields.items():
            flat[layer + SEP + field] = t.detach().float().contiguous()
    save_file(flat, path)


def load(path, device="cpu"):
    """Inverse of save (kvq/scales.py:41-46)."""
    by_layer = {}
    for key, t in load_file(path, device=device).items():
        layer, field = key.split(SEP)
        by_layer.setdefault(layer, {})[field] = t
    return by_layer


def shard(t, tp_rank, tp_size):
    """Rows (kv heads) that tensor-parallel rank `tp_rank` owns (kvq/scales.py:49-56). With at least as many
    kv heads as ranks each rank takes a contiguous block; with fewer, heads are replicated over
    tp_size / heads consecutive ranks and the rank gets the single row of its replica group."""
    heads = t.shape[0]
    if heads >= tp_size:
        if heads % tp_size:
            raise ValueError(f"{heads} kv heads do not divide over {tp_size} ranks")
        per = heads // tp_size
        return t[tp_rank * per:(tp_rank + 1) * per]
    row = tp_rank * heads // tp_size
    return t[row:row + 1]


def for_layer(all_scales, name, tp_rank, tp_size, device):
    """This rank's slice of one layer's scales, on `device` (kvq/scales.py:78-80)."""
    return {field: shard(t, tp_rank, tp_size).to(device) for field, t in all_scales[name].items()}


def _scale_from_absmax(amax):
    return (amax / QMAX).clamp(min=1e-8)


def from_stats(st, samples=None, granularity="per_channel", method="max", smooth_k=False):
    """One layer's static scales from capture statistics (kvq/scales.py:13-34).

    st: {"tokens", "k_sum", "k_max", "k_min", "k_absmax", "v_absmax"} with [H, D] tensors. method "max" uses
    the absolute maximum; "q<fraction>" (e.g. "q0.999") a per-channel quantile over `samples` {"k", "v"}
    shaped [rows, H, D]. smooth_k removes the per-channel mean of K first and stores it as k_mu."""
    out = {}
    mu = None
    if smooth_k:
        mu = (st["k_sum"] / st["tokens"]).float()
        out["k_mu"] = mu
    for side in ("k", "v"):
        centred = side == "k" and mu is not None
        if method == "max":
            amax = torch.maximum(st["k_max"] - mu, mu - st["k_min"]) if centred else st[f"{side}_absmax"].float()
        else:
            frac = float(method[1:])
            x = samples[side].float()
            if centred:
                x = x - mu
            a = x.abs()
            kth = max(1, min(a.shape[0], int(round(frac * a.shape[0]))))
            amax = a.kthvalue(kth, dim=0).values if frac < 1.0 else a.amax(0)
        if granularity == "per_head":
            amax = amax.amax(-1, keepdim=True)
        out[f"{side}_scale"] = _scale_from_absmax(amax)
    return out


def merge_tp(per_rank, num_kv_heads):
    """Combine per-rank calibration results (kvq/scales.py:59-75): ranks hold disjoint kv heads, so statistics
    and sample rows are concatenated along heads in rank order; replicated heads keep one replica."""
    ranks = sorted(per_rank, key=lambda r: r["tp_rank"])
    if len(ranks) > num_kv_heads:
        ranks = ranks[::len(ranks) // num_kv_heads]
    if len(ranks) == 1:
        return ranks[0]["stats"], ranks[0]["samples"]
    stats, samples = {}, {}
    for layer in ranks[0]["stats"]:
        per = [r["stats"][layer] for r in ranks]
        merged = {"tokens": per[0]["tokens"]}
        for field in per[0]:
            if field != "tokens":
                merged[field] = torch.cat([p[field] for p in per], dim=0)
        stats[layer] = merged
        samples[layer] = {side: torch.cat([r["samples"][layer][side] for r in ranks], dim=1) for side in ("k", "v")}
    return stats, samples
