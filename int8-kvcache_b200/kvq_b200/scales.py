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
        if all(layer in r["samples"] for r in ranks):   # sampled rows are optional (quantile scales only)
            samples[layer] = {side: torch.cat([r["samples"][layer][side] for r in ranks], dim=1) for side in ("k", "v")}
    return stats, samples


# The scale-file variants a calibration run writes, as (granularity, method, smooth_k)
# (the six of the reference's scripts/calibrate.py:23-26).
CALIBRATION_VARIANTS = (("per_channel", "max", False), ("per_channel", "max", True), ("per_channel", "q0.999", True),
                        ("per_channel", "q0.9999", True), ("per_head", "max", False), ("per_head", "max", True))


def variant_file_name(prefix, granularity, method, smooth_k):
    """<prefix>_<granularity>_<method>[_smooth].safetensors, the naming of the reference's scale files
    (e.g. math_per_channel_max_smooth.safetensors)."""
    return f"{prefix}_{granularity}_{method}{'_smooth' if smooth_k else ''}.safetensors"


def calibrate_from(per_rank, num_kv_heads, out_dir, prefix="calib", variants=CALIBRATION_VARIANTS):
    """From what every tensor-parallel rank's capture.collect() returned to one scale file per variant in out_dir
    (the second half of the reference's scripts/calibrate.py:59-76; the first half, running a calibration set through
    the engine with KVQ_CAPTURE=1, belongs to the serving stack). Quantile variants need the sampled rows and are
    skipped for layers without samples. Returns {"tokens": rows seen by the first layer, "variants": [file names]}."""
    import os

    stats, samples = merge_tp(per_rank, num_kv_heads)
    if not stats:
        raise ValueError("calibrate_from: the capture holds no layer statistics (was KVQ_CAPTURE=1 set before the run?)")
    os.makedirs(out_dir, exist_ok=True)
    written = []
    for granularity, method, smooth_k in variants:
        needs_samples = method != "max"
        if needs_samples and any(name not in samples for name in stats):
            continue
        layer_scales = {name: from_stats(stats[name], samples.get(name), granularity, method, smooth_k) for name in stats}
        name = variant_file_name(prefix, granularity, method, smooth_k)
        save(os.path.join(out_dir, name), layer_scales)
        written.append(name)
    return {"tokens": int(next(iter(stats.values()))["tokens"]), "variants": written}
