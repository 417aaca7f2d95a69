"""Raw int8 KV pages as a transfer format between a prefill and a decode instance.

With static scales the int8 bytes of a page are all there is to send: the receiving side quantized nothing, holds the
same scale file, and attends over the received pages exactly as the sender would (the reference measured this with
vLLM's KV connector, docs/LOG.md:614-633: half the bytes of a bf16 transfer, same accuracy). This module is the data
path either side of such a connector, per layer:

    sender:    wire = export_pages(k_cache, v_cache, page_ids)        # [P, 2, block, H, D] int8, contiguous
    transport: any byte mover (NCCL send/recv, NIXL, a file)          # header(...) describes the payload
    receiver:  import_pages(wire, k_cache, v_cache, page_ids)         # own page ids, own cache layout

Bytes per token and layer: 2 * H * D (1024 for 4 kv heads of 128 channels; a 28-layer model moves 28,672 bytes per
token against 57,344 in bf16). The scales do not travel; header() carries a digest of them so that a receiver
calibrated differently refuses the pages instead of attending with the wrong scales.
"""
import hashlib
import json

import torch

from . import _native
from .cuda_kernels import _cache_args, _is_cuda, _stream

FORMAT = "kvq-int8-static-pages/1"


def _ids(page_ids, device):
    ids = torch.as_tensor(page_ids, dtype=torch.int32, device=device)
    if ids.dim() != 1:
        raise RuntimeError("kvq_b200: page_ids must be one-dimensional")
    return ids.contiguous()


def export_pages(k_cache, v_cache, page_ids, out=None):
    """Gather pages `page_ids` of one layer's int8 cache ([num_blocks, block, H, D] views, any strides) into a contiguous
    int8 tensor [P, 2, block, H, D] (K then V per page). `out` may be a preallocated buffer of that shape."""
    _is_cuda(k_cache, v_cache)
    kc, kc_sb, kc_sn, kc_sh = _cache_args(k_cache)
    vc, vc_sb, vc_sn, vc_sh = _cache_args(v_cache)
    ids = _ids(page_ids, k_cache.device)
    _, bs, h, d = k_cache.shape
    shape = (ids.numel(), 2, bs, h, d)
    if out is None:
        out = torch.empty(shape, dtype=torch.int8, device=k_cache.device)
    elif tuple(out.shape) != shape or out.dtype != torch.int8 or not out.is_contiguous():
        raise RuntimeError(f"kvq_b200: wire buffer must be a contiguous int8 tensor of shape {shape}")
    _native.check(_native.lib().kvq_pages_to_wire(kc, vc, out.data_ptr(), ids.data_ptr(), ids.numel(), h, d, bs, kc_sb, kc_sn,
                                                  kc_sh, vc_sb, vc_sn, vc_sh, _stream()))
    return out


def import_pages(wire, k_cache, v_cache, page_ids):
    """Scatter a wire buffer [P, 2, block, H, D] into pages `page_ids` of the receiving layer's int8 cache."""
    _is_cuda(wire, k_cache, v_cache)
    kc, kc_sb, kc_sn, kc_sh = _cache_args(k_cache)
    vc, vc_sb, vc_sn, vc_sh = _cache_args(v_cache)
    ids = _ids(page_ids, k_cache.device)
    _, bs, h, d = k_cache.shape
    if tuple(wire.shape) != (ids.numel(), 2, bs, h, d) or wire.dtype != torch.int8 or not wire.is_contiguous():
        raise RuntimeError(f"kvq_b200: wire buffer {tuple(wire.shape)} does not match {ids.numel()} pages of "
                           f"[2, {bs}, {h}, {d}] int8")
    _native.check(_native.lib().kvq_wire_to_pages(wire.data_ptr(), kc, vc, ids.data_ptr(), ids.numel(), h, d, bs, kc_sb, kc_sn,
                                                  kc_sh, vc_sb, vc_sn, vc_sh, _stream()))


def scales_digest(static):
    """sha256 over a layer's k_scale, v_scale and k_mu bytes (fp32, in that order)."""
    h = hashlib.sha256()
    for name in ("k_scale", "v_scale", "k_mu"):
        h.update(static[name].detach().float().contiguous().cpu().numpy().tobytes())
    return h.hexdigest()


def header(layer_name, num_tokens, num_pages, block_size, num_kv_heads, head_dim, static):
    """JSON description of one layer's payload (num_pages pages holding num_tokens tokens; every request's last page
    may be partly filled); check_header() on the receiving side."""
    pages = int(num_pages)
    return json.dumps({"format": FORMAT, "layer": layer_name, "tokens": int(num_tokens), "pages": int(pages),
                       "block_size": int(block_size), "num_kv_heads": int(num_kv_heads), "head_dim": int(head_dim),
                       "dtype": "int8", "bytes": int(pages * 2 * block_size * num_kv_heads * head_dim),
                       "scales_sha256": scales_digest(static)}).encode()


def check_header(raw, block_size, num_kv_heads, head_dim, static):
    """Parsed header if the payload fits this cache and was quantized with the scales this side holds."""
    h = json.loads(raw)
    if h.get("format") != FORMAT:
        raise RuntimeError(f"kvq_b200: unknown KV wire format {h.get('format')!r}")
    want = {"block_size": block_size, "num_kv_heads": num_kv_heads, "head_dim": head_dim}
    for key, value in want.items():
        if h[key] != value:
            raise RuntimeError(f"kvq_b200: KV pages for {key}={h[key]}, this cache has {value}")
    if h["scales_sha256"] != scales_digest(static):
        raise RuntimeError("kvq_b200: the sender quantized with other static scales than this side holds")
    return h
