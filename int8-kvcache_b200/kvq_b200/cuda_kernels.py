"""Operator API of the static INT8 KV cache on B200: the same entry points, argument order and error
behaviour as the reference's kvq/cuda_kernels.py, backed by libkvq_b200.so through its C ABI.

Attention on the INT8 cache is routed by query length, as in the reference (kvq/cuda_kernels.py:1-12):
requests with at most SHORT_Q query tokens run the INT8 tensor-core kernel; longer ones either have their pages
dequantized to a temporary bf16 paged cache that a FlashAttention kernel reads (the reference's route) or run
prefill_attention, which reads the INT8 pages directly. In a mixed batch the long path runs first and the INT8
kernel then writes the short requests' rows.

All tensors must live on the current CUDA device; work is enqueued on torch's current stream, nothing
synchronizes, and every call can be captured in a CUDA graph.
"""
import os
import warnings
from dataclasses import dataclass

import numpy as np
import torch

from . import _native

# q_len at or below SHORT_Q: INT8 kernel; above: the long-query path (kvq/cuda_kernels.py:19-21).
# The INT8 kernel handles at most KERNEL_QMAX query tokens per request, so KVQ_SHORT_Q can only lower the
# threshold: a larger value is clamped (with a warning) and requests with 9 or more query tokens always take the
# long path. Every routing decision (decode_attention, plan_long, long_attention, prefill_attention, the backend's
# CUDA-graph support level) uses this one effective value.
KERNEL_QMAX = 8


def _short_q_from_env():
    asked = int(os.environ.get("KVQ_SHORT_Q", KERNEL_QMAX))
    if asked < 1:
        raise RuntimeError(f"kvq_b200: KVQ_SHORT_Q must be at least 1, got {asked}")
    if asked > KERNEL_QMAX:
        warnings.warn(f"kvq_b200: KVQ_SHORT_Q={asked} exceeds the INT8 kernel's limit of {KERNEL_QMAX} query tokens per "
                      f"request; using {KERNEL_QMAX} (longer queries take the long-query path)", stacklevel=2)
    return min(asked, KERNEL_QMAX)


SHORT_Q = _short_q_from_env()


def ext():
    """The native library (the reference JIT-compiles here, kvq/cuda_kernels.py:26-39; ours is prebuilt)."""
    return _native.lib()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _is_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("kvq_b200: expected CUDA tensors (there is no CPU path)")


def _cache_args(cache):
    """(data_ptr, block/slot/head strides) of a [num_blocks, block, H, D] int8 view."""
    if cache.dtype != torch.int8 or cache.dim() != 4 or cache.stride(3) != 1:
        raise RuntimeError("kvq_b200: cache must be an int8 [num_blocks, block, H, D] view with a contiguous last dim")
    return cache.data_ptr(), cache.stride(0), cache.stride(1), cache.stride(2)


def _scale_flags(static_k, static_v):
    return int(static_k.shape[-1] > 1), int(static_v.shape[-1] > 1)


def _check_scale(t, name):
    if t.dtype != torch.float32 or not t.is_contiguous():
        raise RuntimeError(f"kvq_b200: {name} must be a contiguous fp32 tensor")


def quant_reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, static):
    """Fused static quantize + paged cache write (kvq/cuda_kernels.py:42-44)."""
    ks, vs, kmu = static["k_scale"], static["v_scale"], static["k_mu"]
    _is_cuda(key, value, key_cache, value_cache, slot_mapping, ks, vs, kmu)
    if key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
        raise RuntimeError("kvq_b200: key/value must be bf16")
    if key.size(2) != key_cache.size(3) or key.stride(2) != 1 or value.stride(2) != 1:
        raise RuntimeError("kvq_b200: contiguous last dim")
    if slot_mapping.dtype != torch.int64 or not slot_mapping.is_contiguous():
        raise RuntimeError("kvq_b200: slot_mapping must be contiguous int64")
    for t, n in ((ks, "k_scale"), (vs, "v_scale"), (kmu, "k_mu")):
        _check_scale(t, n)
    kc, kc_sb, kc_sn, kc_sh = _cache_args(key_cache)
    vc, vc_sb, vc_sn, vc_sh = _cache_args(value_cache)
    pk, pv = _scale_flags(ks, vs)
    _native.check(ext().kvq_quant_cache(
        key.data_ptr(), value.data_ptr(), kc, vc, slot_mapping.data_ptr(), ks.data_ptr(), vs.data_ptr(), kmu.data_ptr(),
        slot_mapping.size(0), key.size(1), key.size(2), key_cache.size(1), key.stride(0), key.stride(1), value.stride(0),
        value.stride(1), kc_sb, kc_sn, kc_sh, vc_sb, vc_sn, vc_sh, pk, pv, _stream()))


def quant_q(q, k_scale, group=None):
    """Standalone q quantization (kvq/cuda_kernels.py:47-48): returns (q_i8 [T, Hq, D], q_scale [T, Hq, D/group])."""
    _is_cuda(q, k_scale)
    group = group or q.shape[-1]
    if q.dtype != torch.bfloat16 or q.stride(2) != 1:
        raise RuntimeError("kvq_b200: q must be bf16 with a contiguous last dim")
    _check_scale(k_scale, "k_scale")
    T, hq, d = q.shape
    if d != 128 or group not in (128, 32):
        raise RuntimeError("kvq_b200: standalone q quantization: head_dim 128, group 128 or 32")
    q_i8 = torch.empty(T, hq, d, dtype=torch.int8, device=q.device)
    q_s = torch.empty(T, hq, d // group, dtype=torch.float32, device=q.device)
    _native.check(ext().kvq_quant_q(q.data_ptr(), k_scale.data_ptr(), q_i8.data_ptr(), q_s.data_ptr(), T, hq,
                                    k_scale.size(0), d, group, q.stride(0), q.stride(1), int(k_scale.shape[-1] > 1),
                                    _stream()))
    return q_i8, q_s


class _StreamWorkspaces:
    """Scratch buffers of one kernel family, one per (device, stream): calls on different streams of a device can
    overlap on the GPU, so they must not share scratch; calls on one stream are ordered by it.

    A buffer that has been handed out is never freed or replaced in place: a CUDA graph that captured a call
    replays with the buffer's raw address, whatever Python does afterwards. When a larger batch needs more, a new
    buffer is allocated and the old one is kept alive in `retired`. A buffer first needed while its stream is
    capturing is allocated inside the capture, i.e. from the graph's memory pool, and stays referenced here."""

    def __init__(self, size_fn, floor_args):
        self.size_fn, self.floor_args = size_fn, floor_args
        self.live, self.retired = {}, []

    @staticmethod
    def _key(device, stream_ptr=None):
        if not isinstance(device, torch.device):
            device = torch.device(device)   # "cuda", "cuda:1" and torch.device objects name the same buffers
        index = device.index if device.index is not None else torch.cuda.current_device()
        return index, (torch.cuda.current_stream(device).cuda_stream if stream_ptr is None else stream_ptr)

    def get(self, device, need, stream_ptr=None):
        """The buffer of (device, stream); stream_ptr: the raw handle of torch's current stream on `device` when the
        caller has looked it up already."""
        key = self._key(device, stream_ptr)
        ws = self.live.get(key)
        if ws is None or ws.numel() < need:
            if ws is not None:
                self.retired.append(ws)
            ws = torch.empty(max(need, self.size_fn(*self.floor_args)), dtype=torch.uint8, device=device)
            self.live[key] = ws
        return ws

    def peek(self, device):
        return self.live.get(self._key(device))


# sized for a generous batch (4096 requests, ~39 MB) so that it rarely grows
_WORKSPACES = _StreamWorkspaces(lambda n, d: ext().kvq_decode_workspace_size(n, d), (4096, 128))


_WORKSPACE_BYTES = {}   # (num_seqs, head_dim) -> kvq_decode_workspace_size: asked once per batch size


def decode_workspace(device, num_seqs, head_dim, stream_ptr=None):
    """Scratch of the attention kernels (work plan and split-KV partials) for torch's current stream on `device`."""
    need = _WORKSPACE_BYTES.get((num_seqs, head_dim))
    if need is None:
        need = ext().kvq_decode_workspace_size(num_seqs, head_dim)
        if need == 0:
            raise RuntimeError("kvq_b200: " + ext().kvq_last_error().decode())
        _WORKSPACE_BYTES[(num_seqs, head_dim)] = need
    return _WORKSPACES.get(device, need, stream_ptr)


# Channels per q scale inside the attention kernel: unset / 0 = one scale per (token, head) row, the reference CUDA
# kernel's numerics; 32 = the reference's q_gran="group32" accuracy option (kvq/int8_ref.py:120-130).
Q_GROUP = int(os.environ.get("KVQ_Q_GROUP", 0))


def decode_attention(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, softmax_scale, static,
                     segm=None, max_query_len=1, q_group=None):
    """INT8 attention for the requests with at most SHORT_Q query tokens; others are skipped and their rows of
    `out` left untouched (kvq/cuda_kernels.py:51-58). max_query_len bounds the short queries' length.

    `segm` (vLLM's split-KV scratch in the reference) is accepted for signature compatibility and not used:
    the kernel divides the work over the SMs itself and keeps its partial results in its own workspace.
    q_group (default: KVQ_Q_GROUP, normally unset) = 32 quantizes q with one scale per 32 channels."""
    ks, vs = static["k_scale"], static["v_scale"]
    _is_cuda(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, ks, vs)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise RuntimeError("kvq_b200: q/out must be bf16")
    if q.size(2) != k_cache.size(3) or q.stride(2) != 1 or out.stride(2) != 1:
        raise RuntimeError("kvq_b200: unsupported shape/layout")
    for t, n in ((cu_seqlens_q, "cu_seqlens_q"), (seq_lens, "seq_lens"), (block_table, "block_table")):
        if t.dtype != torch.int32:
            raise RuntimeError(f"kvq_b200: {n} must be int32")
    if block_table.stride(1) != 1 or not cu_seqlens_q.is_contiguous() or not seq_lens.is_contiguous():
        raise RuntimeError("kvq_b200: metadata tensors must be contiguous")
    _check_scale(ks, "k_scale")
    _check_scale(vs, "v_scale")
    num_seqs = cu_seqlens_q.size(0) - 1
    if num_seqs <= 0:
        return out
    kc, kc_sb, kc_sn, kc_sh = _cache_args(k_cache)
    vc, vc_sb, vc_sn, vc_sh = _cache_args(v_cache)
    pk, pv = _scale_flags(ks, vs)
    stream = torch.cuda.current_stream(q.device).cuda_stream   # looked up once: launch stream and workspace key
    ws = decode_workspace(q.device, num_seqs, q.size(2), stream)
    _native.check(ext().kvq_int8_decode_attention_qgroup(
        q.data_ptr(), kc, vc, out.data_ptr(), cu_seqlens_q.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(),
        ks.data_ptr(), vs.data_ptr(), float(softmax_scale), num_seqs, q.size(1), k_cache.size(2), q.size(2),
        k_cache.size(1), k_cache.size(0), q.stride(0), q.stride(1), out.stride(0), out.stride(1), kc_sb, kc_sn, kc_sh,
        vc_sb, vc_sn, vc_sh, block_table.stride(0), pk, pv, int(max_query_len), SHORT_Q,
        int(Q_GROUP if q_group is None else q_group), ws.data_ptr(), ws.numel(), stream))
    return out


def decode_status(device=None):
    """Debug: status word of the last attention call on `device` and torch's current stream (0 = clean).
    Synchronizes the stream."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    ws = _WORKSPACES.peek(device)
    if ws is None:
        return 0
    import ctypes

    status = ctypes.c_int(0)
    _native.check(ext().kvq_decode_status(ws.data_ptr(), ctypes.byref(status), _stream()))
    return status.value


@dataclass
class LongPlan:
    """Temporary bf16 paged cache for the long-query requests of one step (kvq/cuda_kernels.py:61-77). Built on
    the host by the metadata builder; device copies are made lazily by the first layer's forward."""
    src_req: np.ndarray         # [P] request of temporary page p
    src_j: np.ndarray           # [P] index of temporary page p among that request's pages
    block_table: np.ndarray     # [num_reqs, max_pages] page table of the temporary cache
    max_seqlen_k: int           # from the host-side (possibly optimistic) lengths
    has_short: bool             # any request left for the INT8 kernel
    block_size: int             # page size of both caches
    _gpu: tuple = None

    def gpu(self, device):
        if self._gpu is None:
            self._gpu = tuple(torch.from_numpy(a).to(device) for a in (self.src_req, self.src_j, self.block_table))
        return self._gpu


FA_TILE = 256  # FlashAttention looks up pages for a whole KV tile, also past the last key


def plan_long(query_start_loc_cpu, seq_lens_cpu, block_size):
    """Page table of the temporary cache, or None when no request has more than SHORT_Q query tokens
    (kvq/cuda_kernels.py:80-103). Host-side lengths may be upper bounds: they only size the copy."""
    starts = np.asarray(query_start_loc_cpu, dtype=np.int64)
    n = starts.shape[0] - 1
    q_lens = starts[1:] - starts[:-1]
    is_long = q_lens > SHORT_Q
    if not bool(is_long.any()):
        return None
    ctx = np.asarray(seq_lens_cpu, dtype=np.int64)[:n]
    n_pages = np.where(is_long, (ctx + block_size - 1) // block_size, 0)
    total = int(n_pages.sum())
    first = np.cumsum(n_pages) - n_pages                      # first temporary page of each request
    src_req = np.repeat(np.arange(n, dtype=np.int32), n_pages)
    src_j = (np.arange(total, dtype=np.int64) - first[src_req]).astype(np.int32)
    # one FlashAttention KV tile of slack; the extra entries (and short requests' rows) point at temporary page 0
    table = np.zeros((n, int(n_pages.max()) + (FA_TILE + block_size - 1) // block_size), dtype=np.int32)
    table[src_req, src_j] = np.arange(total, dtype=np.int32)
    return LongPlan(src_req=src_req, src_j=src_j, block_table=table, max_seqlen_k=int(ctx[is_long].max()),
                    has_short=bool((q_lens[~is_long] > 0).any()), block_size=int(block_size))


def dequant_pages(k_cache, v_cache, k_out, v_out, block_table, src_req, src_j, static):
    """Copy pages block_table[src_req[p], src_j[p]] of the INT8 cache into contiguous bf16 pages
    (the reference's ext().dequant_pages, kvq/cuda/int8_kv.cu:650-672)."""
    ks, vs = static["k_scale"], static["v_scale"]
    _is_cuda(k_cache, v_cache, k_out, v_out, block_table, src_req, src_j, ks, vs)
    if not (k_out.is_contiguous() and v_out.is_contiguous()) or src_j.size(0) != src_req.size(0):
        raise RuntimeError("kvq_b200: layout")
    if k_out.dtype != torch.bfloat16 or v_out.dtype != torch.bfloat16:
        raise RuntimeError("kvq_b200: temporary pages must be bf16")
    for t in (block_table, src_req, src_j):
        if t.dtype != torch.int32:
            raise RuntimeError("kvq_b200: page tables must be int32")
    _check_scale(ks, "k_scale")
    _check_scale(vs, "v_scale")
    kc, kc_sb, kc_sn, kc_sh = _cache_args(k_cache)
    vc, vc_sb, vc_sn, vc_sh = _cache_args(v_cache)
    pk, pv = _scale_flags(ks, vs)
    _native.check(ext().kvq_dequant_pages(
        kc, vc, k_out.data_ptr(), v_out.data_ptr(), block_table.data_ptr(), src_req.data_ptr(), src_j.data_ptr(),
        ks.data_ptr(), vs.data_ptr(), src_req.size(0), k_cache.size(2), k_cache.size(3), k_cache.size(1), kc_sb, kc_sn,
        kc_sh, vc_sb, vc_sn, vc_sh, block_table.stride(0), pk, pv, _stream()))


def _flash_attn_varlen():
    """Paged varlen FlashAttention for the long-query path: vLLM's fork (page size 16), as the reference uses."""
    try:
        from vllm.v1.attention.backends.fa_utils import flash_attn_varlen_func, get_flash_attn_version
        return flash_attn_varlen_func, get_flash_attn_version()
    except Exception:  # noqa: BLE001
        from vllm.vllm_flash_attn import flash_attn_varlen_func
        return flash_attn_varlen_func, 2


def long_attention(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, max_query_len, plan, softmax_scale,
                   static):
    """Dequantize the long requests' pages, then FlashAttention over the whole batch
    (kvq/cuda_kernels.py:106-131). Short requests read as many keys as they have query tokens from temporary
    page 0 there (a row with zero keys makes FlashAttention-2 write out of bounds) and are overwritten by
    decode_attention afterwards."""
    fa, fa_version = _flash_attn_varlen()
    bs, h, d = k_cache.shape[1:]
    assert bs == plan.block_size, (bs, plan.block_size)
    src_req, src_j, tmp_bt = plan.gpu(q.device)
    q_lens = cu_seqlens_q[1:] - cu_seqlens_q[:-1]
    seqused_k = torch.where(q_lens > SHORT_Q, seq_lens[:q_lens.shape[0]], q_lens).to(torch.int32)
    kt = torch.empty(src_req.shape[0], bs, h, d, dtype=q.dtype, device=q.device)
    vt = torch.empty_like(kt)
    dequant_pages(k_cache, v_cache, kt, vt, block_table, src_req, src_j, static)
    fa(q=q, k=kt, v=vt, out=out, cu_seqlens_q=cu_seqlens_q, max_seqlen_q=max_query_len, seqused_k=seqused_k,
       max_seqlen_k=plan.max_seqlen_k, softmax_scale=softmax_scale, causal=True, block_table=tmp_bt,
       fa_version=fa_version)
    return out


_PREFILL_WS = _StreamWorkspaces(lambda n: ext().kvq_prefill_workspace_size(n), (4096,))


def prefill_attention(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, softmax_scale, static,
                      min_query_len=None):
    """Causal attention for the requests with more than SHORT_Q query tokens, read straight from the INT8 pages
    (tcgen05 tensor-core kernel; no temporary bf16 cache, no plan). Requests with at most SHORT_Q query tokens are
    skipped and their rows of `out` left untouched. Same result as long_attention up to bf16/fp16 rounding:
    q against K = k_i8 * k_scale, V = v_i8 * v_scale ("implementation A", kvq/int8_ref.py:62-91).

    min_query_len (default SHORT_Q) moves the threshold: 0 serves every request, decode included, with
    implementation A numerics (unquantized q and P; the reference's A_* configurations, kvq/int8_ref.py:201-222). That
    is an accuracy reference for the INT8 kernel, not a fast path: single-token queries fill 7 of a tile's 128 rows."""
    ks, vs = static["k_scale"], static["v_scale"]
    _is_cuda(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, ks, vs)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise RuntimeError("kvq_b200: q/out must be bf16")
    if q.size(2) != k_cache.size(3) or q.stride(2) != 1 or out.stride(2) != 1:
        raise RuntimeError("kvq_b200: unsupported shape/layout")
    for t, n in ((cu_seqlens_q, "cu_seqlens_q"), (seq_lens, "seq_lens"), (block_table, "block_table")):
        if t.dtype != torch.int32:
            raise RuntimeError(f"kvq_b200: {n} must be int32")
    if block_table.stride(1) != 1 or not cu_seqlens_q.is_contiguous() or not seq_lens.is_contiguous():
        raise RuntimeError("kvq_b200: metadata tensors must be contiguous")
    _check_scale(ks, "k_scale")
    _check_scale(vs, "v_scale")
    num_seqs = cu_seqlens_q.size(0) - 1
    if num_seqs <= 0 or q.size(0) == 0:
        return out
    kc, kc_sb, kc_sn, kc_sh = _cache_args(k_cache)
    vc, vc_sb, vc_sn, vc_sh = _cache_args(v_cache)
    pk, pv = _scale_flags(ks, vs)
    ws = _PREFILL_WS.get(q.device, ext().kvq_prefill_workspace_size(num_seqs))
    _native.check(ext().kvq_int8_prefill_attention(
        q.data_ptr(), kc, vc, out.data_ptr(), cu_seqlens_q.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(),
        ks.data_ptr(), vs.data_ptr(), float(softmax_scale), num_seqs, q.size(0), q.size(1), k_cache.size(2), q.size(2),
        k_cache.size(1), k_cache.size(0), q.stride(0), q.stride(1), out.stride(0), out.stride(1), kc_sb, kc_sn, kc_sh,
        vc_sb, vc_sn, vc_sh, block_table.stride(0), pk, pv, SHORT_Q if min_query_len is None else int(min_query_len),
        ws.data_ptr(), ws.numel(), _stream()))
    return out


def prefill_status(device=None):
    """Debug: status word of the last prefill_attention call on `device` (0 = clean). Synchronizes the stream."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    ws = _PREFILL_WS.peek(device)
    if ws is None:
        return 0
    torch.cuda.current_stream(device).synchronize()
    return int(ws[:4].view(torch.int32).item())


def check_inputs(q, k_cache, cu_seqlens_q, seq_lens, block_table, plan):
    """KVQ_DEBUG=1: host-side bounds checks of one batch before the kernels run; raises
    RuntimeError("kvq input check: ...") like the reference (kvq/cuda_kernels.py:134-169). Synchronizes, so it
    is skipped while a CUDA graph is being captured."""
    if q.is_cuda and torch.cuda.is_current_stream_capturing():
        return
    starts = cu_seqlens_q.cpu().numpy().astype(np.int64)
    ctx = seq_lens.cpu().numpy().astype(np.int64)
    table = block_table.cpu().numpy().astype(np.int64)
    num_blocks, bs = k_cache.shape[:2]
    n = starts.shape[0] - 1
    q_lens = starts[1:] - starts[:-1]
    problems = []
    if starts[-1] > q.shape[0]:
        problems.append(f"cu_seqlens_q[-1] {int(starts[-1])} > {q.shape[0]} query rows")
    if ctx.shape[0] < n or table.shape[0] < n:
        problems.append(f"seq_lens {ctx.shape[0]} / block_table {tuple(table.shape)} rows < {n} requests")
    else:
        for r in np.nonzero(q_lens > 0)[0].tolist():
            L, ql = int(ctx[r]), int(q_lens[r])
            pages = (L + bs - 1) // bs
            if L < ql:
                problems.append(f"req {r}: seq_len {L} < q_len {ql}")
            if pages > table.shape[1]:
                problems.append(f"req {r}: {pages} pages > block_table width {table.shape[1]}")
            elif pages and (table[r, :pages].min() < 0 or table[r, :pages].max() >= num_blocks):
                problems.append(f"req {r} (q_len {ql}, seq_len {L}): page ids {table[r, :pages].tolist()[:8]}... "
                                f"outside [0, {num_blocks})")
        if plan is not None:
            ids = table[plan.src_req.astype(np.int64), plan.src_j.astype(np.int64)]
            if ids.size and (ids.min() < 0 or ids.max() >= num_blocks):
                problems.append(f"pages to dequantize outside [0, {num_blocks})")
            copied = np.bincount(plan.src_req, minlength=n)[:n]
            short = np.nonzero((q_lens > SHORT_Q) & (copied * bs < ctx[:n]))[0].tolist()
            if short:
                r = short[0]
                problems.append(f"{len(short)} long requests with fewer copied pages than keys, e.g. req {r}: "
                                f"{int(copied[r])} pages for {int(ctx[r])} keys")
    if problems:
        raise RuntimeError("kvq input check: " + "; ".join(problems[:8]))


# Longest query for which the INT8-page kernel is the default long path when FlashAttention is also available.
# Measured on B200 (Qwen2.5-7B layer shape): 16 requests x 64 query tokens over 4096 keys 0.13 ms against 0.23 ms
# for dequantize + FlashAttention; 32 x 512 over 512 keys 0.33 against 0.32 ms; 4 x 2048 over 8192 1.10 against 0.84.
INT8_LONG_MAX_Q = int(os.environ.get("KVQ_INT8_LONG_MAX_Q", 256))


def long_path(max_query_len=None):
    """Which kernel serves long queries: "int8" (prefill_attention: reads the INT8 pages directly, needs nothing
    outside this package, no temporary cache) or "fa" (dequantize + vLLM's paged FlashAttention, as the reference
    does). The environment variable KVQ_LONG_PATH picks one; by default ("auto") the INT8-page kernel serves
    batches whose longest query has at most INT8_LONG_MAX_Q tokens (chunked prefill, where it is the faster of
    the two), and every batch when vLLM's kernel cannot be imported; larger prefills go to FlashAttention."""
    choice = os.environ.get("KVQ_LONG_PATH", "auto")
    if choice in ("int8", "fa"):
        return choice
    if choice != "auto":
        raise RuntimeError(f"kvq_b200: KVQ_LONG_PATH must be int8, fa or auto, got {choice!r}")
    if max_query_len is not None and max_query_len <= INT8_LONG_MAX_Q:
        return "int8"
    global _FA_IMPORTABLE
    if _FA_IMPORTABLE is None:
        try:
            _flash_attn_varlen()
            _FA_IMPORTABLE = True
        except Exception:  # noqa: BLE001
            _FA_IMPORTABLE = False
    return "fa" if _FA_IMPORTABLE else "int8"


_FA_IMPORTABLE = None


def paged_attention(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, max_query_len, softmax_scale,
                    static, plan=None, segm=None):
    """Both paths for one batch, as the backend runs them (kvq/cuda_kernels.py:172-183); plan from plan_long,
    None if every request is short. The long requests go to long_attention or prefill_attention (see long_path)."""
    if os.environ.get("KVQ_DEBUG") == "1":
        check_inputs(q, k_cache, cu_seqlens_q, seq_lens, block_table, plan)
    if plan is not None:
        if long_path(max_query_len) == "int8":
            prefill_attention(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, softmax_scale, static)
        else:
            long_attention(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, max_query_len, plan,
                           softmax_scale, static)
    if plan is None or plan.has_short:
        decode_attention(q, k_cache, v_cache, out, cu_seqlens_q, seq_lens, block_table, softmax_scale, static, segm,
                         max_query_len)
    return out
