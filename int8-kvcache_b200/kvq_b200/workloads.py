"""Seeded synthetic inputs for the static INT8 KV-cache path.

Everything is drawn from a CPU torch.Generator so that a CPU checker and the GPU kernels see the
same bytes. Shapes and value distributions follow the benchmark configurations of this
repository: K ~ N(0, sigma_c^2) with sigma_c log-uniform per (kv head, channel) (outlier channels),
V likewise with a narrower range, static scales = absmax / 127 over the generated data, q ~ N(0, 1).
These tensors stand in for real model activations; no dataset or checkpoint is involved.
"""
import math

import torch

QMAX = 127.0


def fill_quantize(x, scale, mu=None):
    """int8 cache contents from bf16/fp32 rows with a static scale: clamp(round((x - mu) / s), +-127).
    Plain torch (any device); used to pre-fill caches for benchmarks and tests."""
    xf = x.float()
    if mu is not None:
        xf = xf - mu
    return torch.clamp(torch.round(xf / scale), -QMAX, QMAX).to(torch.int8)


def channel_sigmas(gen, hkv, d, lo, hi):
    """sigma[h, c] = exp(U[ln lo, ln hi])."""
    u = torch.rand(hkv, d, generator=gen)
    return torch.exp(math.log(lo) + u * (math.log(hi) - math.log(lo)))


def static_from_data(k_rows, v_rows, per_channel=True, smooth=False):
    """Static scales from data rows [..., Hkv, D] (stand-in for a calibration run).
    Returns {"k_scale", "v_scale", "k_mu"} as fp32 [Hkv, D] (or [Hkv, 1] per head; k_mu always [Hkv, D])."""
    k = k_rows.reshape(-1, *k_rows.shape[-2:]).float()
    v = v_rows.reshape(-1, *v_rows.shape[-2:]).float()
    mu = k.mean(0) if smooth else torch.zeros_like(k[0])
    ka, va = (k - mu).abs().amax(0), v.abs().amax(0)
    if not per_channel:
        ka, va = ka.amax(-1, keepdim=True), va.amax(-1, keepdim=True)
    return {"k_scale": (ka / QMAX).clamp(min=1e-8).contiguous(), "v_scale": (va / QMAX).clamp(min=1e-8).contiguous(),
            "k_mu": mu.contiguous()}


def paged_case(seed, hq, hkv, d, q_lens, seq_lens, block_size=16, num_blocks=None, k_sigma=(0.1, 10.0),
               v_sigma=(0.5, 2.0), per_channel=True, smooth=False, q_std=1.0):
    """One batch over a paged cache whose pages are scattered through a larger pool.

    Returns a dict of CPU tensors: q bf16 [T, Hq, D]; k, v bf16 [num_blocks, block, Hkv, D]; kq, vq int8
    (the same pool quantized with `static`); cu_seqlens_q, seq_lens int32; block_table int32 [B, max_pages]
    (unused entries point at page 0); static (fp32 scales)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    pages = [(s + block_size - 1) // block_size for s in seq_lens]
    if num_blocks is None:
        num_blocks = 2 * sum(pages) + 8
    assert num_blocks >= sum(pages)
    perm = torch.randperm(num_blocks, generator=gen).to(torch.int32)
    bt = torch.zeros(len(seq_lens), max(max(pages), 1), dtype=torch.int32)
    off = 0
    for i, p in enumerate(pages):
        bt[i, :p] = perm[off:off + p]
        off += p
    cu = torch.zeros(len(q_lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(q_lens, dtype=torch.int32), 0)
    q = (torch.randn(int(cu[-1]), hq, d, generator=gen) * q_std).to(torch.bfloat16)
    ksig = channel_sigmas(gen, hkv, d, *k_sigma)
    vsig = channel_sigmas(gen, hkv, d, *v_sigma)
    k = (torch.randn(num_blocks, block_size, hkv, d, generator=gen) * ksig).to(torch.bfloat16)
    v = (torch.randn(num_blocks, block_size, hkv, d, generator=gen) * vsig).to(torch.bfloat16)
    if smooth:   # give K a per-channel offset so that the smooth-K mean matters
        k = (k.float() + channel_sigmas(gen, hkv, d, 0.1, 3.0)).to(torch.bfloat16)
    static = static_from_data(k, v, per_channel, smooth)
    return {"q": q, "k": k, "v": v, "kq": fill_quantize(k, static["k_scale"], static["k_mu"]),
            "vq": fill_quantize(v, static["v_scale"]), "cu_seqlens_q": cu,
            "seq_lens": torch.tensor(seq_lens, dtype=torch.int32), "block_table": bt, "static": static,
            "softmax_scale": d ** -0.5, "q_lens": list(q_lens)}


def write_case(seed, tokens, hkv, d, num_blocks, block_size=16, per_channel=True, smooth=True, pad_rows=0,
               drop_every=0, k_sigma=(0.1, 10.0), v_sigma=(0.5, 2.0)):
    """New K/V rows for one step plus an injective slot mapping into a [num_blocks, block] cache.
    pad_rows extra input rows lie beyond the slot mapping; drop_every > 0 marks every n-th slot -1."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    ksig = channel_sigmas(gen, hkv, d, *k_sigma)
    vsig = channel_sigmas(gen, hkv, d, *v_sigma)
    key = (torch.randn(tokens + pad_rows, hkv, d, generator=gen) * ksig).to(torch.bfloat16)
    value = (torch.randn(tokens + pad_rows, hkv, d, generator=gen) * vsig).to(torch.bfloat16)
    if smooth:
        key = (key.float() + channel_sigmas(gen, hkv, d, 0.1, 3.0)).to(torch.bfloat16)
    slots = torch.randperm(num_blocks * block_size, generator=gen)[:tokens].long()
    if drop_every:
        slots[::drop_every] = -1
    static = static_from_data(key[:tokens], value[:tokens], per_channel, smooth)
    return {"key": key, "value": value, "slots": slots, "static": static, "num_blocks": num_blocks,
            "block_size": block_size}


def serving_lengths(seed=0, chunks=68, decodes=188):
    """(q_lens, seq_lens) of one chunked-prefill serving step: `chunks` prompt chunks of 39..73 query tokens whose
    context is the chunk plus 0..19 earlier tokens, among `decodes` single-token requests with contexts of
    100..399, in a seeded random order. Short requests between long ones are the batch shape on which a
    FlashAttention call over the whole batch must not see requests with zero keys."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    q_chunks = torch.randint(39, 74, (chunks,), generator=gen)
    ctx_chunks = q_chunks + torch.randint(0, 20, (chunks,), generator=gen)
    ctx_dec = torch.randint(100, 400, (decodes,), generator=gen)
    q = torch.cat([q_chunks, torch.ones(decodes, dtype=torch.int64)])
    ctx = torch.cat([ctx_chunks, ctx_dec])
    order = torch.randperm(chunks + decodes, generator=gen)
    return q[order].tolist(), ctx[order].tolist()


# Benchmark configurations (geometry of one Qwen2.5-7B attention layer).
HQ, HKV, D, BLOCK = 28, 4, 128, 16


def config0(seed=1000):
    """CPU-sized decode case: 4 requests, contexts 128..512, pool of 256 blocks."""
    return paged_case(seed, HQ, HKV, D, [1, 1, 1, 1], [128, 256, 384, 512], BLOCK, num_blocks=256)


def config1(seed=1001):
    """8192 new tokens into a 4096 x 16 slot cache."""
    return write_case(seed, 8192, HKV, D, num_blocks=4096, block_size=BLOCK, smooth=False)


def decode_batch_on_device(batch, ctx, device, seed=1002, q_len=1, ctx_range=None, hq=HQ, hkv=HKV, d=D,
                           block_size=BLOCK, chunk_blocks=16384, head_major=False):
    """Large decode / short-query batch built directly on `device` (the pool is several GB).

    K/V pools are generated and quantized chunk by chunk with per-chunk seeds; the static scales use the
    analytic bound 4.5 sigma_c / 127 instead of a data pass, so no bf16 copy of the pool is ever held.
    ctx_range=(lo, hi) draws per-request contexts uniformly from [lo, hi]; otherwise all are `ctx`.
    head_major=True stores each (page, head) tile contiguously (2 KB for 16 x 128 int8) instead of token-major.
    Returns the same keys as paged_case minus the bf16 pools."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    if ctx_range is not None:
        seq = torch.randint(ctx_range[0], ctx_range[1] + 1, (batch,), generator=gen).tolist()
    else:
        seq = [ctx] * batch
    pages = [(s + block_size - 1) // block_size for s in seq]
    num_blocks = sum(pages) + 1
    perm = (torch.randperm(num_blocks - 1, generator=gen) + 1).to(torch.int32)
    bt = torch.zeros(batch, max(pages), dtype=torch.int32)
    off = 0
    for i, p in enumerate(pages):
        bt[i, :p] = perm[off:off + p]
        off += p
    cu = torch.arange(0, (batch + 1) * q_len, q_len, dtype=torch.int32)
    q = torch.randn(batch * q_len, hq, d, generator=gen).to(torch.bfloat16)
    ksig = channel_sigmas(gen, hkv, d, 0.1, 10.0)
    vsig = channel_sigmas(gen, hkv, d, 0.5, 2.0)
    static = {"k_scale": (4.5 * ksig / QMAX).contiguous(), "v_scale": (4.5 * vsig / QMAX).contiguous(),
              "k_mu": torch.zeros(hkv, d)}
    if head_major:   # pages stored [block, head, slot, channel]; the kernels see the usual [block, slot, head, channel] view
        kq = torch.empty(num_blocks, hkv, block_size, d, dtype=torch.int8, device=device).transpose(1, 2)
        vq = torch.empty(num_blocks, hkv, block_size, d, dtype=torch.int8, device=device).transpose(1, 2)
    else:
        kq = torch.empty(num_blocks, block_size, hkv, d, dtype=torch.int8, device=device)
        vq = torch.empty_like(kq)
    dgen = torch.Generator(device=device)
    ks_d, vs_d = static["k_scale"].to(device), static["v_scale"].to(device)
    ksig_d, vsig_d = ksig.to(device), vsig.to(device)
    for b0 in range(0, num_blocks, chunk_blocks):
        b1 = min(num_blocks, b0 + chunk_blocks)
        dgen.manual_seed(seed * 100003 + b0)
        shape = (b1 - b0, block_size, hkv, d)
        kq[b0:b1] = fill_quantize((torch.randn(shape, generator=dgen, device=device) * ksig_d).to(torch.bfloat16), ks_d)
        vq[b0:b1] = fill_quantize((torch.randn(shape, generator=dgen, device=device) * vsig_d).to(torch.bfloat16), vs_d)
    dev = lambda t: t.to(device)  # noqa: E731
    return {"q": dev(q), "kq": kq, "vq": vq, "cu_seqlens_q": dev(cu), "seq_lens": dev(torch.tensor(seq, dtype=torch.int32)),
            "block_table": dev(bt), "static": {k: dev(v) for k, v in static.items()}, "softmax_scale": d ** -0.5,
            "q_lens": [q_len] * batch, "seq_lens_list": seq}
