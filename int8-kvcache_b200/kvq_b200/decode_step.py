"""A caller of the hot path: one decode step of a Qwen2.5-7B-geometry decoder with an int8_static paged KV cache.

Random-initialised bf16 weights (no checkpoint), library kernels for everything that is not the KV path (embedding,
fused RMSNorm, QKV / output / MLP GEMMs through cuBLAS with the residual adds in their epilogues, RoPE and SwiGLU
through vLLM's fused ops where vLLM is importable and plain torch otherwise, greedy sampling); per layer the new K/V go
through `quant_reshape_and_cache` and attention through `decode_attention`. The whole step is captured in one CUDA graph.
This is benchmark scaffolding for "decode tokens/s on N GPUs with requests sharded": every rank holds the full
weights and its own requests and pages; there is no collective inside the step.
"""
import math

import torch
import torch.nn.functional as F

from . import cuda_kernels as ck


def _library_ops():
    """vLLM's fused elementwise kernels (in-place rotary embedding, silu-and-mul), or None where vLLM is not there."""
    try:
        import vllm._custom_ops as ops   # noqa: F401  (registers torch.ops._C)

        return ops if hasattr(torch.ops, "_C") and hasattr(torch.ops._C, "silu_and_mul") else None
    except Exception:  # noqa: BLE001
        return None

QWEN25_7B = dict(layers=28, hidden=3584, hq=28, hkv=4, head_dim=128, mlp=18944, vocab=152064, rope_theta=1e6,
                 rms_eps=1e-6)


class DecodeStep:
    def __init__(self, device, batch, ctx, block_size=16, seed=0, geometry=None, cache_fill_chunk=1 << 28):
        g = dict(QWEN25_7B, **(geometry or {}))
        self.g, self.device, self.batch, self.ctx, self.block = g, device, batch, ctx, block_size
        gen = torch.Generator(device=device).manual_seed(seed)
        L, H, hq, hkv, d, mlp = g["layers"], g["hidden"], g["hq"], g["hkv"], g["head_dim"], g["mlp"]

        def w(*shape, std=0.02):
            return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std).to(torch.bfloat16)

        self.embed, self.lm_head = w(g["vocab"], H), w(H, g["vocab"])
        self.final_norm = torch.ones(H, dtype=torch.bfloat16, device=device)
        self.layers = []
        for _ in range(L):
            self.layers.append(dict(
                ln1=torch.ones(H, dtype=torch.bfloat16, device=device), ln2=torch.ones(H, dtype=torch.bfloat16, device=device),
                wqkv=w(H, (hq + 2 * hkv) * d), bqkv=w((hq + 2 * hkv) * d), wo=w(hq * d, H), wgu=w(H, 2 * mlp),
                wdown=w(mlp, H),
                static={"k_scale": torch.rand(hkv, d, generator=gen, device=device) * 0.05 + 0.01,
                        "v_scale": torch.rand(hkv, d, generator=gen, device=device) * 0.02 + 0.005,
                        "k_mu": torch.randn(hkv, d, generator=gen, device=device) * 0.1}))
        # paged int8 cache: room for ctx + 1 tokens per request, pages randomly permuted, contents random bytes
        pages = (ctx + 1 + block_size - 1) // block_size
        self.num_blocks = batch * pages + 1
        self.kv = torch.empty(L, 2, self.num_blocks, block_size, hkv, d, dtype=torch.int8, device=device)
        flat = self.kv.view(-1)
        for s in range(0, flat.numel(), cache_fill_chunk):
            n = min(cache_fill_chunk, flat.numel() - s)
            flat[s:s + n] = torch.randint(-127, 128, (n,), generator=gen, device=device, dtype=torch.int8)
        perm = (torch.randperm(self.num_blocks - 1, generator=gen, device=device) + 1).to(torch.int32)
        self.block_table = perm[:batch * pages].view(batch, pages).contiguous()
        self.seq_lens = torch.full((batch,), ctx + 1, dtype=torch.int32, device=device)   # including the new token
        self.positions = torch.full((batch,), ctx, dtype=torch.int64, device=device)
        self.slots = (self.block_table[:, ctx // block_size].long() * block_size + ctx % block_size).contiguous()
        self.cu = torch.arange(batch + 1, dtype=torch.int32, device=device)
        inv = 1.0 / (g["rope_theta"] ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
        ang = self.positions.float()[:, None] * inv[None]
        self.cos, self.sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        self.ops = _library_ops()
        # rotary table for the fused op: row p = [cos(p * inv) | sin(p * inv)]; every request sits at position ctx
        table = torch.arange(ctx + 1, device=device, dtype=torch.float32)[:, None] * inv[None]
        self.cos_sin = torch.cat([table.cos(), table.sin()], -1).to(torch.bfloat16)
        self.tokens = torch.randint(0, g["vocab"], (batch,), generator=gen, device=device)
        self.next_tokens = torch.zeros_like(self.tokens)
        self.attn_out = torch.empty(batch, hq, d, dtype=torch.bfloat16, device=device)
        self.graph = None
        self.trace = None   # set to a list before an eager forward() to keep every layer's (q, k, v, attn_out)

    def kv_bytes_per_step(self):
        g = self.g
        return self.batch * (self.ctx + 1) * g["hkv"] * g["head_dim"] * 2 * g["layers"]

    def weight_bytes(self):
        return sum(t.numel() * 2 for l in self.layers for k, t in l.items() if k != "static") + \
            self.lm_head.numel() * 2

    def _rms(self, x, weight):
        return F.rms_norm(x, (x.shape[-1],), weight, self.g["rms_eps"])

    def _rope(self, x):   # x [B, heads, D], rotate-half convention
        d = x.shape[-1]
        x1, x2 = x[..., :d // 2].float(), x[..., d // 2:].float()
        return torch.cat([x1 * self.cos - x2 * self.sin, x2 * self.cos + x1 * self.sin], -1).to(torch.bfloat16)

    def forward(self):
        g = self.g
        hq, hkv, d = g["hq"], g["hkv"], g["head_dim"]
        x = self.embed[self.tokens]
        scale = 1.0 / math.sqrt(d)
        for i, l in enumerate(self.layers):
            qkv = torch.addmm(l["bqkv"], self._rms(x, l["ln1"]), l["wqkv"])
            if self.ops is not None:   # rotate q and k in place inside the fused activation
                self.ops.rotary_embedding(self.positions, qkv[:, :hq * d], qkv[:, hq * d:(hq + hkv) * d], d, self.cos_sin, True)
                qkv = qkv.view(self.batch, hq + 2 * hkv, d)
                q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
            else:
                qkv = qkv.view(self.batch, hq + 2 * hkv, d)
                qk = self._rope(qkv[:, :hq + hkv])
                q, k, v = qk[:, :hq], qk[:, hq:], qkv[:, hq + hkv:]
            kc, vc = self.kv[i, 0], self.kv[i, 1]
            ck.quant_reshape_and_cache(k, v, kc, vc, self.slots, l["static"])
            ck.decode_attention(q, kc, vc, self.attn_out, self.cu, self.seq_lens, self.block_table, scale, l["static"])
            if self.trace is not None:
                self.trace.append(dict(q=q.clone(), k=k.clone(), v=v.clone(), attn_out=self.attn_out.clone()))
            x = torch.addmm(x, self.attn_out.view(self.batch, hq * d), l["wo"])
            gu = self._rms(x, l["ln2"]) @ l["wgu"]
            if self.ops is not None:
                act = torch.empty(self.batch, g["mlp"], dtype=gu.dtype, device=gu.device)
                torch.ops._C.silu_and_mul(act, gu)
            else:
                act = F.silu(gu[:, :g["mlp"]]) * gu[:, g["mlp"]:]
            x = torch.addmm(x, act, l["wdown"])
        logits = self._rms(x, self.final_norm) @ self.lm_head
        self.next_tokens.copy_(logits.argmax(-1))
        return self.next_tokens

    def capture(self):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.forward()
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.forward()
        return self

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.forward()
        return self.next_tokens
