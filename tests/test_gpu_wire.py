"""Raw int8 pages as a transfer format (prefill / decode disaggregation), and implementation-A numerics for decode.

A sender's pages are exported to a contiguous buffer, imported into a receiver's cache that uses other page ids and
another memory layout, and attention on the receiver must give the sender's output bit for bit: the int8 bytes are
all that travels, both sides hold the same static scales (reference: docs/LOG.md:614-633)."""
import numpy as np
import pytest
import torch
from gpu_util import DEV, assert_close, oracle_attention, run_decode, to_dev

from kvq_b200 import cuda_kernels as ck
from kvq_b200 import wire, workloads
from oracle import kvq_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,block_size", [(128, 16), (64, 32)])
def test_pages_cross_the_wire_unchanged(d, block_size):
    case = workloads.paged_case(80 + d, 28 if d == 128 else 14, 4 if d == 128 else 2, d, [1, 3, 1, 8], [700, 90, 33, 1024],
                                block_size=block_size, smooth=True, q_std=2.0)
    hkv = case["kq"].shape[2]
    static = to_dev(case["static"])
    # sender: vLLM-style interleaved K|V cache
    kv = torch.cat([case["kq"], case["vq"]], dim=-1).to(DEV)
    k_src, v_src = kv.split(d, dim=-1)
    bt = case["block_table"]
    lens = case["seq_lens"].tolist()
    send_ids = torch.cat([bt[r, :(lens[r] + block_size - 1) // block_size] for r in range(len(lens))])
    payload = wire.export_pages(k_src, v_src, send_ids)
    assert payload.shape == (send_ids.numel(), 2, block_size, hkv, d) and payload.dtype == torch.int8
    assert torch.equal(payload[:, 0].cpu(), case["kq"][send_ids.long()]) and torch.equal(payload[:, 1].cpu(), case["vq"][send_ids.long()])
    meta = wire.header("model.layers.0.self_attn.attn", sum(lens), send_ids.numel(), block_size, hkv, d, static)
    assert wire.check_header(meta, block_size, hkv, d, static)["bytes"] == payload.numel()
    with pytest.raises(RuntimeError, match="other static scales"):
        wire.check_header(meta, block_size, hkv, d, dict(static, v_scale=static["v_scale"] * 2))

    # receiver: separate head-major K and V pools, its own page numbering
    nb = send_ids.numel() + 5
    k_dst = torch.full((nb, hkv, block_size, d), 99, dtype=torch.int8, device=DEV).transpose(1, 2)
    v_dst = torch.full((nb, hkv, block_size, d), 99, dtype=torch.int8, device=DEV).transpose(1, 2)
    recv_ids = torch.randperm(nb, generator=torch.Generator().manual_seed(1))[:send_ids.numel()].to(torch.int32)
    wire.import_pages(payload, k_dst, v_dst, recv_ids)
    assert torch.equal(k_dst[recv_ids.long()].cpu(), case["kq"][send_ids.long()])
    untouched = torch.ones(nb, dtype=torch.bool)
    untouched[recv_ids.long()] = False
    assert (k_dst[untouched.to(DEV)] == 99).all() and (v_dst[untouched.to(DEV)] == 99).all()

    recv_bt = torch.zeros_like(bt)
    off = 0
    for r, L in enumerate(lens):
        n = (L + block_size - 1) // block_size
        recv_bt[r, :n] = recv_ids[off:off + n]
        off += n
    want = run_decode(case)
    q = case["q"].to(DEV)
    out = torch.zeros_like(q)
    ck.decode_attention(q, k_dst, v_dst, out, case["cu_seqlens_q"].to(DEV), case["seq_lens"].to(DEV), recv_bt.to(DEV),
                        case["softmax_scale"], static, max_query_len=max(case["q_lens"]))
    torch.cuda.synchronize()
    assert np.array_equal(out.float().cpu().numpy(), want)
    assert_close(oracle_attention(case), want, "sender output")
    wire.export_pages(k_src, v_src, send_ids[:0])     # nothing to send: a no-op


def test_implementation_a_for_decode_and_short_queries():
    """prefill_attention with min_query_len = 0 serves every request with implementation A numerics (bf16 q against
    dequantized K/V, no q or P quantization): checked against the oracle's implementation A with unrounded dequantized
    K/V (the quantity a kernel reading the int8 pages computes; bound as in the long-query tests)."""
    case = workloads.paged_case(85, 28, 4, 128, [1, 1, 4, 8, 1, 20], [300, 33, 513, 1000, 16, 150], smooth=True, q_std=2.0)
    ref = oracle_attention(case, short_q=0, long_kv_bf16=False)
    q = case["q"].to(DEV)
    out = torch.zeros_like(q)
    ck.prefill_attention(q, case["kq"].to(DEV), case["vq"].to(DEV), out, case["cu_seqlens_q"].to(DEV),
                         case["seq_lens"].to(DEV), case["block_table"].to(DEV), case["softmax_scale"],
                         to_dev(case["static"]), min_query_len=0)
    torch.cuda.synchronize()
    assert ck.prefill_status() == 0
    assert orc.compare(ref, out.float().cpu().numpy())["rel_l2"] < 3e-3
