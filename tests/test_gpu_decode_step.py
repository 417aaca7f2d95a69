"""The full decode step (benchmark configuration 4's harness, kvq_b200/decode_step.py) at a size the CPU oracle can
follow: a 2-layer decoder of the same layer geometry, 4 requests. After one eager step, the bytes each layer wrote
into its int8 cache equal the oracle's quantization of that layer's new K/V rows, and each layer's attention output
meets the attention bar against the oracle run on the same cache; the captured graph then reproduces the eager
step's tokens."""
import numpy as np
import pytest
import torch
from gpu_util import DEV, assert_close

from kvq_b200.decode_step import DecodeStep
from oracle import kvq_oracle as orc

pytestmark = pytest.mark.gpu


def test_decode_step_layers_match_oracle():
    batch, ctx, bs = 4, 300, 16
    step = DecodeStep(torch.device(DEV, 0), batch, ctx, block_size=bs, seed=3, geometry=dict(layers=2, vocab=4096))
    g = step.g
    before = step.kv.cpu().numpy().copy()
    step.trace = []
    tokens_eager = step.forward().clone()
    torch.cuda.synchronize()
    after = step.kv.cpu().numpy()
    slots = step.slots.cpu().numpy()
    bt, sl, cu = step.block_table.cpu().numpy(), step.seq_lens.cpu().numpy(), step.cu.cpu().numpy()
    assert len(step.trace) == 2
    for i, tr in enumerate(step.trace):
        st = {k: v.cpu().numpy() for k, v in step.layers[i]["static"].items()}
        # cache bytes: exactly the oracle's quantization of the new rows, nothing else touched
        want_k, want_v = before[i, 0].copy(), before[i, 1].copy()
        orc.quant_cache_write(tr["k"].float().cpu().numpy(), tr["v"].float().cpu().numpy(), want_k, want_v, slots,
                              st["k_scale"], st["v_scale"], st["k_mu"])
        assert np.array_equal(after[i, 0], want_k) and np.array_equal(after[i, 1], want_v), f"layer {i} cache bytes"
        assert (after[i, 0] != before[i, 0]).any()
        # attention over the updated cache
        ref = orc.paged_static_attention(tr["q"].float().cpu().numpy(), after[i, 0], after[i, 1], cu, sl, bt,
                                         1.0 / np.sqrt(g["head_dim"]), st["k_scale"], st["v_scale"])
        assert_close(ref, tr["attn_out"].float().cpu().numpy(), f"layer {i} attention")
    # the graph replays the same step (the cache rows it rewrites get the same bytes)
    step.trace = None
    step.capture()
    tokens_graph = step.step().clone()
    torch.cuda.synchronize()
    assert torch.equal(tokens_graph, tokens_eager)
    assert np.array_equal(step.kv.cpu().numpy(), after)
