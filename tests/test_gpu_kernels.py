"""GPU parity tests: the sm_100a kernels, called through the C ABI, against the CPU oracle and the golden
fixtures made by the reference's own code.

Bars: cache bytes, quantized q and dequantized pages bit-exact; attention output by gpu_util.assert_close
(max-abs 1e-2 and mean-abs 1e-3 against the fp32 oracle where |ref| < 2, within one bf16 step of the bf16-rounded
oracle above that, and the reference's own rel_l2 < 5e-3)."""
import numpy as np
import pytest
import torch
from conftest import load_golden
from gpu_util import DEV, assert_close, fixture_case, oracle_attention, run_decode, short_row_mask, to_dev

from kvq_b200 import cuda_kernels as ck
from kvq_b200 import workloads
from oracle import kvq_oracle as orc

pytestmark = pytest.mark.gpu

DECODE = ([1] * 11, [1, 16, 17, 31, 32, 33, 250, 1023, 2049, 700, 3100])
SHORT = ([2, 4, 8, 3, 1, 5, 7, 1, 6], [37, 650, 1025, 9, 2050, 100, 2800, 16, 513])
MIXED = ([1, 1, 7, 40, 130, 1, 290, 9, 4, 0], [590, 33, 7, 480, 130, 1400, 910, 1900, 70, 12])

def bf16_t(bits):
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16)


# ---------------------------------------------------------------------------------------------------
# fused quantize + cache write, page dequantization
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("gran", ["channel", "head"])
@pytest.mark.parametrize("layout", ["interleaved", "separate"])
def test_quant_cache_golden(d, gran, layout):
    """Reference-generated fixture: 200 tokens + 8 padded rows, every 17th slot -1, both cache layouts."""
    fx = load_golden(f"write_d{d}_{gran}.npz")
    key, value = bf16_t(fx["key"]).to(DEV), bf16_t(fx["value"]).to(DEV)
    nb, bs, H = fx["k_cache"].shape[:3]
    if layout == "interleaved":   # vLLM 0.32 logical [nb, H, bs, 2D] over physical [nb, bs, H, 2D]
        kv = torch.zeros(nb, bs, H, 2 * d, dtype=torch.int8, device=DEV)
        kc, vc = kv.split(d, dim=-1)
    else:
        kc = torch.zeros(nb, bs, H, d, dtype=torch.int8, device=DEV)
        vc = torch.zeros_like(kc)
    st = to_dev({k: torch.from_numpy(fx[k]) for k in ("k_scale", "v_scale", "k_mu")})
    ck.quant_reshape_and_cache(key, value, kc, vc, torch.from_numpy(fx["slots"]).to(DEV), st)
    assert np.array_equal(kc.cpu().numpy(), fx["k_cache"]) and np.array_equal(vc.cpu().numpy(), fx["v_cache"])
    # dequantize all pages through an identity table: bit-exact bf16
    ko = torch.empty(nb, bs, H, d, dtype=torch.bfloat16, device=DEV)
    vo = torch.empty_like(ko)
    ident = torch.arange(nb, dtype=torch.int32, device=DEV)
    ck.dequant_pages(kc, vc, ko, vo, ident[None].contiguous(), torch.zeros_like(ident), ident, st)
    assert np.array_equal(ko.cpu().view(torch.int16).numpy().view(np.uint16), fx["k_dequant"])
    assert np.array_equal(vo.cpu().view(torch.int16).numpy().view(np.uint16), fx["v_dequant"])


def test_quant_cache_config1_round_trip():
    """Benchmark configuration 1 (cache write round trip): 8192 tokens into a 65536-slot cache, bit-exact against the oracle, then the pages
    dequantized back to bf16 (also bit-exact). A strided key (fused qkv row stride) is used."""
    c = workloads.config1()
    st, bs, nb = c["static"], c["block_size"], c["num_blocks"]
    T, H, D = c["key"].shape
    qkv = torch.zeros(T, 3 * H * D + 64, dtype=torch.bfloat16, device=DEV)
    key = qkv[:, H * D:2 * H * D].view(T, H, D)
    value = qkv[:, 2 * H * D:3 * H * D].view(T, H, D)
    key.copy_(c["key"]), value.copy_(c["value"])
    kc = torch.zeros(nb, bs, H, D, dtype=torch.int8, device=DEV)
    vc = torch.zeros_like(kc)
    ck.quant_reshape_and_cache(key, value, kc, vc, c["slots"].to(DEV), to_dev(st))
    ref_k, ref_v = np.zeros((nb, bs, H, D), np.int8), np.zeros((nb, bs, H, D), np.int8)
    orc.quant_cache_write(c["key"].float().numpy(), c["value"].float().numpy(), ref_k, ref_v, c["slots"].numpy(),
                          st["k_scale"].numpy(), st["v_scale"].numpy(), st["k_mu"].numpy())
    assert np.array_equal(kc.cpu().numpy(), ref_k) and np.array_equal(vc.cpu().numpy(), ref_v)
    # pages that hold the tokens, in slot order
    pages = torch.unique(c["slots"] // bs).to(torch.int32)
    P = pages.numel()
    ko = torch.empty(P, bs, H, D, dtype=torch.bfloat16, device=DEV)
    vo = torch.empty_like(ko)
    idx = torch.arange(P, dtype=torch.int32, device=DEV)
    ck.dequant_pages(kc, vc, ko, vo, pages[None].contiguous().to(DEV), torch.zeros_like(idx), idx, to_dev(st))
    rk, rv = orc.dequant_pages(ref_k, ref_v, pages[None].numpy(), np.zeros(P, np.int32), np.arange(P, dtype=np.int32),
                               st["k_scale"].numpy(), st["v_scale"].numpy())
    assert np.array_equal(ko.float().cpu().numpy(), rk) and np.array_equal(vo.float().cpu().numpy(), rv)


def test_quant_cache_all_padding_and_empty():
    c = workloads.write_case(3, 64, 4, 128, num_blocks=8)
    kc = torch.zeros(8, 16, 4, 128, dtype=torch.int8, device=DEV)
    vc = torch.zeros_like(kc)
    slots = torch.full((64,), -1, dtype=torch.int64, device=DEV)
    ck.quant_reshape_and_cache(c["key"].to(DEV), c["value"].to(DEV), kc, vc, slots, to_dev(c["static"]))
    assert not kc.any() and not vc.any()
    slots[:10] = torch.arange(10, device=DEV) * 3
    ck.quant_reshape_and_cache(c["key"].to(DEV), c["value"].to(DEV), kc, vc, slots, to_dev(c["static"]))
    assert int((kc != 0).flatten(2).any(-1).sum()) == 10
    ck.quant_reshape_and_cache(c["key"].to(DEV), c["value"].to(DEV), kc, vc, slots[:0], to_dev(c["static"]))  # no tokens


def test_layout_violations_raise():
    c = workloads.write_case(3, 8, 4, 128, num_blocks=2)
    kc = torch.zeros(2, 16, 4, 128, dtype=torch.int8, device=DEV)
    with pytest.raises(RuntimeError):   # cache with a strided last dim
        ck.quant_reshape_and_cache(c["key"].to(DEV), c["value"].to(DEV), kc.transpose(2, 3), kc, c["slots"].to(DEV),
                                   to_dev(c["static"]))
    with pytest.raises(RuntimeError):   # head_dim 96 is not supported
        ck.quant_q(torch.zeros(4, 8, 96, dtype=torch.bfloat16, device=DEV), torch.ones(2, 96, device=DEV))


# ---------------------------------------------------------------------------------------------------
# q quantization
# ---------------------------------------------------------------------------------------------------
def test_quant_q_golden():
    fx = load_golden("quant_q.npz")
    q = bf16_t(fx["q"]).to(DEV)
    ks = torch.from_numpy(fx["k_scale"]).to(DEV)
    for group in (128, 32):
        qi, qs = ck.quant_q(q, ks, group)
        assert np.array_equal(qi.cpu().numpy(), fx[f"q_i8_g{group}"])
        assert np.array_equal(qs.cpu().numpy(), fx[f"q_scale_g{group}"])
    qi, qs = ck.quant_q(q, torch.ones(4, 1, device=DEV))
    assert np.array_equal(qi.cpu().numpy(), fx["q_i8_per_head"])
    assert np.array_equal(qs.cpu().numpy(), fx["q_scale_per_head"])


def test_quant_q_strided_rows_vs_oracle():
    g = torch.Generator().manual_seed(5)
    T = 2048 + 3
    qkv = (torch.randn(T, 40, 128, generator=g) * 3).to(torch.bfloat16)
    q = qkv[:, :28].to(DEV)                      # contiguous copy
    q_strided = qkv.to(DEV)[:, :28]              # token stride 40 * 128
    ks = (torch.rand(4, 128, generator=g) + 0.01)
    ri, rs = orc.quant_q(qkv[:, :28].float().numpy(), ks.numpy(), 128)
    for t in (q, q_strided):
        qi, qs = ck.quant_q(t, ks.to(DEV))
        assert np.array_equal(qi.cpu().numpy(), ri) and np.array_equal(qs.cpu().numpy(), rs)


# ---------------------------------------------------------------------------------------------------
# INT8 attention
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["attn_short_smooth.npz", "attn_per_head_d64.npz"])
def test_attention_golden(name):
    """Against outputs of the reference's implementation B itself (tests/golden)."""
    fx = load_golden(name)
    out = run_decode(fixture_case(fx))
    assert_close(fx["ref_out"], out, name)


def test_attention_config0_golden():
    """Benchmark configuration 0 (4 requests, contexts 128..512): reference output, then the bf16 golden within the
    reference's own quantization tolerance."""
    fx = load_golden("attn_config0.npz")
    out = run_decode(workloads.config0())
    assert_close(fx["ref_out"], out, "config0")
    assert orc.compare(fx["bf16_golden"], out)["rel_l2"] < 0.05
    # beyond the tolerance: the bf16 output is the bf16 rounding of the reference's fp32 result almost everywhere
    assert (orc.round_to_bf16(fx["ref_out"]) == out).mean() > 0.999


def test_mixed_batch_leaves_long_requests_alone():
    fx = load_golden("attn_mixed_long.npz")
    case = fixture_case(fx)
    out = torch.full_like(case["q"], 7.0).to(DEV)
    got = run_decode(case, out=out)
    short = short_row_mask(case)
    assert (got[~short] == 7.0).all() and not (got[short] == 7.0).all(-1).all(-1).any()
    assert_close(fx["ref_out"][short], got[short], "mixed short rows")


@pytest.mark.parametrize("shape", [(28, 4, 128), (12, 2, 128), (32, 8, 128), (16, 1, 128), (14, 2, 64), (16, 4, 64)])
@pytest.mark.parametrize("batch", ["decode", "short"])
@pytest.mark.parametrize("variant", ["per_channel", "per_head", "interleaved"])
def test_short_queries_match_oracle(shape, batch, variant):
    """Decode and short multi-token queries (causal inside the request, several m tiles when q_len * G > 16),
    head_dim 128 and 64, per-channel and per-head scales, smooth-K, both cache layouts."""
    hq, hkv, d = shape
    q_lens, seq_lens = DECODE if batch == "decode" else SHORT
    case = workloads.paged_case(100 + hq + d, hq, hkv, d, q_lens, seq_lens, per_channel=variant != "per_head",
                                smooth=True, q_std=3.0)
    out = run_decode(case, interleaved=variant == "interleaved")
    assert_close(oracle_attention(case), out, (shape, batch, variant))


def test_mixed_lengths_and_padding_requests():
    case = workloads.paged_case(9, 28, 4, 128, *MIXED, q_std=3.0)
    out = torch.full_like(case["q"], 7.0).to(DEV)
    got = run_decode(case, out=out)
    short = short_row_mask(case)
    assert (got[~short] == 7.0).all()
    assert_close(oracle_attention(case)[short], got[short], "mixed")


@pytest.mark.parametrize("block_size", [32, 64, 128])
def test_larger_pages(block_size):
    case = workloads.paged_case(31, 28, 4, 128, [1, 3, 1, 8], [100, 777, 2048, 333], block_size=block_size)
    assert_close(oracle_attention(case), run_decode(case), block_size)


def test_wider_tables_and_extra_rows():
    """vLLM hands tables wider than the request and seq_lens/block_table with more rows than requests."""
    case = workloads.paged_case(32, 28, 4, 128, [1, 5, 1], [300, 90, 1000])
    ref = oracle_attention(case)
    bt = case["block_table"]
    case["block_table"] = torch.cat([torch.cat([bt, bt[:, :1].expand(-1, 5)], 1), bt.new_zeros(2, bt.shape[1] + 5)], 0)
    case["seq_lens"] = torch.cat([case["seq_lens"], case["seq_lens"].new_zeros(2)])
    assert_close(ref, run_decode(case), "wide table")


def test_single_long_request_is_split_over_many_ctas():
    """One request with a 20k context: every (kv head) item is cut across dozens of CTAs and merged."""
    case = workloads.paged_case(33, 28, 4, 128, [1], [20000])
    assert_close(oracle_attention(case), run_decode(case), "split")
    case = workloads.paged_case(34, 28, 4, 128, [6], [9000])
    assert_close(oracle_attention(case), run_decode(case), "split short-q")


def test_kernel_split_equals_host_restatement():
    """The records the attention kernel leaves for the merge kernel (which item each CTA's range end cut, and the
    last CTA that item reaches) agree with the host restatement of the split (kvq_debug_decode_split), for decode
    batches on the fused path and beyond 1024 requests on the planned one."""
    import ctypes

    lib = ck.ext()
    sms = torch.cuda.get_device_properties(DEV).multi_processor_count
    nctas = 2 * sms                                    # the 8-row kernel runs two CTAs per SM
    for seed, lens in ((61, [32768] * 3), (62, [5000, 20000, 777, 12345, 64]), (63, None)):
        if lens is None:                               # planned path: more than 1024 requests
            lens = np.random.default_rng(seed).integers(1, 400, 1200).tolist()
        b = len(lens)
        case = workloads.paged_case(seed, 28, 4, 128, [1] * b, lens)
        run_decode(case)
        torch.cuda.synchronize()
        ws = ck.decode_workspace(DEV, b, 128)
        raw = ws.view(torch.int32).cpu().numpy()
        bnd0 = (256 + -(-((b + 1) * 8) // 256) * 256) // 4
        rec = raw[bnd0:bnd0 + nctas * 8].reshape(nctas, 8)
        ql = np.ones(b, dtype=np.int32)
        sl = np.asarray(lens, dtype=np.int32)
        ub = np.zeros(nctas, dtype=np.int32)
        ue = np.zeros(nctas, dtype=np.int32)
        assert lib.kvq_debug_decode_split(ql.ctypes.data_as(ctypes.c_void_p), sl.ctypes.data_as(ctypes.c_void_p), b, 7, 4, 8,
                                          0, 0, -1, nctas, ub.ctypes.data_as(ctypes.c_void_p),
                                          ue.ctypes.data_as(ctypes.c_void_p)) == 0
        # items in unit order: (first unit, chunks, request, kv head)
        items, u = [], 0
        for r, L in enumerate(lens):
            n = max(1, -(-L // 32))
            for h in range(4):
                items.append((u, n, r, h))
                u += n
        firsts = np.asarray([it[0] for it in items])
        cuts = 0
        for c in range(nctas - 1):
            e = int(ue[c])
            k = int(np.searchsorted(firsts, e, side="right")) - 1
            first, n, r, h = items[k]
            cut_here = ub[c] < ue[c] and first < e < first + n and first >= ub[c]   # first boundary inside the item
            if cut_here:
                cuts += 1
                last = first + n - 1
                last_cta = next(cc for cc in range(nctas) if ub[cc] <= last < ue[cc])
                assert (rec[c, 0], rec[c, 1], rec[c, 3]) == (r, h, first), (c, rec[c], (r, h, first))
                assert rec[c, 4] == last_cta, (c, rec[c], last_cta)
            else:
                assert rec[c, 0] < 0, (c, rec[c])
        assert cuts > 0


def test_headline_shape_subset_vs_oracle():
    """Full-size contexts (32768) at a batch the oracle finishes in seconds; the decode kernel sees 8 requests."""
    case = workloads.paged_case(35, 28, 4, 128, [1] * 8, [32768] * 8, num_blocks=8 * 2048 + 8)
    assert_close(oracle_attention(case), run_decode(case), "8x32k")


def test_cuda_graph_replay_is_bit_identical():
    """Replay with new inputs equals an eager call: no host-side state, no atomics in the data path."""
    for q_len in (1, 4, 5):
        case = workloads.paged_case(40 + q_len, 28, 4, 128, [q_len] * 8, [100, 2000, 37, 512, 1500, 64, 999, 3000],
                                    q_std=3.0)
        q, kq, vq = case["q"].to(DEV), case["kq"].to(DEV), case["vq"].to(DEV)
        cu, sl, bt = case["cu_seqlens_q"].to(DEV), case["seq_lens"].to(DEV), case["block_table"].to(DEV)
        st = to_dev(case["static"])
        out = torch.zeros_like(q)
        fn = lambda o: ck.decode_attention(q, kq, vq, o, cu, sl, bt, case["softmax_scale"], st, max_query_len=q_len)  # noqa: E731
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn(out)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn(out)
        q2 = workloads.paged_case(77, 28, 4, 128, [q_len] * 8, [100] * 8, q_std=3.0)["q"]
        q.copy_(q2)
        sl.sub_(1)          # same shapes, new contents
        g.replay()
        ref = fn(torch.zeros_like(q))
        torch.cuda.synchronize()
        assert torch.equal(ref, out)
        # scales are read through their storage: an in-place update reaches the captured graph
        st["v_scale"].mul_(2)
        g.replay()
        ref2 = fn(torch.zeros_like(q))
        torch.cuda.synchronize()
        assert torch.equal(ref2, out) and not torch.equal(ref2, ref)


def test_check_inputs_reports_bad_pages():
    case = workloads.paged_case(50, 28, 4, 128, [1, 1], [100, 50])
    bt = case["block_table"].clone()
    bt[1, 0] = 10 ** 6
    with pytest.raises(RuntimeError, match="kvq input check"):
        ck.check_inputs(case["q"].to(DEV), case["kq"].to(DEV), case["cu_seqlens_q"].to(DEV), case["seq_lens"].to(DEV),
                        bt.to(DEV), None)


def test_strided_q_and_out_rows():
    """q as a slice of a fused qkv activation and out as a slice of a wider buffer (token / head strides)."""
    case = workloads.paged_case(51, 28, 4, 128, [1, 4, 1, 8], [200, 513, 31, 1000], q_std=2.0)
    ref = oracle_attention(case)
    T = case["q"].shape[0]
    qkv = torch.zeros(T, 28 + 8, 128, dtype=torch.bfloat16, device=DEV)
    qkv[:, :28] = case["q"].to(DEV)
    wide = torch.full((T, 28, 256), 7.0, dtype=torch.bfloat16, device=DEV)
    out = wide[:, :, :128]
    ck.decode_attention(qkv[:, :28], case["kq"].to(DEV), case["vq"].to(DEV), out, case["cu_seqlens_q"].to(DEV),
                        case["seq_lens"].to(DEV), case["block_table"].to(DEV), case["softmax_scale"], to_dev(case["static"]),
                        max_query_len=8)
    torch.cuda.synchronize()
    assert ck.decode_status() == 0
    assert_close(ref, out.float().cpu().numpy(), "strided")
    assert (wide[:, :, 128:] == 7.0).all()          # nothing written outside the rows


def test_garbage_table_entries_past_the_context_are_harmless():
    """Entries of the block table beyond a request's pages may hold anything (vLLM leaves stale ids there): they are
    either never read or land in masked keys; out-of-range ids make TMA zero-fill instead of faulting."""
    case = workloads.paged_case(52, 28, 4, 128, [1, 1, 3], [100, 16, 530])
    ref = oracle_attention(case)
    bt = case["block_table"].clone()
    for r, L in enumerate(case["seq_lens"].tolist()):
        pages = (L + 15) // 16
        bt[r, pages:] = torch.tensor([-1, 2 ** 30, 12345678][r % 3], dtype=torch.int32)
    case["block_table"] = bt
    assert_close(ref, run_decode(case), "garbage table")


def test_all_requests_skipped_leaves_output_alone():
    """A batch with only padding (q_len 0) and long (q_len > 8) requests: the call is a no-op on `out`."""
    case = workloads.paged_case(53, 28, 4, 128, [0, 12, 0], [40, 300, 9])
    out = torch.full_like(case["q"], 7.0).to(DEV)
    got = run_decode(case, out=out, max_query_len=12)
    assert (got == 7.0).all()


def test_head_major_pages():
    """Caches stored [block, head, slot, channel] (each (page, head) tile contiguous) and passed as the usual
    [block, slot, head, channel] views: slot stride < head stride, so the tensor maps order their dims differently."""
    case = workloads.paged_case(54, 32, 8, 128, [1, 1, 6, 1], [700, 90, 333, 2049])
    ref = oracle_attention(case)
    q = case["q"].to(DEV)
    kq = case["kq"].to(DEV).permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    vq = case["vq"].to(DEV).permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert kq.stride(1) == 128 and kq.stride(2) == 16 * 128
    out = torch.zeros_like(q)
    ck.decode_attention(q, kq, vq, out, case["cu_seqlens_q"].to(DEV), case["seq_lens"].to(DEV),
                        case["block_table"].to(DEV), case["softmax_scale"], to_dev(case["static"]), max_query_len=6)
    torch.cuda.synchronize()
    assert ck.decode_status() == 0
    assert_close(ref, out.float().cpu().numpy(), "head-major")
    # the write kernel into the same layout
    w = workloads.write_case(55, 100, 8, 128, num_blocks=16)
    kc = torch.zeros(16, 8, 16, 128, dtype=torch.int8, device=DEV).transpose(1, 2)
    vc = torch.zeros(16, 8, 16, 128, dtype=torch.int8, device=DEV).transpose(1, 2)
    ck.quant_reshape_and_cache(w["key"].to(DEV), w["value"].to(DEV), kc, vc, w["slots"].to(DEV), to_dev(w["static"]))
    rk, rv = np.zeros((16, 16, 8, 128), np.int8), np.zeros((16, 16, 8, 128), np.int8)
    st = w["static"]
    orc.quant_cache_write(w["key"].float().numpy(), w["value"].float().numpy(), rk, rv, w["slots"].numpy(),
                          st["k_scale"].numpy(), st["v_scale"].numpy(), st["k_mu"].numpy())
    assert np.array_equal(kc.cpu().numpy(), rk) and np.array_equal(vc.cpu().numpy(), rv)


def config3_subset(requests=32, seed=1003):
    """Benchmark configuration 3 at a size the oracle finishes in seconds: q_len 8 (56 rows = 4 m tiles per kv
    head), contexts uniform in [1024, 8192], layer geometry 28 / 4 / 128."""
    gen = torch.Generator().manual_seed(seed)
    ctx = torch.randint(1024, 8193, (requests,), generator=gen).tolist()
    return workloads.paged_case(seed, 28, 4, 128, [8] * requests, ctx, num_blocks=sum((c + 15) // 16 for c in ctx) + 8)


def test_config3_subset_vs_oracle():
    """Spec-decode verification batch: every CTA range holds many variable-length items of four m tiles each, cut
    items are merged. 32 of the configuration's 256 requests."""
    case = config3_subset()
    assert_close(oracle_attention(case), run_decode(case), "config 3 subset")


def test_workspaces_are_per_stream_and_never_freed():
    """The host layer keeps one scratch buffer per (device, stream) and keeps superseded buffers alive, because a
    captured CUDA graph replays with the raw address of the buffer it saw."""
    dev = torch.device(DEV, torch.cuda.current_device())
    pool = ck._StreamWorkspaces(lambda n, d: ck.ext().kvq_decode_workspace_size(n, d), (16, 128))
    small = pool.get(dev, ck.ext().kvq_decode_workspace_size(16, 128))
    assert pool.get(dev, 1024) is small
    grown = pool.get(dev, small.numel() + 4096)
    assert grown is not small and grown.numel() >= small.numel() + 4096
    assert any(t is small for t in pool.retired) and pool.peek(dev) is grown
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        other = pool.get(dev, 1024)
    assert other.data_ptr() not in (small.data_ptr(), grown.data_ptr())
    assert pool.get(dev, 1024) is grown


def _capture(fn):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def test_rebinding_a_scale_is_not_seen_by_a_captured_graph():
    """The reference's contract for scales under CUDA graphs (tests/test_cudagraph.py:56-70): a graph reads the
    scale tensors it captured. Replacing static["v_scale"] by a new tensor leaves the replay on the old values;
    only an in-place update (covered by test_cuda_graph_replay_is_bit_identical) reaches it."""
    case = workloads.paged_case(45, 28, 4, 128, [1] * 8, [100, 2000, 37, 512, 1500, 64, 999, 3000], q_std=3.0)
    q, kq, vq = case["q"].to(DEV), case["kq"].to(DEV), case["vq"].to(DEV)
    cu, sl, bt = case["cu_seqlens_q"].to(DEV), case["seq_lens"].to(DEV), case["block_table"].to(DEV)
    st = to_dev(case["static"])
    out = torch.zeros_like(q)
    fn = lambda o: ck.decode_attention(q, kq, vq, o, cu, sl, bt, case["softmax_scale"], st)  # noqa: E731
    g = _capture(lambda: fn(out))
    g.replay()
    torch.cuda.synchronize()
    before = out.clone()
    st["v_scale"] = st["v_scale"] * 2          # rebinding: new storage
    g.replay()
    expected = fn(torch.zeros_like(q))
    torch.cuda.synchronize()
    assert torch.equal(out, before) and not torch.allclose(out.float(), expected.float())


def test_cache_write_under_graph_capture_skips_padded_slots():
    """Under a full CUDA graph the slot mapping is padded with -1 up to the captured size
    (reference: tests/test_cudagraph.py:87-101): captured with every slot -1, replayed with 10 real tokens."""
    T, H, D, nb, bs = 64, 4, 128, 32, 16
    c = workloads.write_case(46, T, H, D, num_blocks=nb, block_size=bs)
    key, value, st = c["key"].to(DEV), c["value"].to(DEV), to_dev(c["static"])
    slots = torch.full((T,), -1, dtype=torch.int64, device=DEV)
    kc = torch.zeros(nb, bs, H, D, dtype=torch.int8, device=DEV)
    vc = torch.zeros_like(kc)
    g = _capture(lambda: ck.quant_reshape_and_cache(key, value, kc, vc, slots, st))
    torch.cuda.synchronize()
    assert not kc.any() and not vc.any()
    slots[:10] = torch.arange(10, device=DEV) * 3
    g.replay()
    torch.cuda.synchronize()
    assert int((kc != 0).flatten(2).any(-1).sum()) == 10
    rk, rv = np.zeros((nb, bs, H, D), np.int8), np.zeros((nb, bs, H, D), np.int8)
    s = c["static"]
    orc.quant_cache_write(c["key"].float().numpy(), c["value"].float().numpy(), rk, rv, slots.cpu().numpy(),
                          s["k_scale"].numpy(), s["v_scale"].numpy(), s["k_mu"].numpy())
    assert np.array_equal(kc.cpu().numpy(), rk) and np.array_equal(vc.cpu().numpy(), rv)


def test_large_batch_takes_the_planned_path():
    """More requests than a CTA sums by itself (1024): the plan kernel runs first and the CTAs look their first
    request up in its prefix sums. 1500 decode requests with short ragged contexts, padding requests in between."""
    gen = torch.Generator().manual_seed(47)
    n = 1500
    ctx = torch.randint(1, 200, (n,), generator=gen).tolist()
    q_lens = [0 if i % 97 == 5 else 1 for i in range(n)]
    case = workloads.paged_case(47, 28, 4, 128, q_lens, ctx)
    out = torch.full_like(case["q"], 7.0).to(DEV)
    got = run_decode(case, out=out)
    assert_close(oracle_attention(case), got, "planned path")


def test_items_follow_each_other_without_draining_the_stream():
    """Decode batch in which every CTA meets several items: many requests of a few chunks each, so that a warp's
    stream runs across item and request boundaries (next item's pages and q rows are fetched while the current one
    runs), including requests too short to give every warp a chunk and requests that are skipped."""
    gen = torch.Generator().manual_seed(48)
    n = 700
    ctx = torch.randint(1, 700, (n,), generator=gen).tolist()
    q_lens = [1] * n
    for i in range(0, n, 41):
        q_lens[i] = 0          # padding request
    for i in range(7, n, 53):
        q_lens[i] = 12         # long request: not this kernel's
    case = workloads.paged_case(48, 28, 4, 128, q_lens, ctx, q_std=2.0)
    out = torch.full_like(case["q"], 7.0).to(DEV)
    got = run_decode(case, out=out, max_query_len=1)
    short = short_row_mask(case)
    assert (got[~short] == 7.0).all()
    assert_close(oracle_attention(case)[short], got[short], "stream across items")


# ---------------------------------------------------------------------------------------------------
# one q scale per 32 channels inside the attention kernel (kvq_int8_decode_attention_qgroup)
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["attn_qgroup32.npz", "attn_qgroup32_per_head.npz"])
def test_group32_q_scales_golden(name):
    """Against outputs of the reference's own implementation with q_gran="group32" (tests/golden), and the option
    really changes the result: the per-row kernel does not meet them as closely."""
    fx = load_golden(name)
    case = fixture_case(fx)
    out = run_decode(case, q_group=32)
    err = assert_close(fx["ref_out"], out, name)
    per_row = orc.compare(fx["ref_out"], run_decode(case))
    assert err["rel_l2"] < per_row["rel_l2"]


@pytest.mark.parametrize("shape", [(28, 4, 128), (32, 8, 128), (14, 2, 64)])
@pytest.mark.parametrize("batch", ["decode", "short"])
@pytest.mark.parametrize("per_channel", [True, False])
def test_group32_q_scales_match_oracle(shape, batch, per_channel):
    """Decode (8-row kernel, incl. head pairs at 8 kv heads) and multi-token queries (16-row kernel, warp groups),
    head_dim 128 and 64, per-channel and per-head K/V scales, smooth-K."""
    hq, hkv, d = shape
    q_lens, seq_lens = DECODE if batch == "decode" else SHORT
    case = workloads.paged_case(300 + hq + d, hq, hkv, d, q_lens, seq_lens, per_channel=per_channel, smooth=True, q_std=3.0)
    out = run_decode(case, q_group=32)
    assert_close(oracle_attention(case, q_group=32), out, (shape, batch, per_channel))


def test_group32_rejects_other_group_sizes():
    case = workloads.paged_case(301, 28, 4, 128, [1], [64])
    with pytest.raises(RuntimeError, match="q_group"):
        run_decode(case, q_group=16)
    assert_close(oracle_attention(case), run_decode(case, q_group=128), "q_group = head_dim is the per-row kernel")
