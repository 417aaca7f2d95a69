"""CPU tests: the C-ABI library loads and exports what include/kvq_b200.h declares (no compute calls), and the host
logic of the package (page plan, scale files and their TP sharding, input checks, loud failure without the native
library, vLLM surface)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch
from conftest import ROOT, load_golden

from kvq_b200 import _native, scales
from kvq_b200 import cuda_kernels as ck

HEADER = os.path.join(ROOT, "include", "kvq_b200.h")


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:int|size_t|const char\*)\s+(kvq_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        params = m.group(2).strip()
        out[m.group(1)] = 0 if params == "void" else len([p for p in params.split(",") if p.strip()])
    return out


def test_library_exports_every_declared_symbol():
    decl = declared_functions()
    assert len(decl) >= 10 and "kvq_int8_decode_attention" in decl and "kvq_quant_cache" in decl
    handle = ctypes.CDLL(_native.LIB_PATH)
    for name in decl:
        assert hasattr(handle, name), f"{name} declared in kvq_b200.h but not exported"
    lib = _native.lib()
    assert lib.kvq_version() >= 100 and lib.kvq_last_error() == b""


def test_ctypes_signatures_match_header():
    decl = declared_functions()
    assert set(decl) == set(_native.SIGNATURES), set(decl) ^ set(_native.SIGNATURES)
    for name, nparams in decl.items():
        assert len(_native.SIGNATURES[name][1]) == nparams, name


def test_argument_errors_are_reported_without_a_gpu():
    """Validation happens before any CUDA call: bad head_dim -> KVQ_ERR_INVALID_ARGUMENT + message."""
    lib = _native.lib()
    rc = lib.kvq_quant_q(None, None, None, None, 4, 28, 4, 96, 128, 0, 0, 1, None)
    assert rc == 1 and b"head_dim 128" in lib.kvq_last_error()
    with pytest.raises(RuntimeError, match="kvq_b200"):
        _native.check(rc)
    assert lib.kvq_quant_cache(*([None] * 8), 0, 4, 128, 16, *([0] * 10), 1, 1, None) == 0   # empty batch: silent


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_native, "_LIB", None)
    monkeypatch.setattr(_native, "LIB_PATH", "/nonexistent/libkvq_b200.so")
    with pytest.raises(RuntimeError, match="no non-CUDA fallback"):
        _native.lib()


def test_cpu_tensors_are_rejected():
    case_q = torch.zeros(2, 28, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ck.quant_q(case_q, torch.ones(4, 128))


def test_plan_long_matches_reference_tables():
    fx = load_golden("plan_long.npz")
    for key in ("a", "b", "c", "none"):
        plan = ck.plan_long(fx[f"{key}_cu"], fx[f"{key}_sl"], int(fx[f"{key}_bs"]))
        if bool(fx[f"{key}_is_none"]):
            assert plan is None
            continue
        assert np.array_equal(plan.src_req, fx[f"{key}_src_req"]) and plan.src_req.dtype == np.int32
        assert np.array_equal(plan.src_j, fx[f"{key}_src_j"]) and np.array_equal(plan.block_table, fx[f"{key}_bt"])
        assert plan.max_seqlen_k == int(fx[f"{key}_max_seqlen_k"]) and plan.has_short == bool(fx[f"{key}_has_short"])
    # the reference's literal known answers (tests/test_cuda_kernels.py:88-97 there)
    plan = ck.plan_long(torch.tensor([0, 1, 13, 14, 314], dtype=torch.int32), torch.tensor([50, 40, 9, 330]), 16)
    assert plan.src_req.tolist() == [1] * 3 + [3] * 21 and plan.src_j.tolist() == list(range(3)) + list(range(21))
    assert plan.block_table.shape[1] * 16 >= 330 + 256 and not plan.block_table[3, 21:].any()
    assert ck.plan_long(torch.tensor([0, 1, 9]), torch.tensor([5, 8]), 16) is None   # q_len 8 is still short


def test_scale_sharding_matches_reference():
    fx = load_golden("scale_shards.npz")
    for name in ("t8", "t2"):
        t = torch.from_numpy(fx[name])
        for tp in (1, 2, 4, 8):
            for rank in range(tp):
                assert np.array_equal(scales.shard(t, rank, tp).numpy(), fx[f"{name}_tp{tp}_r{rank}"])
    with pytest.raises(ValueError):
        scales.shard(torch.zeros(6, 4), 0, 4)


def test_scale_file_round_trip(tmp_path):
    g = torch.Generator().manual_seed(0)
    layers = {f"model.layers.{i}.self_attn.attn": {"k_scale": torch.rand(4, 128, generator=g), "v_scale": torch.rand(4, 128, generator=g),
                                                   "k_mu": torch.randn(4, 128, generator=g)} for i in range(3)}
    path = str(tmp_path / "scales.safetensors")
    scales.save(path, layers)
    back = scales.load(path)
    assert set(back) == set(layers)
    for name, fields in layers.items():
        for f, t in fields.items():
            assert back[name][f].dtype == torch.float32 and torch.equal(back[name][f], t)
    mine = scales.for_layer(back, "model.layers.1.self_attn.attn", 1, 2, "cpu")
    assert torch.equal(mine["k_scale"], layers["model.layers.1.self_attn.attn"]["k_scale"][2:4])
    # key format of the file: "<layer>|<field>"
    from safetensors.torch import load_file
    assert "model.layers.0.self_attn.attn|k_mu" in load_file(path)


def test_from_stats_and_merge_tp():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(500, 4, 16, generator=g) * 3 + 1
    st = {"tokens": 500, "k_sum": x.sum(0), "k_max": x.amax(0), "k_min": x.amin(0), "k_absmax": x.abs().amax(0),
          "v_absmax": x.abs().amax(0)}
    s = scales.from_stats(st, smooth_k=True)
    mu = x.mean(0)
    assert torch.allclose(s["k_mu"], mu, atol=1e-5)
    assert torch.allclose(s["k_scale"], ((x - mu).abs().amax(0) / 127).clamp(min=1e-8), rtol=1e-5)
    assert scales.from_stats(st, granularity="per_head")["v_scale"].shape == (4, 1)
    halves = [{"tp_rank": r, "stats": {"l": {k: (v if k == "tokens" else v[2 * r:2 * r + 2]) for k, v in st.items()}},
               "samples": {"l": {"k": x[:, 2 * r:2 * r + 2], "v": x[:, 2 * r:2 * r + 2]}}} for r in (1, 0)]
    stats, samples = scales.merge_tp(halves, 4)
    assert torch.equal(stats["l"]["k_absmax"], st["k_absmax"]) and torch.equal(samples["l"]["k"], x)


def test_check_inputs_messages():
    c = {"q": torch.zeros(3, 28, 128), "k": torch.zeros(8, 16, 4, 128, dtype=torch.int8)}
    cu = torch.tensor([0, 1, 3], dtype=torch.int32)
    ok_bt = torch.tensor([[0, 1, 2], [3, 4, 5]], dtype=torch.int32)
    ck.check_inputs(c["q"], c["k"], cu, torch.tensor([40, 20], dtype=torch.int32), ok_bt, None)
    with pytest.raises(RuntimeError, match="kvq input check: .*outside"):
        ck.check_inputs(c["q"], c["k"], cu, torch.tensor([40, 20], dtype=torch.int32), ok_bt + 6, None)
    with pytest.raises(RuntimeError, match="seq_len 1 < q_len 2"):
        ck.check_inputs(c["q"], c["k"], cu, torch.tensor([40, 1], dtype=torch.int32), ok_bt, None)
    with pytest.raises(RuntimeError, match="pages > block_table width"):
        ck.check_inputs(c["q"], c["k"], cu, torch.tensor([400, 20], dtype=torch.int32), ok_bt, None)


def test_vllm_surface():
    pytest.importorskip("vllm")
    from kvq_b200 import vllm_plugin
    from kvq_b200.vllm_int8 import backend as b

    assert b.Int8StaticBackend.get_name() == "CUSTOM" and b.Int8StaticBackend.supported_kv_cache_dtypes == ["int8_static"]
    assert b.Int8StaticBackend.get_impl_cls() is b.Int8StaticImpl and b.Int8StaticBackend.get_builder_cls() is b.Int8StaticBuilder
    assert vllm_plugin.BACKEND_PATH.endswith("Int8StaticBackend")
    kv = torch.arange(2 * 2 * 16 * 4 * 8, dtype=torch.int32).to(torch.int8).reshape(2, 2, 16, 4, 8)
    k, v = b.split_kv_cache(kv, 8)
    assert k.shape == (2, 16, 4, 8) and torch.equal(k, kv[:, 0]) and torch.equal(v, kv[:, 1])
    kv32 = torch.zeros(2, 16, 4, 16, dtype=torch.int8).transpose(1, 2)     # logical [nb, H, block, 2D]
    k, v = b.split_kv_cache(kv32, 8)
    assert k.shape == (2, 16, 4, 8) and k.stride() == (1024, 64, 16, 1) and v.storage_offset() == 8


def test_long_path_policy(monkeypatch):
    """Chunked prefill goes to the INT8-page kernel by default, an explicit choice wins, a typo is an error."""
    monkeypatch.delenv("KVQ_LONG_PATH", raising=False)
    assert ck.long_path(64) == "int8" and ck.long_path(ck.INT8_LONG_MAX_Q) == "int8"
    monkeypatch.setattr(ck, "_FA_IMPORTABLE", False)
    assert ck.long_path(4096) == "int8"            # nothing else to run it on
    monkeypatch.setattr(ck, "_FA_IMPORTABLE", True)
    assert ck.long_path(4096) == "fa"
    monkeypatch.setenv("KVQ_LONG_PATH", "int8")
    assert ck.long_path(4096) == "int8"
    monkeypatch.setenv("KVQ_LONG_PATH", "fa")
    assert ck.long_path(16) == "fa"
    monkeypatch.setenv("KVQ_LONG_PATH", "flash")
    with pytest.raises(RuntimeError, match="KVQ_LONG_PATH"):
        ck.long_path(16)


def test_prefill_argument_errors_are_reported_without_a_gpu():
    lib = _native.lib()
    assert lib.kvq_prefill_workspace_size(100) >= 256 + 101 * 4 and lib.kvq_prefill_workspace_size(-1) == 0
    args = [1] * 9 + [0.1, 1, 16, 28, 4, 96, 16, 8] + [128] * 12 + [1, 1, 8, 1, 1024, None]
    assert lib.kvq_int8_prefill_attention(*args) == 1 and b"head_dim" in lib.kvq_last_error()
    args[14] = 128
    args[12] = 30                                   # 30 q heads over 4 kv heads
    assert lib.kvq_int8_prefill_attention(*args) == 1 and b"group" in lib.kvq_last_error()
    args[10] = 0                                    # empty batch: silent success, like the reference's early returns
    assert lib.kvq_int8_prefill_attention(*args) == 0


def test_short_q_is_one_threshold_everywhere():
    """KVQ_SHORT_Q above the INT8 kernel's limit is clamped with a warning, and every routing decision uses the
    clamped value: a request with 9 query tokens is planned as long (never left to a kernel that would skip it),
    one with 8 as short. A lower value is honoured; zero or less is rejected."""
    import subprocess
    import sys

    code = (
        "import sys, warnings; sys.path.insert(0, %r)\n"
        "with warnings.catch_warnings(record=True) as w:\n"
        "    warnings.simplefilter('always')\n"
        "    from kvq_b200 import cuda_kernels as ck\n"
        "import numpy as np\n"
        "plan = ck.plan_long(np.array([0, 9, 17, 18]), np.array([40, 50, 60]), 16)\n"
        "print(ck.SHORT_Q, ck.KERNEL_QMAX, len(w), None if plan is None else plan.src_req.tolist())\n"
    ) % os.path.join(ROOT, "int8-kvcache_b200")

    def run(value):
        env = dict(os.environ, KVQ_SHORT_Q=value)
        return subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)

    res = run("1000000")
    assert res.returncode == 0, res.stderr
    assert res.stdout.split(None, 3) == ["8", "8", "1", "[0, 0, 0]\n"], res.stdout   # 9 tokens -> 3 pages copied, 8 -> none
    res = run("4")
    assert res.stdout.split(None, 3) == ["4", "8", "0", "[0, 0, 0, 1, 1, 1, 1]\n"], res.stdout
    assert run("0").returncode != 0


# ---------------------------------------------------------------------------------------------------
# vLLM glue without an engine: scale hand-out, cache dtype registration, capture hook, calibration files
# ---------------------------------------------------------------------------------------------------
class _FakeImpl:
    """Stands in for a layer's Int8StaticImpl: records what set_static receives, completed like the real one."""

    def __init__(self, num_kv_heads, head_size=8):
        self.num_kv_heads, self.head_size, self.static = num_kv_heads, head_size, None

    def set_static(self, static):
        from kvq_b200.vllm_int8 import backend as b

        self.static = b.complete_static(static, self.num_kv_heads, self.head_size)


def _layer_table(layers, heads=4, dim=8, with_mu=True, offset=0.0):
    table = {}
    for i in range(layers):
        base = torch.arange(heads * dim, dtype=torch.float32).reshape(heads, dim) + 100 * i + offset
        table[f"model.layers.{i}.self_attn.attn"] = {"k_scale": base + 1, "v_scale": base + 2,
                                                     **({"k_mu": base + 3} if with_mu else {})}
    return table


def test_builder_hands_every_layer_its_rank_slice(tmp_path):
    """What Int8StaticBuilder.__init__ does with the scale files (reference: kvq/vllm_int8/backend.py:90-105): every
    layer gets its tensor-parallel rows; layers the target file does not know come from the draft file, looked up
    without the draft prefix; files without k_mu get zeros; replicated kv heads follow the replica rule."""
    pytest.importorskip("vllm")
    from kvq_b200.vllm_int8 import backend as b

    main_path, draft_path = str(tmp_path / "main.safetensors"), str(tmp_path / "draft.safetensors")
    scales.save(main_path, _layer_table(3))
    scales.save(draft_path, _layer_table(1, with_mu=False, offset=0.5))
    files = b.ScaleFiles.from_env({"KVQ_SCALES": main_path, "KVQ_DRAFT_SCALES": draft_path})
    names = [f"model.layers.{i}.self_attn.attn" for i in range(3)] + ["draft_model.model.layers.0.self_attn.attn"]
    for tp_size, rows in ((1, 4), (2, 2), (4, 1), (8, 1)):
        for rank in range(tp_size):
            impls = {n: _FakeImpl(rows) for n in names}
            drafted = b.assign_layer_scales(impls.__getitem__, names, files, rank, tp_size, torch.device("cpu"))
            assert drafted == 1
            full = _layer_table(3)
            for i in range(3):
                got, want = impls[names[i]].static, full[names[i]]
                for field in ("k_scale", "v_scale", "k_mu"):
                    assert torch.equal(got[field], scales.shard(want[field], rank, tp_size)), (tp_size, rank, field)
                    assert got[field].dtype == torch.float32 and got[field].is_contiguous()
            d = impls[names[3]].static
            assert torch.equal(d["k_scale"], scales.shard(_layer_table(1, offset=0.5)[names[0]]["k_scale"], rank, tp_size))
            assert d["k_mu"].shape == (rows, 8) and not d["k_mu"].any()          # no smooth-K in the draft file
    with pytest.raises(ValueError, match="kv heads"):
        _FakeImpl(3).set_static(scales.for_layer(_layer_table(1), names[0], 0, 1, "cpu"))
    with pytest.raises(KeyError):
        b.assign_layer_scales({"other.layer": _FakeImpl(4)}.__getitem__, ["other.layer"], files, 0, 1, "cpu")
    with pytest.raises(RuntimeError, match="KVQ_SCALES"):
        b.ScaleFiles.from_env({})


def test_graph_support_level_follows_the_short_query_limit():
    pytest.importorskip("vllm")
    from vllm.v1.attention.backend import AttentionCGSupport
    from kvq_b200.vllm_int8 import backend as b

    assert b.graph_support_level(0, AttentionCGSupport) == AttentionCGSupport.UNIFORM_BATCH
    assert b.graph_support_level(ck.SHORT_Q - 1, AttentionCGSupport) == AttentionCGSupport.UNIFORM_BATCH
    assert b.graph_support_level(ck.SHORT_Q, AttentionCGSupport) == AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    class Cfg:   # what the builder classmethod reads from vllm_config
        class speculative_config:
            num_speculative_tokens = 3

    assert b.Int8StaticBuilder.get_cudagraph_support(Cfg, None) == AttentionCGSupport.UNIFORM_BATCH
    Cfg.speculative_config = None
    assert b.Int8StaticBuilder.get_cudagraph_support(Cfg, None) == AttentionCGSupport.UNIFORM_BATCH


def test_plugin_registers_backend_and_cache_dtype():
    """register() in a fresh interpreter (it edits vLLM's config classes): the CUSTOM backend resolves to this
    package's class and an unpatched vLLM accepts kv_cache_dtype="int8_static" as an int8 cache."""
    pytest.importorskip("vllm")
    import subprocess
    import sys

    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "from kvq_b200 import vllm_plugin\n"
        "vllm_plugin.register(); vllm_plugin.register()\n"
        "import torch\n"
        "from vllm.config.cache import CacheConfig\n"
        "from vllm.utils.torch_utils import STR_DTYPE_TO_TORCH_DTYPE\n"
        "from vllm.v1.attention.backends.registry import AttentionBackendEnum\n"
        "assert CacheConfig(cache_dtype='int8_static').cache_dtype == 'int8_static'\n"
        "assert STR_DTYPE_TO_TORCH_DTYPE['int8_static'] is torch.int8\n"
        "cls = AttentionBackendEnum.CUSTOM.get_class()\n"
        "assert cls.__name__ == 'Int8StaticBackend' and cls.supports_kv_cache_dtype('int8_static')\n"
        "print('registered')\n"
    ) % os.path.join(ROOT, "int8-kvcache_b200")
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert res.returncode == 0 and "registered" in res.stdout, res.stderr[-2000:]


def test_capture_hook_wraps_the_cache_update(monkeypatch):
    """capture.install() against a stand-in for vLLM's FlashAttentionImpl (the reference's hook,
    kvq/capture.py:87-106): the original update still runs, with the same arguments, after the rows are recorded."""
    import sys
    import types

    from kvq_b200 import capture

    calls = []

    class FlashAttentionImpl:
        def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
            calls.append(("orig", layer.layer_name, key, value, kv_cache, slot_mapping))
            return "written"

    fake = types.ModuleType("vllm.v1.attention.backends.flash_attn")
    fake.FlashAttentionImpl = FlashAttentionImpl
    for name in ("vllm", "vllm.v1", "vllm.v1.attention", "vllm.v1.attention.backends"):
        monkeypatch.setitem(sys.modules, name, sys.modules.get(name) or types.ModuleType(name))
    monkeypatch.setitem(sys.modules, "vllm.v1.attention.backends.flash_attn", fake)
    monkeypatch.setattr(capture, "record", lambda *a: calls.append(("record",) + a))
    capture.install()
    layer = types.SimpleNamespace(layer_name="model.layers.0.self_attn.attn")
    assert FlashAttentionImpl().do_kv_cache_update(layer, "k", "v", "cache", "slots") == "written"
    assert calls == [("record", "model.layers.0.self_attn.attn", "k", "v", "slots"),
                     ("orig", "model.layers.0.self_attn.attn", "k", "v", "cache", "slots")]
    del FlashAttentionImpl.do_kv_cache_update     # a backend without the method: loud failure, not a silent no-op
    with pytest.raises(RuntimeError, match="do_kv_cache_update"):
        capture.install()


def test_calibrate_from_writes_the_six_variants(tmp_path):
    """Per-rank capture results -> one scale file per (granularity, method, smooth) variant, merged over two
    tensor-parallel ranks; file names follow the reference's scale files; quantile variants are skipped without
    samples."""
    gen = torch.Generator().manual_seed(3)
    rows, heads, dim = 50, 2, 8

    def rank_result(rank):
        k = torch.randn(rows, heads, dim, generator=gen) * 2 + 1
        v = torch.randn(rows, heads, dim, generator=gen)
        st = {"tokens": rows, "k_absmax": k.abs().amax(0), "k_max": k.amax(0), "k_min": k.amin(0), "k_sum": k.double().sum(0),
              "v_absmax": v.abs().amax(0), "v_max": v.amax(0), "v_min": v.amin(0), "v_sum": v.double().sum(0)}
        return {"stats": {"L0": st}, "samples": {"L0": {"k": k.half(), "v": v.half()}}, "tp_rank": rank, "tp_size": 2}

    per_rank = [rank_result(1), rank_result(0)]
    summary = scales.calibrate_from(per_rank, num_kv_heads=4, out_dir=str(tmp_path), prefix="math")
    assert summary["tokens"] == rows and len(summary["variants"]) == 6
    assert "math_per_channel_max_smooth.safetensors" in summary["variants"]
    assert "math_per_head_max.safetensors" in summary["variants"]
    loaded = scales.load(str(tmp_path / "math_per_channel_max_smooth.safetensors"))["L0"]
    assert loaded["k_scale"].shape == (4, dim) and loaded["k_mu"].shape == (4, dim)       # two ranks x two heads
    by_rank = sorted(per_rank, key=lambda r: r["tp_rank"])
    want = torch.cat([r["stats"]["L0"]["v_absmax"] for r in by_rank]) / 127.0
    assert torch.allclose(loaded["v_scale"], want)
    assert scales.load(str(tmp_path / "math_per_head_max.safetensors"))["L0"]["k_scale"].shape == (4, 1)
    for r in per_rank:
        r["samples"] = {}
    assert len(scales.calibrate_from(per_rank, 4, str(tmp_path / "nosamples"))["variants"]) == 4


def test_wire_header_round_trip_and_refusals():
    """The payload description of the int8 page wire format: geometry and a digest of the layer's scales travel with
    the pages, and a receiver with another geometry, other scales or an unknown format tag refuses them."""
    import json

    from kvq_b200 import wire

    static = {"k_scale": torch.rand(4, 128) + 0.01, "v_scale": torch.rand(4, 128) + 0.01, "k_mu": torch.randn(4, 128)}
    raw = wire.header("model.layers.3.self_attn.attn", num_tokens=100, num_pages=7, block_size=16, num_kv_heads=4,
                      head_dim=128, static=static)
    h = wire.check_header(raw, 16, 4, 128, static)
    assert h["pages"] == 7 and h["tokens"] == 100 and h["bytes"] == 7 * 2 * 16 * 4 * 128 and h["dtype"] == "int8"
    with pytest.raises(RuntimeError, match="head_dim"):
        wire.check_header(raw, 16, 4, 64, static)
    with pytest.raises(RuntimeError, match="other static scales"):
        wire.check_header(raw, 16, 4, 128, dict(static, k_mu=static["k_mu"] + 1))
    bad = json.loads(raw)
    bad["format"] = "something-else/9"
    with pytest.raises(RuntimeError, match="unknown KV wire format"):
        wire.check_header(json.dumps(bad).encode(), 16, 4, 128, static)
    with pytest.raises(RuntimeError, match="no CPU path"):
        wire.export_pages(torch.zeros(2, 16, 4, 128, dtype=torch.int8), torch.zeros(2, 16, 4, 128, dtype=torch.int8), [0])


def _split_reference(q_lens, seq_lens, G, Hkv, qmax, item_cost, nctas):
    """Pure-Python statement of how the attention kernel divides a single-token-decode batch over its CTAs: an item
    (request, kv head) is `item_cost` of start-up followed by ceil(L / 32) chunks; CTAs take equal shares of that
    cost; a share boundary inside a start-up belongs to the item's first chunk."""
    items = []   # (first global unit, chunks) per item, in order
    unit = 0
    for ql, L in zip(q_lens, seq_lens):
        if ql < 1 or ql > qmax:
            continue
        n = max(1, -(-L // 32))
        for _ in range(Hkv):
            items.append((unit, n))
            unit += n
    total = unit
    total_f = total + item_cost * len(items)
    wf = max(-(-total_f // nctas), 4)

    def unit_of(f):
        if f >= total_f:
            return total
        c = 0
        for first, n in items:
            if f < c + item_cost + n:
                return first + max(0, f - c - item_cost)
            c += item_cost + n
        return total
    return [unit_of(b * wf) for b in range(nctas)], [unit_of((b + 1) * wf) for b in range(nctas)], total, items


def test_decode_split_is_contiguous_cost_balanced_and_snaps_to_items():
    """kvq_debug_decode_split (the host restatement of the kernel's own split, same inline functions): the ranges tile
    the units in order, equal the pure-Python statement, no range costs more than a share, and with an item cost
    ranges begin at item starts far more often than an even split of the units would."""
    import ctypes

    from kvq_b200 import _native
    lib = _native.lib()
    rng = np.random.default_rng(7)
    for (b, lo, hi, nctas, cost) in [(1, 32768, 32768, 296, 20), (8, 32768, 32768, 296, 20), (16, 32768, 32768, 296, 14),
                                     (128, 32768, 32768, 296, 20), (37, 1, 5000, 296, 20), (300, 17, 900, 296, 0),
                                     (5, 1, 40, 296, 20), (64, 4096, 4096, 148, 28)]:
        seq = rng.integers(lo, hi + 1, b).astype(np.int32)
        ql = np.ones(b, dtype=np.int32)
        if b > 4:
            ql[3] = 0          # a padded request has no work
        ub = np.zeros(nctas, dtype=np.int32)
        ue = np.zeros(nctas, dtype=np.int32)
        rc = lib.kvq_debug_decode_split(ql.ctypes.data_as(ctypes.c_void_p), seq.ctypes.data_as(ctypes.c_void_p), b, 7, 4, 8,
                                        0, 0, cost, nctas, ub.ctypes.data_as(ctypes.c_void_p), ue.ctypes.data_as(ctypes.c_void_p))
        assert rc == 0
        rb, re_, total, items = _split_reference(ql.tolist(), seq.tolist(), 7, 4, 8, cost, nctas)
        assert ub.tolist() == rb and ue.tolist() == re_
        assert ub[0] == 0 and ue[-1] == total and np.all(ub[1:] == ue[:-1]) and np.all(ue >= ub)
        starts = {first for first, _ in items}
        share = max(-(-(total + cost * len(items)) // nctas), 4)
        for lo_u, hi_u in zip(ub.tolist(), ue.tolist()):
            inside = sum(1 for s in starts if lo_u < s < hi_u)      # item starts strictly inside the range
            assert (hi_u - lo_u) + cost * inside <= share
    # snapping: 8 x 32768 over 296 CTAs; ranges that begin exactly at an item start
    seq = np.full(8, 32768, dtype=np.int32)
    ql = np.ones(8, dtype=np.int32)
    snapped = {}
    for cost in (0, 20):
        rb, _, _, items = _split_reference(ql.tolist(), seq.tolist(), 7, 4, 8, cost, 296)
        starts = {first for first, _ in items}
        snapped[cost] = sum(1 for u in rb if u in starts)
    assert snapped[20] >= 4 * snapped[0]


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` (the reference's CPU implementation on the host cores) runs without a GPU and prints
    one JSON line with the keys the measurement contract names."""
    import json
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=root)
    assert res.returncode == 0, res.stderr[-500:]
    line = json.loads([ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["metric"] == "int8_paged_decode_attention_kv_bandwidth_128x32k" and line["steps"] == 1
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert "workload" in line["config"] and line["gpu_launches"] == 0
