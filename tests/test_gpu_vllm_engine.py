"""The backend inside a running vLLM engine (the installed vLLM, unpatched): calibrate on the stock bf16 cache with the
capture hook, write the scale files, then serve the same prompts from an int8_static cache through the CUSTOM backend,
eagerly and under vLLM's CUDA graphs.

The model is a 2-layer decoder with the attention geometry of the benchmark layer (28 q heads, 4 kv heads, head_dim
128) and vLLM's random "dummy" weights; prompts are random token ids. No checkpoint, tokenizer or dataset is involved.
What is checked:
  * the capture hook sees every layer and every prompt token, and calibrate_from writes loadable scale files;
  * vLLM accepts kv_cache_dtype="int8_static" after the plugin's register(), allocates int8 cache tensors and selects
    Int8StaticBackend; every layer received scales; do_kv_cache_update and forward run for prefill and decode;
  * one decode step of layer 0, recorded in the eager engine (queries, the int8 pages vLLM's block table points at,
    metadata, output), meets the attention bar against the CPU oracle;
  * the engine with full CUDA graphs for uniform decode batches (forward reached during capture) generates the same
    tokens as the eager int8 engine: the kernels are deterministic, so replayed steps equal eager steps.
"""
import gc
import json
import os

import numpy as np
import pytest
import torch
from gpu_util import assert_close

from oracle import kvq_oracle as orc

pytestmark = pytest.mark.gpu

MODEL_CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 3584, "intermediate_size": 1024,
    "num_hidden_layers": 2, "num_attention_heads": 28, "num_key_value_heads": 4, "vocab_size": 1024,
    "max_position_embeddings": 4096, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "hidden_act": "silu",
    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
}
LAYER0 = "model.layers.0.self_attn.attn"


def _prompts():
    rng = np.random.default_rng(7)
    return [{"prompt_token_ids": rng.integers(3, 1024, size=n).tolist()} for n in (23, 150, 64, 301, 9, 77, 512, 40)]


def _engine(model_dir, **kw):
    from vllm import LLM

    return LLM(model=model_dir, skip_tokenizer_init=True, load_format="dummy", dtype="bfloat16", max_model_len=2048,
               max_num_seqs=16, gpu_memory_utilization=0.15, seed=0, enable_prefix_caching=False, **kw)


def _generate(llm, max_tokens=12):
    from vllm import SamplingParams

    outs = llm.generate(_prompts(), SamplingParams(temperature=0, max_tokens=max_tokens, detokenize=False, ignore_eos=True))
    return [list(o.outputs[0].token_ids) for o in outs]


def _release(llm):
    """Tear an in-process engine down before the next one takes its memory snapshot. The caller drops its own
    reference with `llm = _release(llm)`."""
    try:
        llm.llm_engine.engine_core.shutdown()
    except Exception:  # noqa: BLE001  (best effort: the garbage collector below does the rest)
        pass
    del llm
    for _ in range(2):
        gc.collect()
    torch.cuda.empty_cache()
    torch.cuda.synchronize()
    return None


def test_calibrate_then_serve_from_the_int8_cache(tmp_path, monkeypatch):
    pytest.importorskip("vllm")
    monkeypatch.setenv("VLLM_ENABLE_V1_MULTIPROCESSING", "0")     # engine core in this process: hooks and counters are visible
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(MODEL_CONFIG))

    from kvq_b200 import capture, scales, vllm_plugin

    # ---- 1. calibration on the stock bf16 cache, FlashAttention backend hooked by the plugin ----
    monkeypatch.setenv("KVQ_CAPTURE", "1")
    capture.reset()
    vllm_plugin.register()
    llm = _engine(str(model_dir), enforce_eager=True, attention_config={"backend": "FLASH_ATTN"})
    _generate(llm, max_tokens=4)
    result = capture.collect(tp_rank=0, tp_size=1)
    llm = _release(llm)
    monkeypatch.delenv("KVQ_CAPTURE")
    prompt_tokens = sum(len(p["prompt_token_ids"]) for p in _prompts())
    assert set(result["stats"]) == {LAYER0, "model.layers.1.self_attn.attn"}
    assert result["stats"][LAYER0]["tokens"] >= prompt_tokens            # every prompt token (plus the generated ones)
    summary = scales.calibrate_from([result], num_kv_heads=4, out_dir=str(tmp_path / "scales"), prefix="dummy")
    assert len(summary["variants"]) == 6
    scale_file = str(tmp_path / "scales" / "dummy_per_channel_max_smooth.safetensors")
    assert set(scales.load(scale_file)[LAYER0]) == {"k_scale", "v_scale", "k_mu"}

    # ---- 2. int8_static cache through the CUSTOM backend, eager: reachability and one recorded decode step ----
    monkeypatch.setenv("KVQ_SCALES", scale_file)
    from kvq_b200.vllm_int8 import backend as b

    seen = {"update": 0, "forward": 0, "forward_capturing": 0, "cache_dtypes": set(), "step": None}
    real_forward, real_update = b.Int8StaticImpl.forward, b.Int8StaticImpl.do_kv_cache_update

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output, *a, **kw):
        out = real_forward(self, layer, query, key, value, kv_cache, attn_metadata, output, *a, **kw)
        if attn_metadata is None:
            return out
        seen["forward"] += 1
        seen["cache_dtypes"].add(kv_cache.dtype)
        if torch.cuda.is_current_stream_capturing():
            seen["forward_capturing"] += 1
        elif seen["step"] is None and layer.layer_name == LAYER0 and attn_metadata.max_query_len == 1:
            torch.cuda.synchronize()
            md, n = attn_metadata, attn_metadata.num_actual_tokens
            reqs = md.query_start_loc.shape[0] - 1
            k_pages, v_pages = b.split_kv_cache(kv_cache, self.head_size)
            table = md.block_table[:reqs].cpu().numpy()
            lens = md.seq_lens[:reqs].cpu().numpy()
            used = np.unique(np.concatenate([table[r, :(lens[r] + k_pages.shape[1] - 1) // k_pages.shape[1]] for r in range(reqs)]))
            remap = {int(p): i for i, p in enumerate(used)}
            compact = np.vectorize(lambda p: remap.get(int(p), 0))(table).astype(np.int32)
            idx = torch.as_tensor(used, device=kv_cache.device).long()
            seen["step"] = dict(q=query[:n].float().cpu().numpy(), out=output[:n].float().cpu().numpy(),
                                k=k_pages[idx].cpu().numpy(), v=v_pages[idx].cpu().numpy(), table=compact, lens=lens,
                                cu=md.query_start_loc.cpu().numpy(), scale=self.scale,
                                static={k: t.cpu().numpy() for k, t in self.static.items()})
        return out

    def update(self, *a, **kw):
        seen["update"] += 1
        return real_update(self, *a, **kw)

    monkeypatch.setattr(b.Int8StaticImpl, "forward", forward)
    monkeypatch.setattr(b.Int8StaticImpl, "do_kv_cache_update", update)
    llm = _engine(str(model_dir), enforce_eager=True, kv_cache_dtype="int8_static", attention_config={"backend": "CUSTOM"})
    eager_tokens = _generate(llm)
    llm = _release(llm)
    assert seen["cache_dtypes"] == {torch.int8} and seen["update"] > 0 and seen["forward"] > 0
    step = seen["step"]
    assert step is not None, "no decode step of layer 0 was seen"
    ref = orc.paged_static_attention(step["q"], step["k"], step["v"], step["cu"], step["lens"], step["table"], step["scale"],
                                     step["static"]["k_scale"], step["static"]["v_scale"])
    assert_close(ref, step["out"], "layer 0 decode step inside the engine")

    # ---- 3. the same engine with CUDA graphs: forward is captured, replayed steps reproduce the eager tokens ----
    seen.update(forward=0, forward_capturing=0, step="skip")
    llm = _engine(str(model_dir), kv_cache_dtype="int8_static", attention_config={"backend": "CUSTOM"})
    graph_tokens = _generate(llm)
    llm = _release(llm)
    assert seen["forward_capturing"] > 0, "forward was never reached under CUDA graph capture"
    assert graph_tokens == eager_tokens
