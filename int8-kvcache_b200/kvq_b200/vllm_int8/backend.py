"""Static INT8 KV-cache attention backend for vLLM, registered as AttentionBackendEnum.CUSTOM.

Drop-in for the reference's kvq/vllm_int8/backend.py:48-184: the same class names, get_name() == "CUSTOM",
supported_kv_cache_dtypes == ["int8_static"], the KVQ_SCALES / KVQ_DRAFT_SCALES files, scales handed to every
layer when the metadata builder is created, the CUDA-graph support level and the routing by query length.
Run with kv_cache_dtype="int8_static" and attention_config={"backend": "CUSTOM"}.

How this module is organised (everything vLLM-free lives in plain functions so that it can be tested without an
engine):
  ScaleFiles            the calibration files of a run: which file and which key serve a layer name
  assign_layer_scales   hands every attention layer its tensor-parallel slice of the scales
  complete_static       what a layer keeps: contiguous fp32 tensors, k_mu zero-filled when the file has none
  split_kv_cache        K and V views of vLLM's combined cache tensor, for either cache layout
  graph_support_level   full CUDA graphs for which batches
and the three vLLM classes only adapt those to vLLM's interfaces.

Differences from the reference, on purpose:
  * there is no PyTorch ("KVQ_KERNEL=torch") path and no KVQ_CFG switch: the CUDA kernels are the only
    implementation, with the numerics of the reference's CUDA path (implementation B, per-(token, head) q scale,
    P quantized per 32-key tile);
  * split-KV needs no vLLM scratch: the kernel balances work over the SMs itself;
  * both vLLM cache layouts are understood: [num_blocks, 2, block, H, D] (vLLM 0.2x) and the logical
    [num_blocks, H, block, 2 * D] of vLLM 0.32 (kvq/vllm_int8/backend.py:145-147).
"""
import os
from typing import ClassVar

import torch

from kvq_b200 import cuda_kernels, scales

KV_CACHE_DTYPE = "int8_static"
DRAFT_ANCHOR = "model.layers"   # a draft model's layer names are "<prefix>.model.layers.N...."; its file has no prefix


class ScaleFiles:
    """The scale files of one run: the target model's (KVQ_SCALES) and, optionally, the speculative-decoding draft
    model's own calibration (KVQ_DRAFT_SCALES). Files are parsed once per process."""

    _parsed = {}

    def __init__(self, main_path, draft_path=None):
        self.main_path, self.draft_path = main_path, draft_path

    @classmethod
    def from_env(cls, env=os.environ):
        if "KVQ_SCALES" not in env:
            raise RuntimeError("kvq_b200: the int8_static backend needs KVQ_SCALES=<calibrated scale file>")
        return cls(env["KVQ_SCALES"], env.get("KVQ_DRAFT_SCALES") or None)

    @classmethod
    def table(cls, path):
        if path not in cls._parsed:
            cls._parsed[path] = scales.load(path)
        return cls._parsed[path]

    def lookup(self, layer_name):
        """(table, key) that hold the scales of `layer_name`. A name the target model's file does not know belongs to
        the draft model when a draft file was given: it is looked up there without the draft prefix."""
        main = self.table(self.main_path)
        if layer_name in main or not self.draft_path:
            return main, layer_name          # a missing name fails in for_layer with the layer's name in the KeyError
        if DRAFT_ANCHOR not in layer_name:
            raise KeyError(f"{layer_name}: not in {self.main_path} and not a draft-model layer name")
        return self.table(self.draft_path), layer_name[layer_name.index(DRAFT_ANCHOR):]


def complete_static(static, num_kv_heads, head_size):
    """A layer's scales as the kernels want them: contiguous fp32; k_mu (smooth-K mean) all zeros when the file was
    calibrated without smooth-K, so that one code path serves both (kvq/vllm_int8/backend.py:136-142)."""
    rows = static["k_scale"].shape[0]
    if rows != num_kv_heads:
        raise ValueError(f"scale rows {tuple(static['k_scale'].shape)} != {num_kv_heads} kv heads of this rank")
    out = {name: t.float().contiguous() for name, t in static.items()}
    if "k_mu" not in out:
        out["k_mu"] = torch.zeros(rows, head_size, dtype=torch.float32, device=out["k_scale"].device)
    return out


def assign_layer_scales(impl_of, layer_names, files, tp_rank, tp_size, device):
    """Give every attention layer (impl_of(name) -> its Int8StaticImpl) this rank's rows of its scales
    (scales.for_layer applies the tensor-parallel rule, incl. replicated kv heads). Returns the number of layers that
    came from the draft file."""
    from_draft = 0
    for name in layer_names:
        table, key = files.lookup(name)
        from_draft += table is not files.table(files.main_path)
        impl_of(name).set_static(scales.for_layer(table, key, tp_rank, tp_size, device))
    return from_draft


def split_kv_cache(kv_cache, head_size):
    """Two [num_blocks, block, H, D] int8 views (K, V) of vLLM's combined cache tensor, whichever layout it has."""
    if kv_cache.dim() == 5:                      # [num_blocks, 2, block, H, D]
        return kv_cache[:, 0], kv_cache[:, 1]
    return kv_cache.transpose(1, 2).split(head_size, dim=-1)   # logical [num_blocks, H, block, 2 * D]


def graph_support_level(num_speculative_tokens, levels):
    """Full CUDA graphs cover the batches the INT8 kernel serves alone: uniform batches of 1 + k query tokens per
    request while that fits the kernel (cuda_kernels.SHORT_Q), single-token decode otherwise. The long-query path
    sizes buffers from host-side lengths, so batches that contain it run attention eagerly
    (kvq/vllm_int8/backend.py:78-88). `levels` is vLLM's AttentionCGSupport."""
    uniform_q_len = 1 + (num_speculative_tokens or 0)
    return levels.UNIFORM_BATCH if uniform_q_len <= cuda_kernels.SHORT_Q else levels.UNIFORM_SINGLE_TOKEN_DECODE


try:   # the vLLM classes exist only where vLLM is installed; the helpers above do not need it
    from vllm.logger import init_logger
    from vllm.v1.attention.backend import AttentionCGSupport
    from vllm.v1.attention.backends.triton_attn import (
        TritonAttentionBackend,
        TritonAttentionImpl,
        TritonAttentionMetadataBuilder,
    )
except ImportError as e:   # noqa: F841
    _VLLM_IMPORT_ERROR = e
else:
    _VLLM_IMPORT_ERROR = None
    logger = init_logger("vllm.kvq")

    class Int8StaticBackend(TritonAttentionBackend):
        """Backend descriptor. The metadata (lengths, block table) is vLLM's Triton backend's, which this subclasses;
        the cache spec is left alone because the scales live in the backend, not inside the KV pages."""
        supported_kv_cache_dtypes: ClassVar[list] = [KV_CACHE_DTYPE]

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_impl_cls():
            return Int8StaticImpl

        @staticmethod
        def get_builder_cls():
            return Int8StaticBuilder

        @classmethod
        def customize_spec(cls, spec):
            return spec

    class Int8StaticBuilder(TritonAttentionMetadataBuilder):
        """Triton-backend metadata plus, for a batch with long queries, the page table of the temporary bf16 cache
        (cuda_kernels.plan_long), computed once per step for all layers. vLLM creates the builder after the model is
        loaded and before CUDA graphs are captured: the moment every layer receives its static scales as persistent
        tensors (kvq/vllm_int8/backend.py:68-115)."""

        # a draft-decode step that reused an earlier metadata object would reuse its long-query plan too
        supports_draft_decode_metadata_update = False

        @classmethod
        def get_cudagraph_support(cls, vllm_config, kv_cache_spec):
            spec = vllm_config.speculative_config
            return graph_support_level(spec.num_speculative_tokens if spec is not None else 0, AttentionCGSupport)

        def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
            super().__init__(kv_cache_spec, layer_names, vllm_config, device)
            from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size

            files = ScaleFiles.from_env()
            layers = vllm_config.compilation_config.static_forward_context
            rank, size = get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
            drafted = assign_layer_scales(lambda name: layers[name].impl, layer_names, files, rank, size, device)
            logger.info("kvq_b200: static INT8 scales for %d layers from %s (%d from the draft file), tp rank %d of %d",
                        len(layer_names), files.main_path, drafted, rank, size)

        def build(self, common_prefix_len, common_attn_metadata, fast_build=False):
            md = super().build(common_prefix_len, common_attn_metadata, fast_build)
            batch = common_attn_metadata
            md.kvq_long = None
            if batch.max_query_len > cuda_kernels.SHORT_Q:
                # host-side lengths may be upper bounds (asynchronous scheduling): they only size the page copy
                host_lens = getattr(batch, "seq_lens_cpu_upper_bound", None)
                if host_lens is None:
                    host_lens = batch.seq_lens.cpu()
                md.kvq_long = cuda_kernels.plan_long(batch.query_start_loc_cpu, host_lens, self.block_size)
            return md

    class Int8StaticImpl(TritonAttentionImpl):
        """Per-layer attention: new K/V are quantized with the layer's static scales on their way into the int8 cache,
        attention reads the int8 pages (kvq/vllm_int8/backend.py:118-184)."""

        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            if self.kv_cache_dtype != KV_CACHE_DTYPE:
                raise ValueError(f"Int8StaticImpl needs kv_cache_dtype={KV_CACHE_DTYPE!r}, got {self.kv_cache_dtype!r}")
            self.static = None
            cuda_kernels.ext()   # load the native library at model build time, long before any graph capture

        def fused_output_quant_supported(self, quant_key):
            return False   # the kernels write bf16 output only

        def set_static(self, static):
            self.static = complete_static(static, self.num_kv_heads, self.head_size)

        def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
            k_pages, v_pages = split_kv_cache(kv_cache, self.head_size)
            cuda_kernels.quant_reshape_and_cache(key, value, k_pages, v_pages, slot_mapping, self.static)

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
                    output_block_scale=None):
            if attn_metadata is None:      # vLLM's memory-profiling run
                return output.fill_(0)
            rows = attn_metadata.num_actual_tokens
            k_pages, v_pages = split_kv_cache(kv_cache, self.head_size)
            cuda_kernels.paged_attention(query[:rows], k_pages, v_pages, output[:rows], attn_metadata.query_start_loc,
                                         attn_metadata.seq_lens, attn_metadata.block_table, attn_metadata.max_query_len,
                                         self.scale, self.static, plan=getattr(attn_metadata, "kvq_long", None))
            return output


def __getattr__(name):
    if name in ("Int8StaticBackend", "Int8StaticBuilder", "Int8StaticImpl") and _VLLM_IMPORT_ERROR is not None:
        raise ImportError(f"kvq_b200.vllm_int8.backend.{name} needs vLLM: {_VLLM_IMPORT_ERROR}")
    raise AttributeError(name)
