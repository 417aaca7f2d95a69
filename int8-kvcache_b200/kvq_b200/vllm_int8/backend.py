"""Static INT8 KV-cache attention backend for vLLM, registered as AttentionBackendEnum.CUSTOM.

Same surface as the reference's kvq/vllm_int8/backend.py:48-184 (class names, get_name() == "CUSTOM",
supported_kv_cache_dtypes == ["int8_static"], KVQ_SCALES / KVQ_DRAFT_SCALES, scales handed to every layer by
the metadata builder, CUDA-graph support level, routing by query length), with the kernels of kvq_b200.
Run with kv_cache_dtype="int8_static" and attention_config={"backend": "CUSTOM"}.

Differences from the reference, on purpose:
  * there is no PyTorch ("KVQ_KERNEL=torch") path: the CUDA kernels are the only implementation;
  * split-KV needs no vLLM scratch: the kernel balances work over the SMs itself;
  * both vLLM cache layouts are understood: [num_blocks, 2, block, H, D] (vLLM <= 0.2x Triton backend) and
    the logical [num_blocks, H, block, 2 * D] of vLLM 0.32 (kvq/vllm_int8/backend.py:145-147).
The metadata (lengths, block table) is reused from vLLM's Triton backend, which this subclasses.
"""
import os
from typing import ClassVar

import torch
from vllm.logger import init_logger
from vllm.v1.attention.backend import AttentionCGSupport
from vllm.v1.attention.backends.triton_attn import (
    TritonAttentionBackend,
    TritonAttentionImpl,
    TritonAttentionMetadataBuilder,
)

from kvq_b200 import cuda_kernels, scales

logger = init_logger("vllm.kvq")
_SCALES_CACHE = {}
KV_CACHE_DTYPE = "int8_static"


def _load_scales(path):
    if path not in _SCALES_CACHE:
        _SCALES_CACHE[path] = scales.load(path)
    return _SCALES_CACHE[path]


def split_kv_cache(kv_cache, head_size):
    """Two [num_blocks, block, H, D] int8 views (K, V) of vLLM's combined cache tensor, whichever layout it has."""
    if kv_cache.dim() == 5:                      # [num_blocks, 2, block, H, D]
        return kv_cache[:, 0], kv_cache[:, 1]
    return kv_cache.transpose(1, 2).split(head_size, dim=-1)   # logical [num_blocks, H, block, 2 * D]


class Int8StaticBackend(TritonAttentionBackend):
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
        return spec   # the scales live in the backend, not inside the KV pages


class Int8StaticBuilder(TritonAttentionMetadataBuilder):
    """Triton-backend metadata plus, for a batch with long queries, the page table of the temporary bf16
    cache (cuda_kernels.plan_long), computed once per step for all layers. The builder is created after the
    model is loaded and before CUDA graphs are captured, so it is where every layer receives its static
    scales as persistent tensors (kvq/vllm_int8/backend.py:68-115)."""

    supports_draft_decode_metadata_update = False

    @classmethod
    def get_cudagraph_support(cls, vllm_config, kv_cache_spec):
        # Full graphs for uniform batches the INT8 kernel covers alone; the long-query path sizes buffers from
        # host-side lengths, so mixed batches run attention eagerly.
        spec = vllm_config.speculative_config
        q_len = 1 + (spec.num_speculative_tokens if spec is not None else 0)
        if q_len <= cuda_kernels.SHORT_Q:
            return AttentionCGSupport.UNIFORM_BATCH
        return AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size

        path = os.environ["KVQ_SCALES"]
        all_scales = _load_scales(path)
        ctx = vllm_config.compilation_config.static_forward_context
        rank, size = get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
        for name in layer_names:
            src, key = all_scales, name
            if name not in all_scales and os.environ.get("KVQ_DRAFT_SCALES"):
                # speculative-decoding draft model ("draft_model." prefix): its own calibration file
                src, key = _load_scales(os.environ["KVQ_DRAFT_SCALES"]), name[name.index("model.layers"):]
            ctx[name].impl.set_static(scales.for_layer(src, key, rank, size, device))
        logger.info("kvq_b200: static INT8 scales for %d layers from %s (tp %d/%d)", len(layer_names), path, rank, size)

    def build(self, common_prefix_len, common_attn_metadata, fast_build=False):
        md = super().build(common_prefix_len, common_attn_metadata, fast_build)
        md.kvq_long = None
        c = common_attn_metadata
        if c.max_query_len > cuda_kernels.SHORT_Q:
            upper = getattr(c, "seq_lens_cpu_upper_bound", None)
            seq_cpu = upper if upper is not None else c.seq_lens.cpu()
            md.kvq_long = cuda_kernels.plan_long(c.query_start_loc_cpu, seq_cpu, self.block_size)
        return md


class Int8StaticImpl(TritonAttentionImpl):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        if self.kv_cache_dtype != KV_CACHE_DTYPE:
            raise ValueError(f"Int8StaticImpl needs kv_cache_dtype={KV_CACHE_DTYPE!r}, got {self.kv_cache_dtype!r}")
        self.static = None
        cuda_kernels.ext()   # load the native library at model build time, long before any graph capture

    def fused_output_quant_supported(self, quant_key):
        return False   # the kernels write bf16 output only

    def set_static(self, static):
        if static["k_scale"].shape[0] != self.num_kv_heads:
            raise ValueError(f"scale rows {tuple(static['k_scale'].shape)} != {self.num_kv_heads} kv heads")
        static = {k: v.float().contiguous() for k, v in static.items()}
        if "k_mu" not in static:
            static["k_mu"] = torch.zeros_like(static["k_scale"].expand(-1, self.head_size)).contiguous()
        self.static = static

    def _caches(self, kv_cache):
        return split_kv_cache(kv_cache, self.head_size)

    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
        key_cache, value_cache = self._caches(kv_cache)
        cuda_kernels.quant_reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, self.static)

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
                output_block_scale=None):
        if attn_metadata is None:
            return output.fill_(0)   # profiling run
        md = attn_metadata
        n = md.num_actual_tokens
        key_cache, value_cache = self._caches(kv_cache)
        cuda_kernels.paged_attention(query[:n], key_cache, value_cache, output[:n], md.query_start_loc, md.seq_lens,
                                     md.block_table, md.max_query_len, self.scale, self.static,
                                     getattr(md, "kvq_long", None), None)
        return output
