"""vLLM general-plugin entry point: registers the static INT8 backend as AttentionBackendEnum.CUSTOM.

vLLM calls register() in every process it starts, before the model is built (same contract as the
reference's kvq/vllm_plugin.py:9-13). Registration is by class path, so the backend module is imported only
when vLLM selects it. With KVQ_CAPTURE=1 the calibration capture hook is installed as in the reference
(kvq/vllm_plugin.py:14-17); its attention-override and MLA study hooks are debugging tools and are not part
of this package.

The reference adds the "int8_static" cache dtype to vLLM with a source patch
(patches/vllm-0.32.0-int8-static-kv.patch: one entry in CacheDType, one in the string -> torch dtype table, one
quantization-mode enum value). register_cache_dtype() makes the first two additions at run time, in the process
that calls it, so that an unpatched vLLM accepts kv_cache_dtype="int8_static" and allocates the cache as torch.int8;
the third is not needed (an unknown dtype string maps to "no vLLM-side KV quantization", which is what a backend
that owns its scales wants).
"""
import os

BACKEND_PATH = "kvq_b200.vllm_int8.backend.Int8StaticBackend"
KV_CACHE_DTYPE = "int8_static"


def register_cache_dtype():
    """Teach this process's vLLM the "int8_static" cache dtype. Idempotent. Returns True when vLLM already knew it or
    now accepts it; raises RuntimeError naming the check that still refuses it otherwise."""
    import typing

    import torch
    from vllm.config import cache as vllm_cache
    from vllm.utils import torch_utils

    torch_utils.STR_DTYPE_TO_TORCH_DTYPE.setdefault(KV_CACHE_DTYPE, torch.int8)
    literal = vllm_cache.CacheDType
    if KV_CACHE_DTYPE not in typing.get_args(literal):
        # CacheDType is a typing.Literal; pydantic compiled its allowed values into the validators of every config
        # dataclass that mentions it, so those are rebuilt after the value is appended
        literal.__args__ = tuple(literal.__args__) + (KV_CACHE_DTYPE,)
        from pydantic.dataclasses import rebuild_dataclass

        rebuild_dataclass(vllm_cache.CacheConfig, force=True)
        try:
            from vllm.config.vllm import VllmConfig

            rebuild_dataclass(VllmConfig, force=True)
        except Exception:  # noqa: BLE001  (older layouts keep VllmConfig elsewhere; CacheConfig is what validates the string)
            pass
    try:
        vllm_cache.CacheConfig(cache_dtype=KV_CACHE_DTYPE)
    except Exception as e:  # noqa: BLE001
        raise RuntimeError(f"kvq_b200: this vLLM still rejects kv_cache_dtype={KV_CACHE_DTYPE!r} in CacheConfig: {e}") from e
    return True


def register():
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(AttentionBackendEnum.CUSTOM, BACKEND_PATH)
    register_cache_dtype()
    if os.environ.get("KVQ_CAPTURE") == "1":
        from . import capture

        capture.install()
