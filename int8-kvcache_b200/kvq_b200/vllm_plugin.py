"""vLLM general-plugin entry point: registers the static INT8 backend as AttentionBackendEnum.CUSTOM.

vLLM calls register() in every process it starts, before the model is built (same contract as the
reference's kvq/vllm_plugin.py:9-13). Registration is by class path, so the backend module is imported only
when vLLM selects it. With KVQ_CAPTURE=1 the calibration capture hook is installed as in the reference
(kvq/vllm_plugin.py:14-17); its attention-override and MLA study hooks are debugging tools and are not part
of this package.
"""
import os

BACKEND_PATH = "kvq_b200.vllm_int8.backend.Int8StaticBackend"


def register():
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(AttentionBackendEnum.CUSTOM, BACKEND_PATH)
    if os.environ.get("KVQ_CAPTURE") == "1":
        from . import capture

        capture.install()
