"""B200-native `hygemm_vllm` plugin: drop-in for the reference's vLLM hybrid-linear path."""
import os


def register():
    """Entry point of the `vllm.general_plugins` group (reference: hygemm_vllm/__init__.py:1-14).
    Runs in the parent process and in every vLLM worker."""
    from . import quantization  # noqa: F401  registers the `hygemm` quantization config
    from . import offline  # noqa: F401  registers `hygemm_offline` (MXFP4 rows from an offline bank)
    if os.environ.get("HYGEMM_FUSE_SILU", "0") == "1":
        from .producer import install
        install(llama=os.environ.get("HYGEMM_FUSE_LLAMA", "0") == "1")
