"""B200 (sm_100a) decode-schedule package for the QiMeng-MegaKernel `--route mk` path.

Exposes the attributes the reference's decode runtime reads from a decode-schedule package
(qimeng_megakernel/models/LLM/registry.py:84-94, 238-262; decode.py:600-642): `Globals`, `ModelConfig`,
`mk_kernel.get_mk / call_mk`, and `STATIC_MEGAKERNEL = True` (the kernel owns its scheduler and
dependency counters, so the runtime neither builds instruction queues nor zeroes barriers).
There is no CPU route in this package.
"""
from .globs import Globals
from .model_config import LlamaConfig

ModelConfig = LlamaConfig
STATIC_MEGAKERNEL = True
HARDWARE = "B200"

__all__ = ["Globals", "ModelConfig", "LlamaConfig", "STATIC_MEGAKERNEL", "HARDWARE", "mk_kernel"]


def __getattr__(name: str):
    import importlib
    if name in ("mk_kernel", "decode", "synthetic", "rope", "prefill", "registry"):
        return importlib.import_module(f".{name}", __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
