"""Registers the B200 route inside an importable QiMeng-MegaKernel checkout without editing its files.

What a maintainer would commit to the reference are the package files under integration/qimeng_megakernel/ (copied to
the same paths) and three small edits; this module applies the same three edits at run time, so that the drop-in can be
exercised against an unmodified checkout:

  1. the B200 decode-schedule packages are made importable under their reference paths by appending this overlay's
     directories to the `__path__` of the reference's model packages;
  2. registry.json (qimeng_megakernel/models/LLM/registry.py:92-96 `_load_registry`) gains a "B200" implementation
     beside "A100" / "H100" for every model the B200 library serves, with the A100 `preprocess` module (the weight
     layout is the same);
  3. `_supports_multibatch` (registry.py:197-202) accepts B200 for those models and the 16-sequence cap of
     `decode_schedule_package_name` (registry.py:212) becomes 64 for B200.
`examples/llm.py:23` would also list "B200" among its `--hardware` choices; that file is a script, not patched here.
"""
from __future__ import annotations

import copy
import importlib
import os

OVERLAY = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qimeng_megakernel")
B200_MODELS = {("llama", "llama-3.2-1b"): "llama3_2__1b", ("qwen", "qwen3-0.6b"): "qwen3__0_6b"}
MAX_BATCH = 64


def enable() -> None:
    """Idempotent.  Raises ImportError when the reference package is not importable."""
    registry = importlib.import_module("qimeng_megakernel.models.LLM.registry")
    if getattr(registry, "_b200_enabled", False):
        return
    # 1. overlay packages
    for (family, _), module in B200_MODELS.items():
        pkg = importlib.import_module(f"qimeng_megakernel.models.LLM.{family}.{module}")
        extra = os.path.join(OVERLAY, "models", "LLM", family, module)
        if extra not in pkg.__path__:
            pkg.__path__.append(extra)
    # 2. registry entries
    load = registry._load_registry

    def load_with_b200():
        data = copy.deepcopy(load())
        for (family, key) in B200_MODELS:
            impls = data["families"][family]["models"][key]["implementations"]
            for arch_impls in impls.values():
                if "B200" not in arch_impls and "A100" in arch_impls:
                    arch_impls["B200"] = dict(arch_impls["A100"])
        return data

    registry._load_registry = load_with_b200
    # 3. multi-batch support and the batch cap
    supports = registry._supports_multibatch
    registry._supports_multibatch = lambda impl: (impl.hardware == "B200" and (impl.family, impl.model_key) in B200_MODELS) or supports(impl)
    name_of = registry.decode_schedule_package_name

    def package_name(model_name: str, hardware: str, batch_size: int = 1) -> str:
        if hardware == "B200" and batch_size > 16:
            if batch_size > MAX_BATCH:
                raise NotImplementedError(f"multi-batch decode on B200 supports batch_size<={MAX_BATCH}")
            return name_of(model_name, hardware, 16)        # same package for every batch 2..64
        return name_of(model_name, hardware, batch_size)

    registry.decode_schedule_package_name = package_name
    registry._b200_enabled = True
