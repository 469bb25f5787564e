"""Model / hardware -> decode-schedule package, for the B200 route.

Mirrors the part of the reference's registry the `mk` route uses
(qimeng_megakernel/models/LLM/registry.py:84-94 LLMDecodeSchedule, 197-225 decode_schedule_package_name,
238-262 import_decode_schedule): same dataclass fields, same errors.  The reference only knows the
hardware keys A100 and H100 (registry.json:11-16, examples/llm.py:23, 48-58); this module adds B200 and its
name-based auto-detection.  The B200 package has no scheduler / layer_scheduler / python_vm attributes:
it sets STATIC_MEGAKERNEL and has no CPU routes.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Any

from .model_config import LLAMA_3_2_1B, OLMOE_1B_7B, QWEN3_0_6B

HARDWARE_CHOICES = ("auto", "B200")
# architectures with a kernel (the batch-1 kernel's compiled shape, or the batched kernel's runtime shapes): model key -> config
MODELS = {"llama-3.2-1b": LLAMA_3_2_1B, "qwen3-0.6b": QWEN3_0_6B, "olmoe-1b-7b": OLMOE_1B_7B}
_ALIASES = {"meta-llama/llama-3.2-1b": "llama-3.2-1b", "meta-llama/llama-3.2-1b-instruct": "llama-3.2-1b",
            "llama3_2__1b": "llama-3.2-1b", "synthetic-llama-3.2-1b": "llama-3.2-1b",
            "qwen/qwen3-0.6b": "qwen3-0.6b", "allenai/olmoe-1b-7b-0924": "olmoe-1b-7b", "synthetic-olmoe-1b-7b": "olmoe-1b-7b", "qwen3__0_6b": "qwen3-0.6b", "synthetic-qwen3-0.6b": "qwen3-0.6b"}
# sequences per GPU in one launch (the reference stops at 16, registry.py:212; more sequences shard over GPUs)
MAX_BATCH = 64


@dataclass(frozen=True)
class LLMDecodeSchedule:
    package_name: str
    package: Any
    scheduler: Any | None
    layer_scheduler: Any | None
    python_vm: Any | None
    get_mk: Any | None
    call_mk: Any | None
    config: Any | None
    globs_cls: Any | None


def resolve_model_key(model_name: str) -> str:
    key = str(model_name).strip().rstrip("/").split("/")[-1].lower() if "/" in str(model_name) else str(model_name).lower()
    full = str(model_name).lower()
    for cand in (full, key):
        if cand in MODELS:
            return cand
        if cand in _ALIASES:
            return _ALIASES[cand]
    raise NotImplementedError(f"no B200 decode schedule for model {model_name!r}; known: {sorted(MODELS)}")


def resolve_hardware(hardware: str = "auto", device_name: str | None = None) -> str:
    """`auto` picks B200 from the CUDA device name, like the reference's CLI does for A100 / H100."""
    if hardware != "auto":
        if hardware != "B200":
            raise ValueError(f"this package implements hardware 'B200' only (got {hardware!r})")
        return hardware
    if device_name is None:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("hardware='auto' needs a CUDA device")
        device_name = torch.cuda.get_device_name(0)
    if "B200" in device_name.upper():
        return "B200"
    raise RuntimeError(f"device {device_name!r} is not a B200; the sm_100a kernel cannot run on it")


def decode_schedule_package_name(model_name: str, hardware: str, batch_size: int = 1) -> str:
    resolve_model_key(model_name)
    resolve_hardware(hardware, device_name="B200" if hardware == "auto" else None)
    if batch_size > MAX_BATCH:
        raise NotImplementedError(f"B200 decode supports batch_size<={MAX_BATCH} per GPU (more sequences shard over GPUs)")
    return "qimeng_megakernel_b200"


def import_decode_schedule(model_name: str, hardware: str, batch_size: int = 1) -> LLMDecodeSchedule:
    package_name = decode_schedule_package_name(model_name, hardware, batch_size)
    package = importlib.import_module(package_name)
    mk_kernel = importlib.import_module(f"{package_name}.mk_kernel")
    return LLMDecodeSchedule(package_name=package_name, package=package, scheduler=None, layer_scheduler=None,
                             python_vm=None, get_mk=mk_kernel.get_mk, call_mk=mk_kernel.call_mk,
                             config=getattr(package, "ModelConfig", None), globs_cls=getattr(package, "Globals", None))
