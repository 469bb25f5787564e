"""ctypes binding of libqmk_b200.so (the C ABI in include/qmk_b200.h).

There is no fallback: if the library cannot be loaded the product path raises.  The reference
loads a prebuilt pybind module and raises ImportError when it is missing
(qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_schedule/mk_kernel.py:40-53).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from ._build import LIB_PATH

ABI_VERSION = 5
ARCH_LLAMA = 0
ARCH_QWEN3 = 1
ARCH_MOE = 2
MAX_BATCH = 64
PHASES_PER_LAYER = 5
PHASE_QKV, PHASE_ATTN, PHASE_OPROJ, PHASE_UPGATE, PHASE_DOWN = range(5)

ERR_DEVICE_TIMEOUT = -7
ERR_SCRATCH_TOO_LARGE = -9
STATIC_SCRATCH_MAX_BYTES = 2 << 20


class ModelDesc(C.Structure):
    _fields_ = [("abi_version", C.c_int32), ("arch", C.c_int32), ("num_layers", C.c_int32),
                ("hidden_size", C.c_int32), ("intermediate_size", C.c_int32),
                ("num_attention_heads", C.c_int32), ("num_key_value_heads", C.c_int32),
                ("head_dim", C.c_int32), ("vocab_size", C.c_int32), ("rope_rows", C.c_int32),
                ("rms_norm_eps", C.c_float), ("attn_scale", C.c_float), ("qk_norm_eps", C.c_float),
                ("num_experts", C.c_int32), ("num_experts_per_tok", C.c_int32), ("moe_intermediate_size", C.c_int32),
                ("ep_world", C.c_int32), ("ep_rank", C.c_int32),
                ("tp_world", C.c_int32), ("tp_rank", C.c_int32), ("embed_rows", C.c_int32)]


class WeightPtrs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_norm", "qkv", "o_proj", "mlp_norm", "up_proj", "gate_proj",
                                          "down_proj", "lm_head_norm", "lm_head", "embed_tokens",
                                          "rope_cos", "rope_sin", "q_norm", "k_norm", "router", "expert_gate_up",
                                          "expert_down")]


class StatePtrs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("hidden_states", "q_post_rope", "k_cache", "v_cache", "attn_out",
                                          "silu_out", "logits", "next_token", "token_in", "out_tokens")] + \
               [("out_tokens_len", C.c_int64), ("batch", C.c_int32), ("kv_seq_len", C.c_int32),
                ("position_ids", C.c_void_p), ("active_mask", C.c_void_p), ("kv_slots", C.c_void_p), ("kv_batch", C.c_int32)]


class Status(C.Structure):
    _fields_ = [("code", C.c_int32), ("sm", C.c_int32), ("warp", C.c_int32), ("phase", C.c_int32),
                ("seen", C.c_uint32), ("expected", C.c_uint32), ("detail", C.c_int32), ("reserved", C.c_int32)]


# Every symbol include/qmk_b200.h declares: (name, restype, argtypes).
SYMBOLS = [
    ("qmk_create", C.c_int, [C.POINTER(ModelDesc), C.POINTER(WeightPtrs), C.c_int, C.POINTER(C.c_void_p)]),
    ("qmk_bind_state", C.c_int, [C.c_void_p, C.POINTER(StatePtrs)]),
    ("qmk_decode_step", C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    ("qmk_run_phases", C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    ("qmk_generate_host", C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                    C.c_void_p, C.c_void_p]),
    ("qmk_poll_status", C.c_int, [C.c_void_p, C.POINTER(Status)]),
    ("qmk_set_timeout_cycles", C.c_int, [C.c_void_p, C.c_int64]),
    ("qmk_set_trace", C.c_int, [C.c_void_p, C.c_void_p, C.c_int64]),
    ("qmk_set_cooperative_launch", C.c_int, [C.c_void_p, C.c_int32]),
    ("qmk_set_kernel_variant", C.c_int, [C.c_void_p, C.c_int32]),
    ("qmk_set_wait_first_dependency", C.c_int, [C.c_void_p, C.c_int32]),
    ("qmk_step_bytes", C.c_int64, [C.c_void_p, C.c_int32]),
    ("qmk_last_expert_count", C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
    ("qmk_last_expert_routing", C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_float)]),
    ("qmk_ep_export", C.c_int, [C.c_void_p, C.c_void_p]),
    ("qmk_ep_connect", C.c_int, [C.c_void_p, C.c_void_p]),
    ("qmk_expert_reads", C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.c_int32]),
    ("qmk_launch_count", C.c_int64, [C.c_void_p]),
    ("qmk_launch_geometry", C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                      C.POINTER(C.c_int32)]),
    ("qmk_decode_step_static", C.c_int, [C.POINTER(ModelDesc), C.POINTER(WeightPtrs), C.POINTER(StatePtrs), C.c_int32,
                                         C.c_int, C.c_void_p]),
    ("qmk_static_poll_status", C.c_int, [C.c_int, C.POINTER(Status)]),
    ("qmk_static_set_timeout_cycles", C.c_int, [C.c_int, C.c_int64]),
    ("qmk_static_set_wait_first_dependency", C.c_int, [C.c_int, C.c_int32]),
    ("qmk_generate_device", C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    ("qmk_static_last_cuda_error", C.c_char_p, []),
    ("qmk_destroy", None, [C.c_void_p]),
    ("qmk_strerror", C.c_char_p, [C.c_int]),
    ("qmk_last_cuda_error", C.c_char_p, [C.c_void_p]),
    ("qmk_abi_version", C.c_int, []),
]

_lib = None


def load(path: Path | None = None) -> C.CDLL:
    """dlopen the library and type every export; raises ImportError if it is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    dso = Path(path) if path is not None else LIB_PATH
    if not dso.is_file():
        raise ImportError(f"missing prebuilt kernel library {dso}; run `python -m qimeng_megakernel_b200._build`")
    lib = C.CDLL(str(dso))
    for name, restype, argtypes in SYMBOLS:
        fn = getattr(lib, name)          # AttributeError if the export is missing
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.qmk_abi_version() != ABI_VERSION:
        raise ImportError(f"{dso}: ABI version {lib.qmk_abi_version()} != {ABI_VERSION}")
    if path is None:
        _lib = lib
    return lib


class QmkError(RuntimeError):
    def __init__(self, code: int, detail: str = ""):
        self.code = code
        msg = load().qmk_strerror(code).decode()
        super().__init__(f"qmk error {code}: {msg}" + (f" ({detail})" if detail else ""))


def check(code: int, handle=None) -> None:
    if code != 0:
        detail = ""
        if handle is not None and code == -3:
            detail = load().qmk_last_cuda_error(handle).decode()
        raise QmkError(code, detail)
