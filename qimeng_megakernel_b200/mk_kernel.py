"""Load and call the B200 decode megakernel.

Same two functions the reference's decode runtime reads from a decode-schedule package
(qimeng_megakernel/models/LLM/llama/llama3_2__1b/A100/single_batch/decode_schedule/mk_kernel.py:40-94):
`get_mk(mk_dir)` returns the kernel callable, `call_mk(globs, mk)` launches one decode step on the
current CUDA stream using `globs.position_id`.  The callable wraps the C ABI of libqmk_b200.so through
ctypes; tensors cross as raw device pointers.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from pathlib import Path
from typing import Any

import torch

from . import _lib
from .globs import Globals
from .model_config import LlamaConfig

_WEIGHT_FIELDS = (("attn_norm", "attn_norm_weights"), ("qkv", "qkv_weights"), ("o_proj", "o_proj_weights"),
                  ("mlp_norm", "mlp_norm_weights"), ("up_proj", "up_proj_weights"),
                  ("gate_proj", "gate_proj_weights"), ("down_proj", "down_proj_weights"),
                  ("lm_head_norm", "lm_head_norm_weights"), ("lm_head", "lm_head_weights"),
                  ("embed_tokens", "embed_tokens"), ("rope_cos", "rope_cos"), ("rope_sin", "rope_sin"),
                  ("q_norm", "q_norm_weights"), ("k_norm", "k_norm_weights"), ("router", "router_weights"),
                  ("expert_gate_up", "expert_gate_up_proj_weights"), ("expert_down", "expert_down_proj_weights"))
_STATE_FIELDS = ("hidden_states", "q_post_rope", "k_cache", "v_cache", "attn_out", "silu_out", "logits",
                 "next_token", "token_in", "out_tokens", "position_ids", "active_mask", "kv_slots")


def _check_tensor(name: str, t: torch.Tensor, dtype: torch.dtype, shape: tuple) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"globs.{name} must be a tensor")
    if not t.is_cuda:
        raise ValueError(f"globs.{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"globs.{name}: expected {dtype}, got {t.dtype}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"globs.{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"globs.{name} must be contiguous")


def _ptr(t) -> int | None:
    if t is None:
        return None
    if isinstance(t, torch.nn.Parameter):
        t = t.data
    return t.data_ptr()


def _sig(t):
    """Identity of a bound tensor: address, shape and dtype (a view with another shape must re-validate)."""
    if t is None:
        return None
    return (t.data_ptr(), tuple(t.shape), t.dtype)


class MegaKernel:
    """Callable returned by get_mk(): owns one native handle per set of weights."""

    def __init__(self, lib: C.CDLL):
        self._lib = lib
        self._handle = None
        self._weights_key = None
        self._state_key = None
        self._device = None
        self._variant = 0
        self._timeout_cycles = int(os.environ.get("QMK_TIMEOUT_CYCLES", "0"))   # device wait budget override (0 = default)

    # -- handle management -------------------------------------------------------------------
    def _validate(self, g: Globals) -> tuple:
        cfg = LlamaConfig
        L, H, I = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size
        NH, NKV, HD, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.vocab_size
        bf = torch.bfloat16
        _check_tensor("attn_norm_weights", g.attn_norm_weights, bf, (L, H))
        _check_tensor("qkv_weights", g.qkv_weights, bf, (L, (NH + 2 * NKV) * HD, H))
        _check_tensor("o_proj_weights", g.o_proj_weights, bf, (L, H, NH * HD))
        _check_tensor("mlp_norm_weights", g.mlp_norm_weights, bf, (L, H))
        if cfg.num_experts:
            E, Ie = cfg.num_experts, cfg.moe_intermediate_size
            El = E // cfg.ep_world if cfg.ep_world > 1 else E      # experts this rank holds (expert parallelism)
            _check_tensor("router_weights", g.router_weights, bf, (L, E, H))
            _check_tensor("expert_gate_up_proj_weights", g.expert_gate_up_proj_weights, bf, (L, El, 2 * Ie, H))
            _check_tensor("expert_down_proj_weights", g.expert_down_proj_weights, bf, (L, El, H, Ie))
        else:
            _check_tensor("up_proj_weights", g.up_proj_weights, bf, (L, I, H))
            _check_tensor("gate_proj_weights", g.gate_proj_weights, bf, (L, I, H))
            _check_tensor("down_proj_weights", g.down_proj_weights, bf, (L, H, I))
        _check_tensor("lm_head_norm_weights", g.lm_head_norm_weights, bf, (H,))
        _check_tensor("lm_head_weights", g.lm_head_weights, bf, (V, H))
        if g.embed_tokens is not None:
            _check_tensor("embed_tokens", g.embed_tokens, bf, (cfg.embed_rows or V, H))
        rows = int(g.rope_cos.shape[0])
        _check_tensor("rope_cos", g.rope_cos, torch.float32, (rows, HD))
        _check_tensor("rope_sin", g.rope_sin, torch.float32, (rows, HD))
        if cfg.qk_norm:
            _check_tensor("q_norm_weights", g.q_norm_weights, bf, (L, HD))
            _check_tensor("k_norm_weights", g.k_norm_weights, bf, (L, HD))
        if g.k_cache.dim() != 5:
            raise ValueError("globs.k_cache must be [L, B, S, NKV, HD]")
        Bc, S = int(g.k_cache.shape[1]), int(g.k_cache.shape[2])
        # rows of the step: one per sequence of the cache, unless kv_slots says which sequence every row belongs to
        slots = getattr(g, "kv_slots", None)
        B = int(slots.numel()) if slots is not None else Bc
        if not 1 <= B <= _lib.MAX_BATCH:
            raise ValueError(f"batch {B} outside 1..{_lib.MAX_BATCH}")
        _check_tensor("k_cache", g.k_cache, bf, (L, Bc, S, NKV, HD))
        _check_tensor("v_cache", g.v_cache, bf, (L, Bc, S, NKV, HD))
        if slots is not None:
            _check_tensor("kv_slots", slots, torch.int32, (B,))

        def state(name, width):
            t = getattr(g, name)
            # one sequence may keep the reference's single-batch shapes ([H]), B sequences are [B, H]
            shape = (width,) if (B == 1 and isinstance(t, torch.Tensor) and t.dim() == 1) else (B, width)
            _check_tensor(name, t, bf, shape)

        state("hidden_states", H)
        state("q_post_rope", NH * HD)
        state("attn_out", NH * HD)
        state("silu_out", I)
        state("logits", V)
        for name in ("next_token", "token_in"):
            t = getattr(g, name, None)
            if t is not None:
                _check_tensor(name, t, torch.int64, (B,))
        if getattr(g, "out_tokens", None) is not None:
            n = g.out_tokens.numel() // B
            _check_tensor("out_tokens", g.out_tokens, torch.int64, (n,) if (B == 1 and g.out_tokens.dim() == 1) else (B, n))
        if getattr(g, "position_ids", None) is not None:
            _check_tensor("position_ids", g.position_ids, torch.int32, (B,))
        if getattr(g, "active_mask", None) is not None:
            if g.active_mask.dtype not in (torch.uint8, torch.bool):
                raise TypeError("globs.active_mask must be uint8 or bool")
            _check_tensor("active_mask", g.active_mask, g.active_mask.dtype, (B,))
        return rows, S, B, Bc

    def _ensure(self, g: Globals) -> None:
        wkey = tuple(_ptr(getattr(g, f, None)) for _, f in _WEIGHT_FIELDS) + tuple(
            LlamaConfig.as_dict().items())
        skey = tuple(_sig(getattr(g, f, None)) for f in _STATE_FIELDS)
        if wkey == self._weights_key and skey == self._state_key:
            return
        rows, S, B, Bc = self._validate(g)
        dev = g.hidden_states.device
        if wkey != self._weights_key:
            self.close()
            cfg = LlamaConfig
            arch = _lib.ARCH_MOE if cfg.num_experts else (_lib.ARCH_QWEN3 if cfg.qk_norm else _lib.ARCH_LLAMA)
            desc = _lib.ModelDesc(_lib.ABI_VERSION, arch,
                                  cfg.num_hidden_layers, cfg.hidden_size,
                                  cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                                  cfg.head_dim, cfg.vocab_size, rows, float(cfg.rms_norm_eps),
                                  1.0 / math.sqrt(cfg.head_dim), float(cfg.rms_norm_eps), int(cfg.num_experts),
                                  int(cfg.num_experts_per_tok), int(cfg.moe_intermediate_size),
                                  int(cfg.ep_world), int(cfg.ep_rank), int(cfg.tp_world), int(cfg.tp_rank),
                                  int(cfg.embed_rows))
            w = _lib.WeightPtrs(**{c: _ptr(getattr(g, f, None)) for c, f in _WEIGHT_FIELDS})
            h = C.c_void_p()
            _lib.check(self._lib.qmk_create(C.byref(desc), C.byref(w), dev.index or 0, C.byref(h)))
            self._handle = h
            self._weights_key = wkey
            self._state_key = None
            self._device = dev
            if self._variant:
                _lib.check(self._lib.qmk_set_kernel_variant(self._handle, self._variant), self._handle)
            if self._timeout_cycles:
                _lib.check(self._lib.qmk_set_timeout_cycles(self._handle, self._timeout_cycles))
        if skey != self._state_key:
            st = _lib.StatePtrs(**{f: _ptr(getattr(g, f, None)) for f in _STATE_FIELDS})
            st.out_tokens_len = int(g.out_tokens.numel()) // B if getattr(g, "out_tokens", None) is not None else 0
            st.batch = B
            st.kv_seq_len = S
            st.kv_batch = Bc
            _lib.check(self._lib.qmk_bind_state(self._handle, C.byref(st)), self._handle)
            self._state_key = skey

    def close(self) -> None:
        if self._handle is not None:
            self._lib.qmk_destroy(self._handle)
            self._handle = None
            self._weights_key = self._state_key = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- launches ----------------------------------------------------------------------------
    def _stream(self) -> int:
        return torch.cuda.current_stream(self._device).cuda_stream

    def __call__(self, g: Globals, pos_id: int | None = None) -> None:
        self._ensure(g)
        pos = int(g.position_id if pos_id is None else pos_id) if (g.position_id is not None or pos_id is not None) else 0
        _lib.check(self._lib.qmk_decode_step(self._handle, pos, self._stream()), self._handle)

    def run_phases(self, g: Globals, phase_begin: int, phase_end: int, mode: int = 0) -> None:
        """Run a sub-range of phases (per-op verification), see qmk_run_phases."""
        self._ensure(g)
        pos = int(g.position_id or 0)
        _lib.check(self._lib.qmk_run_phases(self._handle, pos, phase_begin, phase_end, mode, self._stream()),
                   self._handle)

    def generate_host(self, g: Globals, host_tokens: torch.Tensor, first_pos: int, n_steps: int,
                      teacher_forced: bool = False, host_argmax: torch.Tensor | None = None) -> None:
        """Greedy decode with host token buffers (int64 CPU tensors, ideally pinned)."""
        self._ensure(g)
        if host_tokens.dtype != torch.int64 or host_tokens.is_cuda or not host_tokens.is_contiguous():
            raise TypeError("host_tokens must be a contiguous int64 CPU tensor")
        ha = host_argmax.data_ptr() if host_argmax is not None else None
        _lib.check(self._lib.qmk_generate_host(self._handle, host_tokens.data_ptr(), host_tokens.numel(),
                                               first_pos, n_steps, 1 if teacher_forced else 0, ha,
                                               self._stream()), self._handle)

    def generate_device(self, g: Globals, first_pos: int, n_steps: int) -> None:
        """n_steps greedy steps from first_pos with the token loop on the device (g.token_in feeds the first step, every
        later one takes the arg-max of the step before): one persistent launch on the batch-1 kernel."""
        self._ensure(g)
        _lib.check(self._lib.qmk_generate_device(self._handle, int(first_pos), int(n_steps), self._stream()), self._handle)

    def poll_status(self) -> dict:
        st = _lib.Status()
        rc = self._lib.qmk_poll_status(self._handle, C.byref(st)) if self._handle is not None else 0   # nothing launched yet
        d = {f: getattr(st, f) for f, _ in _lib.Status._fields_}
        d["rc"] = rc
        return d

    def check_status(self) -> None:
        d = self.poll_status()
        if d["rc"] != 0:
            raise _lib.QmkError(d["rc"], f"status={d}")

    def set_timeout_cycles(self, cycles: int) -> None:
        self._timeout_cycles = int(cycles)
        if self._handle is not None:
            _lib.check(self._lib.qmk_set_timeout_cycles(self._handle, int(cycles)))

    def set_kernel_variant(self, variant: int) -> None:
        """0: the batch-1 kernel when the shape and batch allow it; 1: always the batched kernel."""
        self._variant = int(variant)
        if self._handle is not None:
            _lib.check(self._lib.qmk_set_kernel_variant(self._handle, self._variant), self._handle)

    def set_cooperative_launch(self, on: bool) -> None:
        _lib.check(self._lib.qmk_set_cooperative_launch(self._handle, 1 if on else 0))

    def set_wait_first_dependency(self, on: bool) -> None:
        _lib.check(self._lib.qmk_set_wait_first_dependency(self._handle, 1 if on else 0))

    def set_trace(self, buf: torch.Tensor | None) -> None:
        """buf: int64 CUDA tensor [CTAs, phases, 8] receiving globaltimer stamps, or None to stop."""
        if buf is None:
            _lib.check(self._lib.qmk_set_trace(self._handle, None, 0))
        else:
            _lib.check(self._lib.qmk_set_trace(self._handle, buf.data_ptr(), buf.numel() * 8))

    def step_bytes(self, pos: int) -> int:
        return int(self._lib.qmk_step_bytes(self._handle, pos)) if self._handle is not None else 0

    def decode_step(self, pos: int) -> None:
        """One more decode step at position `pos` on the state bound by the last `mk(globs)` call (no tensor
        re-validation: the form a device-resident token loop and the benchmark's timed loops use)."""
        if self._handle is None:
            raise RuntimeError("decode_step needs a bound state: call mk(globs) once first")
        _lib.check(self._lib.qmk_decode_step(self._handle, int(pos), self._stream()), self._handle)

    def run_phases_bound(self, pos: int, phase_begin: int, phase_end: int, mode: int = 0) -> None:
        """run_phases on the state bound by the last `mk(globs)` / `run_phases(globs, ...)` call, without tensor
        re-validation (a profiling loop that launches single phases back to back)."""
        if self._handle is None:
            raise RuntimeError("run_phases_bound needs a bound state: call run_phases(globs, ...) once first")
        _lib.check(self._lib.qmk_run_phases(self._handle, int(pos), int(phase_begin), int(phase_end), int(mode),
                                            self._stream()), self._handle)

    def last_expert_count(self) -> int:
        """MoE: distinct experts selected by the last layer's router in the last step (synchronises)."""
        n = C.c_int32()
        _lib.check(self._lib.qmk_last_expert_count(self._handle, C.byref(n)), self._handle)
        return n.value

    def ep_export(self, g: Globals) -> bytes:
        """Expert parallelism: creates the handle for `g` if need be and returns the 64-byte inter-process handle of this
        rank's exchange buffer (to be gathered over all ranks and passed to ep_connect)."""
        self._ensure(g)
        buf = C.create_string_buffer(64)
        _lib.check(self._lib.qmk_ep_export(self._handle, buf), self._handle)
        return buf.raw

    def ep_connect(self, handles: list[bytes]) -> None:
        """Expert parallelism: maps the exchange buffers of all ranks (their handles in rank order)."""
        blob = b"".join(handles)
        _lib.check(self._lib.qmk_ep_connect(self._handle, C.c_char_p(blob)), self._handle)

    def expert_reads(self, reset: bool = False) -> int:
        """MoE: distinct experts read, summed over every router phase since the last reset (synchronises)."""
        n = C.c_int64()
        _lib.check(self._lib.qmk_expert_reads(self._handle, C.byref(n), 1 if reset else 0), self._handle)
        return n.value

    def last_expert_routing(self) -> list[dict]:
        """MoE: per row of the last step, {expert index: router weight} as the last router phase selected them."""
        E = int(LlamaConfig.num_experts)
        n = C.c_int32()
        experts = (C.c_int32 * E)()
        weights = (C.c_float * (E * _lib.MAX_BATCH))()
        _lib.check(self._lib.qmk_last_expert_routing(self._handle, C.byref(n), experts, weights), self._handle)
        rows = [dict() for _ in range(_lib.MAX_BATCH)]
        for slot in range(n.value):
            for b in range(_lib.MAX_BATCH):
                wgt = weights[slot * _lib.MAX_BATCH + b]
                if wgt > 0.0:
                    rows[b][int(experts[slot])] = float(wgt)
        return rows

    @property
    def launch_count(self) -> int:
        return int(self._lib.qmk_launch_count(self._handle)) if self._handle is not None else 0

    def geometry(self) -> tuple[int, int, int]:
        a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
        _lib.check(self._lib.qmk_launch_geometry(self._handle, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value


def get_mk(mk_dir: Path | None = None) -> MegaKernel:
    """Return the prebuilt kernel (raises ImportError when libqmk_b200.so is missing)."""
    path = None if mk_dir is None else Path(mk_dir) / "libqmk_b200.so"
    return MegaKernel(_lib.load(path))


def call_mk(globs: Globals, mk: Any) -> None:
    """Launch one decode step with the current Globals (position from globs.position_id)."""
    mk(globs)
