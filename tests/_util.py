"""Shared helpers of the parity tests: build the CPU oracle state and the GPU Globals from the
same seeded weights, copy state between them, and the comparison metrics."""
from __future__ import annotations

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import fused_oracle as fo  # noqa: E402

STATE_BUFFERS = ("hidden_states", "q_post_rope", "attn_out", "silu_out", "logits", "k_cache", "v_cache")


def oracle_config(config: dict) -> fo.OracleConfig:
    return fo.OracleConfig(qk_norm=bool(config.get("qk_norm", False)),
                           **{k: config[k] for k in ("num_hidden_layers", "hidden_size", "intermediate_size",
                                                      "head_dim", "num_attention_heads", "num_key_value_heads",
                                                      "vocab_size", "rms_norm_eps")})


def oracle_state(config: dict, weights: dict, kv_seq_len: int, dtype=torch.bfloat16, batch=None) -> fo.OracleState:
    return fo.make_state(oracle_config(config), weights, kv_seq_len, dtype, batch)


def push_state(st: fo.OracleState, g) -> None:
    """Copy the oracle's current buffers into the GPU Globals (identical inputs for a per-op check)."""
    for name in STATE_BUFFERS:
        getattr(g, name).copy_(getattr(st, name).to(torch.bfloat16))
    g.position_id = st.position_id
    if st.position_ids is not None:
        g.position_ids.copy_(torch.tensor(st.position_ids, dtype=torch.int32))
        g.position_id = max(st.position_ids)
    if st.active_mask is not None:
        g.active_mask.copy_(torch.tensor(st.active_mask, dtype=torch.uint8))


def max_rel_with_abs_floor(actual: torch.Tensor, expected: torch.Tensor, floor: float) -> float:
    """Piecewise metric of the reference's verifier (qimeng_megakernel/verifier/common/compare.py:978-1019):
    relative error where |expected| > floor, absolute error (scaled by 1/floor) below it."""
    a, e = actual.float().cpu().flatten(), expected.float().cpu().flatten()
    d = (a - e).abs()
    big = e.abs() > floor
    rel = torch.where(big, d / e.abs().clamp_min(1e-30), d / floor)
    return float(rel.max()) if rel.numel() else 0.0


def rel_l2(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a, e = actual.float().cpu().flatten(), expected.float().cpu().flatten()
    return float((a - e).norm() / e.norm().clamp_min(1e-30))


def untied(top: float, second: float, units: int = 2) -> bool:
    """True if the two best bf16 logits are more than `units` bf16 units of the larger one apart.  Kernel and oracle
    each round a logit to bf16 after sums taken in different orders, so either value may land one unit away from the
    other side's; a gap of two units or less can therefore tie or flip without either side being wrong."""
    import math
    top, second = float(top), float(second)
    if top == 0.0:
        return False
    unit = 2.0 ** (math.floor(math.log2(abs(top))) - 7)
    return top - second > units * unit


def bf16_ulps(actual: torch.Tensor, expected: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 units-in-the-last-place of `expected` (both bf16)."""
    a = actual.cpu().view(torch.int16).to(torch.int32)
    e = expected.cpu().view(torch.int16).to(torch.int32)
    def key(x):
        return torch.where(x < 0, -(x & 0x7fff), x)
    return (key(a) - key(e)).abs()
