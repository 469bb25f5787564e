"""CPU oracle for the MoE block of a decode step -- TEST INFRASTRUCTURE, not part of the product.

Only tests/ may import this module.  It restates, in plain PyTorch on the CPU, the reference's fused MoE block
(paths inside the QiMeng-MegaKernel project):
  qimeng_megakernel/models/LLM/qwen/qwen1_5_moe_a2_7b/A100/single_batch/decode_schedule/fused/operations.py
      fused_shared_mlp               151-172   shared expert: SiLU(gate) * up in fp32, rounded, down-projection
      fused_router                   175-194   fp32 softmax over ALL experts, torch.topk, no renormalisation
      fused_routed_expert_upgate     197-219   one expert: fused gate|up rows, SiLU(gate) * up in fp32, rounded
      fused_routed_expert_downproj   222-240   down-projection times the router weight, fp32 accumulator
      fused_moe_block                243-268   shared + routed, sigmoid gate on the shared branch, residual adds
The attention half of that model is the dense path already restated in oracle/fused_oracle.py (MHA, head_dim 128).

Parity pin: tests/test_oracle_golden.py::test_moe_block checks this restatement bit for bit against the fixture
tests/golden/moe_block.npz, which tests/golden/make_golden.py made from the real reference.  The batched CUDA
kernel's MoE phases (router, expert up/gate, expert down-projection) are held to this module by
tests/test_gpu_moe.py; the kernel has no shared expert, so that test gives the shared branch zero weights.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .fused_oracle import rms_norm


@dataclass
class MoeConfig:
    hidden_size: int = 2048
    intermediate_size: int = 5632          # shared expert
    moe_intermediate_size: int = 1408      # routed experts
    num_experts: int = 60
    num_experts_per_tok: int = 4
    rms_norm_eps: float = 1e-6


@dataclass
class MoeLayerWeights:
    """One layer of the reference's MoE Globals (globs.py:23-34)."""
    mlp_norm: torch.Tensor                 # [H]
    shared_gate_proj: torch.Tensor         # [I, H]
    shared_up_proj: torch.Tensor           # [I, H]
    shared_down_proj: torch.Tensor         # [H, I]
    shared_expert_gate: torch.Tensor       # [H, 1]  sigmoid gate of the shared branch
    router: torch.Tensor                   # [E, H]
    expert_gate_up: torch.Tensor           # [E, 2 * Ie, H]  gate rows first, then up rows
    expert_down: torch.Tensor              # [E, H, Ie]


def router(cfg: MoeConfig, w: MoeLayerWeights, normed: torch.Tensor):
    """fused_router: logits and softmax in fp32 over all experts, top-k of the probabilities as they are."""
    logits = F.linear(normed.float().unsqueeze(0), w.router.float()).squeeze(0)
    probs = F.softmax(logits, dim=-1)
    top_probs, top_indices = torch.topk(probs, cfg.num_experts_per_tok, dim=-1)
    return top_indices, top_probs


def shared_mlp(w: MoeLayerWeights, normed: torch.Tensor) -> torch.Tensor:
    n1 = normed.unsqueeze(0)
    gate = F.linear(n1, w.shared_gate_proj).squeeze(0)
    up = F.linear(n1, w.shared_up_proj).squeeze(0)
    x = F.silu(gate.to(torch.float32)) * up.to(torch.float32)
    return F.linear(x.to(normed.dtype).unsqueeze(0), w.shared_down_proj).squeeze(0)


def routed_expert(cfg: MoeConfig, w: MoeLayerWeights, normed: torch.Tensor, eid: int) -> torch.Tensor:
    """One expert: returns its down-projection (before the router weight), in the state dtype."""
    mid = cfg.moe_intermediate_size
    gate_up = F.linear(normed.unsqueeze(0), w.expert_gate_up[eid]).squeeze(0)
    silu = (F.silu(gate_up[:mid].to(torch.float32)) * gate_up[mid:].to(torch.float32)).to(normed.dtype)
    return F.linear(silu.unsqueeze(0), w.expert_down[eid]).squeeze(0)


def moe_block(cfg: MoeConfig, w: MoeLayerWeights, hidden: torch.Tensor) -> dict:
    """fused_moe_block on one hidden vector [H]; returns every intermediate the reference keeps in its Globals and
    the new hidden state (the input is not modified)."""
    dtype = hidden.dtype
    normed = rms_norm(hidden, w.mlp_norm, cfg.rms_norm_eps)
    shared_out = shared_mlp(w, normed).to(dtype)
    idx, probs = router(cfg, w, normed)
    acc = torch.zeros(cfg.hidden_size, dtype=torch.float32)
    for j in range(cfg.num_experts_per_tok):
        acc.add_(routed_expert(cfg, w, normed, int(idx[j])).float() * probs[j])
    routed_out = acc.to(dtype)
    # As written in the reference (operations.py:262-265): the gate tensor is stored [H, 1] (globs.py:28), squeeze(0)
    # leaves it [H, 1], and its product with normed [H] broadcasts to [H, H] before the sum, so the logit is
    # sum(gate) * sum(normed), not their dot product.  Restated literally: parity is with what the reference computes.
    gate_logit = (w.shared_expert_gate.squeeze(0).float() * normed.float()).sum()
    gate_scale = torch.sigmoid(gate_logit).to(dtype)
    out = hidden.clone()
    out.add_(routed_out)
    out.add_(shared_out * gate_scale)
    return {"hidden": out, "shared_out": shared_out, "routed_out": routed_out, "expert_indices": idx,
            "expert_weights": probs, "normed": normed}
