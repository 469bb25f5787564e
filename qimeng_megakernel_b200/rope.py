"""RoPE tables in the interleaved layout the decode kernels read.

Layout contract of the reference: standard tables cos/sin(cat[freqs, freqs]) re-ordered with the
per-head permutation [0, half, 1, half+1, ...] so that entries 2i and 2i+1 both hold frequency i
(qimeng_megakernel/models/LLM/llama/load_weights.py:37-74, llama/preprocess.py:21-44).  The reference's
disk loader uses plain theta; the llama3 frequency scaling below is the published Llama-3.1 rule
(the reference only inherits it from the HuggingFace rotary module, llama/preprocess.py:134-149).
The table is an input of the kernel, so kernel-vs-oracle parity does not depend on it.
"""
from __future__ import annotations

import math

import torch


def inv_frequencies(head_dim: int, theta: float, scaling: tuple | None = None) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    if scaling is None:
        return inv
    factor, low_f, high_f, orig = scaling
    low_wavelen = orig / low_f
    high_wavelen = orig / high_f
    wavelen = 2 * math.pi / inv
    scaled = torch.where(wavelen > low_wavelen, inv / factor, inv)
    smooth = (orig / wavelen - low_f) / (high_f - low_f)
    smoothed = (1 - smooth) * inv / factor + smooth * inv
    medium = (wavelen <= low_wavelen) & (wavelen >= high_wavelen)
    return torch.where(medium, smoothed, scaled)


def rope_tables_interleaved(head_dim: int, max_positions: int, theta: float,
                            scaling: tuple | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 [max_positions, head_dim] cos and sin, interleaved layout."""
    inv = inv_frequencies(head_dim, theta, scaling)
    freqs = torch.outer(torch.arange(max_positions, dtype=torch.float32), inv)
    cos = freqs.cos().repeat_interleave(2, dim=-1).contiguous()
    sin = freqs.sin().repeat_interleave(2, dim=-1).contiguous()
    return cos, sin
