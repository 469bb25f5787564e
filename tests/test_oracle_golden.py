"""Pins the CPU oracle (oracle/fused_oracle.py) to outputs of the REAL reference.

tests/golden/*.npz were produced by tests/golden/make_golden.py, which imports the reference's own fused
PyTorch ops and runs them on the seeded synthetic weights.  The oracle's restatement must reproduce them:
bit for bit where both ran on the same machine, and otherwise within one bf16 unit in the last place on
at most 0.1 % of the elements (a different BLAS may order an fp32 sum differently)."""
import os

import numpy as np
import pytest
import torch

from tests import _util as U
from oracle import fused_oracle as fo

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _as_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def _assert_bits(actual: torch.Tensor, golden_bits: np.ndarray, what: str):
    exp = _as_bf16(golden_bits).reshape(actual.shape)
    ulps = U.bf16_ulps(actual, exp)
    frac = float((ulps > 0).float().mean())
    assert int(ulps.max()) <= 1 and frac <= 1e-3, f"{what}: max {int(ulps.max())} ulp, {frac:.2%} of elements differ"


def test_small_model_every_buffer(small_config, small_weights):
    z = np.load(os.path.join(GOLD, "small_l2_v4096.npz"))
    assert int(z["weights_seed"]) == 1234
    tokens = z["tokens"].tolist()
    st = U.oracle_state(small_config, small_weights, 64, torch.bfloat16)
    st32 = U.oracle_state(small_config, small_weights, 64, torch.float32)
    L = small_config["num_hidden_layers"]
    for pos, tok in enumerate(tokens):
        st.hidden_states.copy_(st.embed_tokens[tok]); st.position_id = pos
        hid = []
        for layer in range(L):
            fo.qkv_rope(st, layer)
            if layer == L - 1:
                _assert_bits(st.q_post_rope, z["bf16_q_post_rope"][pos], f"q_post_rope step {pos}")
                _assert_bits(st.k_cache[layer, 0, pos], z["bf16_k_row"][pos], f"k row step {pos}")
                _assert_bits(st.v_cache[layer, 0, pos], z["bf16_v_row"][pos], f"v row step {pos}")
            fo.decode_attention(st, layer)
            if layer == L - 1:
                _assert_bits(st.attn_out, z["bf16_attn_out"][pos], f"attn_out step {pos}")
            fo.oproj_residual(st, layer)
            if layer == L - 1:
                _assert_bits(st.hidden_states, z["bf16_hidden_after_oproj"][pos], f"hidden after o-proj step {pos}")
            fo.mlp_upgate(st, layer)
            if layer == L - 1:
                _assert_bits(st.silu_out, z["bf16_silu_out"][pos], f"silu_out step {pos}")
            fo.mlp_down_residual(st, layer)
            hid.append(st.hidden_states.clone())
        fo.lm_head(st)
        _assert_bits(torch.stack(hid), z["bf16_layer_hidden"][pos], f"layer hidden step {pos}")
        _assert_bits(st.logits, z["bf16_logits"][pos], f"logits step {pos}")
        assert int(st.logits.argmax()) == int(z["bf16_argmax"][pos])
        # fp32 yardstick
        nxt32 = fo.feed_token(st32, tok, pos, record_layers=True)
        got = torch.stack(st32.layer_hidden)
        exp = torch.from_numpy(z["fp32_layer_hidden"][pos])
        assert torch.allclose(got, exp, rtol=1e-5, atol=1e-5), f"fp32 layer hidden step {pos}"
        assert nxt32 == int(z["fp32_argmax"][pos])


def test_full_fixture_is_self_consistent():
    """Shape and content checks of the full-size Llama-3.2-1B fixture the GPU tests compare against (the
    oracle itself needs ~3 s per full-size step, so its full-size run is left to the GPU suite)."""
    z = np.load(os.path.join(GOLD, "llama1b_cfg1.npz"))
    tokens = z["tokens"]
    assert tokens.shape[0] == 16 + 16 + 1 and (z["prompt"] == tokens[:16]).all()
    # greedy: token t+1 is the bf16 arg-max of step t from the end of the prompt on
    for pos in range(15, 32):
        assert tokens[pos + 1] == z["bf16_top8_indices"][pos][0]
    assert z["bf16_layer_hidden"].shape == (4, 16, 2048) and z["fp32_layer_hidden"].shape == (4, 16, 2048)
    # the reference's own bf16 route stays within the stated tolerance of its fp32 self
    b = _as_bf16(z["bf16_layer_hidden"]).float()
    f = torch.from_numpy(z["fp32_layer_hidden"])
    assert float((b - f).norm() / f.norm()) < 2e-2


def test_oracle_edge_positions(small_config, small_weights):
    """First position (one key) and the last position of the cache."""
    st = U.oracle_state(small_config, small_weights, 8, torch.bfloat16)
    for pos in range(8):
        tok = (pos * 997) % small_config["vocab_size"]
        nxt = fo.feed_token(st, tok, pos)
        assert 0 <= nxt < small_config["vocab_size"]
        assert torch.isfinite(st.logits.float()).all()
    with pytest.raises((IndexError, RuntimeError)):
        fo.feed_token(st, 1, 8)            # beyond the cache
