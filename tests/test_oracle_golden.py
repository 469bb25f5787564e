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


def _walk_layers(st, L, z, step, rows_of, names):
    """Run one step of the oracle layer by layer; compare the last layer's buffers with the fixture."""
    hid = []
    for layer in range(L):
        fo.qkv_rope(st, layer)
        if layer == L - 1:
            _assert_bits(st.q_post_rope, z["bf16_q_post_rope"][step], f"q_post_rope step {step}")
            k_row, v_row = rows_of(st, layer)
            _assert_bits(k_row, z["bf16_k_row"][step], f"k row step {step}")
            _assert_bits(v_row, z["bf16_v_row"][step], f"v row step {step}")
        fo.decode_attention(st, layer)
        if layer == L - 1:
            _assert_bits(st.attn_out, z["bf16_attn_out"][step], f"attn_out step {step}")
        fo.oproj_residual(st, layer)
        if layer == L - 1 and "hidden_after_oproj" in names:
            _assert_bits(st.hidden_states, z["bf16_hidden_after_oproj"][step], f"hidden after o-proj step {step}")
        fo.mlp_upgate(st, layer)
        if layer == L - 1:
            _assert_bits(st.silu_out, z["bf16_silu_out"][step], f"silu_out step {step}")
        fo.mlp_down_residual(st, layer)
        hid.append(st.hidden_states.clone())
    fo.lm_head(st)
    _assert_bits(torch.stack(hid), z["bf16_layer_hidden"][step], f"layer hidden step {step}")
    _assert_bits(st.logits, z["bf16_logits"][step], f"logits step {step}")


def test_ragged_batch_every_buffer():
    """Three sequences in [B, H] state with per-row positions, a late start and an early finish: the fixture is the
    reference's fused ops on its multi-batch Globals."""
    from qimeng_megakernel_b200 import synthetic
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B
    z = np.load(os.path.join(GOLD, "batch3_l2_v4096.npz"))
    cfg = dict(LLAMA_3_2_1B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=4096)
    w = synthetic.make_weights(cfg, seed=int(z["weights_seed"]), device="cpu", gain_jitter=0.1)
    prompts = torch.from_numpy(z["prompts"])
    B, L = prompts.shape[0], cfg["num_hidden_layers"]
    st = U.oracle_state(cfg, w, 16, torch.bfloat16, batch=B)
    st32 = U.oracle_state(cfg, w, 16, torch.float32, batch=B)
    for step, (positions, active) in enumerate(zip(z["positions"].tolist(), z["active"].tolist())):
        toks = [int(prompts[b, positions[b]]) for b in range(B)]
        st.hidden_states.copy_(st.embed_tokens[torch.tensor(toks)])
        st.position_ids, st.active_mask = positions, [bool(a) for a in active]
        rows = lambda s, layer: (torch.stack([s.k_cache[layer, b, positions[b]] for b in range(B)]),
                                 torch.stack([s.v_cache[layer, b, positions[b]] for b in range(B)]))
        _walk_layers(st, L, z, step, rows, {"hidden_after_oproj"})
        assert st.logits.argmax(dim=-1).tolist() == z["bf16_argmax"][step].tolist()
        for b in range(B):
            if not active[b]:   # a finished row: logits pinned to -1e9, nothing else moves
                assert bool((st.logits[b].float() <= -9e8).all())
        got = fo.feed_tokens(st32, toks, positions, active, record_layers=True)
        exp = torch.from_numpy(z["fp32_layer_hidden"][step])
        assert torch.allclose(torch.stack(st32.layer_hidden), exp, rtol=1e-5, atol=1e-5), f"fp32 hidden step {step}"
        assert got == z["fp32_argmax"][step].tolist()


def test_qwen3_every_buffer():
    """Qwen3 layer shape (head_dim 128, per-head Q/K RMSNorm before RoPE) against the reference's Qwen3 fused ops."""
    from qimeng_megakernel_b200 import synthetic
    from qimeng_megakernel_b200.model_config import QWEN3_0_6B
    z = np.load(os.path.join(GOLD, "qwen3_l2_v4096.npz"))
    cfg = dict(QWEN3_0_6B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=4096)
    w = synthetic.make_weights(cfg, seed=int(z["weights_seed"]), device="cpu", gain_jitter=0.1)
    L = cfg["num_hidden_layers"]
    st = U.oracle_state(cfg, w, 16, torch.bfloat16)
    st32 = U.oracle_state(cfg, w, 16, torch.float32)
    for pos, tok in enumerate(z["tokens"].tolist()):
        st.hidden_states.copy_(st.embed_tokens[tok]); st.position_id = pos
        rows = lambda s, layer: (s.k_cache[layer, 0, pos], s.v_cache[layer, 0, pos])
        _walk_layers(st, L, z, pos, rows, set())
        assert int(st.logits.argmax()) == int(z["bf16_argmax"][pos])
        nxt32 = fo.feed_token(st32, tok, pos, record_layers=True)
        exp = torch.from_numpy(z["fp32_layer_hidden"][pos])
        assert torch.allclose(torch.stack(st32.layer_hidden), exp, rtol=1e-5, atol=1e-5), f"fp32 hidden step {pos}"
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


def test_moe_block():
    """The MoE block oracle (oracle/moe_oracle.py) against the reference's fused_moe_block: with a shared expert
    (16 experts, top-4) and shaped like an OLMoE layer in miniature (64 experts, top-8, no shared expert)."""
    import importlib.util
    from oracle import moe_oracle as mo
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLD, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    z = np.load(os.path.join(GOLD, "moe_block.npz"))
    for case in mg.MOE_CASES:
        w = mg.moe_weights(case)
        cfg = mo.MoeConfig(hidden_size=case["hidden_size"], intermediate_size=case["intermediate_size"],
                           moe_intermediate_size=case["moe_intermediate_size"], num_experts=case["num_experts"],
                           num_experts_per_tok=case["num_experts_per_tok"], rms_norm_eps=1e-6)
        for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
            lw = mo.MoeLayerWeights(**{k: w[k].to(dtype) for k in (
                "mlp_norm", "shared_gate_proj", "shared_up_proj", "shared_down_proj", "shared_expert_gate", "router",
                "expert_gate_up", "expert_down")})
            for i, x in enumerate(w["inputs"]):
                r = mo.moe_block(cfg, lw, x.to(dtype))
                key = f"{case['name']}_{name}_"
                assert r["expert_indices"].tolist() == z[key + "expert_indices"][i].tolist(), f"{key} experts, input {i}"
                assert np.allclose(r["expert_weights"].numpy(), z[key + "expert_weights"][i], rtol=1e-6, atol=0)
                assert len(set(r["expert_indices"].tolist())) == case["num_experts_per_tok"]
                for buf in ("shared_out", "routed_out", "hidden"):
                    if dtype == torch.bfloat16:
                        _assert_bits(r[buf], z[key + buf][i], f"{key}{buf} input {i}")
                    else:
                        assert torch.allclose(r[buf], torch.from_numpy(z[key + buf][i]), rtol=1e-5, atol=1e-6), f"{key}{buf}"
                if not case["shared"]:
                    assert float(r["shared_out"].float().abs().max()) == 0.0


def test_moe_block_olmoe_layer_shape():
    """The MoE block oracle at the full OLMoE-1B-7B layer shape (hidden 2048, 64 experts, top-8, expert intermediate
    1024) against the reference's fused_moe_block (tests/golden/moe_olmoe_layer.npz)."""
    import importlib.util
    from oracle import moe_oracle as mo
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLD, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    z = np.load(os.path.join(GOLD, "moe_olmoe_layer.npz"))
    case = mg.MOE_LAYER_CASE
    w = mg.moe_weights(case)
    inputs = _as_bf16(z["inputs"])
    cfg = mo.MoeConfig(hidden_size=case["hidden_size"], intermediate_size=case["intermediate_size"],
                       moe_intermediate_size=case["moe_intermediate_size"], num_experts=case["num_experts"],
                       num_experts_per_tok=case["num_experts_per_tok"], rms_norm_eps=1e-5)
    lw = mo.MoeLayerWeights(**{k: w[k] for k in ("mlp_norm", "shared_gate_proj", "shared_up_proj", "shared_down_proj",
                                                "shared_expert_gate", "router", "expert_gate_up", "expert_down")})
    distinct = set()
    for i, x in enumerate(inputs):
        r = mo.moe_block(cfg, lw, x)
        assert r["expert_indices"].tolist() == z["bf16_expert_indices"][i].tolist(), f"experts, input {i}"
        assert np.allclose(r["expert_weights"].numpy(), z["bf16_expert_weights"][i], rtol=1e-6, atol=0)
        _assert_bits(r["routed_out"], z["bf16_routed_out"][i], f"routed_out input {i}")
        _assert_bits(r["hidden"], z["bf16_hidden"][i], f"hidden input {i}")
        distinct |= set(r["expert_indices"].tolist())
    assert len(distinct) > 24      # near-uniform routing: eight rows touch a good part of the 64 experts
