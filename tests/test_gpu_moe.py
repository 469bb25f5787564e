"""GPU parity of the mixture-of-experts path of the batched kernel (router, grouped expert up/gate, expert
down-projection as one GEMM over the selected experts) against the CPU oracle, through the C ABI.

Oracle: the attention half is oracle/fused_oracle.py (MHA, head_dim 128), the MLP half oracle/moe_oracle.py, which
is pinned to the reference's fused_moe_block (tests/test_oracle_golden.py::test_moe_block); the model has no shared
expert (OLMoE-like), so that branch's weights are zero.  Tolerances: the MoE block as one op with identical inputs,
|d| <= 2e-2*|ref - input| + 1e-2*|ref| + 2e-3*max|ref| (the kernel multiplies the router weight into the bf16
activations of the down-projection, the reference into the fp32 output of each expert: one extra bf16 rounding per
expert term); whole steps: per-layer hidden states within relative L2 2e-2 of the fp32 oracle.
"""
import pytest
import torch

from tests import _util as U
from oracle import fused_oracle as fo
from oracle import moe_oracle as mo

pytestmark = pytest.mark.gpu

MOE_SMALL = dict(num_hidden_layers=2, hidden_size=256, intermediate_size=64, head_dim=128, num_attention_heads=2,
                 num_key_value_heads=2, vocab_size=777, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
                 max_position_embeddings=256, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128)


def moe_layer_weights(cfg, w, layer, dtype):
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    z = lambda *s: torch.zeros(*s, dtype=dtype)
    return mo.MoeLayerWeights(mlp_norm=w["mlp_norm_weights"][layer].to(dtype), shared_gate_proj=z(I, H),
                              shared_up_proj=z(I, H), shared_down_proj=z(H, I), shared_expert_gate=z(H, 1),
                              router=w["router_weights"][layer].to(dtype),
                              expert_gate_up=w["expert_gate_up_proj_weights"][layer].to(dtype),
                              expert_down=w["expert_down_proj_weights"][layer].to(dtype))


def moe_cfg(cfg):
    return mo.MoeConfig(hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"],
                        moe_intermediate_size=cfg["moe_intermediate_size"], num_experts=cfg["num_experts"],
                        num_experts_per_tok=cfg["num_experts_per_tok"], rms_norm_eps=cfg["rms_norm_eps"])


def moe_mlp(st, cfg, w, layer):
    """The MoE block of one layer on every active row of the oracle state."""
    lw = moe_layer_weights(cfg, w, layer, st.hidden_states.dtype)
    rows = fo._bh(st.hidden_states)
    picks = []
    for b in range(rows.shape[0]):
        if st.active(b):
            r = mo.moe_block(moe_cfg(cfg), lw, rows[b])
            rows[b].copy_(r["hidden"])
            picks.append(sorted(r["expert_indices"].tolist()))
    return picks


def oracle_step(st, cfg, w, record=False):
    L = cfg["num_hidden_layers"]
    hid = []
    for layer in range(L):
        fo.qkv_rope(st, layer); fo.decode_attention(st, layer); fo.oproj_residual(st, layer)
        moe_mlp(st, cfg, w, layer)
        hid.append(st.hidden_states.clone())
    fo.lm_head(st)
    return hid


@pytest.mark.parametrize("batch", [5, None, 33])
def test_moe_block_and_steps(batch):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import mk_kernel, synthetic
    from qimeng_megakernel_b200.model_config import LlamaConfig
    cfg = MOE_SMALL
    nb = batch or 1
    w = synthetic.make_weights(cfg, seed=77, device="cpu", gain_jitter=0.1, max_positions=256)
    g = synthetic.make_globals(cfg, w, kv_seq_len=64, device="cuda", batch=batch)
    g.position_ids = torch.zeros(nb, dtype=torch.int32, device="cuda")
    g.active_mask = torch.ones(nb, dtype=torch.uint8, device="cuda")
    st = U.oracle_state(cfg, w, 64, torch.bfloat16, batch=batch)
    st32 = U.oracle_state(cfg, w, 64, torch.float32, batch=batch)
    mk = mk_kernel.get_mk()
    try:
        LlamaConfig.update_from_dict(cfg)
        gen = torch.Generator().manual_seed(9)
        L = cfg["num_hidden_layers"]
        # ---- the MoE block alone, identical inputs (phases router, expert up/gate, expert down of each layer)
        positions = [int(x) for x in torch.randint(0, 20, (nb,), generator=gen)]
        active = [1] * nb
        if nb > 2:
            active[2] = 0
        st.position_ids, st.active_mask = positions, [bool(a) for a in active]
        st.hidden_states.copy_((torch.randn(st.hidden_states.shape, generator=gen) * 0.7).to(torch.bfloat16))
        for layer in range(L):
            for mode in (0, 1):
                h_in = st.hidden_states.clone()
                U.push_state(st, g)
                picks = moe_mlp(st, cfg, w, layer)
                mk.run_phases(g, layer * 6 + 3, layer * 6 + 6, mode)
                a, e, x = g.hidden_states.float().cpu(), st.hidden_states.float(), h_in.float()
                tol = 2e-2 * (e - x).abs() + 1e-2 * e.abs() + 2e-3 * float(e.abs().max())
                bad = (a - e).abs() > tol
                assert not bool(bad.any()), (f"MoE block layer {layer} mode {mode}: {int(bad.sum())} of {bad.numel()} out of "
                                             f"tolerance, max diff {float((a - e).abs().max()):.4g}; experts {picks[:2]}")
                if mode == 0:
                    st.hidden_states.copy_(h_in)
        mk.check_status()
        # ---- whole teacher-forced steps
        for s in (st, st32):
            s.k_cache.zero_(); s.v_cache.zero_()
        g.k_cache.zero_(); g.v_cache.zero_()
        g.token_in = torch.zeros(nb, dtype=torch.int64, device="cuda")
        prompts = synthetic.make_prompts(cfg["vocab_size"], nb, 6, seed=3)
        for step in range(6):
            positions = [step] * nb
            for s in (st, st32):
                s.position_ids, s.active_mask = positions, [bool(a) for a in active]
                s.hidden_states.copy_(fo._bh(s.embed_tokens[prompts[:, step]]).reshape(s.hidden_states.shape))
            hid16 = oracle_step(st, cfg, w)
            hid32 = oracle_step(st32, cfg, w)
            g.token_in.copy_(prompts[:, step])
            g.position_ids.fill_(step)
            g.active_mask.copy_(torch.tensor(active, dtype=torch.uint8))
            g.position_id = step
            mk(g)
            torch.cuda.synchronize()
            got = fo._bh(g.hidden_states).float().cpu()
            for b in range(nb):
                if not active[b]:
                    continue
                h32, h16 = fo._bh(hid32[-1])[b].float(), fo._bh(hid16[-1])[b].float()
                gap = U.rel_l2(h16, h32)
                assert U.rel_l2(got[b], h32) <= max(2e-2, 1.5 * gap), f"step {step} row {b}: hidden vs fp32 oracle"
            ref_logits = fo._bh(st.logits).float()
            own = fo._bh(g.logits).float().argmax(dim=-1)
            assert g.next_token.tolist() == own.tolist()
            for b in range(nb):
                top2 = ref_logits[b].topk(2).values
                if active[b] and float(top2[0] - top2[1]) > 4 * 2.0 ** -8 * abs(float(top2[0])):
                    assert int(g.next_token[b]) == int(ref_logits[b].argmax()), f"step {step} row {b} arg-max"
        mk.check_status()
    finally:
        mk.close()
