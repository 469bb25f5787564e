"""GPU parity of the mixture-of-experts path of the batched kernel (router, grouped expert up/gate, expert
down-projection as one GEMM over the selected experts) against the CPU oracle, through the C ABI.

Oracle: the attention half is oracle/fused_oracle.py (MHA, head_dim 128), the MLP half oracle/moe_oracle.py, which
is pinned to the reference's fused_moe_block (tests/test_oracle_golden.py::test_moe_block and
::test_moe_block_olmoe_layer_shape); the model has no shared expert (OLMoE-like), so that branch's weights are zero.
Shapes: a small one (hidden 256, 16 experts, top-4) and the OLMoE-1B-7B layer itself (hidden 2048, 16 heads of 128,
64 experts, top-8, expert intermediate 1024; 2 layers, small vocabulary) at batch 1 and 32, plus the reference's own
outputs for the MoE block (tests/golden/moe_block.npz, moe_olmoe_layer.npz).  The experts every row selects and their
router weights are compared exactly / to 1e-4 with the oracle's top-k (qmk_last_expert_routing).  Tolerances: the MoE block as one op with identical inputs,
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


def moe_mlp(st, cfg, w, layer, routing=None):
    """The MoE block of one layer on every active row of the oracle state.  routing: optional list that receives, per
    row, (sorted probabilities of ALL experts descending, {expert: weight} of the selected ones) or None if inactive."""
    lw = moe_layer_weights(cfg, w, layer, st.hidden_states.dtype)
    rows = fo._bh(st.hidden_states)
    picks = []
    for b in range(rows.shape[0]):
        if st.active(b):
            r = mo.moe_block(moe_cfg(cfg), lw, rows[b])
            rows[b].copy_(r["hidden"])
            picks.append(sorted(r["expert_indices"].tolist()))
            if routing is not None:
                logits = torch.nn.functional.linear(r["normed"].float().unsqueeze(0), lw.router.float()).squeeze(0)
                allp = torch.softmax(logits, dim=-1).sort(descending=True).values
                routing.append((allp, dict(zip(r["expert_indices"].tolist(), r["expert_weights"].tolist()))))
        elif routing is not None:
            routing.append(None)
    return picks


def assert_routing(mk, routing, k, what):
    """The experts each row selected on the device and their weights against the oracle's top-k: the set must be
    identical unless the oracle's k-th and (k+1)-th probabilities are closer than 1e-5 relative (then either may win);
    the union over rows is what the expert phases read."""
    got = mk.last_expert_routing()
    union = set()
    for b, ref in enumerate(routing):
        if ref is None:
            assert got[b] == {}, f"{what}: finished row {b} must select no expert"
            continue
        allp, picks = ref
        union |= set(got[b])
        assert len(got[b]) == k, f"{what} row {b}: {len(got[b])} experts selected, expected {k}"
        if float(allp[k - 1] - allp[k]) > 1e-5 * float(allp[k - 1]):
            assert set(got[b]) == set(picks), f"{what} row {b}: experts {sorted(got[b])} != oracle {sorted(picks)}"
        for e_id, wgt in got[b].items():
            if e_id in picks:
                assert abs(wgt - picks[e_id]) <= 1e-4 * picks[e_id] + 1e-7, f"{what} row {b} expert {e_id}: weight"
    assert mk.last_expert_count() == len(union), f"{what}: distinct-expert count"


def oracle_step(st, cfg, w, near_tie=None):
    """One decode step of the oracle.  near_tie: optional set that receives the rows whose k-th and (k+1)-th router
    probabilities lie within 1 % of each other in some layer: there the selected set depends on the last bits of the
    layer's input, and two correct implementations may route differently."""
    L, k = cfg["num_hidden_layers"], cfg["num_experts_per_tok"]
    hid = []
    for layer in range(L):
        fo.qkv_rope(st, layer); fo.decode_attention(st, layer); fo.oproj_residual(st, layer)
        routing = []
        moe_mlp(st, cfg, w, layer, routing)
        if near_tie is not None:
            for b, r in enumerate(routing):
                if r is not None and float(r[0][k - 1] - r[0][k]) < 1e-2 * float(r[0][k - 1]):
                    near_tie.add(b)
        hid.append(st.hidden_states.clone())
    fo.lm_head(st)
    return hid


def olmoe_layer_cfg():
    from qimeng_megakernel_b200.model_config import OLMOE_1B_7B
    return dict(OLMOE_1B_7B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=256)


@pytest.mark.parametrize("shape,batch", [("small", 5), ("small", None), ("small", 33), ("olmoe", None), ("olmoe", 32)])
def test_moe_block_and_steps(shape, batch):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import mk_kernel, synthetic
    from qimeng_megakernel_b200.model_config import LlamaConfig
    cfg = MOE_SMALL if shape == "small" else olmoe_layer_cfg()
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
                routing = []
                picks = moe_mlp(st, cfg, w, layer, routing)
                mk.run_phases(g, layer * 6 + 3, layer * 6 + 6, mode)
                assert_routing(mk, routing, cfg["num_experts_per_tok"], f"layer {layer} mode {mode}")
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
        worst = worst_tie = 0.0
        checked = ties = 0
        for step in range(6):
            positions = [step] * nb
            for s in (st, st32):
                s.position_ids, s.active_mask = positions, [bool(a) for a in active]
                s.hidden_states.copy_(fo._bh(s.embed_tokens[prompts[:, step]]).reshape(s.hidden_states.shape))
            near_tie = set()
            hid16 = oracle_step(st, cfg, w, near_tie)
            hid32 = oracle_step(st32, cfg, w, near_tie)
            assert nb < 8 or len(near_tie) <= 0.6 * nb, f"step {step}: {len(near_tie)} of {nb} rows route on a near tie"
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
                # a row that routes on a near tie may legitimately pick the other expert: one expert term of the
                # weighted sum then differs, a few per cent of the hidden state
                bound = 6e-2 if b in near_tie else max(2e-2, 1.5 * gap)
                if b in near_tie:
                    worst_tie, ties = max(worst_tie, U.rel_l2(got[b], h32)), ties + 1
                else:
                    worst, checked = max(worst, U.rel_l2(got[b], h32)), checked + 1
                assert U.rel_l2(got[b], h32) <= bound, f"step {step} row {b}: hidden vs fp32 oracle"
            ref_logits = fo._bh(st.logits).float()
            own = fo._bh(g.logits).float().argmax(dim=-1)
            assert g.next_token.tolist() == own.tolist()
            for b in range(nb):
                top2 = ref_logits[b].topk(2).values
                if active[b] and b not in near_tie and float(top2[0] - top2[1]) > 4 * 2.0 ** -8 * abs(float(top2[0])):
                    assert int(g.next_token[b]) == int(ref_logits[b].argmax()), f"step {step} row {b} arg-max"
        mk.check_status()
        print(f"measured: MoE whole steps, {nb} rows: hidden state vs fp32 relative L2 max {worst:.4g} over {checked} rows "
              f"(rows that route on a near tie: {worst_tie:.4g} over {ties})")
    finally:
        mk.close()


def _load_make_golden():
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_golden.py")
    spec = importlib.util.spec_from_file_location("make_golden", path)
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    return mg, os.path.dirname(path)


@pytest.mark.parametrize("which", ["olmoe_like", "olmoe_layer"])
def test_moe_block_against_reference_fixture(which):
    """The reference's own fused_moe_block outputs: the 64-expert / top-8 miniature of tests/golden/moe_block.npz and the
    full OLMoE layer shape of tests/golden/moe_olmoe_layer.npz.  The fixture's input rows are one batch; the three MoE
    phases of a one-layer model built around the fixture's weights run on them; experts and weights per row must be the
    reference's, the new hidden state within the MoE-block tolerance of its bf16 output."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import numpy as np
    from qimeng_megakernel_b200 import mk_kernel, synthetic
    from qimeng_megakernel_b200.model_config import LlamaConfig
    mg, gold = _load_make_golden()
    if which == "olmoe_like":
        case = [c for c in mg.MOE_CASES if c["name"] == "olmoe_like"][0]
        z, key, eps = np.load(gold + "/moe_block.npz"), "olmoe_like_bf16_", 1e-6
        mw = mg.moe_weights(case)
        inputs = mw["inputs"]
    else:
        case = mg.MOE_LAYER_CASE
        z, key, eps = np.load(gold + "/moe_olmoe_layer.npz"), "bf16_", 1e-5
        mw = mg.moe_weights(case)
        inputs = torch.from_numpy(z["inputs"].copy()).view(torch.bfloat16)
    H, E, K, Ie = case["hidden_size"], case["num_experts"], case["num_experts_per_tok"], case["moe_intermediate_size"]
    cfg = dict(num_hidden_layers=1, hidden_size=H, intermediate_size=64, head_dim=128, num_attention_heads=H // 128,
               num_key_value_heads=H // 128, vocab_size=512, rms_norm_eps=eps, rope_theta=10000.0, rope_scaling=None,
               max_position_embeddings=64, num_experts=E, num_experts_per_tok=K, moe_intermediate_size=Ie)
    w = synthetic.make_weights(dict(cfg, num_experts=8, moe_intermediate_size=64), seed=5, device="cpu", max_positions=64)
    w["mlp_norm_weights"] = mw["mlp_norm"].view(1, H)
    w["router_weights"] = mw["router"].view(1, E, H)
    w["expert_gate_up_proj_weights"] = mw["expert_gate_up"].view(1, E, 2 * Ie, H)
    w["expert_down_proj_weights"] = mw["expert_down"].view(1, E, H, Ie)
    B = inputs.shape[0]
    g = synthetic.make_globals(cfg, w, kv_seq_len=8, device="cuda", batch=B)
    mk = mk_kernel.get_mk()
    try:
        LlamaConfig.update_from_dict(cfg)
        ref_h = torch.from_numpy(z[key + "hidden"].copy()).view(torch.bfloat16).float()
        for mode in (0, 1):
            g.hidden_states.copy_(inputs)
            g.position_id = 0
            mk.run_phases(g, 3, 6, mode)
            torch.cuda.synchronize()
            mk.check_status()
            got = mk.last_expert_routing()
            for b in range(B):
                ref_e = z[key + "expert_indices"][b].tolist()
                ref_w = z[key + "expert_weights"][b].tolist()
                assert sorted(got[b]) == sorted(ref_e), f"{which} mode {mode} row {b}: experts {sorted(got[b])} != {sorted(ref_e)}"
                for e_id, wgt in zip(ref_e, ref_w):
                    assert abs(got[b][e_id] - wgt) <= 1e-4 * wgt + 1e-7
            a, e, x = g.hidden_states.float().cpu(), ref_h, inputs.float()
            tol = 2e-2 * (e - x).abs() + 1e-2 * e.abs() + 2e-3 * float(e.abs().max())
            bad = (a - e).abs() > tol
            assert not bool(bad.any()), f"{which} mode {mode}: {int(bad.sum())} of {bad.numel()} elements out of tolerance"
    finally:
        mk.close()
