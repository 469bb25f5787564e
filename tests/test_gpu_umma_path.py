"""The tcgen05.mma variant of the weight stream (libqmk_b200.so built with -DQMK_UMMA=1 into csrc/umma/)
held to the per-op parity bar of the default path, plus a whole-step check against the default library."""
import pytest
import torch

from tests import _util as U
from tests.test_gpu_parity import assert_op_close, _phase
from oracle import fused_oracle as fo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(small_config, small_weights):
    from qimeng_megakernel_b200 import _build, mk_kernel, synthetic
    if not _build.UMMA_LIB_PATH.exists():
        pytest.skip("tcgen05 variant not built (python -m qimeng_megakernel_b200._build)")
    S = 128
    g = synthetic.make_globals(small_config, small_weights, kv_seq_len=S, device="cuda")
    g2 = synthetic.make_globals(small_config, small_weights, kv_seq_len=S, device="cuda")
    mk = mk_kernel.get_mk(_build.UMMA_DIR)
    ref = mk_kernel.get_mk()
    st = U.oracle_state(small_config, small_weights, S, torch.bfloat16)
    yield dict(cfg=small_config, g=g, g2=g2, mk=mk, ref=ref, st=st)
    mk.close()


@pytest.mark.parametrize("mode", [0, 1])
def test_umma_per_op_parity(env, mode):
    g, mk, st, cfg = env["g"], env["mk"], env["st"], env["cfg"]
    L = cfg["num_hidden_layers"]
    st.k_cache.zero_(); st.v_cache.zero_(); g.k_cache.zero_(); g.v_cache.zero_()
    prompt = [int(t) for t in torch.randint(0, cfg["vocab_size"], (36,), generator=torch.Generator().manual_seed(9))]
    for pos, tok in enumerate(prompt):
        st.hidden_states.copy_(st.embed_tokens[tok])
        st.position_id = pos
        if pos not in (0, 3, 32, 35):
            fo.decode_step(st)
            continue
        for layer in range(L):
            U.push_state(st, g); fo.qkv_rope(st, layer)
            mk.run_phases(g, _phase(layer, 0), _phase(layer, 0) + 1, mode)
            assert_op_close(g.q_post_rope, st.q_post_rope, f"q_post_rope pos {pos} layer {layer}")
            assert_op_close(g.k_cache[layer, 0, pos], st.k_cache[layer, 0, pos], f"k row pos {pos} layer {layer}")
            assert_op_close(g.v_cache[layer, 0, pos], st.v_cache[layer, 0, pos], f"v row pos {pos} layer {layer}")
            U.push_state(st, g); fo.decode_attention(st, layer)
            mk.run_phases(g, _phase(layer, 1), _phase(layer, 1) + 1, mode)
            assert_op_close(g.attn_out, st.attn_out, f"attn_out pos {pos} layer {layer}")
            U.push_state(st, g); h_in = st.hidden_states.clone(); fo.oproj_residual(st, layer)
            mk.run_phases(g, _phase(layer, 2), _phase(layer, 2) + 1, mode)
            assert_op_close(g.hidden_states, st.hidden_states, f"o-proj hidden pos {pos} layer {layer}", h_in)
            U.push_state(st, g); fo.mlp_upgate(st, layer)
            mk.run_phases(g, _phase(layer, 3), _phase(layer, 3) + 1, mode)
            assert_op_close(g.silu_out, st.silu_out, f"silu_out pos {pos} layer {layer}")
            U.push_state(st, g); h_in = st.hidden_states.clone(); fo.mlp_down_residual(st, layer)
            mk.run_phases(g, _phase(layer, 4), _phase(layer, 4) + 1, mode)
            assert_op_close(g.hidden_states, st.hidden_states, f"down hidden pos {pos} layer {layer}", h_in)
        U.push_state(st, g); fo.lm_head(st)
        mk.run_phases(g, 5 * L, 5 * L + 1, mode)
        assert_op_close(g.logits, st.logits, f"logits pos {pos}")
        assert int(g.next_token.item()) == int(g.logits.float().argmax().item())
    mk.check_status()


def test_umma_whole_step_matches_default_library(env):
    """24 persistent steps on both libraries from the same state: logits within rel L2 1e-2 of each other."""
    g, g2, mk, ref, cfg = env["g"], env["g2"], env["mk"], env["ref"], env["cfg"]
    for x in (g, g2):
        x.k_cache.zero_(); x.v_cache.zero_()
    toks = [int(t) for t in torch.randint(0, cfg["vocab_size"], (24,), generator=torch.Generator().manual_seed(3))]
    for pos, tok in enumerate(toks):
        for x, k in ((g, mk), (g2, ref)):
            x.hidden_states.copy_(x.embed_tokens[tok]); x.position_id = pos
            k(x)
        assert U.rel_l2(g.logits, g2.logits) <= 1e-2, f"pos {pos}: {U.rel_l2(g.logits, g2.logits):.4g}"
        assert int(g.next_token.item()) == int(g.logits.float().argmax().item())
    mk.check_status(); ref.check_status()
