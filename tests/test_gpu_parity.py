"""GPU parity of the sm_100a decode kernel against the CPU oracle, through the C ABI (ctypes).

Per-op tests give both sides identical inputs (the oracle's state is copied to the device before
each phase), in the manner of the reference's pyvm_to_megakernel op tests
(qimeng_megakernel/verifier/LLM/llama/llama3_2__1b/A100/single_batch/pyvm_to_megakernel/test_op_qkv_rope.py:22-62).
Tolerances (stated once here): a per-op output may differ from the bf16 oracle by bf16 rounding of a
differently-ordered fp32 sum: |d| <= 1e-2*|ref| + 2e-3*max|ref|.  The residual phases round the projection
to bf16 BEFORE adding it to the stream (operations.py:251-262, 285-295), so there the rounding unit is that of
the projection term, which can be much larger than the sum: the bound gains 1e-2*|ref - residual input|.  Whole-step hidden states are held to
rtol 2e-2 against the fp32 oracle: relative L2 error <= 2e-2 and elementwise |d| <= 2e-2*|ref| + 5e-2*rms(ref)
(the reference's own bf16 route sits at relative L2 ~1e-2 and elementwise ~3.3e-2*(|ref|+rms) from fp32 on
these weights, so a tighter elementwise bound would reject the reference itself); and to relative L2 <= 1e-2
against the bf16 oracle.
"""
import pytest
import torch

from tests import _util as U
from oracle import fused_oracle as fo

pytestmark = pytest.mark.gpu

OP_RTOL, OP_ATOL_FRAC = 1e-2, 2e-3


def assert_op_close(actual, expected, what, residual_in=None):
    a, e = actual.float().cpu(), expected.float().cpu()
    tol = OP_RTOL * e.abs() + OP_ATOL_FRAC * float(e.abs().max())
    if residual_in is not None:   # bf16 rounding of the projection term that was added to residual_in
        tol = tol + OP_RTOL * (e - residual_in.float().cpu()).abs()
    bad = (a - e).abs() > tol
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} of {bad.numel()} elements out of tolerance; "
        f"max abs diff {float((a - e).abs().max()):.4g}, max |ref| {float(e.abs().max()):.4g}")


@pytest.fixture(scope="module")
def env(small_config, small_weights):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import mk_kernel, synthetic
    S = 4096
    g = synthetic.make_globals(small_config, small_weights, kv_seq_len=S, device="cuda")
    mk = mk_kernel.get_mk()
    st = U.oracle_state(small_config, small_weights, S, torch.bfloat16)
    st32 = U.oracle_state(small_config, small_weights, S, torch.float32)
    yield dict(cfg=small_config, w=small_weights, g=g, mk=mk, st=st, st32=st32, S=S)
    mk.close()


def _reset(env):
    for st in (env["st"], env["st32"]):
        st.k_cache.zero_(); st.v_cache.zero_()
    env["g"].k_cache.zero_(); env["g"].v_cache.zero_()


def _phase(layer, kind):
    return layer * 5 + kind


@pytest.mark.parametrize("mode", [0, 1])
def test_per_op_parity(env, mode):
    """Each phase alone, identical inputs, positions 0..5 then 31, 32, 33 (attention block edges)."""
    _reset(env)
    g, mk, st, cfg = env["g"], env["mk"], env["st"], env["cfg"]
    L = cfg["num_hidden_layers"]
    prompt = [int(t) for t in torch.randint(0, cfg["vocab_size"], (40,), generator=torch.Generator().manual_seed(5))]
    check_at = {0, 1, 2, 5, 31, 32, 33, 39}
    for pos, tok in enumerate(prompt):
        st.hidden_states.copy_(st.embed_tokens[tok])
        st.position_id = pos
        if pos not in check_at:
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
        # fused argmax = argmax of the kernel's own bf16 logits, lowest index on ties
        assert int(g.next_token.item()) == int(g.logits.float().argmax().item())
    mk.check_status()


def test_long_context_attention(env):
    """Split-KV with many partials and more than one block per partial: random KV, positions that
    are not multiples of the block size, including the last position of the cache."""
    g, mk, st, cfg = env["g"], env["mk"], env["st"], env["cfg"]
    gen = torch.Generator().manual_seed(11)
    st.k_cache.copy_(torch.randn(st.k_cache.shape, generator=gen) * 0.5)
    st.v_cache.copy_(torch.randn(st.v_cache.shape, generator=gen) * 0.5)
    for pos in (63, 64, 777, 2047, 2048, 2100, env["S"] - 1):
        st.position_id = pos
        st.q_post_rope.copy_(torch.randn(st.q_post_rope.shape, generator=gen))
        for layer in range(cfg["num_hidden_layers"]):
            U.push_state(st, g); fo.decode_attention(st, layer)
            for mode in (0, 1):
                g.attn_out.zero_()
                mk.run_phases(g, _phase(layer, 1), _phase(layer, 1) + 1, mode)
                assert_op_close(g.attn_out, st.attn_out, f"attn_out pos {pos} layer {layer} mode {mode}")
    mk.check_status()


def test_full_step_teacher_forced(env):
    """Whole persistent step, 48 teacher-forced tokens: hidden states per layer vs the fp32 oracle
    (rtol 2e-2), logits vs the bf16 oracle, exact argmax where the oracle's top-2 logits are not tied, and where
    they are tied (within 2 bf16 ulps) the kernel's token must be one of the tied ones: on random weights near-ties
    are common, so a plain agreement rate would measure the weights, not the kernel."""
    _reset(env)
    g, mk, st, st32, cfg = env["g"], env["mk"], env["st"], env["st32"], env["cfg"]
    L, V = cfg["num_hidden_layers"], cfg["vocab_size"]
    gen = torch.Generator().manual_seed(7)
    tokens = [int(t) for t in torch.randint(0, V, (16,), generator=gen)]
    n_steps, agree, untied, untied_agree = 48, 0, 0, 0
    for pos in range(n_steps):
        tok = tokens[pos]
        nxt = fo.feed_token(st, tok, pos, record_layers=True)
        fo.feed_token(st32, tok, pos, record_layers=True)
        # per-layer hidden state through a synchronised sub-range launch (layers 0..l)
        if pos in (0, 17, 47):
            kc, vc = g.k_cache.clone(), g.v_cache.clone()
            for l in range(L):
                g.hidden_states.copy_(g.embed_tokens[tok]); g.position_id = pos
                mk.run_phases(g, 0, 5 * (l + 1), 1)
                ref = st32.layer_hidden[l]
                got = g.hidden_states.float().cpu()
                assert U.rel_l2(got, ref) <= 2e-2, f"layer {l} pos {pos}: rel L2 {U.rel_l2(got, ref):.4g}"
                tol = 2e-2 * ref.abs() + 5e-2 * float(ref.pow(2).mean().sqrt())
                assert bool(((got - ref).abs() <= tol).all()), f"layer {l} pos {pos}: elementwise rtol 2e-2 + floor"
                ref16 = st.layer_hidden[l]
                assert U.rel_l2(got, ref16) <= 1e-2, f"layer {l} pos {pos}: vs bf16 oracle {U.rel_l2(got, ref16):.4g}"
            g.k_cache.copy_(kc); g.v_cache.copy_(vc)
        g.hidden_states.copy_(g.embed_tokens[tok]); g.position_id = pos
        mk(g)
        got_tok = int(g.next_token.item())
        assert got_tok == int(g.logits.float().argmax().item())
        lg = g.logits.float().cpu()
        assert U.rel_l2(lg, st.logits) <= 2e-2, f"logits pos {pos}: rel L2 {U.rel_l2(lg, st.logits):.4g}"
        top2 = st.logits.float().topk(2).values
        agree += int(got_tok == nxt)
        if got_tok != nxt:   # only acceptable between logits the oracle itself cannot tell apart at bf16 resolution
            gap = float(top2[0] - st.logits.float()[got_tok])
            assert gap <= 2 * 2 ** -8 * float(top2[0].abs()), f"pos {pos}: token {got_tok} is {gap:.4g} below the oracle's best logit"
        if float(top2[0] - top2[1]) > 2 * 2 ** -8 * float(top2[0].abs()):
            untied += 1
            untied_agree += int(got_tok == nxt)
        if pos + 1 >= len(tokens):
            tokens.append(nxt)          # teacher forcing: the oracle's token is replayed
    mk.check_status()
    assert agree / n_steps >= 0.9, f"top-1 agreement {agree}/{n_steps}"
    assert untied_agree == untied, f"argmax differs on {untied - untied_agree} untied steps"


def test_device_token_loop_and_host_generate(env):
    """Token-input mode (the kernel embeds the token and writes the next one) must reproduce the
    hidden-state-input path exactly, both device-resident and through host token buffers."""
    _reset(env)
    g, mk, cfg = env["g"], env["mk"], env["cfg"]
    prompt = [int(t) for t in torch.randint(0, cfg["vocab_size"], (8,), generator=torch.Generator().manual_seed(3))]
    n_new = 24
    # path A: host loop as in generate_greedy_fast
    out_a = list(prompt)
    for pos in range(len(prompt) + n_new - 1):
        g.hidden_states.copy_(g.embed_tokens[out_a[pos]]); g.position_id = pos
        mk(g)
        if pos + 1 >= len(out_a):
            out_a.append(int(g.next_token.item()))
    # path B: host token buffers through qmk_generate_host
    g.k_cache.zero_(); g.v_cache.zero_()
    host = torch.zeros(len(prompt) + n_new, dtype=torch.int64).pin_memory()
    host[:len(prompt)] = torch.tensor(prompt)
    scratch = torch.zeros(len(prompt), dtype=torch.int64).pin_memory()
    mk.generate_host(g, host, 0, len(prompt) - 1, teacher_forced=True, host_argmax=scratch)
    mk.generate_host(g, host, len(prompt) - 1, n_new)
    assert host.tolist() == out_a
    # path C: device-resident loop, no host involvement between steps
    g.k_cache.zero_(); g.v_cache.zero_()
    dev_tokens = torch.zeros(len(prompt) + n_new, dtype=torch.int64, device="cuda")
    dev_tokens[:len(prompt)] = torch.tensor(prompt)
    g.out_tokens = dev_tokens
    g.token_in = torch.zeros(1, dtype=torch.int64, device="cuda")
    for pos in range(len(prompt) - 1):
        g.token_in.copy_(dev_tokens[pos:pos + 1]); g.position_id = pos
        saved = dev_tokens[pos + 1].clone()
        mk(g)
        dev_tokens[pos + 1] = saved      # prompt positions keep their token
    g.token_in.copy_(dev_tokens[len(prompt) - 1:len(prompt)])
    g.next_token = g.token_in            # feed the argmax straight back
    for pos in range(len(prompt) - 1, len(prompt) + n_new - 1):
        g.position_id = pos
        mk(g)
    assert dev_tokens.tolist() == out_a
    logits_c = g.logits.clone()
    # path D: the same run as persistent multi-step launches (qmk_generate_device): the token crosses the step boundary
    # inside the kernel.  Chunks of 1, 5, 7 and the rest; tokens and the last logits must be the single-step loop's, bit for bit.
    g.k_cache.zero_(); g.v_cache.zero_()
    dev_tokens[len(prompt):] = 0
    g.next_token = torch.zeros(1, dtype=torch.int64, device="cuda")
    for pos in range(len(prompt) - 1):
        g.token_in.copy_(dev_tokens[pos:pos + 1]); g.position_id = pos
        saved = dev_tokens[pos + 1].clone()
        mk(g)
        dev_tokens[pos + 1] = saved
    g.token_in.copy_(dev_tokens[len(prompt) - 1:len(prompt)])
    g.next_token = g.token_in
    pos, left = len(prompt) - 1, n_new
    for chunk in (1, 5, 7, n_new):
        n = min(chunk, left)
        if n <= 0:
            break
        mk.generate_device(g, pos, n)
        pos, left = pos + n, left - n
    torch.cuda.synchronize()
    mk.check_status()
    assert dev_tokens.tolist() == out_a, "multi-step launches disagree with the one-step loop"
    assert torch.equal(g.logits.view(torch.int16), logits_c.view(torch.int16))
    g.token_in = None; g.out_tokens = None
    g.next_token = torch.zeros(1, dtype=torch.int64, device="cuda")
    mk.check_status()


def test_bounded_wait_reports_status(env):
    """Failure detection without a fault: a dependency nothing publishes makes the controller's bounded
    wait expire; the status record comes back, and the same handle then runs a correct step."""
    g, mk, st, cfg = env["g"], env["mk"], env["st"], env["cfg"]
    from qimeng_megakernel_b200 import _lib
    g.position_id = 0
    mk.run_phases(g, 0, 1, 0)                      # make sure the handle exists
    mk.set_timeout_cycles(2_000_000)               # about a millisecond
    mk.set_wait_first_dependency(True)
    mk.run_phases(g, 2, 3, 1)                      # o-proj waits for an attention phase that never ran
    status = mk.poll_status()
    mk.set_wait_first_dependency(False)
    mk.set_timeout_cycles(2_000_000_000)
    assert status["rc"] == _lib.ERR_DEVICE_TIMEOUT
    assert status["code"] == 1 and status["phase"] == 2
    assert status["seen"] < status["expected"]
    # healthy afterwards
    _reset(env)
    tok = 17
    nxt = fo.feed_token(st, tok, 0)
    g.hidden_states.copy_(g.embed_tokens[tok]); g.position_id = 0
    mk(g)
    mk.check_status()
    assert U.rel_l2(g.logits, st.logits) <= 2e-2


def test_argument_validation(env):
    from qimeng_megakernel_b200 import _lib
    g, mk = env["g"], env["mk"]
    g.position_id = env["S"]                       # outside the KV cache
    with pytest.raises(_lib.QmkError):
        mk(g)
    g.position_id = 0
    good = g.logits
    g.logits = good.float()
    with pytest.raises(TypeError):
        mk(g)
    g.logits = good[:-1]
    with pytest.raises(ValueError):
        mk(g)
    g.logits = good
    mk(g)
    mk.check_status()


def test_full_size_against_reference_fixture():
    """The full-size Llama-3.2-1B workload (16 layers, vocabulary 128256) against outputs of the real
    reference (tests/golden/llama1b_cfg1.npz): 32 teacher-forced steps.  Top-1 agreement >= 99 % per step
    (exact where the reference's top-2 logits are not tied), top-8 logit values within bf16 tolerance,
    per-layer hidden states within rtol 2e-2 (relative L2) of the reference's fp32 run (see the bound below)
    and of its bf16 run."""
    import os
    import numpy as np
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import mk_kernel, synthetic
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "llama1b_cfg1.npz"))
    cfg = dict(LLAMA_3_2_1B)
    w = synthetic.make_weights(cfg, seed=int(z["weights_seed"]), device="cpu", max_positions=2048)
    g = synthetic.make_globals(cfg, w, kv_seq_len=40, device="cuda")
    del w
    mk = mk_kernel.get_mk()
    tokens = z["tokens"].tolist()
    L = cfg["num_hidden_layers"]
    hid_steps = z["hidden_steps"].tolist()
    agree = untied = untied_agree = 0
    worst32 = worst_gap = 0.0
    n_steps = 32
    for pos in range(n_steps):
        tok = tokens[pos]
        if pos in hid_steps:
            k = hid_steps.index(pos)
            ref32 = torch.from_numpy(z["fp32_layer_hidden"][k])
            ref16 = torch.from_numpy(z["bf16_layer_hidden"][k].copy()).view(torch.bfloat16).float()
            kc, vc = g.k_cache.clone(), g.v_cache.clone()
            for l in (0, 7, 15):
                g.hidden_states.copy_(g.embed_tokens[tok]); g.position_id = pos
                mk.run_phases(g, 0, 5 * (l + 1), 1)
                got = g.hidden_states.float().cpu()
                # rtol 2e-2 against fp32; the reference's own bf16 route is 2.2-2.5e-2 away from its fp32
                # self at layer 15 on these weights, so the bound is never tighter than 1.25x that distance
                bound = max(2e-2, 1.25 * U.rel_l2(ref16[l], ref32[l]))
                worst32, worst_gap = max(worst32, U.rel_l2(got, ref32[l])), max(worst_gap, U.rel_l2(ref16[l], ref32[l]))
                assert U.rel_l2(got, ref32[l]) <= bound, f"layer {l} pos {pos}: {U.rel_l2(got, ref32[l]):.4g} vs fp32"
                # two bf16 routes that order their fp32 sums differently are independent perturbations of
                # the fp32 result: their mutual distance is bounded by 1.5x the reference route's own
                assert U.rel_l2(got, ref16[l]) <= max(2e-2, 1.5 * U.rel_l2(ref16[l], ref32[l])), \
                    f"layer {l} pos {pos}: {U.rel_l2(got, ref16[l]):.4g} vs bf16"
            g.k_cache.copy_(kc); g.v_cache.copy_(vc)
        g.hidden_states.copy_(g.embed_tokens[tok]); g.position_id = pos
        mk(g)
        got_tok = int(g.next_token.item())
        logits = g.logits.float().cpu()
        assert got_tok == int(logits.argmax())
        ref_idx = z["bf16_top8_indices"][pos]; ref_val = torch.from_numpy(z["bf16_top8_values"][pos])
        got_val = logits[torch.from_numpy(ref_idx)]
        scale = float(ref_val.abs().max())
        assert float((got_val - ref_val).abs().max()) <= 3e-2 * scale + 1e-3, f"top-8 logits pos {pos}"
        agree += int(got_tok == int(ref_idx[0]))
        if float(ref_val[0] - ref_val[1]) > 2 * 2 ** -8 * float(ref_val[0].abs()):
            untied += 1
            untied_agree += int(got_tok == int(ref_idx[0]))
    mk.check_status()
    mk.close()
    print(f"measured: full-size Llama-3.2-1B, {n_steps} steps: top-1 agreement {agree}/{n_steps}, untied {untied_agree}/{untied}; "
          f"hidden states vs fp32 relative L2 max {worst32:.4g} (the reference's own bf16 route: {worst_gap:.4g})")
    assert agree / n_steps >= 0.99 or untied_agree == untied, f"top-1 agreement {agree}/{n_steps}"
    assert untied_agree == untied, f"arg-max differs on {untied - untied_agree} untied steps"


def test_decode_api_host_and_device_loops(small_config, small_weights):
    """`decode(route='mk', hardware='B200')`: the reference's host loop (embed / call_mk / arg-max in PyTorch)
    and the device-resident loop generate the same tokens as the CPU oracle's greedy loop, and the timing
    dictionary carries the reference's keys."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import synthetic
    from qimeng_megakernel_b200.decode import decode
    from qimeng_megakernel_b200.prefill import run_prefill_synthetic
    prompt = synthetic.make_prompt(small_config["vocab_size"], 16, seed=21)
    n_new = 24
    st = U.oracle_state(small_config, small_weights, 16 + n_new, torch.bfloat16)
    seq = prompt.tolist()
    for pos in range(16 + n_new - 1):
        nxt = fo.feed_token(st, seq[pos], pos)
        if pos + 1 >= len(seq):
            seq.append(nxt)
    outs = []
    for host_loop in (True, False):
        pre = run_prefill_synthetic(small_config, small_weights, prompt, n_new, device="cuda:0")
        out = decode("llama-3.2-1b", prefill=pre, max_new_tokens=n_new, decode_route="mk", hardware="B200",
                     decode_time=True, ignore_eos=True, host_loop=host_loop)
        assert out["generated_ids"].shape == (1, 16 + n_new)
        assert out["per_row_new_tokens"].tolist() == [n_new]
        t = out["timing"]
        for key in ("decode_wall_s", "decode_gpu_s", "mk_kernel_gpu_s", "effective_new_tokens",
                    "decode_window_new_tokens", "effective_tok_s_wall", "effective_tok_s_gpu", "kernel_tok_s", "kernel_steps"):
            assert key in t
        assert t["decode_window_new_tokens"] == n_new - 1 and t["kernel_steps"] == n_new - 1 and t["kernel_tok_s"] > 0
        outs.append(out["generated_ids"][0].tolist())
        pre.mk.close()
    assert outs[0] == outs[1]
    agree = sum(int(a == b) for a, b in zip(outs[0], seq)) / len(seq)
    assert agree >= 0.99 or outs[0][:17] == seq[:17], f"greedy tokens agree with the oracle on {agree:.0%}"
    # EOS handling: stop at the first EOS, pad after it
    pre = run_prefill_synthetic(small_config, small_weights, prompt, n_new, device="cuda:0")
    eos = outs[0][16 + 5]
    out = decode("llama-3.2-1b", prefill=pre, max_new_tokens=n_new, eos_token_ids=[eos], pad_token_id=0)
    first = outs[0][16:].index(eos)
    assert out["per_row_new_tokens"].tolist() == [first + 1]
    assert out["new_tokens"].shape[1] == first + 1
    pre.mk.close()


def test_full_size_step_at_kv1040_against_reference_fixture():
    """One full-size decode step (16 layers, vocabulary 128256) at position 1039, over a KV cache whose first 1039 rows
    are the seeded random rows the fixture was made with (tests/golden/llama1b_kv1040.npz, outputs of the real
    reference): the long end of the decode-length sweep at full size.  Per-layer hidden states within rtol 2e-2
    (relative L2) of the reference's fp32 run -- or 1.25x the reference's own bf16-to-fp32 distance where that is
    larger -- top-8 logits within bf16 tolerance, arg-max exact unless the reference's top two are tied."""
    import os
    import numpy as np
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import mk_kernel, synthetic
    from qimeng_megakernel_b200.model_config import LLAMA_3_2_1B
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "llama1b_kv1040.npz"))
    cfg = dict(LLAMA_3_2_1B)
    pos, tok = int(z["pos"]), int(z["token"])
    w = synthetic.make_weights(cfg, seed=0, device="cpu", max_positions=2048)
    g = synthetic.make_globals(cfg, w, kv_seq_len=pos + 1, device="cuda")
    del w
    k, v = synthetic.random_kv_rows(cfg, pos, int(z["kv_seed"]))
    g.k_cache[:, :, :pos].copy_(k)
    g.v_cache[:, :, :pos].copy_(v)
    mk = mk_kernel.get_mk()
    ref32 = torch.from_numpy(z["fp32_layer_hidden"])
    ref16 = torch.from_numpy(z["bf16_layer_hidden"].copy()).view(torch.bfloat16).float()
    for l in (0, 7, 15):
        g.hidden_states.copy_(g.embed_tokens[tok]); g.position_id = pos
        mk.run_phases(g, 0, 5 * (l + 1), 1)
        got = g.hidden_states.float().cpu()
        gap = U.rel_l2(ref16[l], ref32[l])
        assert U.rel_l2(got, ref32[l]) <= max(2e-2, 1.25 * gap), f"layer {l}: {U.rel_l2(got, ref32[l]):.4g} vs fp32"
        assert U.rel_l2(got, ref16[l]) <= max(2e-2, 1.5 * gap), f"layer {l}: {U.rel_l2(got, ref16[l]):.4g} vs bf16"
        if l == 15:
            ref_attn = torch.from_numpy(z["bf16_attn_out_last_layer"].copy()).view(torch.bfloat16).float()
            assert U.rel_l2(g.attn_out, ref_attn) <= 3e-2, "attention output of the last layer over 1040 keys"
    g.hidden_states.copy_(g.embed_tokens[tok]); g.position_id = pos
    mk(g)
    torch.cuda.synchronize()
    mk.check_status()
    logits = g.logits.float().cpu()
    ref_idx, ref_val = z["bf16_top8_indices"], torch.from_numpy(z["bf16_top8_values"])
    got_val = logits[torch.from_numpy(ref_idx)]
    assert float((got_val - ref_val).abs().max()) <= 3e-2 * float(ref_val.abs().max()) + 1e-3
    assert int(g.next_token.item()) == int(logits.argmax())
    if float(ref_val[0] - ref_val[1]) > 2 * 2 ** -8 * float(ref_val[0].abs()):
        assert int(g.next_token.item()) == int(z["bf16_argmax"])
    mk.close()


def test_decode_api_sampling(small_config, small_weights):
    """`decode()` with sampling arguments: the kernel still feeds the fed token itself, the next token is drawn from
    the kernel's logits on the device.  top_k = 1 is greedy in distribution and must reproduce the greedy text; a fixed
    seed reproduces the draws; a strong presence penalty forbids repeating the penalised token."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import synthetic
    from qimeng_megakernel_b200.decode import decode
    from qimeng_megakernel_b200.prefill import run_prefill_synthetic
    prompt = synthetic.make_prompt(small_config["vocab_size"], 16, seed=23)
    n_new = 12

    def run(**kw):
        pre = run_prefill_synthetic(small_config, small_weights, prompt, n_new, device="cuda:0")
        out = decode("llama-3.2-1b", prefill=pre, max_new_tokens=n_new, ignore_eos=True, decode_time=True, **kw)
        pre.mk.close()
        assert out["timing"]["kernel_steps"] == n_new - 1
        return out["generated_ids"][0].tolist()

    greedy = run()
    assert run(temperature=0.8, top_k=1) == greedy
    a, b = run(temperature=1.5, top_p=0.95, seed=7), run(temperature=1.5, top_p=0.95, seed=7)
    assert a == b and a[:17] == greedy[:17] and a != greedy     # prompt and first token come from prefill
    pen = run(temperature=0.0, presence_penalty=50.0)
    new = pen[16:]
    assert len(set(new[1:])) == len(new[1:]), "with a prohibitive presence penalty no generated token may repeat"
    two = synthetic.make_prompts(small_config["vocab_size"], 2, 16, seed=29)
    pre = run_prefill_synthetic(small_config, small_weights, two, n_new, device="cuda:0")
    out = decode("llama-3.2-1b", prefill=pre, max_new_tokens=n_new, ignore_eos=True, temperature=1.0, top_k=20, seed=3)
    assert out["generated_ids"].shape == (2, 16 + n_new) and int(out["generated_ids"].max()) < small_config["vocab_size"]
    pre.mk.close()
