"""The entry point for callers that must not allocate device memory (qmk_decode_step_static).

Some callers cannot let a library call cudaMalloc on their behalf: a serving loop whose device memory is
owned by a pool allocator, an embedder with a fixed memory budget, or code that runs where an allocation
would synchronise the device.  For them the library keeps its scratch in a fixed 2 MiB __device__ array
inside its own image.  This test drives that entry point through the C ABI and checks that two decode
steps in a row produce what the handle-based entry point (qmk_create / qmk_decode_step) produces on the
same inputs; the second step reuses the array with the first step's contents still in it.

The file name makes pytest collect it last, so a run that stops at the first failure has already run every
other test; it passes alone in a fresh process as well as after the other tests.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _structs(g, cfg, lib_mod):
    desc = lib_mod.ModelDesc(lib_mod.ABI_VERSION, lib_mod.ARCH_LLAMA, cfg["num_hidden_layers"], cfg["hidden_size"],
                             cfg["intermediate_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                             cfg["head_dim"], cfg["vocab_size"], int(g.rope_cos.shape[0]), float(cfg["rms_norm_eps"]),
                             1.0 / math.sqrt(cfg["head_dim"]))
    w = lib_mod.WeightPtrs(attn_norm=g.attn_norm_weights.data_ptr(), qkv=g.qkv_weights.data_ptr(),
                           o_proj=g.o_proj_weights.data_ptr(), mlp_norm=g.mlp_norm_weights.data_ptr(),
                           up_proj=g.up_proj_weights.data_ptr(), gate_proj=g.gate_proj_weights.data_ptr(),
                           down_proj=g.down_proj_weights.data_ptr(), lm_head_norm=g.lm_head_norm_weights.data_ptr(),
                           lm_head=g.lm_head_weights.data_ptr(), embed_tokens=g.embed_tokens.data_ptr(),
                           rope_cos=g.rope_cos.data_ptr(), rope_sin=g.rope_sin.data_ptr())
    st = lib_mod.StatePtrs(hidden_states=g.hidden_states.data_ptr(), q_post_rope=g.q_post_rope.data_ptr(),
                           k_cache=g.k_cache.data_ptr(), v_cache=g.v_cache.data_ptr(), attn_out=g.attn_out.data_ptr(),
                           silu_out=g.silu_out.data_ptr(), logits=g.logits.data_ptr(),
                           next_token=g.next_token.data_ptr(), token_in=None, out_tokens=None, out_tokens_len=0,
                           batch=1, kv_seq_len=int(g.k_cache.shape[2]))
    return desc, w, st


def test_static_scratch_entry_matches_handle_entry(small_config, small_weights):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import _lib, mk_kernel, synthetic
    lib = _lib.load()
    cfg = small_config
    tokens = synthetic.make_prompt(cfg["vocab_size"], 2, seed=77).tolist()
    # reference run: the existing, handle-based entry point
    g_ref = synthetic.make_globals(cfg, small_weights, kv_seq_len=16, device="cuda:0")
    mk = mk_kernel.get_mk()
    expected = []
    for pos, tok in enumerate(tokens):
        g_ref.hidden_states.copy_(g_ref.embed_tokens[tok]); g_ref.position_id = pos
        mk(g_ref)
        torch.cuda.synchronize()
        expected.append((g_ref.logits.float().cpu().clone(), int(g_ref.next_token.item()),
                         g_ref.hidden_states.float().cpu().clone()))
    mk.check_status()
    mk.close()
    # the entry point that allocates nothing, on its own state buffers (fresh KV cache), two calls in a row
    g = synthetic.make_globals(cfg, small_weights, kv_seq_len=16, device="cuda:0")
    desc, w, st = _structs(g, cfg, _lib)
    stream = torch.cuda.current_stream().cuda_stream
    rows = [g.embed_tokens[tok].clone() for tok in tokens]
    for pos, tok in enumerate(tokens):
        g.hidden_states.copy_(rows[pos])
        torch.cuda.synchronize()
        # device memory in use must not move across the call (the first call may still load the kernel
        # image, so the check is made on the second one); no PyTorch operation runs inside the bracket
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.qmk_decode_step_static(C.byref(desc), C.byref(w), C.byref(st), pos, 0, stream)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        assert rc == 0, f"qmk_decode_step_static returned {rc}: {lib.qmk_strerror(rc).decode()}"
        if pos > 0:
            assert free_after == free_before, "the static entry point must not allocate device memory"
        logits, token, hidden = expected[pos]
        got = g.logits.float().cpu()
        rel = float((got - logits).norm() / logits.norm())
        assert rel <= 2e-2, f"call {pos}: logits differ from the handle-based entry point, relative L2 {rel:.3g}"
        assert torch.equal(got, logits), f"call {pos}: same kernel, same inputs: logits should be identical"
        assert int(g.next_token.item()) == token
        assert torch.equal(g.hidden_states.float().cpu(), hidden)
    # both steps were healthy: the status record in the fixed array is clean
    status = _lib.Status()
    assert lib.qmk_static_poll_status(0, C.byref(status)) == 0 and status.code == 0
    # a model whose scratch cannot fit the fixed array is refused with its own error code
    big = _lib.ModelDesc(**{f: getattr(desc, f) for f, _ in _lib.ModelDesc._fields_})
    big.num_attention_heads = 4096
    rc = lib.qmk_decode_step_static(C.byref(big), C.byref(w), C.byref(st), 0, 0, stream)
    assert rc == _lib.ERR_SCRATCH_TOO_LARGE
    assert b"fixed array" in lib.qmk_strerror(rc)
    # a position outside the cache is refused before anything is launched
    assert lib.qmk_decode_step_static(C.byref(desc), C.byref(w), C.byref(st), 16, 0, stream) == -6

    # per-row positions / an active mask do not exist in the batch-1 kernel: refused, not ignored
    pid = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    st2 = _lib.StatePtrs(**{f: getattr(st, f) for f, _ in _lib.StatePtrs._fields_})
    st2.position_ids = pid.data_ptr()
    assert lib.qmk_decode_step_static(C.byref(desc), C.byref(w), C.byref(st2), 0, 0, stream) == -1


def test_static_entry_reports_an_expired_wait_and_recovers(small_config, small_weights):
    """A caller of the allocation-free entry point has no handle to poll, so the record of a bounded wait that ran
    out stays in the fixed array until qmk_static_poll_status reads it.  The wait is made to run out on the host's
    terms: the first phase waits, with a one-millisecond budget, for hand-off words that nothing writes; the kernel
    returns by itself and the context stays usable.  A healthy call afterwards matches the handle-based entry point."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from qimeng_megakernel_b200 import _lib, mk_kernel, synthetic
    lib = _lib.load()
    cfg = small_config
    tok = int(synthetic.make_prompt(cfg["vocab_size"], 1, seed=78)[0])
    g = synthetic.make_globals(cfg, small_weights, kv_seq_len=16, device="cuda:0")
    desc, w, st = _structs(g, cfg, _lib)
    stream = torch.cuda.current_stream().cuda_stream
    status = _lib.Status()
    assert lib.qmk_static_set_timeout_cycles(0, 999) == -1            # below the smallest budget
    assert lib.qmk_static_set_timeout_cycles(0, 2_000_000) == 0       # about a millisecond
    assert lib.qmk_static_set_wait_first_dependency(0, 1) == 0
    try:
        g.hidden_states.copy_(g.embed_tokens[tok])
        assert lib.qmk_decode_step_static(C.byref(desc), C.byref(w), C.byref(st), 0, 0, stream) == 0
        # a second step queued behind the failed one must not wipe the record
        lib.qmk_static_set_wait_first_dependency(0, 0)
        assert lib.qmk_decode_step_static(C.byref(desc), C.byref(w), C.byref(st), 1, 0, stream) == 0
        rc = lib.qmk_static_poll_status(0, C.byref(status))
        assert rc == _lib.ERR_DEVICE_TIMEOUT, f"expected the expired wait to be reported, got {rc}"
        assert status.code != 0 and status.phase == 0
        assert lib.qmk_static_poll_status(0, C.byref(status)) == 0 and status.code == 0   # read once, then clean
    finally:
        lib.qmk_static_set_wait_first_dependency(0, 0)
        lib.qmk_static_set_timeout_cycles(0, 0)
    # healthy again: same result as the handle-based entry point on the same input
    g_ref = synthetic.make_globals(cfg, small_weights, kv_seq_len=16, device="cuda:0")
    mk = mk_kernel.get_mk()
    g_ref.hidden_states.copy_(g_ref.embed_tokens[tok]); g_ref.position_id = 0
    mk(g_ref)
    torch.cuda.synchronize()
    mk.check_status()
    g2 = synthetic.make_globals(cfg, small_weights, kv_seq_len=16, device="cuda:0")
    desc2, w2, st2 = _structs(g2, cfg, _lib)
    g2.hidden_states.copy_(g2.embed_tokens[tok])
    assert lib.qmk_decode_step_static(C.byref(desc2), C.byref(w2), C.byref(st2), 0, 0, stream) == 0
    assert lib.qmk_static_poll_status(0, C.byref(status)) == 0 and status.code == 0
    assert torch.equal(g2.logits, g_ref.logits) and int(g2.next_token.item()) == int(g_ref.next_token.item())
    mk.close()
