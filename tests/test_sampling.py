"""Token selection after the LM head (qimeng_megakernel_b200/sampling.py) against the reference's `_sample_logits`.

tests/golden/sampling.npz holds, for a grid of settings, what the real reference hands to torch.multinomial (captured
by tests/golden/make_golden.py) or the token it returns when it decides greedily.  The distribution must match to
fp32 rounding and the greedy decisions exactly; the batched evaluation must equal the row-by-row one."""
import importlib.util
import os

import numpy as np
import torch

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _make_golden():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLD, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    return mg


def test_distribution_and_greedy_decisions_match_the_reference():
    from qimeng_megakernel_b200 import sampling as S
    mg = _make_golden()
    z = np.load(os.path.join(GOLD, "sampling.npz"))
    logits, generated = mg.sampling_inputs()
    sampled_cases = 0
    for ci, case in enumerate(mg.SAMPLING_CASES):
        ref_probs, ref_greedy = z[f"case{ci}_probs"], z[f"case{ci}_greedy"]
        kw = {k: case[k] for k in ("temperature", "top_p", "top_k", "min_p")}
        pen = case["presence_penalty"]
        for b in range(logits.shape[0]):
            if ref_greedy[b] >= 0:      # the reference took the arg-max (possibly after the penalty)
                tok = S.sample_logits(logits[b], presence_penalty=pen, generated_ids=generated[b], **kw)
                assert int(tok) == int(ref_greedy[b]), f"case {ci} row {b}: greedy token"
                continue
            sampled_cases += 1
            work = S.apply_presence_penalty(logits[b:b + 1], generated[b:b + 1], pen) if pen != 0.0 else logits[b:b + 1].float()
            probs = S.filtered_probs(work, **kw).clamp(min=1e-9)[0].numpy()
            assert np.allclose(probs, ref_probs[b], rtol=2e-5, atol=1e-9), f"case {ci} row {b}: distribution"
            assert (probs > 1e-8).sum() == (ref_probs[b] > 1e-8).sum(), f"case {ci} row {b}: support size"
        # all rows at once = row by row
        if ref_greedy[0] < 0:
            work = S.apply_presence_penalty(logits, generated, pen) if pen != 0.0 else logits.float()
            allp = S.filtered_probs(work, **kw).clamp(min=1e-9).numpy()
            assert np.allclose(allp, ref_probs, rtol=2e-5, atol=1e-9), f"case {ci}: batched distribution"
    assert sampled_cases >= 15


def test_draws_follow_the_distribution_and_the_seed():
    from qimeng_megakernel_b200 import sampling as S
    gen = torch.Generator().manual_seed(3)
    logits = torch.randn(2, 50, generator=gen) * 2
    kw = dict(temperature=0.9, top_k=5)
    g1, g2 = torch.Generator().manual_seed(11), torch.Generator().manual_seed(11)
    a = torch.stack([S.sample_logits(logits, generator=g1, **kw) for _ in range(200)])
    b = torch.stack([S.sample_logits(logits, generator=g2, **kw) for _ in range(200)])
    assert torch.equal(a, b)                                   # same seed, same draws
    top5 = logits.topk(5, dim=-1).indices
    for row in range(2):
        assert set(a[:, row].tolist()) <= set(top5[row].tolist())   # never outside the top-k support
        assert len(set(a[:, row].tolist())) > 1                      # and not degenerate
    assert S.sample_logits(logits[0]).dim() == 0 and int(S.sample_logits(logits[0])) == int(logits[0].argmax())
    assert S.is_greedy(0.0) and S.is_greedy(1.0) and not S.is_greedy(1.0, top_p=0.9) and S.is_greedy(1.0, top_k=50, vocab=50)
