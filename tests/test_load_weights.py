"""The checkpoint loader (qimeng_megakernel_b200/load_weights.py) on a synthetic Hugging Face checkpoint directory.

No real checkpoint exists offline, so one is written here: seeded weights in the kernels' layout are permuted back into
the Hugging Face layout (Q / K rows and Qwen3 norm gains de-interleaved), saved as config.json plus two safetensors
shards with an index, and loaded again: every tensor must come back bit for bit.  Where the reference checkout is
importable its own disk loader reads the same directory and must agree tensor for tensor."""
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def write_checkpoint(path, cfg, w, tied, model_type):
    from safetensors.torch import save_file
    from qimeng_megakernel_b200.load_weights import interleave_rows, one_head_interleave
    L, NH, NKV, HD = cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qd, kd = NH * HD, NKV * HD
    inv = lambda perm: torch.argsort(perm)
    q_inv, k_inv, one_inv = inv(interleave_rows(NH, HD)), inv(interleave_rows(NKV, HD)), inv(one_head_interleave(HD))
    sd = {"model.embed_tokens.weight": w["embed_tokens"], "model.norm.weight": w["lm_head_norm_weights"]}
    if not tied:
        sd["lm_head.weight"] = w["lm_head_weights"]
    for i in range(L):
        pre = f"model.layers.{i}."
        qkv = w["qkv_weights"][i]
        sd[pre + "self_attn.q_proj.weight"] = qkv[:qd][q_inv]
        sd[pre + "self_attn.k_proj.weight"] = qkv[qd:qd + kd][k_inv]
        sd[pre + "self_attn.v_proj.weight"] = qkv[qd + kd:]
        sd[pre + "self_attn.o_proj.weight"] = w["o_proj_weights"][i]
        sd[pre + "input_layernorm.weight"] = w["attn_norm_weights"][i]
        sd[pre + "post_attention_layernorm.weight"] = w["mlp_norm_weights"][i]
        sd[pre + "mlp.up_proj.weight"] = w["up_proj_weights"][i]
        sd[pre + "mlp.gate_proj.weight"] = w["gate_proj_weights"][i]
        sd[pre + "mlp.down_proj.weight"] = w["down_proj_weights"][i]
        if cfg.get("qk_norm"):
            sd[pre + "self_attn.q_norm.weight"] = w["q_norm_weights"][i][one_inv]
            sd[pre + "self_attn.k_norm.weight"] = w["k_norm_weights"][i][one_inv]
    sd = {k: v.contiguous().clone() for k, v in sd.items()}
    names = sorted(sd)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fname, keys in shards.items():
        save_file({k: sd[k] for k in keys}, os.path.join(path, fname))
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {k: fname for fname, keys in shards.items() for k in keys}}, f)
    hf = dict(model_type=model_type, num_hidden_layers=L, hidden_size=cfg["hidden_size"],
              intermediate_size=cfg["intermediate_size"], num_attention_heads=NH, num_key_value_heads=NKV, head_dim=HD,
              vocab_size=cfg["vocab_size"], rms_norm_eps=cfg["rms_norm_eps"], rope_theta=cfg["rope_theta"],
              max_position_embeddings=cfg["max_position_embeddings"], tie_word_embeddings=tied)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf, f)


CASES = {
    "llama": dict(num_hidden_layers=3, hidden_size=256, intermediate_size=512, head_dim=64, num_attention_heads=4,
                  num_key_value_heads=2, vocab_size=300, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=None,
                  max_position_embeddings=128),
    "qwen3": dict(num_hidden_layers=2, hidden_size=256, intermediate_size=384, head_dim=128, num_attention_heads=2,
                  num_key_value_heads=1, vocab_size=200, rms_norm_eps=1e-6, rope_theta=1000000.0, rope_scaling=None,
                  max_position_embeddings=64, qk_norm=True),
}


@pytest.mark.parametrize("family,tied", [("llama", True), ("llama", False), ("qwen3", True)])
def test_synthetic_checkpoint_round_trip(tmp_path, family, tied):
    from qimeng_megakernel_b200 import synthetic
    from qimeng_megakernel_b200.load_weights import load_weights_from_disk
    cfg = CASES[family]
    w = synthetic.make_weights(cfg, seed=17, device="cpu", gain_jitter=0.1)
    if not tied:
        w["lm_head_weights"] = (w["embed_tokens"].float() * 0.5).to(torch.bfloat16)
    write_checkpoint(str(tmp_path), cfg, w, tied, "qwen3" if family == "qwen3" else "llama")
    got_cfg, got = load_weights_from_disk(tmp_path, device="cpu")
    for k in ("num_hidden_layers", "hidden_size", "intermediate_size", "head_dim", "num_attention_heads",
              "num_key_value_heads", "vocab_size"):
        assert got_cfg[k] == cfg[k]
    assert got_cfg["qk_norm"] == bool(cfg.get("qk_norm"))
    names = ["qkv_weights", "o_proj_weights", "attn_norm_weights", "mlp_norm_weights", "up_proj_weights",
             "gate_proj_weights", "down_proj_weights", "lm_head_norm_weights", "lm_head_weights", "embed_tokens",
             "rope_cos", "rope_sin"] + (["q_norm_weights", "k_norm_weights"] if cfg.get("qk_norm") else [])
    for n in names:
        assert torch.equal(got[n], w[n]), f"{n} differs after the round trip"
    assert (got["lm_head_weights"].data_ptr() == got["embed_tokens"].data_ptr()) == tied
    # a checkpoint that lacks a tensor is refused
    os.remove(os.path.join(str(tmp_path), "model-00002-of-00002.safetensors"))
    with pytest.raises(FileNotFoundError):
        load_weights_from_disk(tmp_path, device="cpu")


def test_agrees_with_the_reference_loader(tmp_path):
    ref = os.environ.get("QMK_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
    if not os.path.isdir(os.path.join(ref, "qimeng_megakernel")):
        pytest.skip("no reference checkout on this machine")
    if ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        from qimeng_megakernel.models.LLM.llama.load_weights import load_llama_weights_from_disk
    except Exception as e:
        pytest.skip(f"reference loader not importable here: {e}")
    from qimeng_megakernel_b200 import synthetic
    from qimeng_megakernel_b200.load_weights import load_weights_from_disk
    cfg = CASES["llama"]
    w = synthetic.make_weights(cfg, seed=18, device="cpu")
    write_checkpoint(str(tmp_path), cfg, w, True, "llama")
    _, ours = load_weights_from_disk(tmp_path, device="cpu")
    _, theirs = load_llama_weights_from_disk(str(tmp_path), torch.device("cpu"), torch.bfloat16)
    for name, t in theirs.items():
        if name in ("rope_cos", "rope_sin"):
            assert torch.allclose(ours[name], t, rtol=1e-6, atol=1e-6), name
        else:
            assert torch.equal(ours[name], t), name
