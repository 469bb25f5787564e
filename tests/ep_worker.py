"""Worker of tests/test_gpu_expert_parallel.py: one process per GPU (torchrun, gloo for the control plane).

`ep` (default): every rank builds the same seeded mixture-of-experts model and keeps its block of experts.  `tp`: the same
seeded dense model, every rank keeps its slice of every projection (tensor parallelism).  Either way the ranks connect the
exchange buffers and decode the same teacher-forced steps; rank 0 also runs the whole model on its own GPU.  Checks: every rank ends a step
with bit-identical logits (the partial tiles are added in rank order on every rank); the expert-parallel result matches the
one-GPU result (hidden state within 1e-2 relative L2, arg-max equal wherever the one-GPU top two are not tied); and, in
the second part, a rank that does not launch makes the others' bounded wait run out into QMK_ERR_DEVICE_TIMEOUT, after
which a healthy step works again.  Nothing here faults or hangs a GPU: the missing rank simply skips a launch.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from qimeng_megakernel_b200 import _lib, expert_parallel as ep, mk_kernel, synthetic, tensor_parallel as tp  # noqa: E402
from qimeng_megakernel_b200.model_config import LlamaConfig  # noqa: E402

MOE = dict(num_hidden_layers=2, hidden_size=256, intermediate_size=64, head_dim=128, num_attention_heads=2,
           num_key_value_heads=2, vocab_size=777, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
           max_position_embeddings=256, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128)
# dense: 4 query / 2 KV heads of 64, intermediate 512, a vocabulary whose slices are not multiples of the tile height
DENSE = dict(num_hidden_layers=2, hidden_size=256, intermediate_size=512, head_dim=64, num_attention_heads=4,
             num_key_value_heads=2, vocab_size=1500, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
             max_position_embeddings=256)


def main() -> None:
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    B, steps = 5, 6
    mode = sys.argv[1] if len(sys.argv) > 1 else "ep"
    CFG = DENSE if mode == "tp" else MOE
    full = synthetic.make_weights(CFG, seed=77, device="cpu", gain_jitter=0.1, max_positions=64)
    prompts = synthetic.make_prompts(CFG["vocab_size"], B, steps, seed=3)
    # ---- this rank's shard
    if mode == "tp":
        cfg_r = tp.shard_config(CFG, rank, world)
        shard = tp.shard_weights(CFG, full, rank, world)
    else:
        cfg_r = ep.shard_config(CFG, rank, world)
        shard = ep.shard_moe_weights(full, rank, world)
    g = synthetic.make_globals(cfg_r, shard, kv_seq_len=32, device=dev, batch=B)
    g.token_in = torch.zeros(B, dtype=torch.int64, device=dev)
    mk = mk_kernel.get_mk()
    LlamaConfig.update_from_dict(cfg_r)
    ep.connect(mk, g)
    # ---- the whole model on one GPU (rank 0 only)
    if rank == 0:
        g1 = synthetic.make_globals(CFG, full, kv_seq_len=32, device=dev, batch=B)
        g1.token_in = torch.zeros(B, dtype=torch.int64, device=dev)
        mk1 = mk_kernel.get_mk()
    ok = True
    for step in range(steps):
        dist.barrier()                             # ranks launch a step together: the wait for a peer's tiles is bounded
        LlamaConfig.update_from_dict(cfg_r)
        g.token_in.copy_(prompts[:, step]); g.position_id = step
        mk(g)
        torch.cuda.synchronize()
        mk.check_status()
        # what every rank must agree on, bit for bit: the residual stream and the chosen tokens (and, when every rank
        # holds the whole LM head, the logits); as bytes: gloo gathers no 16-bit types
        parts = [g.hidden_states.contiguous().view(torch.uint8).flatten(), g.next_token.view(torch.uint8).flatten()]
        if mode != "tp":
            parts.append(g.logits.contiguous().view(torch.uint8).flatten())
        mine = torch.cat(parts).cpu()
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        if not all(torch.equal(gathered[0], t) for t in gathered):
            print(f"rank {rank} step {step}: ranks disagree on the state after the step", flush=True); ok = False
        if rank == 0:
            LlamaConfig.update_from_dict(CFG)
            g1.token_in.copy_(prompts[:, step]); g1.position_id = step
            mk1(g1)
            torch.cuda.synchronize()
            mk1.check_status()
            a, e = g.hidden_states.float(), g1.hidden_states.float()
            rel = float((a - e).norm() / e.norm())
            if rel > 1e-2:
                print(f"step {step}: hidden state differs from the one-GPU run, relative L2 {rel:.4g}", flush=True); ok = False
            ref = g1.logits.float()
            if mode == "tp":     # this rank's slice of the logits against the same rows of the one-GPU logits
                vl = g.logits.shape[-1]
                gap = float((g.logits.float() - ref[:, :vl]).abs().max())
                if gap > 2e-2 * float(ref.abs().max()):
                    print(f"step {step}: logits slice differs from the one-GPU run by {gap:.4g}", flush=True); ok = False
            top2 = ref.topk(2, dim=-1).values
            for b in range(B):
                if float(top2[b, 0] - top2[b, 1]) > 4 * 2.0 ** -8 * abs(float(top2[b, 0])) and int(g.next_token[b]) != int(g1.next_token[b]):
                    print(f"step {step} row {b}: arg-max differs from the one-GPU run on an untied row", flush=True); ok = False
    # ---- a rank that does not launch: the others' wait runs out, the status says so, the next step is healthy
    dist.barrier()
    LlamaConfig.update_from_dict(cfg_r)
    mk.set_timeout_cycles(40_000_000)          # about 20 ms
    g.token_in.copy_(prompts[:, 0]); g.position_id = steps
    if rank != world - 1:
        mk(g)
        torch.cuda.synchronize()
        st = mk.poll_status()
        if st["rc"] != _lib.ERR_DEVICE_TIMEOUT:
            print(f"rank {rank}: expected the wait for the missing rank to expire, got {st}", flush=True); ok = False
    dist.barrier()
    if rank == world - 1:
        # the launch counter tags the exchange: catch up with the launch the other ranks made (it finds their flags or times out)
        mk(g)
        torch.cuda.synchronize()
        mk.poll_status()
    dist.barrier()
    mk.set_timeout_cycles(2_000_000_000)
    g.position_id = steps + 1
    mk(g)
    torch.cuda.synchronize()
    st = mk.poll_status()
    if st["rc"] != 0:
        print(f"rank {rank}: the step after the failure did not recover: {st}", flush=True); ok = False
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_WORKER_OK" if int(flag) == 1 else "EP_WORKER_FAILED", flush=True)
    mk.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
