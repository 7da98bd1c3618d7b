"""One rank of the tensor-parallel parity check (launched by tests/test_tp_multi.py with torchrun).

Every rank builds its shard of a seeded model; rank 0 also builds the unsharded model.  Checked on
every rank, for each way of doing the all-reduce (NCCL, the one-shot peer-memory kernel, the
exchange folded into the packed GEMVs), eager and from a CUDA graph, at batch 1 and 3: the greedy
tokens of the sharded decoder equal the single-GPU decoder's, the logits agree within 2e-3 of
max|logit|, and no bounded wait ran out.  Prints one JSON line from rank 0 and exits 0 on success.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist


def main():
    from nativebit_b200 import generate as G
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    # heads divisible by 8 ranks, FFN blocks not (11 blocks): uneven whole-block shares
    cfg = G.ModelConfig(vocab_size=1024, n_layers=3, n_embd=1024, n_head=8, ffn_hidden=1408, context_len=64)
    n_gen = 10
    prompt = torch.randint(0, cfg.vocab_size, (1, 9), generator=torch.Generator().manual_seed(0)).to(dev)
    full = G.PackedGPT.random_init(cfg, seed=0, device=dev)           # every rank: the single-GPU answer
    ref = {}
    for B in (1, 3):
        s = G.DecodeSession(full, B, use_graph=False)
        toks = s.generate(prompt.repeat(B, 1), n_gen)
        ref[B] = (toks, s.logits.clone())
    del full
    model = G.PackedGPT.random_init(cfg, seed=0, device=dev, tp_rank=rank, tp_size=world)
    report, ok = {}, True
    for mode in ("nccl", "oneshot", "fused"):
        if mode == "oneshot":
            model.enable_oneshot_allreduce(8)
        if mode == "fused":
            model.enable_fused_allreduce(8)
        for graph in (False, True):
            for B in (1, 3):
                s = G.DecodeSession(model, B, use_graph=graph)
                toks = s.generate(prompt.repeat(B, 1), n_gen)
                torch.cuda.synchronize()
                s.check()
                err = float((s.logits - ref[B][1]).abs().max() / ref[B][1].abs().max())
                same = bool(torch.equal(toks, ref[B][0]))
                flags = torch.tensor([int(same), int(err <= 2e-3)], device=dev)
                dist.all_reduce(flags, op=dist.ReduceOp.MIN)
                good = bool(flags.min().item() == 1)
                ok = ok and good
                report[f"{mode}_{'graph' if graph else 'eager'}_b{B}"] = {"tokens_equal": same, "logit_err": err, "all_ranks": good}
    if rank == 0:
        print(json.dumps({"tp_parity": report, "world": world, "ok": ok}), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if ok else 1)        # communicators captured in CUDA graphs cannot be torn down cleanly


if __name__ == "__main__":
    main()
