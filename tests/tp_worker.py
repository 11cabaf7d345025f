"""One rank of the tensor-parallel parity run (launched by torch.distributed.run).
Every rank builds the same seeded small Gemma-shaped model, keeps its shard on its GPU, and
decodes teacher-forced steps; rank 0 runs the unsharded CPU oracle beside it and compares the
greedy tokens and the gathered logits."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")  # host-side plumbing only; the data path is NCCL in the library
    import hesper_b200 as hb
    from hesper_b200 import tp
    from tp_common import SMALL_GEMMA as S
    ctx = hb.Context(local)
    comm = tp.TensorParallel.from_torch_distributed(ctx)
    w = tp.random_gemma_weights(S, seed=31)
    p = tp.plan(S, rank, world)
    model = hb.GemmaModel(ctx, S, tp.shard_weights(S, w, p), p, comm, batch=2, max_new_tokens=8)
    ok = True
    if rank == 0:
        from oracle.oracle import GemmaOracle
        orcs = [GemmaOracle(S, w) for _ in range(2)]
    toks = np.random.default_rng(6).integers(0, S.vocab, (2,)).astype(np.int32)
    for t in range(24):
        cur = torch.from_numpy(toks.copy()).cuda()
        g_tok, g_local = model.step(cur)
        parts = [None] * world
        dist.all_gather_object(parts, g_local)
        nxt = np.zeros(2, np.int32)
        if rank == 0:
            logits = np.concatenate(parts, axis=1)
            for b in range(2):
                o_tok, o_logits = orcs[b].step(int(toks[b]))
                sd = float(np.std(o_logits))
                if np.max(np.abs(logits[b] - o_logits)) >= 2e-3 * sd:
                    ok = False
                if int(g_tok[b]) != o_tok:
                    top2 = np.partition(o_logits, -2)[-2:]
                    if top2[1] - top2[0] > 4e-3 * sd:
                        ok = False
                nxt[b] = o_tok
        box = [nxt]
        dist.broadcast_object_list(box, src=0)
        toks = box[0]
    comm.check()
    ctx.check()
    flag = [ok]
    dist.broadcast_object_list(flag, src=0)
    model.close()
    comm.close()
    dist.barrier()
    if rank == 0:
        print("TP_PARITY_OK" if flag[0] else "TP_PARITY_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag[0] else 1)


if __name__ == "__main__":
    main()
