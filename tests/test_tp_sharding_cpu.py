"""CPU, world_size 2 over gloo: the tensor-parallel sharding rules and the exchange step.
Each rank shards the same seeded weights, computes its part with the CPU oracle, the partial
vectors of the row-split matvecs are summed with an all-reduce, and the result must equal the
unsharded oracle.  No GPU, no CUDA library call."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hesper_b200 import tp
    from oracle import oracle as orc
    from tp_common import SMALL_GEMMA as S
    orc.set_num_threads(2)
    w = tp.random_gemma_weights(S, seed=11)
    p = tp.plan(S, rank, world)
    sh = tp.shard_weights(S, w, p)
    rng = np.random.default_rng(3)
    D, Hd = S.head_dim, S.hidden
    qd = S.n_heads * D
    L, SL = w["layers"][1], sh["layers"][1]
    ok = True
    # column split (output rows): the shard's outputs are a slice of the full outputs
    x = rng.standard_normal((1, Hd)).astype(np.float32)
    full_q = orc.q4k_matvec(L["wq"], Hd, qd, x)
    mine_q = orc.q4k_matvec(SL["wq"], Hd, p.local_q * D, x)
    ok &= np.array_equal(mine_q[0], full_q[0, p.q_heads.start * D:p.q_heads.stop * D])
    full_g = orc.kquant_gateup_gelu(L["wgate"], L["wup"], 12, Hd, S.ffn, x)
    mine_g = orc.kquant_gateup_gelu(SL["wgate"], SL["wup"], 12, Hd, len(p.ffn_rows), x)
    ok &= np.array_equal(mine_g[0], full_g[0, p.ffn_rows.start:p.ffn_rows.stop])
    # row split (input columns): partial vectors, one sum all-reduce
    att = rng.standard_normal((1, qd)).astype(np.float32)
    part = orc.q4k_matvec(SL["wo"], p.local_q * D, Hd,
                          att[:, p.q_heads.start * D:p.q_heads.stop * D])
    t = torch.from_numpy(part.astype(np.float64))
    dist.all_reduce(t)
    full_o = orc.q4k_matvec(L["wo"], qd, Hd, att)
    ok &= bool(np.max(np.abs(t.numpy() - full_o)) <= 2e-6 * np.max(np.abs(full_o)))
    hfull = rng.standard_normal((1, S.ffn)).astype(np.float32)
    part = orc.q4k_matvec(SL["wdown"], len(p.ffn_rows), Hd,
                          hfull[:, p.ffn_rows.start:p.ffn_rows.stop])
    t = torch.from_numpy(part.astype(np.float64))
    dist.all_reduce(t)
    full_d = orc.q4k_matvec(L["wdown"], S.ffn, Hd, hfull)
    ok &= bool(np.max(np.abs(t.numpy() - full_d)) <= 2e-6 * np.max(np.abs(full_d)))
    # LM head: local argmax keys, max all-reduce picks the global greedy token
    lg = orc.q4k_matvec(sh["lm_head"], Hd, len(p.vocab_rows), x)[0]
    li = int(np.argmax(lg))
    best = torch.tensor([float(lg[li]), -float(p.vocab_rows.start + li)], dtype=torch.float64)
    gathered = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, best)
    win = max(gathered, key=lambda g: (g[0].item(), g[1].item()))
    full_l = orc.q4k_matvec(w["lm_head"], Hd, S.vocab, x)[0]
    ok &= int(-win[1].item()) == int(np.argmax(full_l))
    with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "fail")
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_equals_unsharded_world2(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok"


def test_plans_cover_everything_once():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from hesper_b200 import tp
    S = tp.GemmaShape()
    for T in (1, 2, 4, 8):
        plans = [tp.plan(S, r, T) for r in range(T)]
        assert sorted(h for p in plans for h in p.q_heads) == list(range(S.n_heads))
        assert sorted(r for p in plans for r in p.ffn_rows) == list(range(S.ffn))
        assert sum(len(p.vocab_rows) for p in plans) == S.vocab
        G = S.n_heads // S.n_kv_heads
        for p in plans:
            assert all(h // G in p.kv_heads for h in p.q_heads)
            assert (p.local_q * S.head_dim) % 256 == 0 and len(p.ffn_rows) % 256 == 0
    with pytest.raises(ValueError):
        tp.plan(S, 0, 3)


def test_shard_cols_roundtrip():
    from hesper_b200 import formats, tp
    rng = np.random.default_rng(0)
    N, K = 6, 1024
    b = formats.random_q4k(rng, N, K)
    parts = [tp.shard_cols(b, N, K, range(c, c + 256)).reshape(N, 1, 144) for c in range(0, K, 256)]
    assert np.array_equal(np.concatenate(parts, 1).reshape(-1), b)
    with pytest.raises(ValueError):
        tp.shard_cols(b, N, K, range(128, 384))
