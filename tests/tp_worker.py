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


def check_allreduce(hb, ctx, comm, rank, world):
    """The exchange step on its own: the one-shot peer all-reduce must give, on every rank,
    exactly the f32 sum taken in rank order (and the u64 maximum), call after call and when
    replayed from a CUDA graph."""
    import ctypes as C
    fails = []

    def need(cond, what):
        if not cond:
            fails.append(what)

    need(comm.peer_attached or os.environ.get("HB200_TP_NO_PEER", "0") == "1", "peers attached")
    st = torch.cuda.Stream()
    for it, n in enumerate([2560, 2560 * 2, 2560 * 64, 4, 2560 * 7] * 4):
        parts = [np.random.default_rng(1000 * it + r).standard_normal(n).astype(np.float32)
                 for r in range(world)]
        want = parts[0].copy()
        for r in range(1, world):
            want = (want + parts[r]).astype(np.float32)
        x = torch.from_numpy(parts[rank].copy()).cuda()
        torch.cuda.synchronize()
        comm.allreduce_f32(x, stream=st)
        st.synchronize()
        got = x.cpu().numpy()
        if comm.peer_attached:
            need(np.array_equal(got, want), f"all-reduce n={n} call {it}: rank-order sum, bit for bit")
        else:
            need(np.allclose(got, want, rtol=1e-5, atol=1e-5), f"all-reduce n={n} call {it}")
    # u64 maximum (argmax keys)
    keys = torch.from_numpy(np.random.default_rng(7 + rank).integers(0, 2**62, 8)).cuda()
    allk = [np.random.default_rng(7 + r).integers(0, 2**62, 8) for r in range(world)]
    hb.load().hb200_tp_allreduce_max_u64(comm.handle, C.c_void_p(keys.data_ptr()), C.c_size_t(8),
                                         C.c_void_p(st.cuda_stream))
    st.synchronize()
    need(np.array_equal(keys.cpu().numpy(), np.max(np.stack(allk), axis=0)), "u64 maximum")
    # the exchange fused with the RMSNorm (+ residual) that follows it: rank-order sum, then
    # the stand-alone kernel's arithmetic.  K = 2560 takes the flag-in-data kernel (up to 256
    # tokens), K = 4096 the flagged one (up to 64), 300 tokens the unfused route.
    lib = hb.load()
    for it, (M, K) in enumerate([(1, 2560), (32, 2560), (200, 2560), (256, 2560), (5, 4096),
                                 (64, 2560), (300, 2560), (1, 2560)]):
        parts = [np.random.default_rng(5000 + 10 * it + r).standard_normal((M, K)).astype(np.float32)
                 for r in range(world)]
        total = parts[0].copy()
        for r in range(1, world):
            total = (total + parts[r]).astype(np.float32)
        rng = np.random.default_rng(77 + it)
        gamma = torch.from_numpy((1 + 0.1 * rng.standard_normal(K)).astype(np.float32)).cuda()
        add = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
        x = torch.from_numpy(parts[rank].copy()).cuda()
        y = torch.empty_like(x)
        want = torch.empty_like(x)
        t = torch.from_numpy(total).cuda()
        torch.cuda.synchronize()
        rc = lib.hb200_tp_allreduce_rmsnorm(comm.handle, ctx.handle, C.c_void_p(x.data_ptr()),
                                            C.c_void_p(gamma.data_ptr()), C.c_void_p(add.data_ptr()),
                                            C.c_float(1e-6), M, K, C.c_void_p(y.data_ptr()),
                                            C.c_void_p(st.cuda_stream))
        need(rc == 0, f"fused exchange M={M} K={K}: rc {rc}")
        rc = lib.hb200_rmsnorm(ctx.handle, C.c_void_p(t.data_ptr()), C.c_void_p(gamma.data_ptr()),
                               C.c_void_p(add.data_ptr()), C.c_float(1e-6), M, K,
                               C.c_void_p(want.data_ptr()), C.c_void_p(st.cuda_stream))
        need(rc == 0, "rmsnorm")
        st.synchronize()
        # the peer kernels add in rank order; 300 tokens go through NCCL, whose order is its own
        if comm.peer_attached and K == 2560 and M <= 256:
            need(bool(torch.equal(y, want)), f"fused exchange M={M} K={K}: bits of the stand-alone kernel")
        else:
            need(bool(torch.allclose(y, want, rtol=1e-5, atol=1e-5)), f"fused exchange M={M} K={K}")
    # graph replay: the sequence number advances on the device
    x = torch.full((2560,), float(rank + 1), device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(3):
                comm.allreduce_f32(x, stream=st)
        for _ in range(4):
            g.replay()
        st.synchronize()
    tot = float(sum(range(1, world + 1)))
    expect = tot * float(world) ** 11  # 12 all-reduces: the first sums the ranks, 11 multiply by W
    need(bool(torch.all(x == expect).item()), f"graph replay: {float(x[0].item())} != {expect}")
    ctx.check()
    if fails:
        print(f"rank {rank}: exchange checks failed: {fails[:8]}", flush=True)
    return not fails


def withheld_exchange(hb, ctx, comm, rank, world):
    """Failure detection without a GPU fault: rank 1 does not take part in three exchanges (a
    host-side decision), rank 0's kernels must give up by themselves when their deadline
    passes, flag the context, let the later exchanges through at once, and leave the GPU and
    the process usable.  Plain peer stores only (NVLS is off for this run)."""
    import ctypes as C
    import time
    from hesper_b200 import HesperB200Error
    lib = hb.load()
    if not comm.peer_attached:
        return True  # nothing to time out on the NCCL route: not the subject of this check
    comm.set_timeout_ms(50)
    M, K = 4, 2560
    st = torch.cuda.Stream()
    x = torch.ones(M, K, device="cuda") * (rank + 1)
    gamma = torch.ones(K, device="cuda")
    y = torch.empty_like(x)

    def exchange():
        rc = lib.hb200_tp_allreduce_rmsnorm(comm.handle, ctx.handle, C.c_void_p(x.data_ptr()),
                                            C.c_void_p(gamma.data_ptr()), None, C.c_float(1e-6),
                                            M, K, C.c_void_p(y.data_ptr()),
                                            C.c_void_p(st.cuda_stream))
        assert rc == 0, lib.hb200_last_error()

    torch.cuda.synchronize()
    exchange()                      # everybody takes part: completes, no flag
    st.synchronize()
    ok = ctx.check() == 0
    dist.barrier()
    if rank == 0:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        for i in range(3):          # rank 1 withholds these three
            ev[i].record(st)
            exchange()
        ev[3].record(st)
        t0 = time.perf_counter()
        st.synchronize()            # returns: the waits are bounded
        ok = ok and (time.perf_counter() - t0) < 5.0
        first, second, third = (ev[i].elapsed_time(ev[i + 1]) for i in range(3))
        ok = ok and 30.0 <= first <= 500.0          # waited for its 50 ms deadline, once
        ok = ok and second < 10.0 and third < 10.0  # context already in error: look once, go on
        try:
            ctx.check()
            ok = False                              # the expired wait must be reported
        except HesperB200Error as e:
            ok = ok and e.code == -4                # HB200_ERR_TIMEOUT
        ok = ok and ctx.check() == 0                # reported once, then cleared
        # the GPU and the library are still usable
        t = torch.ones(8, device="cuda")
        ok = ok and float((t * 2).sum().item()) == 16.0
    dist.barrier()                  # rank 1 stays (its buffer mapped) until rank 0 is done
    return ok


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
    if "--withhold" in sys.argv:
        ok = withheld_exchange(hb, ctx, comm, rank, world)
        oks = [None] * world
        dist.all_gather_object(oks, bool(ok))
        comm.close()
        dist.barrier()
        if rank == 0:
            print("TP_TIMEOUT_OK" if all(oks) else "TP_TIMEOUT_FAIL", flush=True)
        dist.destroy_process_group()
        sys.exit(0 if all(oks) else 1)
    ok_ar = check_allreduce(hb, ctx, comm, rank, world)
    if "--full-shape" in sys.argv:
        # the benchmark model's widths (hidden 2560, 8/2 heads of 256, FFN 10240, vocab 262144)
        # with two layers, one sliding-window and one global: every sharding rule of TP 2, 4 and
        # 8 is exercised (KV heads replicated beyond 2 ranks, 5-block row splits at 8)
        import dataclasses
        S = dataclasses.replace(tp.GemmaShape(), n_layers=2, max_seq=128, window=16,
                                global_every=2)
    w = tp.random_gemma_weights(S, seed=31)
    p = tp.plan(S, rank, world)
    model = hb.GemmaModel(ctx, S, tp.shard_weights(S, w, p), p, comm, batch=2, max_new_tokens=8)
    ok = True
    why = []
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
                dev = float(np.max(np.abs(logits[b] - o_logits))) / sd
                if dev >= 2e-3:
                    ok = False
                    why.append(f"step {t} seq {b}: logits off by {dev:.2e} of their spread")
                if int(g_tok[b]) != o_tok:
                    top2 = np.partition(o_logits, -2)[-2:]
                    if top2[1] - top2[0] > 4e-3 * sd:
                        ok = False
                        why.append(f"step {t} seq {b}: token {int(g_tok[b])} != {o_tok}")
                nxt[b] = o_tok
        box = [nxt]
        dist.broadcast_object_list(box, src=0)
        toks = box[0]
    comm.check()
    ctx.check()
    comm_attached = comm.peer_attached
    oks = [None] * world
    dist.all_gather_object(oks, bool(ok_ar))
    flag = [ok and all(oks)]
    dist.broadcast_object_list(flag, src=0)
    if rank == 0 and not flag[0]:
        print(f"exchange checks per rank: {oks}; model: {why[:6]}", flush=True)
    model.close()
    comm.close()
    dist.barrier()
    if rank == 0:
        print(("TP_PARITY_OK" if flag[0] else "TP_PARITY_FAIL") +
              f" world={world} layers={S.n_layers} hidden={S.hidden} heads={S.n_heads}/"
              f"{S.n_kv_heads} ffn={S.ffn} vocab={S.vocab} steps=24 batch=2 "
              f"peer_exchange={int(comm_attached)}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag[0] else 1)


if __name__ == "__main__":
    main()
