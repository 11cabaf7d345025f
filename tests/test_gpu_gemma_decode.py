"""GPU parity of the Gemma-shaped decode engine against the unsharded CPU oracle model.
One GPU: TP = 1 in-process.  Two or more GPUs: `tests/tp_worker.py` under torch.distributed.run
(see test_tp2_matches_oracle_when_two_gpus), each rank holding its shard, NCCL all-reduce at
the o_proj / down_proj boundaries.

The Q4_K path has no int8 re-quantiser between layers, so small arithmetic differences stay
small: logits must agree to 2e-3 of their spread and the greedy tokens must be identical under
teacher forcing (a differing argmax counts only if the oracle's top-2 margin exceeds the
logit tolerance)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from hesper_b200 import GemmaModel, tp
from tp_common import SMALL_GEMMA

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LOGIT_TOL = 2e-3


def test_tp1_forced_steps(ctx, oracle):
    from oracle.oracle import GemmaOracle
    S = SMALL_GEMMA
    w = tp.random_gemma_weights(S, seed=21)
    p = tp.plan(S, 0, 1)
    model = GemmaModel(ctx, S, tp.shard_weights(S, w, p), p, None, batch=2, max_new_tokens=8)
    orcs = [GemmaOracle(S, w) for _ in range(2)]
    rng = np.random.default_rng(4)
    toks = rng.integers(0, S.vocab, (2, 1)).astype(np.int32).tolist()
    # 40 steps: past the 16-position window, so the ring cache wraps more than twice
    for t in range(40):
        cur = np.array([toks[b][t] for b in range(2)], np.int32)
        g_tok, g_logits = model.step(torch.from_numpy(cur).cuda())
        for b in range(2):
            o_tok, o_logits = orcs[b].step(int(cur[b]))
            sd = float(np.std(o_logits))
            assert np.max(np.abs(g_logits[b] - o_logits)) < LOGIT_TOL * sd
            if int(g_tok[b]) != o_tok:
                top2 = np.partition(o_logits, -2)[-2:]
                assert top2[1] - top2[0] <= 2 * LOGIT_TOL * sd
            toks[b].append(o_tok)
    ctx.check()
    for o in orcs:
        o.close()
    model.close()


def test_tp1_forced_steps_wide_batch(ctx, oracle):
    """Batch 20: every product on the tensor cores (f16 activations, one power-of-two scale per
    row), the path the batch-32 / batch-256 decode numbers run on; this model's FFN
    intermediates reach a few 1e4, which needed that scale.  The random weights of the test
    model have mean +1.1, so the hidden state is one large common-mode component; for the odd
    token whose activations sum to almost zero the logits are ill-conditioned and the streaming
    kernels and the tensor-core kernels alike miss them by up to 4e-2 of their spread (2 of 20
    sequences, measured with both).  The bar is therefore stated over the run: every logit
    vector finite and within 5e-2, the median deviation under 1e-3 (measured 3e-4, the f16
    rounding of the weights), at most one (step, sequence) pair in ten outside the 2e-3 of
    the narrow-batch test, and the margin rule for tokens only where the logits are inside it."""
    from oracle.oracle import GemmaOracle
    S, batch = SMALL_GEMMA, 20
    w = tp.random_gemma_weights(S, seed=21)
    p = tp.plan(S, 0, 1)
    model = GemmaModel(ctx, S, tp.shard_weights(S, w, p), p, None, batch=batch, max_new_tokens=8)
    orcs = [GemmaOracle(S, w) for _ in range(batch)]
    rng = np.random.default_rng(4)
    toks = rng.integers(0, S.vocab, (batch, 1)).astype(np.int32).tolist()
    devs = []
    for t in range(40):
        cur = np.array([toks[b][t] for b in range(batch)], np.int32)
        g_tok, g_logits = model.step(torch.from_numpy(cur).cuda())
        assert np.isfinite(g_logits).all()
        for b in range(batch):
            o_tok, o_logits = orcs[b].step(int(cur[b]))
            sd = float(np.std(o_logits))
            dev = float(np.max(np.abs(g_logits[b] - o_logits))) / sd
            devs.append(dev)
            if dev < LOGIT_TOL and int(g_tok[b]) != o_tok:
                top2 = np.partition(o_logits, -2)[-2:]
                assert top2[1] - top2[0] <= 2 * LOGIT_TOL * sd
            toks[b].append(o_tok)
    devs = np.array(devs)
    print(f"GEMMA_SMALL_B20 median={np.median(devs):.2e} max={devs.max():.2e} "
          f"outside={np.mean(devs >= LOGIT_TOL):.3f}")
    assert devs.max() < 5e-2
    assert np.median(devs) < 1e-3
    assert np.mean(devs >= LOGIT_TOL) <= 0.1
    ctx.check()
    for o in orcs:
        o.close()
    model.close()


@pytest.mark.parametrize("chunk,batch", [(5, 2), (7, 1), (0, 3)])
def test_prompt_chunks_match_the_oracle(ctx, oracle, chunk, batch, monkeypatch):
    """Prompt passes of several positions per sequence (Gemma4.forwardPrefillBatch,
    Hesper/Models/Gemma4.lean:1333): a 45-token prompt fed in chunks, the logits of every chunk's
    last position and of 8 decode steps after it against the oracle, which takes the same tokens
    one by one.  With chunk 5 / 7 the sliding-window layers run on rings of 16 + chunk - 1 slots
    that wrap twice inside the prompt; chunk 0 = the default (256 / batch rows per pass: the
    whole prompt at once, linear caches because the ring would be as long as max_seq)."""
    from oracle.oracle import GemmaOracle
    S = SMALL_GEMMA
    if chunk:
        monkeypatch.setenv("HB200_GEMMA_CHUNK", str(chunk))
    w = tp.random_gemma_weights(S, seed=23)
    p = tp.plan(S, 0, 1)
    model = GemmaModel(ctx, S, tp.shard_weights(S, w, p), p, None, batch=batch, max_new_tokens=8)
    T = model.chunk
    assert T == (chunk if chunk else 256 // batch)
    orcs = [GemmaOracle(S, w) for _ in range(batch)]
    prompt = np.random.default_rng(6).integers(0, S.vocab, (batch, 45)).astype(np.int32)

    def compare(g_tok, g_logits, o_out):
        for b in range(batch):
            o_tok, o_logits = o_out[b]
            sd = float(np.std(o_logits))
            assert np.max(np.abs(g_logits[b] - o_logits)) < LOGIT_TOL * sd
            if int(g_tok[b]) != o_tok:
                top2 = np.partition(o_logits, -2)[-2:]
                assert top2[1] - top2[0] <= 2 * LOGIT_TOL * sd

    o_out = None
    for p0 in range(0, 45, T):
        part = np.ascontiguousarray(prompt[:, p0:p0 + T])
        g_tok, g_logits = model.prefill(torch.from_numpy(part).cuda())
        for t in range(part.shape[1]):
            o_out = [orcs[b].step(int(part[b, t])) for b in range(batch)]
        compare(g_tok, g_logits, o_out)
    for _ in range(8):  # decode on the caches the chunks left
        cur = np.array([o_out[b][0] for b in range(batch)], np.int32)
        g_tok, g_logits = model.step(torch.from_numpy(cur).cuda())
        o_out = [orcs[b].step(int(cur[b])) for b in range(batch)]
        compare(g_tok, g_logits, o_out)
    ctx.check()
    for o in orcs:
        o.close()
    model.close()


def test_full_shape_gemma_forced_64_steps(ctx, oracle):
    """The shape the benchmark times -- 42 layers, hidden 2560, 8/2 heads of 256, GeGLU FFN
    10240, vocab 262144, window 512, one global layer in six -- in the benchmark's attention
    mode (FAST), 64 teacher-forced greedy steps against the unsharded CPU oracle under the
    margin rule of this file.  (64 positions stay inside the 512-wide window; the ring cache
    wrapping is covered by the small model above.)"""
    import dataclasses
    from oracle.oracle import GemmaOracle
    S = dataclasses.replace(tp.GemmaShape(), max_seq=128)
    w = tp.random_gemma_weights(S, seed=21)
    p = tp.plan(S, 0, 1)
    model = GemmaModel(ctx, S, tp.shard_weights(S, w, p), p, None, batch=1, max_new_tokens=8)
    orc = GemmaOracle(S, w)
    toks, devs, flips = [7], [], 0
    for t in range(64):
        cur = np.array([toks[t]], np.int32)
        g_tok, g_logits = model.step(torch.from_numpy(cur).cuda())
        o_tok, o_logits = orc.step(int(cur[0]))
        sd = float(np.std(o_logits))
        devs.append(float(np.max(np.abs(g_logits[0] - o_logits))) / sd)
        assert devs[-1] < LOGIT_TOL
        if int(g_tok[0]) != o_tok:
            flips += 1
            top2 = np.partition(o_logits, -2)[-2:]
            assert top2[1] - top2[0] <= 2 * LOGIT_TOL * sd
        toks.append(o_tok)
    ctx.check()
    orc.close()
    model.close()
    print(f"GEMMA_FULL_SHAPE_FAST flips={flips}/64 max_logit_dev_over_sd={max(devs):.3e}")
    assert max(devs) < 1e-4  # measured 1e-5: far inside the rule's tolerance


def test_generate_graph_equals_eager(ctx):
    S = SMALL_GEMMA
    w = tp.random_gemma_weights(S, seed=22)
    p = tp.plan(S, 0, 1)
    model = GemmaModel(ctx, S, tp.shard_weights(S, w, p), p, None, batch=3, max_new_tokens=24)
    prompt = np.random.default_rng(5).integers(0, S.vocab, (3, 6)).astype(np.int32)
    a, _, _ = model.generate(prompt, 24, use_graph=True)
    b, _, _ = model.generate(prompt, 24, use_graph=False)
    assert np.array_equal(a, b)
    model.close()


def test_tp2_matches_oracle_when_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port",
                        "29631", os.path.join(ROOT, "tests", "tp_worker.py")],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_PARITY_OK" in r.stdout


def test_withheld_exchange_times_out_cleanly_when_two_gpus():
    """A rank that skips its exchange (decided on the host) makes the peer's kernel run into
    its deadline: status flag, HB200_ERR_TIMEOUT from the context check, later exchanges pass
    at once, both processes exit cleanly.  No trap, no fault, no endless spin; NVLS off."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port",
                        "29633", os.path.join(ROOT, "tests", "tp_worker.py"), "--withhold"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_TIMEOUT_OK" in r.stdout
