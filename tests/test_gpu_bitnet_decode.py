"""GPU parity of the whole decode step of a BitNet-b1.58-shaped model (random-init weights)
against the CPU oracle model: greedy tokens over 64 steps and logits.

Why the attention runs in its EXACT mode here: the model re-quantises its activations to int8
after every block, so it is chaotic at the level of its quantisation noise -- one activation
rounding the other way because attention differed by 1e-6 becomes per-cent logit noise a few
layers later, and a 30-layer random-init model then swaps near-tied tokens every few steps.
With the bit-reproducible attention kernel (mirrored operation for operation by the oracle)
every quantiser sees identical inputs on both sides; what is left is the LM head's f32 versus
f64 accumulation (~1e-6).

Comparison rule (stated before measuring): each step is teacher-forced with the oracle's
token; a differing argmax counts as a mismatch only if the oracle's own top-1/top-2 margin
exceeds MARGIN times the logit standard deviation."""
import numpy as np
import pytest
import torch

from hesper_b200 import BitNetModel, BitNetShape, random_bitnet_weights

pytestmark = pytest.mark.gpu
MARGIN = 1e-4

SMALL = BitNetShape(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=384,
                    vocab=512, max_seq=96, rope_base=500000.0, rms_eps=1e-5)


@pytest.fixture(autouse=True)
def _exact_attention(ctx):
    ctx.set_attn_mode(ctx.ATTN_EXACT)
    yield
    ctx.set_attn_mode(ctx.ATTN_FAST)


def _forced_compare(ctx, oracle, shape, weights, prompt, n_steps, batch=1):
    from oracle.oracle import BitNetOracle
    model = BitNetModel(ctx, shape, weights, batch=batch, max_new_tokens=n_steps + 1)
    oracles = [BitNetOracle(shape, weights) for _ in range(batch)]
    for o in oracles:
        o.set_exact_attention(True)
    toks = [list(prompt[b]) for b in range(batch)]
    mismatches, devs = 0, []
    n_total = prompt.shape[1] + n_steps
    for t in range(n_total):
        cur = np.array([toks[b][t] for b in range(batch)], np.int32)
        g_tok, g_logits = model.step(torch.from_numpy(cur).cuda(), want_logits=True)
        for b in range(batch):
            o_tok, o_logits = oracles[b].step(int(cur[b]))
            sd = float(np.std(o_logits))
            devs.append(float(np.max(np.abs(g_logits[b] - o_logits))) / sd)
            if t >= prompt.shape[1] - 1:
                if t + 1 >= len(toks[b]):
                    toks[b].append(o_tok)  # teacher forcing with the oracle's token
                if int(g_tok[b]) != o_tok:
                    top2 = np.partition(o_logits, -2)[-2:]
                    if (top2[1] - top2[0]) > MARGIN * sd:
                        mismatches += 1
    for o in oracles:
        o.close()
    model.close()
    return mismatches, np.array(devs)


def _check_devs(devs):
    """Logit agreement per step: max |gpu - oracle| over the vocabulary in units of the logit
    spread.  Only the LM head's accumulation order differs between the two sides."""
    assert np.max(devs) < 1e-4


def test_small_model_forced_64_steps(ctx, oracle):
    w = random_bitnet_weights(SMALL, seed=1)
    prompt = np.random.default_rng(0).integers(0, SMALL.vocab, (1, 8)).astype(np.int32)
    mism, devs = _forced_compare(ctx, oracle, SMALL, w, prompt, 64)
    assert mism == 0
    _check_devs(devs)


def test_small_model_batch3(ctx, oracle):
    w = random_bitnet_weights(SMALL, seed=2)
    prompt = np.random.default_rng(1).integers(0, SMALL.vocab, (3, 5)).astype(np.int32)
    mism, devs = _forced_compare(ctx, oracle, SMALL, w, prompt, 16, batch=3)
    assert mism == 0
    _check_devs(devs)


def test_generate_graph_equals_stepwise(ctx):
    """The captured-graph decode loop, the uncaptured loop and explicit steps give the same tokens."""
    w = random_bitnet_weights(SMALL, seed=3)
    prompt = np.random.default_rng(2).integers(0, SMALL.vocab, (2, 7)).astype(np.int32)
    model = BitNetModel(ctx, SMALL, w, batch=2, max_new_tokens=32)
    a, _, _ = model.generate(prompt, 32, use_graph=True)
    b, _, _ = model.generate(prompt, 32, use_graph=False)
    assert np.array_equal(a, b)
    model.reset()
    cur = None
    out = []
    for t in range(prompt.shape[1] + 31):
        inp = torch.from_numpy(prompt[:, t].copy()).cuda() if t < prompt.shape[1] else None
        tok, _ = model.step(inp)
        if t >= prompt.shape[1] - 1:
            out.append(tok.copy())
    assert np.array_equal(np.stack(out, 1), a)
    model.close()


@pytest.mark.parametrize("batch,plen", [(3, 50), (1, 130), (40, 5), (1, 300), (5, 120)])
def test_chunked_prefill_equals_stepwise(ctx, batch, plen):
    """generate() consumes the prompt in chunks of 256 // batch positions through the batched
    tensor-core kernels (passes of 64 rows) and causal prefill attention (ragged last chunk;
    more than one chunk at (1, 300) and (5, 120)); explicit single-token steps over the same
    prompt must give the same tokens."""
    import dataclasses
    shape = dataclasses.replace(SMALL, max_seq=320)
    w = random_bitnet_weights(shape, seed=9)
    prompt = np.random.default_rng(plen).integers(0, shape.vocab, (batch, plen)).astype(np.int32)
    model = BitNetModel(ctx, shape, w, batch=batch, max_new_tokens=12)
    a, _, _ = model.generate(prompt, 12, use_graph=True)
    model.reset()
    out = []
    for t in range(plen + 11):
        inp = torch.from_numpy(prompt[:, t].copy()).cuda() if t < plen else None
        tok, _ = model.step(inp)
        if t >= plen - 1:
            out.append(tok.copy())
    assert np.array_equal(np.stack(out, 1), a)
    model.close()


def test_full_size_bitnet2b_forced_64_steps(ctx, oracle):
    """BitNet-b1.58-2B shape (30 layers, hidden 2560, 20/5 heads, FFN 6912, vocab 128256),
    short prompt, 64 teacher-forced greedy steps against the CPU oracle."""
    shape = BitNetShape.bitnet_2b(max_seq=128)
    w = random_bitnet_weights(shape, seed=4)
    prompt = np.random.default_rng(3).integers(0, shape.vocab, (1, 4)).astype(np.int32)
    mism, devs = _forced_compare(ctx, oracle, shape, w, prompt, 64)
    assert mism == 0
    _check_devs(devs)


@pytest.mark.parametrize("mode", ["FAST", "PRECISE"])
def test_full_size_bitnet2b_other_attention_modes_are_reported(ctx, oracle, mode):
    """The non-reproducible attention modes on the full-size random-init model, against the f64
    oracle: a record, not a parity claim.  Random ternary weights with an int8 re-quantiser
    after every block amplify an attention difference of 1e-6 into logit noise of the order of
    the logit spread, so these modes flip most greedy tokens of THIS model (measured: FAST
    43/64, PRECISE 31/64; logit deviation 1.5 to 2.5 standard deviations) while the EXACT mode
    above flips none.  What is asserted is only that the run is sane (finite logits of the
    oracle's scale); the counts are printed for the results table."""
    from oracle.oracle import BitNetOracle
    shape = BitNetShape.bitnet_2b(max_seq=128)
    w = random_bitnet_weights(shape, seed=4)
    prompt = np.random.default_rng(3).integers(0, shape.vocab, (1, 4)).astype(np.int32)
    ctx.set_attn_mode(ctx.ATTN_FAST if mode == "FAST" else ctx.ATTN_PRECISE)
    model = BitNetModel(ctx, shape, w, batch=1, max_new_tokens=70)
    o = BitNetOracle(shape, w)
    toks, devs, flips, beyond = list(prompt[0]), [], 0, 0
    for t in range(prompt.shape[1] + 64):
        cur = np.array([toks[t]], np.int32)
        g_tok, g_logits = model.step(torch.from_numpy(cur).cuda(), want_logits=True)
        o_tok, o_logits = o.step(int(cur[0]))
        sd = float(np.std(o_logits))
        assert np.isfinite(g_logits).all()
        assert 0.5 * sd < float(np.std(g_logits[0])) < 2.0 * sd
        devs.append(float(np.max(np.abs(g_logits[0] - o_logits))) / sd)
        if t >= prompt.shape[1] - 1:
            if t + 1 >= len(toks):
                toks.append(o_tok)
            if int(g_tok[0]) != o_tok:
                flips += 1
                top2 = np.partition(o_logits, -2)[-2:]
                beyond += int((top2[1] - top2[0]) > MARGIN * sd)
    o.close()
    model.close()
    print(f"BITNET_FULL_SIZE_{mode} flips={flips}/64 beyond_margin={beyond} "
          f"max_logit_dev_over_sd={max(devs):.3f}")
