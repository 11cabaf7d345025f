"""GPU: a context's scratch serves one stream at a time, and the library enforces it.

The batched products stage their activations in the context's scratch; two calls issued back
to back on two different streams would otherwise overlap on the device and the second staging
kernel would overwrite what the first product still reads.  The library orders a call behind
the previous scratch user with an event when the stream changes: results must be bit-identical
to the same calls on one stream."""
import numpy as np
import pytest
import torch

from hesper_b200 import LinearLayer, BitLinear, formats

pytestmark = pytest.mark.gpu


def test_batched_calls_on_two_streams_do_not_share_scratch_in_time(ctx):
    rng = np.random.default_rng(9)
    K, N, M = 2560, 4096, 64
    blocks = formats.random_kquant(rng, 12, N, K)
    layer = LinearLayer.create_from_bytes(ctx, blocks, 12, K, N)
    packed = formats.i2s_pack(formats.random_ternary(rng, N, K))
    bl = BitLinear.create_from_bytes(ctx, packed, 0.05, K, N)
    xs = [torch.randn(M, K, device="cuda") for _ in range(6)]
    torch.cuda.synchronize()
    ref_q = [layer.forward(x).clone() for x in xs]
    ref_t = [bl.forward(x).clone() for x in xs]
    torch.cuda.synchronize()
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(5):
        outs_q, outs_t = [], []
        for i, x in enumerate(xs):
            st = sa if i % 2 == 0 else sb
            outs_q.append(layer.forward(x, stream=st))
            outs_t.append(bl.forward(x, stream=sb if i % 2 == 0 else sa))
        sa.synchronize()
        sb.synchronize()
        for i in range(len(xs)):
            assert torch.equal(outs_q[i], ref_q[i]), f"Q4_K call {i}"
            assert torch.equal(outs_t[i], ref_t[i]), f"ternary call {i}"
    ctx.check()
