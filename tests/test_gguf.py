"""CPU: GGUF ingestion of the three weight formats (round trip through a file written in the
layout the reference's loader reads: Hesper/GGUF/Loader.lean:369-405, Types.lean:86-132)."""
import numpy as np
import pytest

from hesper_b200 import formats, gguf


def test_roundtrip_i2s_q4k_q80(tmp_path, oracle):
    rng = np.random.default_rng(0)
    K, N = 256, 12
    tern = formats.random_ternary(rng, N, K)
    packed = formats.i2s_pack(tern)
    q4 = formats.random_q4k(rng, N, K)
    q8 = formats.random_q80(rng, N, K)
    norm = rng.standard_normal(K).astype(np.float32)
    path = str(tmp_path / "m.gguf")
    gguf.write_gguf(path, {"general.architecture": "bitnet", "bitnet.block_count": 1},
                    [("blk.0.attn_q.weight", (K, N), gguf.T_I2_S, gguf.i2s_payload(packed, 0.0625)),
                     ("blk.0.ffn_up.weight", (K, N), gguf.T_Q4_K, q4.tobytes()),
                     ("blk.0.ffn_down.weight", (K, N), gguf.T_Q8_0, q8.tobytes()),
                     ("blk.0.attn_norm.weight", (K,), gguf.T_F32, norm.tobytes())])
    g = gguf.GGUFFile(path)
    assert g.metadata["general.architecture"] == "bitnet" and g.metadata["bitnet.block_count"] == 1
    p, scale, numel = g.get_i2s("blk.0.attn_q.weight")
    assert numel == N * K and scale == 0.0625 and np.array_equal(p, packed)
    assert np.array_equal(formats.i2s_unpack(p, K, N), tern)
    assert np.array_equal(g.get_blocks("blk.0.ffn_up.weight", gguf.T_Q4_K), q4)
    assert np.array_equal(g.get_blocks("blk.0.ffn_down.weight", gguf.T_Q8_0), q8)
    assert np.array_equal(g.get_f32("blk.0.attn_norm.weight"), norm)
    # the bytes feed the oracle unchanged
    x = rng.standard_normal((1, K)).astype(np.float32)
    y, acc, _ = oracle.bitlinear_forward(p, scale, K, N, x)
    q, _ = oracle.quant_act_i8(x[0])
    assert np.array_equal(acc[0], tern.astype(np.int32) @ q.astype(np.int32))
    with pytest.raises(ValueError):
        g.get_i2s("blk.0.ffn_up.weight")
    with pytest.raises(ValueError):
        g.get_blocks("blk.0.ffn_up.weight", gguf.T_Q8_0)
    g.close()


def test_bad_magic(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(ValueError, match="Invalid GGUF magic"):
        gguf.GGUFFile(str(p))


def _tiny_shape():
    from hesper_b200.models import BitNetShape
    return BitNetShape(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=384,
                       vocab=512, max_seq=64)


def test_bitnet_checkpoint_roundtrip(tmp_path):
    """A whole BitNet-shaped checkpoint under the reference's tensor names
    (Hesper/Models/BitNet.lean:788-941) comes back byte for byte, dimensions from metadata."""
    from hesper_b200.models import random_bitnet_weights
    shape = _tiny_shape()
    w = random_bitnet_weights(shape, seed=5)
    path = str(tmp_path / "tiny.gguf")
    gguf.save_bitnet_gguf(path, shape, w)
    shape2, w2 = gguf.load_bitnet_gguf(path)
    for f in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "max_seq"):
        assert getattr(shape2, f) == getattr(shape, f)
    assert shape2.rope_base == shape.rope_base
    assert np.float32(shape2.rms_eps) == np.float32(shape.rms_eps)
    assert np.array_equal(w2["embed"], w["embed"]) and w2["embed_dtype"] == 0
    assert np.array_equal(w2["final_norm"], w["final_norm"])
    for L, L2 in zip(w["layers"], w2["layers"]):
        for k in L:
            assert np.array_equal(np.asarray(L2[k]), np.asarray(L[k])), k
    assert set(w2["_file"].tensors) >= {"token_embd.weight", "output_norm.weight",
                                        "blk.1.attn_output.weight", "blk.0.ffn_sub_norm.weight"}


@pytest.mark.gpu
def test_bitnet_checkpoint_decodes_like_the_arrays_it_was_written_from(tmp_path, ctx):
    from hesper_b200 import BitNetModel
    from hesper_b200.models import random_bitnet_weights
    shape = _tiny_shape()
    w = random_bitnet_weights(shape, seed=6)
    path = str(tmp_path / "tiny.gguf")
    gguf.save_bitnet_gguf(path, shape, w)
    shape2, w2 = gguf.load_bitnet_gguf(path)
    prompt = np.random.default_rng(1).integers(0, shape.vocab, (2, 5)).astype(np.int32)
    outs = []
    for s_, w_ in ((shape, w), (shape2, w2)):
        m = BitNetModel(ctx, s_, w_, batch=2, max_new_tokens=12)
        toks, _, _ = m.generate(prompt, 12, use_graph=False)
        outs.append(np.array(toks))
        m.close()
    ctx.check()
    assert np.array_equal(outs[0], outs[1])
