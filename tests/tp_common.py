"""Shared pieces of the tensor-parallel tests: a small Gemma-shaped model that satisfies every
sharding constraint at TP 1 and 2 (local attention width and FFN slice multiples of 256)."""
from hesper_b200.tp import GemmaShape

SMALL_GEMMA = GemmaShape(n_layers=3, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024,
                         vocab=1024, max_seq=64, window=16, global_every=3, rope_base=10000.0,
                         rms_eps=1e-6, attn_scale=1.0 / 128 ** 0.5, embed_scale=512 ** 0.5)
