"""Test-case tables taken from the reference's own test files."""

# Tests/BitLinearEquivalence.lean:208-235 -- (name, inDim, outDim, numRows, seed)
BITLINEAR_CASES = [
    ("tiny-M1", 128, 16, 1, 0xDEADBEEF),
    ("tiny-M1-seed2", 128, 16, 1, 0x1337C0DE),
    ("tiny-M1-seed3", 256, 8, 1, 0xBADF00D),
    ("mid-M1", 512, 64, 1, 0xCAFEBABE),
    ("mid-M1-seed2", 512, 64, 1, 0xFEEDFACE),
    ("wide-M1", 1024, 128, 1, 0xABCDEF01),
    ("M2-tiny", 128, 16, 2, 0x11111111),
    ("M8-tiny", 128, 16, 8, 0x22222222),
    ("M8-wider", 256, 32, 8, 0x33333333),
    ("big-M1", 2560, 320, 1, 0x44444444),
    ("M16-tiny", 128, 16, 16, 0x55555555),
    ("M16-wider", 256, 32, 16, 0x66666666),
    ("M16-bignish", 1024, 128, 16, 0x77777777),
    ("M32-mid", 512, 64, 32, 0x88888888),
    ("M16-layer-like", 2560, 320, 16, 0x99999999),
    ("M17-pad", 1024, 128, 17, 0xAAAAAAAA),
    ("M26-prefill", 2560, 320, 26, 0xBBBBBBBB),
    ("M31-near-tile", 512, 64, 31, 0xCCCCCCCC),
]

# Tests/CUDA/CUDAFlashAttnGoldenTest.lean:189-198,225,250,279
# (numHeads, numKVHeads, headDim, maxSeqLen, cacheLen, seed, window)
FLASH_ATTN_CASES = [
    (2, 1, 32, 8, 4, 42, 0),
    (20, 4, 128, 32, 8, 123, 0),
    (4, 2, 64, 16, 8, 777, 4),
]

# Tests/FlashAttentionTest.lean:24-49 and Hesper/WGSL/FlashAttention.lean:95-98
LITERAL_ATTN = {
    "q": [[1.0, 0.5, -0.3, 0.8], [-0.2, 0.7, 0.4, -0.6]],
    "k": [[[0.5, 1.0, 0.2, -0.5], [-0.3, 0.8, 1.0, 0.1], [0.7, -0.2, 0.5, 0.9]],
          [[0.3, 0.6, -0.4, 0.2], [0.8, -0.1, 0.7, -0.3], [-0.5, 0.4, 0.3, 0.6]]],
    "v": [[[1.0, 0.0, 0.5, -0.3], [0.2, 1.0, -0.5, 0.8], [-0.1, 0.5, 1.0, 0.2]],
          [[0.4, -0.2, 0.8, 0.1], [-0.3, 0.6, 0.2, 0.9], [0.7, 0.1, -0.4, 0.5]]],
}
