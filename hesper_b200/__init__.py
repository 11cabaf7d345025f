"""hesper_b200 -- B200-native (sm_100a) quantized-inference hot path of Verilean/hesper.

The product is the CUDA library ``libhesper_b200.so`` behind the C ABI in
``include/hesper_b200.h``.  This package is the thin host-side mirror of the
operator surface the reference's Lean layers expose (BitLinear, LinearLayer,
flash-attention decode); it only marshals device pointers into that ABI.
"""
from ._lib import HesperB200Error, load, LIB_PATH, FMT_Q4_K, FMT_Q8_0, FMT_I2_S  # noqa: F401
from .layers import (  # noqa: F401
    Context, BitLinear, LinearLayer, QuantFormat,
    execute_flash_attention_v11, flash_attention_workspace, flash_attention_prefill,
)

from .models import BitNetModel, BitNetShape, random_bitnet_weights  # noqa: F401
from .tp import GemmaModel, GemmaShape, TensorParallel  # noqa: F401

__version__ = "0.1.0"
