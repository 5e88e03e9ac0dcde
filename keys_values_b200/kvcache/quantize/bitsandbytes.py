"""Optional bitsandbytes block-wise quantizer (``bnb-quantized{4,8}``).

Parity: ``keys_values/kvcache/quantize/bitsandbytes.py:47-550``. The package is an
optional, GPU-only dependency; where it is missing the constructor raises and
the ``torch-quantized*`` buffers are the supported choice.
"""
from __future__ import annotations

from keys_values_b200.kvcache.quantize.quantization import Quantizer


def bitsandbytes_available() -> bool:
    try:
        import bitsandbytes  # noqa: F401

        return True
    except Exception:
        return False


class BitsAndBytesQuantizer(Quantizer):
    def __init__(self, *args, **kwargs):
        if not bitsandbytes_available():
            raise ImportError(
                "bitsandbytes is not installed: use the 'torch-quantized4' / 'torch-quantized8' buffers instead"
            )
        raise NotImplementedError("bnb-quantized buffers: bitsandbytes has no sm_100a build in this environment")
