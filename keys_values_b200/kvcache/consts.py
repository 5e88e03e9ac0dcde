"""Names of the supported buffer kinds (``keys_values/kvcache/consts.py:21-34``)."""
from typing import Tuple

SUPPORTED_QUANTIZERS = ("default", "torch-quantized4", "torch-quantized8", "bnb-quantized4", "bnb-quantized8")


def split_name(name: str) -> Tuple[str, str]:
    """``"h2o-torch-quantized8"`` → ``("h2o", "torch-quantized8")``."""
    for qname in SUPPORTED_QUANTIZERS:
        if name.endswith("-" + qname):
            return name[: -(len(qname) + 1)], qname
    raise ValueError(f"name = {name}: postfix must be one of {SUPPORTED_QUANTIZERS}")
