from keys_values_b200.kvcache.quantize.quantization import Quantizer, QuantizerState
from keys_values_b200.kvcache.quantize.pytorch import TorchBasicQuantizer, TorchBasicQuantizerState

__all__ = ["Quantizer", "QuantizerState", "TorchBasicQuantizer", "TorchBasicQuantizerState"]
