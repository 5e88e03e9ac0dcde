from keys_values_b200.kvcache.quantize.quantization import Quantizer, QuantizerState
from keys_values_b200.kvcache.quantize.pytorch import TorchBasicQuantizer, TorchBasicQuantizerState
from keys_values_b200.kvcache.quantize.bitsandbytes import BitsAndBytesQuantizer

__all__ = ["Quantizer", "QuantizerState", "TorchBasicQuantizer", "TorchBasicQuantizerState", "BitsAndBytesQuantizer"]
