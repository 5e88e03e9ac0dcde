"""keys_values_b200: long-context KV-cache inference and fine-tuning for NVIDIA B200."""
__version__ = "0.1.0"
