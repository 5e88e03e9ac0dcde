from keys_values_b200.models.lora import LoRALinear, LoRAQKVLinear  # noqa: F401
