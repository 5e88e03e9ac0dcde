from keys_values_b200.models.lora import DoRALinear, DoRAQKVLinear, dora_forward, dora_merge, row_lengths  # noqa: F401
