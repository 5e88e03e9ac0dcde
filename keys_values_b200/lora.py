from keys_values_b200.models.lora import *  # noqa: F401,F403
