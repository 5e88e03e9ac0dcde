from keys_values_b200.models.adapter_v2 import *  # noqa: F401,F403
