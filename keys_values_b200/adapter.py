from keys_values_b200.models.adapter import *  # noqa: F401,F403
