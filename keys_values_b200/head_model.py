from keys_values_b200.models.head_model import *  # noqa: F401,F403
