from keys_values_b200.models.model import *  # noqa: F401,F403
