from keys_values_b200.models.pos_encoding import *  # noqa: F401,F403
