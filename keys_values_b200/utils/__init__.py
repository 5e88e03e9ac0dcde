"""Shared helpers (``keys_values/utils.py:37-376``)."""
from keys_values_b200.utils.misc import *  # noqa: F401,F403
