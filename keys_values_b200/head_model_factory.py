from keys_values_b200.models.head_model import HeadModelFactory  # noqa: F401
