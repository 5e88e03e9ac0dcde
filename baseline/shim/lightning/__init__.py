"""Stand-in for the ``lightning`` package: a minimal ``Fabric`` over ``torch.distributed``."""
from lightning.fabric import Fabric, seed_everything  # noqa: F401

__all__ = ["Fabric", "seed_everything"]
