from lightning.pytorch.loggers import CSVLogger  # noqa: F401
