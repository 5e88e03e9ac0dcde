"""Stand-in for ``jsonargparse``: the reference's CLI entry is not driven by the benchmark arm."""


def auto_cli(*args, **kwargs):
    raise NotImplementedError("jsonargparse.auto_cli is not provided by the stand-in package")


def set_config_read_mode(*args, **kwargs) -> None:
    pass


def set_docstring_parse_options(*args, **kwargs) -> None:
    pass
