class BitsandbytesPrecision:
    def __init__(self, *args, **kwargs) -> None:
        raise NotImplementedError("bitsandbytes precision is not provided by the stand-in package")
