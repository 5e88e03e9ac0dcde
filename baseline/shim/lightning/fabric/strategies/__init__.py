class DDPStrategy:
    def __init__(self, *args, **kwargs) -> None:
        self.kwargs = kwargs


class FSDPStrategy(DDPStrategy):
    pass
