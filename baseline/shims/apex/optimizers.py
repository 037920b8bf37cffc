"""`apex.optimizers` without the CUDA extensions: constructors raise the error Apex raises."""


class _NeedsExtensions:
    def __init__(self, *args, **kwargs):
        raise RuntimeError(f"apex.optimizers.{type(self).__name__} requires cuda extensions")


class FusedAdam(_NeedsExtensions):
    pass


class FusedSGD(_NeedsExtensions):
    pass
