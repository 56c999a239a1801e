"""Utilities: rigid maths, feature builders, chunking, checkpointing, weight import, fastnn injection."""


def inject_fastnn(model):
    """``from fastfold.utils import inject_fastnn`` (the spelling of the reference's README) works as well as the
    module path ``fastfold.utils.inject_fastnn.inject_fastnn``."""
    from .inject_fastnn import inject_fastnn as _impl
    return _impl(model)
