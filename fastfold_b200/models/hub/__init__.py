from .alphafold import AlphaFold

__all__ = ["AlphaFold"]
try:
    from .loss import AlphaFoldLoss  # noqa: F401
    from .lr_scheduler import AlphaFoldLRScheduler  # noqa: F401
    __all__ += ["AlphaFoldLoss", "AlphaFoldLRScheduler"]
except ImportError:  # pragma: no cover
    pass
