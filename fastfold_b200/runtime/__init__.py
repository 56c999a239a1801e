from .trainer import FlatAdamTrainer

__all__ = ["FlatAdamTrainer"]
