from .parallel_mode import ParallelMode  # noqa: F401
