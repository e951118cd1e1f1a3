from .batch import StepBatch  # noqa: F401
from .engine import Engine  # noqa: F401
