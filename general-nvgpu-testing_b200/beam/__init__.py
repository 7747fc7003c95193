"""beam — B200-native drop-in for BEAM's fp16 rc GEMM registry (reference: python/beam/__init__.py)."""
from ._C import *  # noqa: F401,F403
from ._C import device_status  # noqa: F401
from .tuner import Operator, OperatorTuner  # noqa: F401
