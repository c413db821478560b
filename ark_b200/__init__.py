"""ark_b200 — B200-native execution engine for ARK models and plan files.

The Python surface mirrors the reference front end (python/ark/__init__.py):
build a model with the functional ops, plan it, run it through `Runtime` or
`Executor`. Execution happens in libark_b200.so (sm_100a loop kernel).
"""
from .data_type import DataType, fp32, fp16, bf16, int32, uint32, int8, uint8, byte  # noqa: F401
from .error import (BaseError, InternalError, InvalidUsageError, ModelError, PlanError, UnsupportedError,  # noqa: F401
                    SystemError, GpuError)
from .model import Model, Tensor  # noqa: F401
from .ops import *  # noqa: F401,F403
from .planner import Plan, Planner, PlannerContext  # noqa: F401
from .executor import Executor, device_info, plan_check, plan_dump, version  # noqa: F401
from .runtime import Runtime  # noqa: F401


def init():
    """Resets the global model and runtime (python/ark/init.py)."""
    rt = runtime._RuntimeState.runtime
    if rt is not None:
        rt.reset()
    Model.reset()


def set_rank(rank):
    Model.set_rank(rank)


def set_world_size(world_size):
    Model.set_world_size(world_size)
