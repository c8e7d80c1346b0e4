from ._ffi import ARCH_LLAMA, ARCH_REFERENCE, DTYPE_BF16, DTYPE_BF16X3, DTYPE_F32, LIB_PATH  # noqa: F401
from .engine import *  # noqa: F401,F403
from .engine import Engine, EngineError, Options, State, StepResult, dp_unique_id, open, pinned_empty  # noqa: F401
