"""Imports every module that registers a CUDA library, so that `build.LIBRARIES`
lists all of them (used by the build check; at run time a library is built when a
model first needs it)."""
from . import build  # noqa: F401
from . import gemm_bf16  # noqa: F401
from . import attention_bf16  # noqa: F401
