"""Library discovery and error types (counterpart of the reference's python/runtime/utils.py)."""
import logging
import os
from pathlib import Path

logger = logging.getLogger("afir_b200.runtime")

SM_100A = "sm_100a"


class ExecutorError(RuntimeError):
    pass


class MemoryAllocationError(ExecutorError):
    pass


class KernelLaunchError(ExecutorError):
    pass


class InvalidBinaryError(ExecutorError):
    pass


class CompilerError(RuntimeError):
    pass


class BinaryNotFoundError(CompilerError):
    pass


def find_afirt_capi_lib() -> Path:
    """Locate libAFIRRuntimeCAPI.so.

    Order (as in the reference, python/runtime/utils.py:60-90): the AFIRT_CAPI_LIB environment
    variable, then the in-tree build output.  Raises ImportError when absent: nothing falls back
    to a CPU implementation.
    """
    env = os.environ.get("AFIRT_CAPI_LIB")
    if env:
        p = Path(env)
        if p.exists():
            return p
        raise ImportError(f"AFIRT_CAPI_LIB set but file not found: {env}")
    pkg = Path(__file__).resolve().parent.parent
    for candidate in (pkg / "lib" / "libAFIRRuntimeCAPI.so", pkg.parent / "build" / "lib" / "libAFIRRuntimeCAPI.so"):
        if candidate.exists():
            return candidate
    raise ImportError(
        "Cannot find libAFIRRuntimeCAPI.so. Build it first (python -m ascend_mlir_b200.build), "
        "or set the AFIRT_CAPI_LIB environment variable."
    )


def read_binary(path) -> bytes:
    return Path(path).read_bytes()
