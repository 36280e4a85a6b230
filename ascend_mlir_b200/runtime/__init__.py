"""Python side of the afirt_* C-ABI (mirrors the reference's python/runtime package)."""
from .utils import (  # noqa: F401
    BinaryNotFoundError,
    CompilerError,
    ExecutorError,
    InvalidBinaryError,
    KernelLaunchError,
    MemoryAllocationError,
    find_afirt_capi_lib,
    read_binary,
)
from .tiling_schema import TilingSchema  # noqa: F401
from .compiler import BishengCompiler, DescriptorCompiler, compile_kernel  # noqa: F401
from .executor import (  # noqa: F401
    MAGIC_ELF_AICUBE,
    MAGIC_ELF_AIVEC,
    AscendRuntime,
    CudaRuntime,
    KernelExecutor,
    execute_kernel,
)
