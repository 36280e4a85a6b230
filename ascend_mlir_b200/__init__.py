"""afir-b200: B200-native device backend for the Ascend-MLIR (AFIR) compiler stack.

The compute lives in libAFIRRuntimeCAPI.so (hand-written sm_100a CUDA kernels behind the afirt_*
C-ABI); this package is the thin Python mirror of the reference's python/runtime interface plus the
launch-descriptor builders.  There is no CPU fallback: without the built library every call raises.
"""
from .runtime import (  # noqa: F401
    AscendRuntime,
    BishengCompiler,
    CompilerError,
    CudaRuntime,
    DescriptorCompiler,
    ExecutorError,
    KernelExecutor,
    TilingSchema,
    compile_kernel,
    execute_kernel,
    find_afirt_capi_lib,
)

__version__ = "0.1"
