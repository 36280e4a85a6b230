"""Kernel "compiler" front (counterpart of the reference's python/runtime/compiler.py).

The reference shells out to bisheng to turn generated AscendC C++ into an ELF; here the source is
the launch descriptor emitted by the translate step and compiling means validating it against the
prebuilt sm_100a kernel library and sealing it into the .bin container the executor takes.
"""
import ctypes
from pathlib import Path

from ._capi import get_lib
from .utils import SM_100A, BinaryNotFoundError, CompilerError, logger


class DescriptorCompiler:
    ARCH_SM100A = "sm_100a"
    # accepted for callers written against the reference
    ARCH_VEC = "dav-c220-vec"
    ARCH_CUBE = "dav-c220-cube"

    def __init__(self, ascend_root=None, soc_version: str = SM_100A):
        self.ascend_root = ascend_root  # unused: kept for signature compatibility
        self.soc_version = soc_version

    def compile_and_link(self, src_file, output_dir, kernel_name: str, arch: str = ARCH_SM100A,
                         opt_level: int = 3, verbose: bool = False) -> Path:
        src_file = Path(src_file)
        output_dir = Path(output_dir)
        output_dir.mkdir(parents=True, exist_ok=True)
        lib = get_lib()
        handle = lib.afirt_compiler_create(self.soc_version.encode(), arch.encode(), opt_level)
        if not handle:
            raise CompilerError("Failed to create compiler instance")
        try:
            buf = ctypes.create_string_buffer(4096)
            ret = lib.afirt_compiler_compile(ctypes.c_void_p(handle), str(src_file.resolve()).encode(),
                                             str(output_dir.resolve()).encode(), kernel_name.encode(), buf,
                                             ctypes.c_size_t(len(buf)))
            if ret != 0:
                raise CompilerError(buf.value.decode(errors="replace"))
            bin_path = Path(buf.value.decode())
        finally:
            lib.afirt_compiler_destroy(ctypes.c_void_p(handle))
        if not bin_path.exists():
            raise BinaryNotFoundError(f"Binary file not generated: {bin_path}")
        if verbose:
            logger.info("Generated binary: %s (%d bytes)", bin_path, bin_path.stat().st_size)
        return bin_path


BishengCompiler = DescriptorCompiler  # name used by callers of the reference package


def compile_kernel(src_file, output_dir, kernel_name: str, ascend_root=None, soc_version: str = SM_100A,
                   arch: str = DescriptorCompiler.ARCH_SM100A, opt_level: int = 3, verbose: bool = False) -> Path:
    return DescriptorCompiler(ascend_root, soc_version).compile_and_link(
        src_file=src_file, output_dir=output_dir, kernel_name=kernel_name, arch=arch, opt_level=opt_level,
        verbose=verbose)
