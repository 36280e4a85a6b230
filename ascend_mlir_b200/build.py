"""In-tree build of libAFIRRuntimeCAPI.so (CUDA kernels for sm_100a + the C++ host runtime).

Explicit nvcc / g++ commands, objects cached under ascend_mlir_b200/build/, the shared library
written to ascend_mlir_b200/lib/.  nvcc cross-compiles without a GPU.
"""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
BUILD = PKG / "build"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libAFIRRuntimeCAPI.so"

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
CXX = "g++"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", str(CSRC), "-I", str(ROOT / "include"),
]
# Bandwidth-bound kernels must round after every op: no mul+add contraction.
NO_FMA = ["-fmad=false"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra", "-I", str(CSRC),
             "-I", str(ROOT / "include"), "-I", str(CUDA_HOME / "include")]

CU_SOURCES = {
    "kernels/elementwise.cu": NO_FMA,
    "kernels/row_reduce.cu": NO_FMA,
    "kernels/gather.cu": NO_FMA,
    "kernels/transpose.cu": [],
    "kernels/transpose_tma.cu": [],
    "kernels/matmul_tcgen05.cu": [],
}
CPP_SOURCES = ["common/json.cpp", "kernels/matmul_plan.cpp", "kernels/body_match.cpp", "codegen/kernel_source.cpp",
               "codegen/nvrtc_compile.cpp", "codegen/embedded_headers.cpp", "runtime/device_module.cpp", "runtime/caller_device.cpp", "runtime/host_staging.cpp", "runtime/descriptor.cpp", "runtime/launcher.cpp", "runtime/executor.cpp",
               "support/npy_io.cpp", "support/tiling_schema.cpp", "execution/output_comparator.cpp",
               "execution/task_graph.cpp", "execution/run_manifest.cpp", "execution/artifact_compiler.cpp",
               "execution/execution_session.cpp", "execution/resource_scheduler.cpp", "execution/global_scheduler.cpp",
               "execution/profile_retention.cpp",
               "front/mlir_text.cpp", "front/group_analysis.cpp", "front/fused_generic.cpp", "front/shape_inference.cpp", "runtime/capi.cpp", "runtime/rowsum_exchange.cpp", "runtime/peer_memory.cpp"]
# command-line tools (reference: tools/runtime-session, tools/autotuner), linked with the same objects
TOOLS = {"runtime-session": "tools/runtime_session_main.cpp", "autotuner": "tools/autotuner_main.cpp",
         "afir-opt": "tools/afir_opt_main.cpp", "afir-translate": "tools/afir_translate_main.cpp"}
# the compiler front-end tools need no CUDA objects
FRONT_ONLY = {"afir-opt", "afir-translate"}
BINDIR = PKG / "bin"


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.inc")) +
                    list((ROOT / "include").rglob("*.h"))):
        h.update(p.read_bytes())
    return h.hexdigest()


def _stale(obj: Path, src: Path, stamp: str) -> bool:
    tag = obj.with_suffix(obj.suffix + ".stamp")
    want = hashlib.sha256(src.read_bytes()).hexdigest() + stamp
    if obj.exists() and tag.exists() and tag.read_text() == want:
        return False
    return True


def _mark(obj: Path, src: Path, stamp: str) -> None:
    obj.with_suffix(obj.suffix + ".stamp").write_text(hashlib.sha256(src.read_bytes()).hexdigest() + stamp)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return res.stdout + res.stderr


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    hdr = _headers_digest()
    jobs, objs = [], []
    for rel, extra in CU_SOURCES.items():
        src = CSRC / rel
        obj = BUILD / (rel.replace("/", "_") + ".o")
        objs.append(obj)
        stamp = hdr + "|".join(NVCC_FLAGS + extra)
        if force or _stale(obj, src, stamp):
            cmd = [NVCC] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", str(src), "-o", str(obj)]
            jobs.append((cmd, obj, src, stamp))
    for rel in CPP_SOURCES:
        src = CSRC / rel
        obj = BUILD / (rel.replace("/", "_") + ".o")
        objs.append(obj)
        stamp = hdr + "|".join(CXX_FLAGS)
        if force or _stale(obj, src, stamp):
            cmd = [CXX] + CXX_FLAGS + ["-c", str(src), "-o", str(obj)]
            jobs.append((cmd, obj, src, stamp))

    def work(job):
        cmd, obj, src, stamp = job
        out = _run(cmd, verbose)
        _mark(obj, src, stamp)
        return out

    logs = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            logs = list(pool.map(work, jobs))
    cuda_libs = ["-L", str(CUDA_HOME / "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    if jobs or not LIB.exists():
        link = [CXX, "-shared", "-o", str(LIB)] + [str(o) for o in objs] + cuda_libs + ["-Wl,--no-undefined", "-Wl,-z,defs"]
        _run(link, verbose)
    BINDIR.mkdir(exist_ok=True)
    lib_objs = [str(o) for o in objs if not str(o).endswith("runtime_capi.cpp.o")]
    for tool, rel in TOOLS.items():
        src = CSRC / rel
        exe = BINDIR / tool
        tobj = BUILD / (rel.replace("/", "_") + ".o")
        stamp = hdr + "|".join(CXX_FLAGS)
        if force or jobs or _stale(tobj, src, stamp) or not exe.exists():
            _run([CXX] + CXX_FLAGS + ["-c", str(src), "-o", str(tobj)], verbose)
            _mark(tobj, src, stamp)
            if tool in FRONT_ONLY:
                # parser, group analysis, descriptor, kernel generator and the NVRTC front: no CUDA objects
                front = [o for o in lib_objs if any(tag in Path(o).name for tag in (
                    "front_", "common_", "codegen_", "runtime_descriptor", "kernels_body_match", "support_tiling_schema"))]
                _run([CXX, "-o", str(exe), str(tobj)] + front + ["-ldl"], verbose)
            else:
                _run([CXX, "-o", str(exe), str(tobj)] + lib_objs + cuda_libs, verbose)
    if ptxas_info:
        print("".join(logs))
    return LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
