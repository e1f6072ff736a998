"""In-tree build of the native module ``symm_mem_recipes_b200/_C*.so``.

``python -m symm_mem_recipes_b200._build`` writes a ninja file under
``build/`` and runs it: every ``.cu`` is compiled by nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``; tcgen05 / TMEM need the ``a``
feature target), every ``.cpp`` by g++, and the objects are linked against the
installed torch.  The result sits next to the Python sources so that it is
found without installation.  nvcc cross-compiles: no GPU is needed to build.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = ROOT / "build" / "smr"
MODULE_NAME = "_C"

# --use_fast_math: flush-to-zero and the approximate exp / rsqrt / division in the glue kernels (RMSNorm,
# RoPE, SiLU, attention softmax).  Their GPU tests compare with the IEEE fp32 CPU oracles within a bf16
# ulp of the output, which the approximations stay well inside; the GEMM, GEMV and all-reduce kernels do
# no fp32 arithmetic that the flag changes (tensor-core MMAs and packed bf16 adds).
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]


def _cuda_home() -> Path:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return Path(cand)
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def sources() -> tuple[list[Path], list[Path]]:
    cu = sorted(CSRC.rglob("*.cu"))
    cpp = sorted(CSRC.rglob("*.cpp"))
    return cu, cpp


def so_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG_DIR / f"{MODULE_NAME}{suffix}"


def write_ninja() -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    cuda = _cuda_home()
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    inc = [f"-I{p}" for p in ce.include_paths()]
    inc += [f"-I{sysconfig.get_paths()['include']}", f"-I{cuda / 'include'}", f"-I{CSRC}"]
    torch_lib = Path(torch.__file__).parent / "lib"
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DTORCH_EXTENSION_NAME={MODULE_NAME}",
            "-DTORCH_API_INCLUDE_EXTENSION_H"]
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    cu, cpp = sources()
    lines = [
        "ninja_required_version = 1.3",
        f"nvcc = {cuda / 'bin' / 'nvcc'}",
        "cxx = g++",
        f"nvcc_flags = {' '.join(NVCC_FLAGS)} -I{CSRC} -D_GLIBCXX_USE_CXX11_ABI={abi}",
        f"cxx_flags = {' '.join(CXX_FLAGS + defs + inc)}",
        f"ld_flags = -shared -L{torch_lib} -Wl,-rpath,{torch_lib} -lc10 -lc10_cuda -ltorch_cpu "
        f"-ltorch_cuda -ltorch -ltorch_python -L{cuda / 'lib64'} -lcudart_static -lrt -lpthread -ldl",
        "",
        "rule nvcc",
        "  command = $nvcc $nvcc_flags -MD -MF $out.d -c $in -o $out > $out.log 2>&1 || (cat $out.log; exit 1)",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = NVCC $in",
        "rule cxx",
        "  command = $cxx $cxx_flags -MMD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = CXX $in",
        "rule link",
        "  command = $cxx $in $ld_flags -o $out",
        "  description = LINK $out",
        "",
    ]
    objs = []
    for src in cu:
        obj = BUILD_DIR / (src.relative_to(CSRC).as_posix().replace("/", "_") + ".o")
        lines.append(f"build {obj}: nvcc {src}")
        objs.append(str(obj))
    for src in cpp:
        obj = BUILD_DIR / (src.relative_to(CSRC).as_posix().replace("/", "_") + ".o")
        lines.append(f"build {obj}: cxx {src}")
        objs.append(str(obj))
    lines.append(f"build {so_path()}: link {' '.join(objs)}")
    lines.append(f"default {so_path()}")
    path = BUILD_DIR / "build.ninja"
    path.write_text("\n".join(lines) + "\n")
    return path


def build(verbose: bool = False) -> Path:
    """Compile (incrementally) and return the path of the shared object."""
    ninja_file = write_ninja()
    cmd = ["ninja", "-f", str(ninja_file)]
    if verbose:
        cmd.append("-v")
    proc = subprocess.run(cmd, cwd=str(BUILD_DIR), capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("native build failed")
    if verbose:
        sys.stdout.write(proc.stdout)
    return so_path()


def ptxas_report() -> str:
    """Registers / spills / shared memory of every kernel, from the build logs."""
    out = []
    for log in sorted(BUILD_DIR.glob("*.o.log")):
        out.append(f"== {log.name}")
        out.append(log.read_text())
    return "\n".join(out)


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv)
    print(p)
