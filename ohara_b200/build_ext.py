"""Builds the sm_100a extension in-tree (``ohara_b200/_C*.so``).

nvcc cross-compiles without a GPU, so this also runs on CPU-only build hosts. The shared object is
git-ignored; ``python -m ohara_b200.build_ext`` (re)builds it. Object files are cached under
``ohara_b200/csrc/build`` and rebuilt only when a source or header is newer.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
OBJ_DIR = SRC_DIR / "build"
EXT_NAME = "_C"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-diag-suppress",
    "20044",
]


def ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG_DIR / f"{EXT_NAME}{suffix}"


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    if candidate.exists():
        return str(candidate)
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found; cannot build the ohara_b200 CUDA extension")
    return found


def _torch_flags() -> tuple[list[str], list[str]]:
    import torch
    from torch.utils import cpp_extension

    includes = [f"-I{p}" for p in cpp_extension.include_paths("cuda")]
    includes.append(f"-I{sysconfig.get_paths()['include']}")
    lib_dir = Path(torch.__file__).parent / "lib"
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    libs = [
        f"-L{lib_dir}",
        f"-Wl,-rpath,{lib_dir}",
        "-lc10",
        "-lc10_cuda",
        "-ltorch_cpu",
        "-ltorch_cuda",
        "-ltorch",
        "-ltorch_python",
        f"-L{cuda_home}/lib64",
        "-lcudart",
    ]
    defines = [
        f"-DTORCH_EXTENSION_NAME={EXT_NAME}",
        "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
    ]
    return includes + defines, libs


def _newest_header_mtime() -> float:
    headers = list(SRC_DIR.glob("*.h")) + list(SRC_DIR.glob("*.cuh"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` / ``*.cpp`` for sm_100a and link ``_C``. Returns the .so path."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    torch_cflags, torch_libs = _torch_flags()
    header_mtime = _newest_header_mtime()
    sources = sorted(SRC_DIR.glob("*.cu")) + sorted(SRC_DIR.glob("*.cpp"))
    jobs: list[tuple[Path, Path, list[str]]] = []
    objects: list[Path] = []
    for src in sources:
        obj = OBJ_DIR / (src.name + ".o")
        objects.append(obj)
        stale = (
            force
            or not obj.exists()
            or obj.stat().st_mtime < max(src.stat().st_mtime, header_mtime)
        )
        if not stale:
            continue
        if src.suffix == ".cu":
            cmd = [nvcc, *NVCC_FLAGS, f"-I{SRC_DIR}", "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
        else:
            cxx = os.environ.get("CXX", "g++")
            cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
            cmd = [
                cxx,
                "-O3",
                "-std=c++17",
                "-fPIC",
                f"-I{SRC_DIR}",
                f"-I{cuda_home}/include",
                *torch_cflags,
                "-c",
                str(src),
                "-o",
                str(obj),
            ]
        jobs.append((src, obj, cmd))

    def run(job):
        src, _, cmd = job
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"compiling {src.name} failed:\n{proc.stdout}\n{proc.stderr}")
        if verbose and (proc.stdout or proc.stderr):
            print(proc.stdout + proc.stderr)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(run, jobs))

    target = ext_path()
    relink = bool(jobs) or not target.exists()
    if relink:
        cxx = os.environ.get("CXX", "g++")
        cmd = [cxx, "-shared", "-o", str(target), *[str(o) for o in objects], *torch_libs]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"linking {target.name} failed:\n{proc.stdout}\n{proc.stderr}")
    return target


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(path)
