"""Build the native library ``soap_tp_b200/_C*.so`` in-tree with nvcc for sm_100a.

    python -m soap_tp_b200.build_ext            # incremental (skips if sources are older than the .so)
    python -m soap_tp_b200.build_ext --force

The library is a plain pybind11 module (no ATen): ``.cu`` files are compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into one shared object next
to this file, so a source checkout plus this command is all a GPU box needs.  nvcc cross-compiles
without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "csrc" / "build"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def target_path() -> Path:
    return HERE / ("_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _includes() -> list[str]:
    import pybind11

    return [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else "nvcc"


def needs_build() -> bool:
    target = target_path()
    if not target.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(sources()) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")))
    return newest > target.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    target = target_path()
    if not force and not needs_build():
        return target
    BUILD.mkdir(parents=True, exist_ok=True)
    common = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr", *ARCH_FLAGS, *_includes()]
    if os.environ.get("SOAP_GEMM_BK"):
        common += [f"-DSOAP_GEMM_BK={int(os.environ['SOAP_GEMM_BK'])}"]
    if os.environ.get("SOAP_GEMM_TERMS"):
        common += [f"-DSOAP_GEMM_TERMS={int(os.environ['SOAP_GEMM_TERMS'])}"]     # timing experiments (see gemm_tf32x3.cu)
    if os.environ.get("SOAP_QR_TRACE", "0") == "1":
        common += ["-DSOAP_QR_TRACE"]     # clock64 stamps in the one-column QR panel kernel (kernel_cases --trace)
    if verbose:
        common += ["-Xptxas", "-v"]

    def compile_one(src: Path) -> Path:
        obj = BUILD / (src.stem + ".o")
        cmd = [_nvcc(), *common, "-x", "cu" if src.suffix == ".cu" else "c++", "-c", str(src), "-o", str(obj)]
        if src.suffix == ".cpp":
            cmd = [_nvcc(), *common, "-c", str(src), "-o", str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{result.stdout}\n{result.stderr}")
        if verbose and result.stderr:
            print(result.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, sources()))
    link = [_nvcc(), "-shared", *ARCH_FLAGS, "-o", str(target), *map(str, objects), "-lcudart"]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    return target


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
