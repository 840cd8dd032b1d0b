"""Build and install ``soap_tp_b200`` together with its native sm_100a library.

    python setup.py build_ext --inplace      # compiles soap_tp_b200/_C*.so next to the sources
    pip install --no-build-isolation .

The reference's ``setup.py`` wires two optional pybind11 extensions against externally built SLATE
and ELPA trees (``setup.py:111-240`` there).  Here there is one extension and no external numerical
library: every ``.cu`` under ``soap_tp_b200/csrc`` is compiled by nvcc with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` (see ``soap_tp_b200/build_ext.py``; nvcc
cross-compiles without a GPU).
"""
import sys
from pathlib import Path

from setuptools import Extension, find_packages, setup
from setuptools.command.build_ext import build_ext as _build_ext

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


class NvccBuild(_build_ext):
    def run(self):  # the whole native library is one nvcc build
        from soap_tp_b200 import build_ext as native

        built = native.build(force=True)
        if not self.inplace:
            target = Path(self.build_lib) / "soap_tp_b200" / built.name
            target.parent.mkdir(parents=True, exist_ok=True)
            self.copy_file(str(built), str(target))


setup(
    name="soap_tp_b200",
    version="0.1.0",
    description="Tensor-parallel SOAP optimizer for NVIDIA B200 (sm_100a)",
    packages=find_packages(include=["soap_tp_b200", "soap_tp_b200.*"]),
    package_data={"soap_tp_b200": ["csrc/*", "bench/launch/*"]},
    ext_modules=[Extension("soap_tp_b200._C", sources=[])],
    cmdclass={"build_ext": NvccBuild},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "pybind11>=2.12", "numpy"],
)
