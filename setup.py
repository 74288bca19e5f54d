"""Build and install flex_block_attn_b200 for NVIDIA B200 (sm_100a) only.

Takes the place of the reference's setup.py (reference setup.py:29-45 picks ``-arch=sm_90a`` and
the ThunderKittens include paths, :60-69 declares one CUDAExtension).  Here there is one target and
no third-party headers: ``flex_block_attn_b200/build.py`` compiles every ``csrc/*.cu`` with the
single ``-gencode arch=compute_100a,code=sm_100a`` and links ``libfba_b200.so``, a plain C-ABI
library that the package binds with ctypes (no torch extension, no pybind).  ``pip install .`` (or
``python setup.py build_py``) runs that build first and ships the library inside the package.
"""
import importlib.util
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


def _build_library():
    spec = importlib.util.spec_from_file_location("_fba_build", ROOT / "flex_block_attn_b200" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build_library()


class BuildPyWithNvcc(build_py):
    def run(self):
        lib = _build_library()
        self.announce(f"built {lib} for sm_100a", level=2)
        super().run()


setup(
    name="flex_block_attn_b200",
    version="0.2.0",
    description="Block-sparse attention (flex_block_attn_func) for NVIDIA B200, sm_100a only",
    packages=["flex_block_attn_b200"],
    package_data={"flex_block_attn_b200": ["libfba_b200.so", "csrc/*.cu", "csrc/*.cuh"]},
    data_files=[("include", ["include/fba.h"])],
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_py": BuildPyWithNvcc},
    zip_safe=False,
)
