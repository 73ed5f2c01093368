"""Build and install llumnix_kv_b200.

The native extension is compiled by ``llumnix_kv_b200/_build.py`` (nvcc for sm_100a + g++, no
torch headers needed) and placed inside the package directory, so ``pip install -e .`` and a
plain in-tree ``python setup.py build_ext --inplace`` give the same result as
``python -c "import __graft_entry__ as g; g.build()"``.
"""
import importlib.util
import os

from setuptools import Extension, find_packages, setup
from setuptools.command.build_ext import build_ext

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_builder():
    spec = importlib.util.spec_from_file_location("_kvx_build", os.path.join(HERE, "llumnix_kv_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildNative(build_ext):
    def run(self):
        target = _load_builder().build(verbose=bool(os.environ.get("KVX_BUILD_VERBOSE")))
        if not self.inplace:
            dst = os.path.join(self.build_lib, "llumnix_kv_b200", os.path.basename(str(target)))
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            self.copy_file(str(target), dst)


setup(
    name="llumnix_kv_b200",
    version="0.1.0",
    description="B200-native KV-cache transfer and storage framework",
    packages=find_packages(include=["llumnix_kv_b200", "llumnix_kv_b200.*"]),
    ext_modules=[Extension("llumnix_kv_b200.kvtransfer_ops", sources=[])],
    cmdclass={"build_ext": BuildNative},
    python_requires=">=3.10",
    install_requires=["torch", "msgspec", "numpy"],
)
