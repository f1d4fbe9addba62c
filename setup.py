"""Packaging for `pip install .`: builds the native extension in-tree for sm_100a and ships
the `bagua_core` (drop-in API) and `bagua_core_b200` packages.

Counterpart of the reference's installer (setup.py:34-235), which downloads NCCL and a network
plugin at install time; nothing is downloaded here — the extension links the NCCL that comes
with the installed torch.
"""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildWithNative(build_py):
    def run(self):
        sys.path.insert(0, ROOT)
        from bagua_core_b200 import _build

        _build.build(verbose=bool(os.environ.get("BAGUA_B200_VERBOSE_BUILD")))
        super().run()


setup(
    name="bagua-core-b200",
    version="0.1.0",
    description="Blackwell-native communication backend with the API of bagua-core",
    packages=find_packages(include=["bagua_core", "bagua_core.*", "bagua_core_b200", "bagua_core_b200.*"]),
    package_data={"bagua_core_b200": ["_bagua_core_b200.so", "csrc/**/*"]},
    python_requires=">=3.9",
    install_requires=["torch", "numpy"],
    cmdclass={"build_py": BuildWithNative},
)
