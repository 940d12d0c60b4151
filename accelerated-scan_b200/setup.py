"""Wheel of the `accelerated_scan` package with the prebuilt sm_100a library inside.

    cd accelerated-scan_b200 && python setup.py bdist_wheel          # or: pip wheel --no-build-isolation .

The build step compiles csrc/ with nvcc (build.py, no GPU needed) and ships
accelerated_scan/libascan_b200.so as package data, so the installed package needs neither
nvcc nor a JIT step at import (the reference compiles its kernel at import time,
warp.py:13-18, and publishes a pure-Python wheel, pyproject.toml).  The wheel is tagged
for the platform because it holds a native library; it does not link against Python or
torch, so one wheel serves every Python version.
"""
import importlib.util
import os
import re

from setuptools import setup
from setuptools.command.build_py import build_py
from setuptools.dist import Distribution

HERE = os.path.dirname(os.path.abspath(__file__))


def _version():
    text = open(os.path.join(HERE, "accelerated_scan", "__init__.py")).read()
    return re.search(r'__version__\s*=\s*"([^"]+)"', text).group(1)


class BuildWithLibrary(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location("ascan_build", os.path.join(HERE, "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
        super().run()


class BinaryDistribution(Distribution):
    def has_ext_modules(self):
        return True


try:
    from wheel.bdist_wheel import bdist_wheel

    class PlatformWheel(bdist_wheel):
        def get_tag(self):
            _, _, plat = super().get_tag()
            return "py3", "none", plat

    CMDCLASS = {"build_py": BuildWithLibrary, "bdist_wheel": PlatformWheel}
except ImportError:
    CMDCLASS = {"build_py": BuildWithLibrary}


setup(
    name="accelerated-scan-b200",
    version=_version(),
    description="First-order parallel scan for NVIDIA B200 (sm_100a): drop-in accelerated_scan.warp / .complex",
    packages=["accelerated_scan"],
    package_dir={"accelerated_scan": "accelerated_scan"},
    package_data={"accelerated_scan": ["libascan_b200.so"]},
    include_package_data=True,
    python_requires=">=3.10",
    install_requires=["torch>=2.9.0"],
    distclass=BinaryDistribution,
    cmdclass=CMDCLASS,
    zip_safe=False,
)
