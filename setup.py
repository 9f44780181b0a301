"""Packaging: builds the native libraries with the Makefile under csrc/ and ships them inside the package.

    python -m pip install --no-build-isolation .        # needs nvcc (sm_100a), g++ and the torch / pybind11 headers

Installs ``nixl_b200`` plus the reference's import names ``nixl`` and ``nixl_ep`` (thin aliases).  The shared objects
locate each other relative to the package directory (``$ORIGIN`` run paths), so the installed tree is self-contained.
"""
import os
import subprocess

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    def run(self):
        jobs = str(os.cpu_count() or 4)
        subprocess.run(["make", "-C", os.path.join(ROOT, "csrc"), "-j", jobs], check=True)
        super().run()


def version():
    with open(os.path.join(ROOT, "nixl_b200", "__init__.py")) as f:
        for line in f:
            if line.startswith("__version__"):
                return line.split("=")[1].strip().strip('"')
    return "0"


setup(
    name="nixl_b200",
    version=version(),
    description="Blackwell-native point-to-point transfer library with the NIXL API",
    packages=find_packages(include=["nixl_b200", "nixl_b200.*", "nixl", "nixl_ep"]),
    package_data={
        "nixl_b200": ["py.typed", "_bindings*.so", "lib/*.so", "lib/plugins/*.so", "lib/standin_plugins/*.so", "bin/*"],
    },
    include_package_data=False,
    python_requires=">=3.10",
    cmdclass={"build_py": BuildNative},
    zip_safe=False,
)
