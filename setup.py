"""Builds the native core in-tree (nvcc, sm_100a) before packaging.

    python setup.py build_ext --inplace      # same as: python -m jaxdecomp_b200.native
"""
from setuptools import setup
from setuptools.command.build_ext import build_ext as _build_ext
from setuptools.command.build_py import build_py as _build_py


def _build_native():
    from jaxdecomp_b200 import native

    native.build(verbose=True)


class build_ext(_build_ext):
    def run(self):
        _build_native()


class build_py(_build_py):
    def run(self):
        try:
            _build_native()
        except Exception as e:  # noqa: BLE001 - a CPU-only install still gets the baseline backend
            print(f"warning: native core not built ({e})")
        super().run()


setup(cmdclass={"build_ext": build_ext, "build_py": build_py})
