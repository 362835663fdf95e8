"""Build script: ``python setup.py build_ext --inplace`` compiles ``mccl_b200/_C.so`` for sm_100a.

The actual compile/link recipe lives in :mod:`mccl_b200._build` (ninja through
``torch.utils.cpp_extension`` with ``-gencode arch=compute_100a,code=sm_100a``);
this file only routes the setuptools commands to it so the extension is always
built in-tree, next to the Python sources.
"""
from setuptools import Command, find_packages, setup


class build_ext(Command):
    description = "build the native extension in-tree for sm_100a"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree"),
                    ("force", "f", "rebuild everything")]

    def initialize_options(self):
        self.inplace = 1
        self.force = 0

    def finalize_options(self):
        pass

    def run(self):
        from mccl_b200 import _build
        print(_build.build(force=bool(self.force), verbose=True))


setup(
    name="mccl_b200",
    version="0.5.0",
    description="Blackwell-native torch.distributed backend 'mccl' (NVLink peer-memory collectives)",
    packages=find_packages(include=["mccl_b200", "mccl_b200.*", "mccl"]),
    package_data={"mccl_b200": ["_C.so"]},
    cmdclass={"build_ext": build_ext},
    python_requires=">=3.10",
)
