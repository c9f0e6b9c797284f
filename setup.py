"""`pip install -e .` builds libonebitmul.so and the onebit_sparse_cuda extension in-tree (the
reference's setup.py:1-36 builds the same extension; here there are no hard-coded include paths
and the only target architecture is sm_100a)."""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        from onebitsparsemul_b200 import build
        build.build_library()
        build.build_torch_extension()
        super().run()


setup(
    name="onebit_sparse_mul",
    version="0.1.0",
    description="One-bit 2:4 sparse x fp16 GEMM for NVIDIA B200 (sm_100a)",
    packages=["onebitsparsemul_b200", "onebit_sparse_mul"],
    package_data={"onebitsparsemul_b200": ["libonebitmul.so", "csrc/*"]},
    install_requires=["numpy", "torch"],
    cmdclass={"build_py": BuildNative},
)
