"""Packaging: ``pip install .`` builds the host runtime (g++) and the sm_100a kernel library (nvcc) in-tree and installs
the ``mxnet_b200`` package together with the ``mxnet`` alias package and both shared objects."""
import os
import subprocess
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    """Compile the native libraries before the Python files are collected, so the shared objects travel as package data."""

    def run(self):
        env = dict(os.environ, PYTHONPATH=HERE + os.pathsep + os.environ.get('PYTHONPATH', ''))
        subprocess.check_call([sys.executable, '-c',
                               'from mxnet_b200.csrc import runtime; runtime.build_runtime(force=True)'], cwd=HERE, env=env)
        if os.environ.get('MXNET_B200_SKIP_KERNELS') != '1':
            subprocess.check_call([sys.executable, '-m', 'mxnet_b200.ops.cuda.build'], cwd=HERE, env=env)
        super().run()


setup(
    name='mxnet-b200',
    version='2.0.0',
    description='Blackwell-native deep-learning framework with the Apache MXNet API',
    packages=find_packages(include=['mxnet_b200', 'mxnet_b200.*', 'mxnet', 'mxnet.*']),
    package_data={'mxnet_b200': ['csrc/*.cc', 'csrc/*.so', 'ops/cuda/*.cu', 'ops/cuda/*.cuh', 'ops/cuda/*.h', 'ops/cuda/*.so',
                                 'include/*.h', 'include/mxnet_b200/*.h']},
    python_requires='>=3.10',
    install_requires=['torch>=2.6', 'numpy'],
    cmdclass={'build_py': BuildNative},
)
