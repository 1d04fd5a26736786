"""Library location and version (``python/mxnet/libinfo.py``)."""
import os

__version__ = '2.0.0'


def find_lib_path(prefix='libmxb200'):
    """Paths of the native libraries that back this package."""
    here = os.path.dirname(os.path.abspath(__file__))
    cands = [os.path.join(here, 'csrc', 'libmxb200_rt.so'), os.path.join(here, 'ops', 'cuda', 'libmxb200_kernels.so')]
    return [c for c in cands if os.path.exists(c)]


def find_include_path():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), 'csrc')
