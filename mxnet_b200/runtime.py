"""Run-time feature detection (``python/mxnet/runtime.py`` over ``src/libinfo.cc:40-163``)."""
import collections

import torch

__all__ = ['Feature', 'Features', 'feature_list']

Feature = collections.namedtuple('Feature', ['name', 'enabled'])


def _nvrtc_bindings():
    """Whether run-time compilation (``mx.rtc.CudaModule``, the pointwise-fusion pass) can load NVRTC."""
    try:
        from cuda import nvrtc  # noqa: F401
        return True
    except Exception:  # pylint: disable=broad-except
        return False


def _probe():
    cuda = torch.cuda.is_available() or torch.version.cuda is not None
    try:
        import torch.distributed as dist
        nccl = dist.is_nccl_available()
    except Exception:  # pylint: disable=broad-except
        nccl = False
    feats = {
        'CUDA': cuda, 'CUDNN': cuda and torch.backends.cudnn.is_available() if torch.cuda.is_available() else cuda,
        'NCCL': nccl, 'TENSORRT': False, 'CUTENSOR': False, 'CUDA_RTC': cuda and _nvrtc_bindings(),
        'CPU_SSE': True, 'CPU_SSE2': True, 'CPU_SSE3': True, 'CPU_SSE4_1': True, 'CPU_SSE4_2': True, 'CPU_SSE4A': False,
        'CPU_AVX': True, 'CPU_AVX2': True, 'OPENMP': True, 'SSE': True, 'F16C': True, 'JEMALLOC': False,
        'BLAS_OPEN': False, 'BLAS_ATLAS': False, 'BLAS_MKL': True, 'BLAS_APPLE': False, 'LAPACK': True,
        'ONEDNN': False, 'OPENCV': False, 'DIST_KVSTORE': True, 'INT64_TENSOR_SIZE': True, 'SIGNAL_HANDLER': True,
        'DEBUG': False, 'TVM_OP': False,
        # what is specific to this build
        'SM100A_KERNELS': True, 'TCGEN05': True, 'CUDA_GRAPHS': cuda, 'FUSED_KVSTORE': True,
    }
    return feats


def feature_list():
    return [Feature(k, v) for k, v in _probe().items()]


class Features(collections.OrderedDict):
    instance = None

    def __new__(cls):
        if cls.instance is None:
            cls.instance = super().__new__(cls)
            super(Features, cls.instance).__init__([(f.name, f) for f in feature_list()])
        return cls.instance

    def __init__(self):
        pass

    def __repr__(self):
        return str(list(self.values()))

    def is_enabled(self, feature_name):
        feature_name = feature_name.upper()
        if feature_name not in self:
            raise RuntimeError("Feature '{}' is unknown, known features are: {}".format(feature_name, list(self.keys())))
        return self[feature_name].enabled


def _git(*args):
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        out = subprocess.run(['git', '-C', root] + list(args), capture_output=True, text=True, timeout=10)
        return out.stdout.strip() if out.returncode == 0 and out.stdout.strip() else 'unknown'
    except Exception:   # pylint: disable=broad-except
        return 'unknown'


def get_branch():
    """Branch of the source tree this package runs from ('unknown' outside a git checkout)."""
    return _git('rev-parse', '--abbrev-ref', 'HEAD')


def get_commit_hash():
    """Commit of the source tree this package runs from ('unknown' outside a git checkout)."""
    return _git('rev-parse', 'HEAD')
