"""mxnet_b200: a Blackwell-native deep-learning framework with Apache MXNet's API.

``import mxnet_b200 as mx`` gives the familiar namespaces: ``mx.nd`` / ``mx.np`` / ``mx.npx`` arrays,
``mx.sym`` graphs, ``mx.autograd``, ``mx.gluon``, ``mx.optimizer``, ``mx.kv``, ``mx.amp``, ``mx.io`` …
"""
__version__ = '2.0.0'

from . import base, env, error
from .base import MXNetError
from . import device
from .device import Device, Context, cpu, gpu, cpu_pinned, cpu_shared, num_gpus, gpu_memory_info, current_device, current_context
from . import context
from . import util
from .util import is_np_shape, set_np_shape, np_shape, use_np_shape, is_np_array, np_array, use_np_array, use_np, set_np, reset_np
from . import engine
from . import ops
from . import ndarray
from . import ndarray as nd
from . import numpy
from . import numpy as np
from . import numpy_extension
from . import numpy_extension as npx
from . import autograd
from . import random
from . import symbol
from . import symbol as sym
from . import initializer
from . import initializer as init
from . import lr_scheduler
from . import optimizer
from . import kvstore
from . import kvstore as kv
from . import gluon
from . import io
from . import recordio
from . import image
from . import image as img
from . import profiler
from . import runtime
from . import callback
from . import model
from . import metric
from . import amp
from . import contrib
from . import test_utils
from . import visualization
from . import visualization as viz
from . import rtc
from . import library
from . import dlpack
from . import operator
from . import executor
from . import name
from . import attribute
from .attribute import AttrScope
from .name import NameManager
from . import _deferred_compute
from . import log
from . import libinfo
from . import registry
from . import parallel
from . import models
from . import onnx
from . import notebook
from . import tvmop
from .ndarray import waitall
from .util import is_np_default_dtype   # noqa: F401
from .kvstore import kvstore_server    # noqa: F401
from . import initialize as _initialize
_initialize.install()
