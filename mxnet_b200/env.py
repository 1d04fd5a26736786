"""Typed registry of the ``MXNET_*`` environment flags.

The reference reads ~100 variables ad hoc through ``dmlc::GetEnv`` (documented in
``docs/static_site/src/pages/api/faq/env_var.md``).  Here every flag is declared once with a type,
a default and a one-line meaning, so ``mx.env.describe()`` lists them and tests can flip them with
:func:`scope`, the counterpart of ``test_utils.environment()`` (``python/mxnet/test_utils.py:2352``)
and of ``MXGetEnv/MXSetEnv`` (``src/c_api/c_api_test.cc:108-120``).
"""
import contextlib
import os

__all__ = ['declare', 'get', 'set', 'scope', 'describe', 'FLAGS']

FLAGS = {}


class _Flag(object):
    __slots__ = ('name', 'type', 'default', 'doc')

    def __init__(self, name, type_, default, doc):
        self.name, self.type, self.default, self.doc = name, type_, default, doc

    def parse(self, raw):
        if self.type is bool:
            return raw.strip().lower() not in ('0', 'false', 'off', 'no', '')
        return self.type(raw)


def declare(name, type_, default, doc=''):
    FLAGS[name] = _Flag(name, type_, default, doc)
    return FLAGS[name]


def get(name, default=None):
    """Current value of a flag (environment wins over the declared default)."""
    flag = FLAGS.get(name)
    raw = os.environ.get(name)
    if flag is None:
        return raw if raw is not None else default
    if raw is None:
        return flag.default if default is None else default
    try:
        return flag.parse(raw)
    except (TypeError, ValueError):
        return flag.default


def set(name, value):  # pylint: disable=redefined-builtin
    if value is None:
        os.environ.pop(name, None)
    else:
        os.environ[name] = str(int(value)) if isinstance(value, bool) else str(value)
    if name == 'MXNET_ENGINE_TYPE':
        _refresh_engine_type()
    if name == 'MXNET_CUDA_ALLOW_TF32':
        _refresh_tf32()


def _refresh_tf32():
    """Mirror ``MXNET_CUDA_ALLOW_TF32`` into the tensor library's math mode for fp32 GEMMs and convolutions (forward and
    backward, on every thread)."""
    import torch
    on = bool(get('MXNET_CUDA_ALLOW_TF32'))
    torch.backends.cuda.matmul.allow_tf32 = on
    torch.backends.cudnn.allow_tf32 = on


def _refresh_engine_type():
    """Mirror ``MXNET_ENGINE_TYPE`` into the flag the operator entry point reads on every call."""
    from . import _state
    _state.naive_engine = os.environ.get('MXNET_ENGINE_TYPE') == 'NaiveEngine'


@contextlib.contextmanager
def scope(*args, **kwargs):
    """``with env.scope('MXNET_X', '1'):`` or ``with env.scope(MXNET_X=1, MXNET_Y=None):``."""
    if args:
        assert len(args) == 2, 'scope(name, value) or scope(**flags)'
        kwargs = dict(kwargs)
        kwargs[args[0]] = args[1]
    saved = {k: os.environ.get(k) for k in kwargs}
    try:
        for k, v in kwargs.items():
            set(k, v)
        yield
    finally:
        for k, v in saved.items():
            set(k, v)


def describe():
    rows = []
    for f in sorted(FLAGS.values(), key=lambda f: f.name):
        rows.append('%-44s %-6s default=%-10r %s' % (f.name, f.type.__name__, f.default, f.doc))
    return '\n'.join(rows)


# ---- engine -------------------------------------------------------------------------------
declare('MXNET_USE_SIGNAL_HANDLER', bool, True,
        'Print the Python stack of every thread when the process receives a fatal signal (SIGSEGV, SIGFPE, SIGABRT, SIGBUS, SIGILL).')
declare('MXNET_ENGINE_TYPE', str, 'ThreadedEnginePerDevice',
        'NaiveEngine = fully synchronous; ThreadedEngine / ThreadedEnginePerDevice / ...Async = stream engine')
declare('MXNET_CPU_WORKER_NTHREADS', int, 1, 'host worker threads of the native dependency engine')
declare('MXNET_GPU_WORKER_NTHREADS', int, 2, 'compute streams per GPU')
declare('MXNET_GPU_COPY_NTHREADS', int, 2, 'copy streams per GPU')
declare('MXNET_CPU_PRIORITY_NTHREADS', int, 4, 'host threads serving prioritised tasks')
declare('MXNET_EXEC_BULK_EXEC_INFERENCE', bool, True, 'bulk (graph-capture) inference segments')
declare('MXNET_EXEC_BULK_EXEC_TRAIN', bool, True, 'bulk (graph-capture) training segments')
declare('MXNET_EXEC_BULK_EXEC_MAX_NODE_TRAIN', int, 15, 'max nodes per bulked segment')
declare('MXNET_ENABLE_CUDA_GRAPHS', bool, True, 'hybridize(static_alloc, static_shape) captures CUDA graphs')
declare('MXNET_CUDA_GRAPHS_AUTO', bool, True, 'a block hybridized without static_alloc / static_shape is also captured once an input signature has repeated three times (at most four signatures per block); 0 = only blocks hybridized with both flags are captured')
declare('MXNET_CUDA_GRAPHS_VERBOSE', bool, False, 'log graph capture / re-capture events')
declare('MXNET_ENGINE_INFO', bool, False, 'verbose engine logging')
# ---- memory -------------------------------------------------------------------------------
declare('MXNET_GPU_MEM_POOL_TYPE', str, 'Naive', 'Naive (round to multiple) | Round (power of two) | Unpooled')
declare('MXNET_CPU_MEM_POOL_TYPE', str, 'Naive', 'same choices for host memory')
declare('MXNET_CPU_PINNED_MEM_POOL_TYPE', str, 'Naive', 'same choices for pinned host memory')
declare('MXNET_GPU_MEM_POOL_RESERVE', int, 5, 'percent of device memory left unpooled')
declare('MXNET_GPU_MEM_POOL_PAGE_SIZE', int, 4096, 'rounding granule of small allocations')
declare('MXNET_GPU_MEM_LARGE_ALLOC_ROUND_SIZE', int, 2097152, 'rounding granule of large allocations')
declare('MXNET_GPU_MEM_POOL_ROUND_LINEAR_CUTOFF', int, 24, 'log2 size above which Round pool goes linear')
declare('MXNET_USE_NAIVE_STORAGE_MANAGER', bool, False, 'bypass pooling entirely')
declare('MXNET_GPU_TEMP_COPY', int, 1, 'temp workspaces per GPU')
declare('MXNET_CPU_TEMP_COPY', int, 4, 'temp workspaces per CPU')
# ---- kvstore ------------------------------------------------------------------------------
declare('MXNET_KVSTORE_REDUCTION_NTHREADS', int, 4, 'threads of the host tree-sum of kvstore local')
declare('MXNET_KVSTORE_BIGARRAY_BOUND', int, 1000000, 'element count above which a key is sliced')
declare('MXNET_KVSTORE_USETREE', bool, False, 'multi-root sliced reduce for kvstore device')
declare('MXNET_KVSTORE_TREE_ARRAY_BOUND', int, 10000000, 'slice bound of the tree reduce')
declare('MXNET_KVSTORE_SLICE_THRESHOLD', int, 40000, 'P3 slice size')
declare('MXNET_KVSTORE_SERIAL_PUSH', bool, False, 'serialise pushes (debug)')
declare('MXNET_ENABLE_GPU_P2P', bool, True, 'map peer memory for kvstore device/nccl')
declare('MXNET_UPDATE_ON_KVSTORE', bool, True, 'default of Trainer.update_on_kvstore')
declare('MXNET_KVSTORE_FUSED', bool, True, 'use the fused reduce-scatter+update+all-gather kernels')
declare('MXNET_KVSTORE_BUCKET_MB', int, 32, 'gradient bucket size of the fused path')
declare('MXNET_KVSTORE_WAIT_MS', int, 20000, 'bound of device-side peer waits before an error status')
declare('MXNET_KVSTORE_NVLS', bool, False, 'fused optimizer step / all-reduce of a multi-process job through the NVLink switch: the arenas are allocated as symmetric memory with a multicast mapping, gradients are summed by multimem.ld_reduce and weights broadcast by multimem.st (falls back to peer loads and stores where the machine has no multicast support). Leave off in jobs whose ranks may exit one by one: a multicast binding must be torn down by all ranks together')
# ---- numerics -----------------------------------------------------------------------------
declare('MXNET_SAFE_ACCUMULATION', bool, True, 'accumulate fp16 reductions in fp32')
declare('MXNET_ENFORCE_DETERMINISM', bool, False, 'refuse non-deterministic kernels')
declare('MXNET_CUDA_ALLOW_TENSOR_CORE', bool, True, 'allow tensor-core GEMM/conv')
declare('MXNET_CUDA_ALLOW_TF32', bool, False, 'fp32 GEMMs and convolutions of the library path on tf32 tensor cores. The reference computes its fp32 cuBLAS products in this mode on CUDA 11+ (src/operator/linalg_impl.h:298, CUBLAS_TF32_TENSOR_OP_MATH); here fp32 stays exact unless this is set')
declare('MXNET_FC_TRUE_FP16', bool, False, 'accumulate FullyConnected in fp16 (never on tcgen05)')
declare('MXNET_B200_KERNELS', bool, True, 'use the hand-written sm_100a kernels (0 = library path)')
declare('MXNET_RNN_UNROLLED', bool, False, 'run the RNN operator as per-step tensor operations even on a GPU (debugging)')
declare('MXNET_B200_ATTENTION', bool, True, 'fused self-attention on the tcgen05 kernel (0 = library attention)')
declare('MXNET_B200_CONV', str, 'auto', 'stride-1 NHWC convolutions on the tcgen05 implicit-GEMM kernels: auto = time against the library per shape and direction, subset of fwd,dgrad,wgrad or 1 = force, 0 = library convolution')
declare('MXNET_B200_CONV_RESIDENT_WEIGHTS', bool, True, 'keep the weight slices of a column tile resident in shared memory in the convolution kernels when they fit (0 = stream them with the activations)')
declare('MXNET_B200_ELEMENTWISE', bool, True, 'GELU, dropout, embedding, add_n, cast and average pooling on the in-tree vector kernels (0 = library kernels)')
declare('MXNET_B200_GEMM_AUTOTUNE', bool, True, 'time the tcgen05 GEMM against the library GEMM per shape and product (forward, data gradient, weight gradient) on first use and keep the faster')
declare('MXNET_B200_GEMM', bool, True, 'route half-precision FullyConnected/dot to the tcgen05 GEMM kernel (0 = library GEMM)')
# ---- graph --------------------------------------------------------------------------------
declare('MXNET_B200_RNN', str, 'auto', 'RNN operator on the in-tree recurrence kernels: auto = time forward + backward against the library recurrence per configuration, 1 = force, 0 = library')
declare('MXNET_B200_RNN_TC', bool, True, 'LSTM recurrence of the in-tree path on the tensor-core kernels (tcgen05; tf32 products for fp32 models, as the library recurrence uses) for layers of 32 units or more where the shape allows; 0 = the fp32-pipe recurrence kernels (exact fp32 products)')
declare('MXNET_USE_FUSION', bool, True, 'pointwise fusion')
declare('MXNET_ELIMINATE_COMMON_EXPR', bool, True, 'common-subexpression elimination on symbols')
declare('MXNET_MEMORY_OPT', bool, False, 'backward mirroring in graph executors and hybridized blocks: runs of cheap stateless operators keep only their inputs and are recomputed in backward')
declare('MXNET_BACKWARD_DO_MIRROR', bool, False, 'legacy spelling of MXNET_MEMORY_OPT')
declare('MXNET_SUBGRAPH_BACKEND', str, '', 'default subgraph backend')
# ---- profiler / misc ----------------------------------------------------------------------
declare('MXNET_PROFILER_AUTOSTART', bool, False, 'start profiling at import')
declare('MXNET_PROFILER_MODE', int, 0, 'bit mask: 1 symbolic, 2 imperative, 4 api, 8 memory')
declare('MXNET_HOME', str, os.path.join(os.path.expanduser('~'), '.mxnet'), 'data / model cache')
declare('MXNET_GLUON_REPO', str, 'https://apache-mxnet.s3-accelerate.dualstack.amazonaws.com/', 'model repo URL')
declare('MXNET_LIBRARY_PATH', str, '', 'override for the native runtime library')
declare('MXNET_MODULE_SEED', int, -1, 'test module seed')
declare('MXNET_TEST_SEED', int, -1, 'test function seed')
declare('MXNET_USE_OPERATOR_TUNING', bool, True, 'tune OpenMP use per CPU op')
declare('MXNET_OMP_MAX_THREADS', int, 0, 'cap of intra-op host threads (0 = auto)')
declare('MXNET_OPTIMIZER_AGGREGATION_SIZE', int, 4, 'tensors per multi-tensor optimizer call')
declare('MXNET_STORAGE_FALLBACK_LOG_VERBOSE', bool, True, 'log dense fallbacks of sparse inputs')


def markdown():
    """The flag table as a Markdown document (``docs/env_var.md`` is this text; the reference documents its flags in
    ``docs/static_site/src/pages/api/faq/env_var.md``)."""
    lines = ['# Environment variables', '',
             'Every flag is read through `mxnet_b200.env.get(name)`; the environment wins over the default, and '
             '`mxnet_b200.env.scope(NAME=value)` / `mxnet_b200.test_utils.environment` set one for a `with` block.', '',
             '| variable | type | default | meaning |', '|---|---|---|---|']
    home = os.path.expanduser('~')
    for f in sorted(FLAGS.values(), key=lambda f: f.name):
        default = f.default
        if isinstance(default, str) and home not in ('', '/') and default.startswith(home):
            default = '~' + default[len(home):]         # the document must not depend on who generated it
        lines.append('| `%s` | %s | `%r` | %s |' % (f.name, f.type.__name__, default, f.doc.replace('|', '\\|')))
    return '\n'.join(lines) + '\n'


if os.environ.get('MXNET_CUDA_ALLOW_TF32') is not None:
    _refresh_tf32()


if __name__ == '__main__':
    import sys
    sys.stdout.write(markdown())
