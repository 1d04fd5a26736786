"""Thread-local runtime state: autograd flags, NumPy-semantics switches, tracing and AMP hooks.

Reference counterparts: ``Imperative::is_recording_/is_training_/is_deferred_compute_``
(``include/mxnet/imperative.h``), ``is_np_shape/is_np_array/is_np_default_dtype``
(``python/mxnet/util.py``).
"""
import threading


class _State(threading.local):
    def __init__(self):
        super().__init__()
        self.recording = False
        self.training = False
        self.np_shape = False
        self.np_array = False
        self.np_default_dtype = False
        self.opt_constraints = 0      # HybridBlock.OptConstraint flags (bit 0: AMP casts off)
        self.tracer = None          # active deferred-compute tracer (symbol/_trace.py) or None
        self.bulk_size = 0
        self.profiler_scope = '<unk>:'
        self.name_prefix = ''


state = _State()

# process-wide hooks (set by mxnet_b200.amp / profiler); kept here to avoid import cycles
naive_engine = __import__('os').environ.get('MXNET_ENGINE_TYPE') == 'NaiveEngine'   # kept current by env.set
amp_hook = None          # callable(opname, tensors:list) -> list, or None
op_monitor = None        # callable(opname, outputs) for register_op_hook style monitors
profiler_hook = None     # callable(opname) -> context manager, or None


def is_recording():
    return state.recording


def is_training():
    return state.training
