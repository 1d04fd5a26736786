"""Deferred-compute tracer: records executed operators into Symbol nodes.

Reference: ``Imperative::RecordDeferredCompute`` / ``GetDeferredComputeSymbol``
(``src/imperative/imperative.cc:336-394``).  Unlike the reference the operators *are* executed
while tracing (results are needed anyway for shapes and for the first output), the trace only adds
bookkeeping: each output array remembers the (node, index) that produced it.
"""
from ..base import MXNetError
from ..name import NameManager
from .symbol import Symbol, _Node, var


class Tracer(object):
    def __init__(self):
        self._entries = {}      # id(array) -> ((node, idx), array)  (array kept alive for id stability)
        self.constants = {}     # name -> array, for inputs that were never declared as variables
        self._names = NameManager()

    def set_variable(self, array, variable):
        self._entries[id(array)] = (variable._outputs[0], array)

    def _entry_of(self, a):
        hit = self._entries.get(id(a))
        if hit is not None:
            return hit[0]
        name = '_const%d' % len(self.constants)
        self.constants[name] = a
        v = var(name)
        self._entries[id(a)] = (v._outputs[0], a)
        return v._outputs[0]

    def record(self, op, args, attrs, outputs):
        from ..ndarray.ndarray import NDArray
        inputs = []
        clean = dict(attrs)
        for a in args:
            if isinstance(a, NDArray):
                inputs.append(self._entry_of(a))
            elif a is None:
                continue
            else:
                raise MXNetError('cannot trace operator %s with a non-array positional input' % op.name)
        name = self._names.get(None, op.name.lower().lstrip('_'))
        node = _Node(op, name, clean, inputs, max(len(outputs), 1))
        for i, o in enumerate(outputs):
            if isinstance(o, NDArray):
                self._entries[id(o)] = ((node, i), o)
                o._sym = (node, i)

    def get_symbol(self, outputs):
        ents = []
        for o in outputs:
            hit = self._entries.get(id(o))
            if hit is None:
                raise MXNetError('output array was not computed inside the tracing scope')
            ents.append(hit[0])
        return Symbol(ents)
