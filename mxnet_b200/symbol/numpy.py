"""``mx.sym.np``: NumPy-named symbolic functions over the ``_npi_*`` operators."""
from ..ops import registry as _reg
from .symbol import _op_frontend

for _name in _reg.list_ops():
    if _name.startswith('_npi_'):
        globals()[_name[5:]] = _op_frontend(_reg.get(_name))
