"""``mx.tvmop`` (``python/mxnet/tvmop.py``): the reference loads TVM-generated operator kernels when it was built with
``USE_TVM_OP``.  This build has no TVM bridge (``mx.runtime.Features()['TVM_OP']`` is off), so nothing is loaded."""


def _load_lib():
    return None


_LIB = _load_lib()
