"""``mx.npx.image``: image operators with NumPy-semantics arrays."""
from ..ops import registry as _reg

for _name in _reg.list_ops():
    if _name.startswith('_image_'):
        globals()[_name[len('_image_'):]] = _reg.make_frontend(_reg.get(_name), 'np')
