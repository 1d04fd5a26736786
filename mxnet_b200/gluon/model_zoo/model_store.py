"""Pretrained-model file lookup (``python/mxnet/gluon/model_zoo/model_store.py``): files are taken
from ``root`` (default ``$MXNET_HOME/models``) and downloaded from the model repository only when
they are missing."""
import os

from ... import env


def get_model_file(name, root=None):
    root = os.path.expanduser(root or os.path.join(env.get('MXNET_HOME'), 'models'))
    for fn in sorted(os.listdir(root)) if os.path.isdir(root) else []:
        if fn.startswith(name) and fn.endswith('.params'):
            return os.path.join(root, fn)
    from ..utils import download
    os.makedirs(root, exist_ok=True)
    url = '%sgluon/models/%s.zip' % (env.get('MXNET_GLUON_REPO'), name)
    zip_path = download(url, path=os.path.join(root, name + '.zip'), overwrite=True)
    import zipfile
    with zipfile.ZipFile(zip_path) as zf:
        zf.extractall(root)
    os.remove(zip_path)
    return get_model_file(name, root)


def purge(root=None):
    root = os.path.expanduser(root or os.path.join(env.get('MXNET_HOME'), 'models'))
    for f in os.listdir(root) if os.path.isdir(root) else []:
        if f.endswith('.params'):
            os.remove(os.path.join(root, f))


def short_hash(name, root=None):
    """The 8-character hash in the file name ``<name>-<hash>.params`` of a pretrained model present under ``root``."""
    root = os.path.expanduser(root or os.path.join(env.get('MXNET_HOME'), 'models'))
    for fn in sorted(os.listdir(root)) if os.path.isdir(root) else []:
        if fn.startswith(name + '-') and fn.endswith('.params'):
            return fn[len(name) + 1:-len('.params')][:8]
    raise ValueError('Pretrained model for {name} is not available.'.format(name=name))
