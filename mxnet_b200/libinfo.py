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


def find_conf_path(prefix='tvmop'):
    """Path of ``<prefix>.conf``: ``$MXNET_CONF_PATH`` when that file exists, else next to the native libraries."""
    import logging
    import os
    conf = os.environ.get('MXNET_CONF_PATH')
    if conf:
        if os.path.isfile(conf):
            if not os.path.isabs(conf):
                logging.warning('MXNET_CONF_PATH should be an absolute path, instead of: %s', conf)
            else:
                return conf
        else:
            logging.warning("MXNET_CONF_PATH '%s' doesn't exist", conf)
    here = os.path.dirname(os.path.abspath(__file__))
    for d in (os.path.join(here, 'csrc'), here):
        cand = os.path.join(d, prefix + '.conf')
        if os.path.isfile(cand):
            return cand
    raise RuntimeError('Cannot find the configuration file %s.conf' % prefix)
