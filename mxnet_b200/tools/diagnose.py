"""Environment report for bug reports:  python -m mxnet_b200.tools.diagnose

Prints platform, Python, framework and dependency versions, the state of the two native libraries, the typed
``MXNET_*`` flags that are set, and what the CUDA runtime reports about the visible GPUs (reference: tools/diagnose.py,
without its network probes)."""
import os
import platform
import sys


def report():
    lines = []

    def sec(title):
        lines.append('----------%s----------' % title)

    sec('Platform')
    lines += ['system   : %s' % platform.platform(), 'machine  : %s' % platform.machine(), 'cpus     : %s' % os.cpu_count()]
    sec('Python')
    lines += ['version  : %s' % sys.version.replace('\n', ' '), 'prefix   : %s' % sys.prefix]
    sec('Framework')
    import mxnet_b200 as mx
    lines.append('mxnet_b200: %s (%s)' % (getattr(mx, '__version__', '?'), os.path.dirname(mx.__file__)))
    for name in ('torch', 'numpy'):
        try:
            mod = __import__(name)
            lines.append('%-10s: %s' % (name, mod.__version__))
        except Exception as e:
            lines.append('%-10s: unavailable (%s)' % (name, e))
    sec('Native libraries')
    here = os.path.dirname(mx.__file__)
    for rel in ('csrc/libmxb200_rt.so', 'ops/cuda/libmxb200_kernels.so'):
        p = os.path.join(here, rel)
        lines.append('%-30s: %s' % (rel, '%d bytes' % os.path.getsize(p) if os.path.exists(p) else 'not built'))
    try:
        feats = mx.runtime.Features()
        lines.append('features : ' + ', '.join(sorted(k for k in feats.keys() if feats.is_enabled(k))))
    except Exception as e:
        lines.append('features : unavailable (%s)' % e)
    sec('Flags set in the environment')
    flags = sorted(k for k in os.environ if k.startswith(('MXNET_', 'DMLC_', 'NCCL_')))
    lines += ['%s=%s' % (k, os.environ[k]) for k in flags] or ['(none)']
    sec('GPUs')
    import torch
    if not torch.cuda.is_available():
        lines.append('no CUDA device visible')
    else:
        lines.append('CUDA runtime %s, %d device(s)' % (torch.version.cuda, torch.cuda.device_count()))
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            lines.append('  [%d] %s  sm_%d%d  %d SMs  %.1f GB' % (i, p.name, p.major, p.minor, p.multi_processor_count,
                                                                  p.total_memory / 2 ** 30))
    return '\n'.join(lines)


def main(argv=None):
    print(report())
    return 0


if __name__ == '__main__':
    sys.exit(main())
