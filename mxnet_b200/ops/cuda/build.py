"""Build the sm_100a kernel library in-tree: ``python -m mxnet_b200.ops.cuda.build``.

nvcc cross-compiles without a GPU.  Each ``.cu`` file is compiled to an object with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into ``libmxb200_kernels.so`` next to
the sources; ``-Xptxas -v`` output (registers, spills, shared memory) is kept in ``build/ptxas.log``."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ['norm.cu', 'softmax.cu', 'optim.cu', 'fused_step.cu', 'gemm_tcgen05.cu', 'pool.cu', 'compress.cu', 'elementwise.cu', 'lstm.cu',
           'attention.cu', 'conv_tcgen05.cu', 'peer_reduce.cu', 'detection.cu', 'gemm_i8.cu', 'lstm_tc.cu', 'image_pipeline.cu', 'sparse.cu']
LIB = os.path.join(HERE, 'libmxb200_kernels.so')
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17', '--use_fast_math',
         '-Xcompiler', '-fPIC', '-Xptxas', '-v']


def _nvcc():
    return os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')


def build(force=False, verbose=False):
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(HERE, s))]
    bdir = os.path.join(HERE, 'build')
    os.makedirs(bdir, exist_ok=True)
    deps = [os.path.join(HERE, h) for h in os.listdir(HERE) if h.endswith(('.cuh', '.h', '.inl'))]

    def stale(obj, src):
        if force or not os.path.exists(obj):
            return True
        t = os.path.getmtime(obj)
        return any(os.path.getmtime(d) > t for d in [src] + deps)

    logs = {}

    def compile_one(name):
        src, obj = os.path.join(HERE, name), os.path.join(bdir, name[:-3] + '.o')
        if not stale(obj, src):
            return name, 0, ''
        r = subprocess.run([_nvcc()] + FLAGS + ['-c', src, '-o', obj], capture_output=True, text=True)
        return name, r.returncode, r.stdout + r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(compile_one, srcs))
    failed = [(n, out) for n, rc, out in results if rc != 0]
    with open(os.path.join(bdir, 'ptxas.log'), 'a') as f:
        for n, rc, out in results:
            if out:
                f.write('==== %s ====\n%s\n' % (n, out))
    if failed:
        raise RuntimeError('nvcc failed:\n' + '\n'.join('--- %s ---\n%s' % f for f in failed))
    objs = [os.path.join(bdir, s[:-3] + '.o') for s in srcs]
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        r = subprocess.run([_nvcc(), '-shared', '-o', LIB + '.tmp'] + objs + ['-lcudart'], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError('link failed:\n' + r.stdout + r.stderr)
        os.replace(LIB + '.tmp', LIB)
    if verbose:
        for n, rc, out in results:
            if out:
                print('====', n)
                print(out)
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
