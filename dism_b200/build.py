"""Build libdism_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
OUT = os.path.join(HERE, 'libdism_b200.so')
SOURCES = ['abi.cu', 'labels.cu', 'labels_tcgen05.cu', 'hard_index.cu', 'hard_scan.cu', 'hard_forward.cu', 'hard_forward_static.cu',
           'hard_backward.cu']
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
         '-Xcompiler', '-fPIC', '-Xptxas', '-v']


def nvcc():
    for candidate in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    raise RuntimeError('nvcc not found')


def stale():
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    inputs = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, '..', 'include', 'dism_b200.h')]
    return any(os.path.getmtime(p) > built for p in inputs)


def build(force=False, verbose=False):
    """Compile every translation unit and link the shared library; returns its path."""
    if not force and not stale():
        return OUT
    objects = os.path.join(HERE, 'csrc', 'build')
    os.makedirs(objects, exist_ok=True)

    def compile_one(source):
        target = os.path.join(objects, source.replace('.cu', '.o'))
        result = subprocess.run([nvcc(), *FLAGS, '-c', os.path.join(CSRC, source), '-o', target],
                                capture_output=True, text=True)
        with open(target.replace('.o', '.ptxas.log'), 'w') as log:
            log.write(result.stdout + result.stderr)
        if result.returncode:
            raise RuntimeError(f'nvcc failed on {source}:\n{result.stderr}')
        return target

    with ThreadPoolExecutor(len(SOURCES)) as pool:
        built = list(pool.map(compile_one, SOURCES))
    subprocess.check_call([nvcc(), '-shared', *FLAGS[:2], '-o', OUT, *built])
    if verbose:
        print('built', OUT)
    return OUT


if __name__ == '__main__':
    build(force='--force' in sys.argv, verbose=True)
