"""Builds bmtk_b200/lib/libbmtk_b200.so from bmtk_b200/csrc/*.cu with nvcc for sm_100a.

    python -m bmtk_b200.build [--force]

The shared object is built in-tree (it is git-ignored) and exports exactly the C ABI declared in
include/bmtk_b200.h. nvcc cross-compiles without a GPU.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(_PKG)
CSRC = os.path.join(_PKG, 'csrc')
OBJ_DIR = os.path.join(CSRC, 'build')
LIB_DIR = os.path.join(_PKG, 'lib')
LIB_PATH = os.path.join(LIB_DIR, 'libbmtk_b200.so')

NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
              '-Xcompiler', '-fPIC', '-Xcompiler', '-fvisibility=hidden']


def _nvcc():
    exe = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(exe):
        raise RuntimeError('nvcc not found: the CUDA toolkit is required to build bmtk_b200')
    return exe


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith('.cu'))


def _newest_header():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(('.cuh', '.h'))]
    hs.append(os.path.join(ROOT, 'include', 'bmtk_b200.h'))
    return max(os.path.getmtime(h) for h in hs)


def _compile(nvcc, src, obj, verbose):
    cmd = [nvcc] + NVCC_FLAGS + (['-Xptxas', '-v'] if verbose else []) + ['-c', src, '-o', obj]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError('nvcc failed for %s:\n%s' % (src, p.stdout))
    return p.stdout


def build(force=False, verbose=False):
    """Compile every CUDA source and link the shared library; returns its path."""
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    hdr_time = _newest_header()
    jobs, objs = [], []
    for f in _sources():
        src = os.path.join(CSRC, f)
        obj = os.path.join(OBJ_DIR, f[:-3] + '.o')
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            jobs.append((src, obj))
    logs = []
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose), jobs))
    if jobs or not os.path.exists(LIB_PATH):
        cmd = [nvcc, '-shared', '-o', LIB_PATH] + objs + ['-gencode', 'arch=compute_100a,code=sm_100a', '-ldl']
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise RuntimeError('link failed:\n' + p.stdout)
    if verbose:
        print('\n'.join(logs))
    return LIB_PATH


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
