"""Build libfga.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python build_native.py [--force] [--verbose]
"""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
OUT = os.path.join(HERE, 'libfga.so')
SOURCES = ('runtime.cu', 'aux_kernels.cu', 'gemm_sm100a.cu')
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
         '-Xcompiler', '-fPIC', '-shared']


def _nvcc():
    found = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(found):
        raise RuntimeError('nvcc not found; libfga.so cannot be built')
    return found


def _stale():
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, '..', 'include', 'fga.h'))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source into libfga.so; returns its path."""
    if not force and not _stale():
        return OUT
    cmd = [_nvcc(), *FLAGS, *(['-Xptxas', '-v'] if verbose else []), '-o', OUT,
           *(os.path.join(CSRC, s) for s in SOURCES)]
    result = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError('nvcc failed while building libfga.so')
    return OUT


if __name__ == '__main__':
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    args = ap.parse_args()
    print(build(args.force, args.verbose))
