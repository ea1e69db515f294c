"""Builds libaether_sort.so for sm_100a with nvcc, in the package folder.

    python -m project_aether_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (see include/aether_sort.h); it is
loaded with ctypes and needs no Python headers.
"""

import argparse
import os
import shutil
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, 'csrc')
LIB = os.path.join(PKG, 'libaether_sort.so')
SOURCES = ['api.cu', 'sort_standard.cu', 'sort_bucketed.cu', 'slab_partition.cu', 'particle_push.cu',
           'static_scratch.cu', 'collide.cu']
NVCC_FLAGS = [
    '-O3', '-std=c++17', '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo',
    '-Xcompiler', '-fPIC', '-shared', '--use_fast_math=false',
]


def _nvcc() -> str:
    for cand in (shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError('nvcc not found; the CUDA library cannot be built')


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(PKG), 'include', 'aether_sort.h'))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every CUDA source into libaether_sort.so; returns its path."""
    if not force and not _stale():
        return LIB
    flags = [f for f in NVCC_FLAGS if not f.startswith('--use_fast_math')]
    if verbose:
        flags += ['-Xptxas', '-v']
    cmd = [_nvcc(), *flags, '-ccbin', 'g++', '-o', LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        print(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError('nvcc failed:\n' + proc.stderr[-4000:])
    return LIB


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
