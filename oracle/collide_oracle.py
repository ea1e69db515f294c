"""NTC collision oracle: ctypes wrapper of collide_oracle.c plus case builders.

TEST INFRASTRUCTURE ONLY.  The arithmetic lives in collide_oracle.c (it needs
the C library's powf/sinf/cosf exactly as the reference's host replay uses
them, project_aether/src/custom_kernels/cuda/dsmc_collide_tma_test.cu:45-84);
this module loads it and builds the seeded cases the tests and the golden
fixture share.
"""

import ctypes
import os
import subprocess
from typing import NamedTuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class CollideCase(NamedTuple):
    velocity: np.ndarray       # (3, padded) float32
    cell_start: np.ndarray     # (C + 1,) int32
    sigma_g_max: np.ndarray    # (C,) float32
    selection_factor: float
    coefficient: float
    exponent: float
    seed: int
    step: int


def _clib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, 'libcollide_oracle.so')
        if not os.path.exists(path):  # a fresh checkout: build it (gcc, a second)
            subprocess.run(['make', '-C', _HERE, 'libcollide_oracle.so'], check=True,
                           capture_output=True)
        lib = ctypes.CDLL(path)
        lib.collide_cells.restype = None
        lib.collide_cells.argtypes = ([ctypes.c_void_p] * 4 + [ctypes.c_int32, ctypes.c_int64] +
                                      [ctypes.c_float] * 3 + [ctypes.c_uint64] * 2 + [ctypes.c_void_p])
        lib.collide_selections.restype = None
        lib.collide_selections.argtypes = ([ctypes.c_void_p] * 3 + [ctypes.c_int32, ctypes.c_float] +
                                           [ctypes.c_uint64] * 2)
        _LIB = lib
    return _LIB


def collide(case: CollideCase, want_pair_sigma: bool = False):
    """Returns (velocity, sigma_g_max, collisions[, pair_sigma_g]) after one collision step."""
    lib = _clib()
    velocity = np.array(case.velocity, dtype=np.float32, order='C', copy=True)
    sigma = np.array(case.sigma_g_max, dtype=np.float32, copy=True)
    start = np.ascontiguousarray(case.cell_start, dtype=np.int32)
    cells = sigma.size
    collisions = np.zeros(cells, dtype=np.int32)
    pair_sigma = np.zeros(velocity.shape[1], dtype=np.float32) if want_pair_sigma else None
    lib.collide_cells(velocity.ctypes.data, start.ctypes.data, sigma.ctypes.data,
                      collisions.ctypes.data, cells, velocity.shape[1],
                      np.float32(case.selection_factor), np.float32(case.coefficient),
                      np.float32(case.exponent), case.seed, case.step,
                      pair_sigma.ctypes.data if want_pair_sigma else None)
    if want_pair_sigma:
        return velocity, sigma, collisions, pair_sigma
    return velocity, sigma, collisions


def selections(case: CollideCase) -> np.ndarray:
    lib = _clib()
    start = np.ascontiguousarray(case.cell_start, dtype=np.int32)
    sigma = np.ascontiguousarray(case.sigma_g_max, dtype=np.float32)
    out = np.zeros(sigma.size, dtype=np.int32)
    lib.collide_selections(start.ctypes.data, sigma.ctypes.data, out.ctypes.data, sigma.size,
                           np.float32(case.selection_factor), case.seed, case.step)
    return out


def make_case(counts, rng_seed: int, thermal: float = 800.0, selection_factor: float = 2.0e12,
              coefficient: float = 1.7e-18, exponent: float = 0.46, majorant: float = 3.0e-16,
              seed: int = 0x5eedf00d, step: int = 7) -> CollideCase:
    """A seeded case with the given particles per cell.  Gas, thermal speed, majorant,
    seed and step default to the numbers of the reference's own kernel test
    (dsmc_collide_tma_test.cu:86-113: air-like VHS gas, 800 m/s thermal speed); the
    selection factor does not (that test's 2e-17 selects no pairs)."""
    counts = np.asarray(counts, dtype=np.int64)
    start = np.zeros(counts.size + 1, dtype=np.int32)
    start[1:] = np.cumsum(counts)
    n = int(start[-1])
    padded = -(-n // 4) * 4
    rng = np.random.default_rng(rng_seed)
    velocity = np.zeros((3, padded), dtype=np.float32)
    velocity[:, :n] = (rng.standard_normal((3, n)) * thermal).astype(np.float32)
    sigma = np.full(counts.size, majorant, dtype=np.float32)
    return CollideCase(velocity, start, sigma, selection_factor, coefficient, exponent, seed, step)
