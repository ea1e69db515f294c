"""Seeded synthetic particle states for the benchmark and parity configurations.

The reference measures its sort on synthetic uniform particles drawn with a
torch generator (project_aether/scripts/phase2_triton_sort_benchmark.py:152-157,
project_aether/tests/test_radix_sort.py:69-70); the five configurations here
keep that protocol and add the shapes and distributions of the benchmark
definition (uniform, drifting Maxwellian, hypersonic-like density with a shock
layer and a body shadow, large uniform, steady-state re-sort).
"""

import math
from typing import NamedTuple, Tuple

import torch

from .cell_grid import CellGrid


class Workload(NamedTuple):
    name: str
    n: int
    grid: CellGrid
    density: str  # 'uniform' or 'hypersonic'
    drift: float  # added to vx, in units of sigma


UNIT = ((0.0, 0.0, 0.0), (1.0, 1.0, 1.0))
WORKLOADS = {
    'c1_1m_64': Workload('c1_1m_64', 1 << 20, CellGrid(*UNIT, (64, 64, 64)), 'uniform', 0.0),
    'c2_16m_128': Workload('c2_16m_128', 1 << 24, CellGrid(*UNIT, (128, 128, 128)), 'uniform', 5.0),
    'c3_64m_hypersonic': Workload('c3_64m_hypersonic', 1 << 26,
                                  CellGrid(*UNIT, (256, 128, 128)), 'hypersonic', 0.0),
    'c4_256m_512': Workload('c4_256m_512', 1 << 28, CellGrid(*UNIT, (512, 256, 256)), 'uniform', 0.0),
    'c5_128m_256': Workload('c5_128m_256', 1 << 27, CellGrid(*UNIT, (256, 256, 256)), 'uniform', 0.0),
}

# Unnormalised piecewise density along x of the hypersonic-like case: free
# stream, a 6x shock layer of width 0.05 at x = 0.4, a body on [0.5, 0.7] with no
# particles, and an exponentially decaying wake behind it.
_WAKE_LENGTH = 0.1
_SEGMENTS = ((0.0, 0.4, 1.0), (0.4, 0.45, 6.0), (0.45, 0.5, 1.0))
_WAKE_START, _WAKE_END = 0.7, 1.0


def hypersonic_x(u: torch.Tensor) -> torch.Tensor:
    """Inverse CDF of the piecewise density, u uniform in [0, 1), in float64."""
    wake_mass = _WAKE_LENGTH * (1.0 - math.exp(-(_WAKE_END - _WAKE_START) / _WAKE_LENGTH))
    total = sum((b - a) * r for a, b, r in _SEGMENTS) + wake_mass
    m = u.to(torch.float64) * total
    x = torch.empty_like(m)
    done = torch.zeros_like(m, dtype=torch.bool)
    acc = 0.0
    for a, b, r in _SEGMENTS:
        mass = (b - a) * r
        sel = (~done) & (m < acc + mass)
        x = torch.where(sel, a + (m - acc) / r, x)
        done |= sel
        acc += mass
    t = ((m - acc) / _WAKE_LENGTH).clamp(0.0, wake_mass / _WAKE_LENGTH * (1 - 1e-12))
    x = torch.where(done, x, _WAKE_START - _WAKE_LENGTH * torch.log1p(-t))
    return x


def make_particles(w: Workload, device, seed: int = 0, n: int = None, padded: int = None
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(x, y, z, velocity(3, padded)) float32 on `device`, drawn with a generator
    seeded with `seed` on that device."""
    n = w.n if n is None else n
    padded = -(-n // 4) * 4 if padded is None else padded
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    lo, hi = w.grid.lo, w.grid.hi
    pos = []
    for axis in range(3):
        u = torch.rand(n, device=device, generator=gen, dtype=torch.float32)
        if axis == 0 and w.density == 'hypersonic':
            u64 = torch.rand(n, device=device, generator=gen, dtype=torch.float64)
            u = hypersonic_x(u64).to(torch.float32).clamp_(max=0.99999994)
        pos.append((u * (hi[axis] - lo[axis]) + lo[axis]).to(torch.float32))
    velocity = torch.zeros((3, padded), dtype=torch.float32, device=device)
    velocity[:, :n] = torch.randn((3, n), device=device, generator=gen, dtype=torch.float32)
    if w.drift:
        velocity[0, :n] += w.drift
    return pos[0], pos[1], pos[2], velocity


def scaled_workload(name: str, log2n: int) -> Workload:
    """A configuration scaled to 2**log2n particles at the same number of particles per cell:
    the grid keeps its x and y extent and its z extent shrinks (or grows) with the particle
    count.  For parity cases and profiler captures smaller than the full configuration."""
    w = WORKLOADS[name]
    n = 1 << log2n
    nx, ny, nz = w.grid.cells
    nz = max(1, nz * n // w.n)
    return w._replace(n=n, grid=CellGrid(w.grid.lo, w.grid.hi, (nx, ny, nz)))


def step_seed(run_seed: int, step: int) -> int:
    """Philox key of a timestep (dsmc_gpu_pipeline.py:106)."""
    return run_seed ^ (step << 20)
