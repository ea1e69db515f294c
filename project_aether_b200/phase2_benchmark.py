"""Binning-stage benchmark: the B200 sort against a multi-threaded CPU pipeline.

Command-line counterpart of the reference's benchmark
(project_aether/scripts/phase2_triton_sort_benchmark.py).  It keeps that
script's argument names (:139-148), its default case (4 M uniform particles in
a 1 x 1 x 0.64 box of 25 x 25 x 16 cells, :150-157) and its definition of the
CPU baseline (:44-59: cell ids, Mersenne-Twister shuffle bits, a stable sort and
a bincount in PyTorch on `--cpu-threads` threads); both pipelines must produce
the same per-cell counts (:161-162).  Measuring and reporting are this
package's own: every pipeline is a `Pipeline` with a `step(i)` callable, timed
by one routine (wall clock for the host pipeline, CUDA events for the device
one), and the report is built from the list of measurements.

With --collisions the collision kernel runs on the sorted particles, as the
reference does (:87-135), and the mean number of accepted pairs per cell is
printed.  The reference compares that mean with its JAX implementation of the
NTC algorithm; JAX is not part of this package, so the statistics are reported
and left to the caller to compare (`run` returns them together with the
kernel's inputs).

    python -m project_aether_b200.phase2_benchmark --cpu-threads 32
"""

import argparse
import dataclasses
import math
import time
from typing import Callable, List, Optional

import numpy as np
import torch

from . import ntc_collide, particle_sort
from .cell_grid import SHUFFLE_BITS, CellGrid, num_passes

BOLTZMANN = ntc_collide.BOLTZMANN
# Single-species VHS model of air (Bird 1994, Table A1), the defaults of the reference's
# GasModel (project_aether/src/physics_engine/dsmc_boltzmann.py:61-75).
GAS_MASS, GAS_D_REF, GAS_OMEGA, GAS_T_REF = 48.1e-27, 4.19e-10, 0.77, 273.0
GAS_TEMPERATURE = 3000.0
GPU_WARMUP_CALLS = 5  # the GPU idles through the host measurement; bring its clocks back up


def cpu_binning(x, y, z, grid: CellGrid, generator: torch.Generator):
    """The CPU baseline as the reference defines it
    (phase2_triton_sort_benchmark.py:44-59): unfused cell ids, shuffle bits from
    torch's host generator, `torch.sort(stable=True)`, `torch.bincount`.
    Returns (sorted keys, permutation, per-cell counts)."""
    axes = []
    for coord, low, high, cells in zip((x, y, z), grid.lo, grid.hi, grid.cells):
        scaled = (coord - low) * (cells / (high - low))
        axes.append(scaled.to(torch.int32).clamp_(0, cells - 1))
    cell = (axes[2] * grid.cells[1] + axes[1]) * grid.cells[0] + axes[0]
    bits = torch.randint(0, 1 << SHUFFLE_BITS, cell.shape, generator=generator, dtype=torch.int32)
    sorted_keys, order = torch.sort((cell << SHUFFLE_BITS) | bits, stable=True)
    return sorted_keys, order, torch.bincount(cell, minlength=grid.num_cells)


@dataclasses.dataclass
class Pipeline:
    """One way of binning the particles: `step(i)` runs call number i and returns its result."""
    label: str
    step: Callable[[int], object]
    on_device: bool
    warmup: int


@dataclasses.dataclass
class Measurement:
    label: str
    seconds_per_step: float
    last_result: object


def measure(pipeline: Pipeline, repeats: int) -> Measurement:
    """Mean time of `repeats` back-to-back calls after the pipeline's warm-up calls."""
    result = None
    for i in range(pipeline.warmup):
        result = pipeline.step(i)
    if pipeline.on_device:
        torch.cuda.synchronize()
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
    else:
        begun = time.perf_counter()
    for i in range(repeats):
        result = pipeline.step(pipeline.warmup + i)
    if pipeline.on_device:
        last.record()
        torch.cuda.synchronize()
        seconds = first.elapsed_time(last) * 1e-3
    else:
        seconds = time.perf_counter() - begun
    return Measurement(pipeline.label, seconds / repeats, result)


@dataclasses.dataclass
class CollisionStatistics:
    """Inputs and outputs of the collision kernel run by --collisions."""
    velocity_before: np.ndarray   # (3, padded) sorted velocities handed to the kernel
    cell_start: np.ndarray        # (cells + 1,)
    sigma_g_max: np.ndarray       # (cells,) majorant handed to the kernel
    params: ntc_collide.CollisionParams
    collisions: np.ndarray        # (cells,) accepted pairs per cell


def collision_statistics(args, grid: CellGrid, order) -> CollisionStatistics:
    """Runs the collision kernel once on thermal velocities put in the sorted order."""
    n = args.particles
    thermal = math.sqrt(BOLTZMANN * GAS_TEMPERATURE / GAS_MASS)
    velocities = np.random.default_rng(1).normal(0.0, thermal, (n, 3)).astype(np.float32)
    coefficient, exponent = ntc_collide.vhs_parameters(GAS_MASS, GAS_D_REF, GAS_OMEGA, GAS_T_REF)
    majorant = np.full(grid.num_cells, coefficient * (4.0 * thermal) ** exponent, np.float32)
    cell_volume = math.prod((h - l) / c for l, h, c in zip(grid.lo, grid.hi, grid.cells))
    params = ntc_collide.CollisionParams(args.fnum * args.dt / cell_volume, coefficient, exponent,
                                         7, 0)
    device = order.keys.device
    padded = -(-n // 4) * 4
    velocity = torch.zeros((3, padded), dtype=torch.float32, device=device)
    permutation = order.particle_index.long().cpu().numpy()
    velocity[:, :n] = torch.as_tensor(np.ascontiguousarray(velocities[permutation].T),
                                      device=device)
    before = velocity.cpu().numpy()
    sigma = torch.as_tensor(majorant, device=device)
    accepted = torch.zeros(grid.num_cells, dtype=torch.int32, device=device)
    library = ntc_collide.load_library(args.cuda_library)
    ntc_collide.collide(library, velocity, order.cell_start, sigma, accepted, n, params)
    return CollisionStatistics(before, order.cell_start.cpu().numpy(), majorant, params,
                               accepted.cpu().numpy())


def render_table(rows, headers) -> str:
    try:
        import tabulate
        return tabulate.tabulate(rows, headers=headers, tablefmt='github')
    except ImportError:
        widths = [max(len(str(r[i])) for r in [headers] + rows) for i in range(len(headers))]
        lines = ['| ' + ' | '.join(str(c).ljust(w) for c, w in zip(r, widths)) + ' |'
                 for r in [headers] + rows]
        lines.insert(1, '|' + '|'.join('-' * (w + 2) for w in widths) + '|')
        return '\n'.join(lines)


@dataclasses.dataclass
class Report:
    measurements: List[Measurement]
    counts_match: bool
    collisions: Optional[CollisionStatistics]
    text: str


def parse_arguments(argv=None):
    # Argument names and defaults of the reference's script (:139-148).
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument('--particles', type=int, default=4_000_000)
    parser.add_argument('--cells', type=int, nargs=3, default=(25, 25, 16))
    parser.add_argument('--cpu-threads', type=int, default=32)
    parser.add_argument('--repeats', type=int, default=5)
    parser.add_argument('--collisions', action='store_true')
    parser.add_argument('--cuda-library', default=None)
    parser.add_argument('--dt', type=float, default=1e-6)
    parser.add_argument('--fnum', type=float, default=1e12)
    return parser.parse_args(argv)


def run(argv=None) -> Report:
    args = parse_arguments(argv)
    if not torch.cuda.is_available():
        raise SystemExit('This benchmark needs a CUDA GPU.')
    grid = CellGrid((0.0, 0.0, 0.0), (1.0, 1.0, 0.64), tuple(args.cells))
    n = args.particles
    draw = torch.Generator(device='cuda').manual_seed(0)
    device_positions = [torch.rand(n, device='cuda', generator=draw) * extent for extent in grid.hi]
    host_positions = [p.cpu() for p in device_positions]
    host_bits = torch.Generator().manual_seed(0)
    torch.set_num_threads(args.cpu_threads)
    pipelines = [
        Pipeline(f'CPU baseline ({args.cpu_threads} threads)',
                 lambda i: cpu_binning(*host_positions, grid, host_bits), False, 1),
        Pipeline('B200 sort (GPU)',
                 lambda i: particle_sort.sort_particles_by_cell(*device_positions, grid, i + 1),
                 True, GPU_WARMUP_CALLS),
    ]
    measured = [measure(p, args.repeats) for p in pipelines]
    host, device = measured
    counts_match = torch.equal(host.last_result[2].to(torch.int32),
                               device.last_result.cell_counts.cpu())
    rows = [[m.label, f'{m.seconds_per_step * 1e3:.3f}', f'{n / m.seconds_per_step / 1e6:.1f}',
             f'{host.seconds_per_step / m.seconds_per_step:.1f}x'] for m in measured]
    lines = [f'{n:,} particles, {grid.num_cells:,} cells, '
             f'{num_passes(grid.num_cells)} digit passes',
             render_table(rows, ['Pipeline', 'ms / step', 'M particles / s', 'Speedup']),
             f'Per-cell counts identical: {counts_match}']
    statistics = None
    if args.collisions:
        statistics = collision_statistics(args, grid, device.last_result)
        lines.append(f'Mean collisions per cell: GPU {statistics.collisions.mean():.3f} '
                     f'({int(statistics.collisions.sum())} accepted pairs in '
                     f'{grid.num_cells:,} cells).')
    return Report(measured, counts_match, statistics, '\n'.join(lines))


def main(argv=None) -> int:
    report = run(argv)
    print(report.text)
    return 0 if report.counts_match else 1


if __name__ == '__main__':
    raise SystemExit(main())
