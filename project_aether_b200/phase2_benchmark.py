"""Binning-stage benchmark: the B200 sort against a multi-threaded CPU pipeline.

Mirror of the reference's command-line benchmark
(project_aether/scripts/phase2_triton_sort_benchmark.py): same case (4 M
particles in a 1 x 1 x 0.64 box of 25 x 25 x 16 cells by default), same CPU
baseline (cell ids, Mersenne-Twister shuffle bits, stable sort, bincount in
PyTorch on T threads, :44-70), same timing protocol (:73-84), same table and
the same per-cell-count check (:161-176).

With --collisions it runs the collision kernel on the sorted particles as the
reference does (:87-135).  The reference compares the mean number of collisions
per cell with its JAX implementation of the NTC algorithm; JAX is not part of
this package, so the comparison here is with a CPU replay of the kernel's own
algorithm when the test oracle is importable, and is skipped otherwise.

    python -m project_aether_b200.phase2_benchmark --cpu-threads 32
"""

import argparse
import math
import time

import numpy as np
import torch

from . import ntc_collide, particle_sort
from .cell_grid import SHUFFLE_BITS, CellGrid, num_passes

BOLTZMANN = ntc_collide.BOLTZMANN
# Single-species VHS model of air (Bird 1994, Table A1), the defaults of the reference's
# GasModel (project_aether/src/physics_engine/dsmc_boltzmann.py:61-75).
GAS_MASS, GAS_D_REF, GAS_OMEGA, GAS_T_REF = 48.1e-27, 4.19e-10, 0.77, 273.0


def cpu_binning(x, y, z, grid: CellGrid, generator: torch.Generator):
    """Unfused CPU pipeline: cell ids, MT19937 shuffle bits, stable sort, counts
    (phase2_triton_sort_benchmark.py:44-59)."""
    nx, ny, _ = grid.cells
    index = []
    for c, l, h, n in zip((x, y, z), grid.lo, grid.hi, grid.cells):
        index.append(((c - l) * (n / (h - l))).to(torch.int32).clamp_(0, n - 1))
    cell = (index[2] * ny + index[1]) * nx + index[0]
    shuffle = torch.randint(0, 1 << SHUFFLE_BITS, cell.shape, generator=generator,
                            dtype=torch.int32)
    keys = (cell << SHUFFLE_BITS) | shuffle
    sorted_keys, order = torch.sort(keys, stable=True)
    return sorted_keys, order, torch.bincount(cell, minlength=grid.num_cells)


def time_cpu(args, positions, grid):
    torch.set_num_threads(args.cpu_threads)
    generator = torch.Generator().manual_seed(0)
    x, y, z = (p.cpu() for p in positions)
    cpu_binning(x, y, z, grid, generator)  # warm up
    start = time.perf_counter()
    for _ in range(args.repeats):
        _, _, counts = cpu_binning(x, y, z, grid, generator)
    return (time.perf_counter() - start) / args.repeats, counts


def time_gpu(args, positions, grid):
    # The GPU has idled through the CPU measurement: a few warm-up calls (the reference makes
    # one) bring its clocks back up before the timed ones.
    for _ in range(5):
        result = particle_sort.sort_particles_by_cell(*positions, grid, 1)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for step in range(args.repeats):
        result = particle_sort.sort_particles_by_cell(*positions, grid, step + 2)
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / 1e3 / args.repeats, result


def check_collision_statistics(args, grid, result) -> str:
    """Collision kernel on the sorted particles (phase2_triton_sort_benchmark.py:87-135)."""
    n = args.particles
    rng = np.random.default_rng(1)
    thermal = math.sqrt(BOLTZMANN * 3000.0 / GAS_MASS)
    vel = rng.normal(0.0, thermal, (n, 3)).astype(np.float32)
    index = result.particle_index.long().cpu().numpy()
    vel_sorted = vel[index]
    coefficient, exponent = ntc_collide.vhs_parameters(GAS_MASS, GAS_D_REF, GAS_OMEGA, GAS_T_REF)
    g_ref = 4.0 * thermal
    sigma_g = coefficient * g_ref ** exponent
    majorant = np.full((grid.num_cells,), sigma_g, np.float32)
    cell_volume = float(np.prod([(h - l) / c for l, h, c in zip(grid.lo, grid.hi, grid.cells)]))
    library = ntc_collide.load_library(args.cuda_library)
    padded = -(-n // 4) * 4
    device = result.keys.device
    velocity = torch.zeros((3, padded), dtype=torch.float32, device=device)
    velocity[:, :n] = torch.as_tensor(np.ascontiguousarray(vel_sorted.T), device=device)
    host_velocity = velocity.cpu().numpy()
    sigma = torch.as_tensor(majorant, device=device)
    collisions = torch.zeros(grid.num_cells, dtype=torch.int32, device=device)
    params = ntc_collide.CollisionParams(args.fnum * args.dt / cell_volume, coefficient, exponent,
                                         7, 0)
    ntc_collide.collide(library, velocity, result.cell_start, sigma, collisions, n, params)
    gpu = collisions.cpu().numpy().astype(np.float64)
    line = f'Mean collisions per cell: GPU {gpu.mean():.3f}'
    try:  # the CPU replay is test infrastructure; it is not shipped with the package
        from oracle import collide_oracle
    except ImportError:
        return line + ' (no CPU replay available to compare with).'
    case = collide_oracle.CollideCase(host_velocity, result.cell_start.cpu().numpy(), majorant,
                                      params.selection_factor, coefficient, exponent, 7, 0)
    ref = collide_oracle.collide(case)[2].astype(np.float64)
    spread = math.sqrt((gpu.var() + ref.var()) / grid.num_cells)
    z = abs(gpu.mean() - ref.mean()) / spread if spread > 0 else 0.0
    return (line + f', CPU replay of the same algorithm {ref.mean():.3f} (z = {z:.2f}; |z| < 3 '
            f'means agreement within stochastic noise; {int((gpu != ref).sum())} of '
            f'{grid.num_cells} cells differ).')


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


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument('--particles', type=int, default=4_000_000)
    parser.add_argument('--cells', type=int, nargs=3, default=(25, 25, 16))
    parser.add_argument('--cpu-threads', type=int, default=32)
    parser.add_argument('--repeats', type=int, default=5)
    parser.add_argument('--collisions', action='store_true')
    parser.add_argument('--cuda-library', default=None)
    parser.add_argument('--dt', type=float, default=1e-6)
    parser.add_argument('--fnum', type=float, default=1e12)
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit('This benchmark needs a CUDA GPU.')

    grid = CellGrid((0.0, 0.0, 0.0), (1.0, 1.0, 0.64), tuple(args.cells))
    gen = torch.Generator(device='cuda').manual_seed(0)
    scale = torch.tensor(grid.hi, device='cuda')
    positions = [torch.rand(args.particles, device='cuda', generator=gen) * scale[i]
                 for i in range(3)]

    cpu_seconds, cpu_counts = time_cpu(args, positions, grid)
    gpu_seconds, result = time_gpu(args, positions, grid)
    counts_match = torch.equal(cpu_counts.to(torch.int32), result.cell_counts.cpu())
    rows = [
        [f'CPU baseline ({args.cpu_threads} threads)', f'{cpu_seconds * 1e3:.2f}',
         f'{args.particles / cpu_seconds / 1e6:.1f}', '1.0x'],
        ['B200 sort (GPU)', f'{gpu_seconds * 1e3:.3f}',
         f'{args.particles / gpu_seconds / 1e6:.1f}', f'{cpu_seconds / gpu_seconds:.1f}x'],
    ]
    print(f'{args.particles:,} particles, {grid.num_cells:,} cells, '
          f'{num_passes(grid.num_cells)} digit passes')
    print(render_table(rows, ['Pipeline', 'ms / step', 'M particles / s', 'Speedup']))
    print(f'Per-cell counts identical: {counts_match}')
    if args.collisions:
        print(check_collision_statistics(args, grid, result))
    return 0 if counts_match else 1


if __name__ == '__main__':
    raise SystemExit(main())
