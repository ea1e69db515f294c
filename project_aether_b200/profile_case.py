"""Runs a few sort calls on a small seeded case, for profiling under ncu.

    python -m project_aether_b200.profile_case --workload c3_64m_hypersonic --log2n 24 --calls 2
    python -m project_aether_b200.profile_case --workload c5_128m_256 --log2n 24 --calls 2 --collide
    python -m project_aether_b200.profile_case --log2n 24 --calls 2 --path digits
    python -m project_aether_b200.profile_case --log2n 24 --calls 1 --extras

The case keeps the workload's grid shape but scales the z extent of the grid
with the particle count so that particles per cell stay what the full
configuration has; inputs stay larger than L2 from 2^23 particles on.
"""

import argparse

import torch

from . import particle_sort, workloads
from .cell_grid import CellGrid


def scaled_case(name: str, log2n: int):
    w = workloads.WORKLOADS[name]
    n = 1 << log2n
    nx, ny, nz = w.grid.cells
    nz = max(1, nz * n // w.n)
    grid = CellGrid(w.grid.lo, w.grid.hi, (nx, ny, nz))
    return w._replace(n=n, grid=grid)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--workload', default='c3_64m_hypersonic')
    ap.add_argument('--log2n', type=int, default=24)
    ap.add_argument('--calls', type=int, default=2)
    ap.add_argument('--path', default='auto', choices=['auto', 'digits'])
    ap.add_argument('--extras', action='store_true',
                    help='also run the move stage and the 8-way slab partition once per call')
    ap.add_argument('--collide', action='store_true',
                    help='also run the collision stage on the sorted output of every call')
    args = ap.parse_args()
    w = scaled_case(args.workload, args.log2n)
    device = torch.device('cuda', 0)
    x, y, z, v = workloads.make_particles(w, device, seed=0)
    path = particle_sort.PATH_AUTO if args.path == 'auto' else particle_sort.PATH_DIGIT_PASSES
    if args.collide:
        # Unit thermal speed: sigma*g = g^0.46 below the majorant 3; about one candidate pair
        # per two cells at 8 particles per cell.
        from . import ntc_collide
        lib = ntc_collide.load_library()
        sigma_g_max = torch.full((w.grid.num_cells,), 3.0, dtype=torch.float32, device=device)
        collisions = torch.zeros(w.grid.num_cells, dtype=torch.int32, device=device)
    for s in range(args.calls):
        out = particle_sort.sort_and_gather_particles(x, y, z, v, w.grid, workloads.step_seed(1234, s),
                                                      path=path)
        if args.extras:
            from . import particle_push, slab_sort
            moved = [t.clone() for t in (x, y, z, v)]
            particle_push.fused_particle_push(moved[:3], [moved[3][k, :w.n] for k in range(3)],
                                              8.2e-5, w.grid.lo, w.grid.hi)
            slab_sort.partition_by_slab(x, y, z, v, w.grid, 8)
        if args.collide:
            ntc_collide.collide(lib, out.velocity, out.order.cell_start, sigma_g_max, collisions,
                                w.n, ntc_collide.CollisionParams(0.006, 1.0, 0.46, 1234, s))
    torch.cuda.synchronize()
    status = particle_sort.last_sort_status(device)
    print(f'{w.name} n={w.n} cells={w.grid.cells} status={status} '
          f'max cell count={int(out.order.cell_counts.max())}')
    raise SystemExit(status)


if __name__ == '__main__':
    main()
