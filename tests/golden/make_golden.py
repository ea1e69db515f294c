"""Generates the golden fixtures in this folder from the reference itself.

Run in a container where the reference tree is mounted:

    make -C oracle            # builds oracle/_ref/philox_ref from the reference's philox.h
    python tests/golden/make_golden.py --reference /path/to/project_aether [--triton]

Outputs (committed):
  philox_kat.json     word 0 of the reference's Philox4x32-10 for several seeds/counters
                      (from oracle/_ref/philox_ref, i.e. the reference header compiled as is)
  replay_cases.npz    inputs and outputs of the reference's NumPy replay
                      `radix_sort_reference.onesweep_reference` on the shapes its own test
                      uses (tests/test_radix_sort.py:22-33), the look-back vector of
                      tests/test_radix_sort.py:36-43, and `num_passes` values
  push_cases.npz      inputs and outputs of the reference's unfused move stage
                      `fused_particle_push.reference_push` (CPU tensors) on seeded cases in
                      which particles leave the box through every face
  triton_interp.npz   (only with --triton) keys / permutation / counts produced by the
                      reference's two Triton kernels run by Triton's CPU interpreter on a
                      small case, with the host code of fused_radix_sort.py:244-279

The tests only read the fixtures; nothing at test time needs the reference tree.
"""

import argparse
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def philox_fixture():
    exe = os.path.join(ROOT, 'oracle', '_ref', 'philox_ref')
    cases = []
    for seed, first, count in [(1234, 0, 16), (0x100000007, 0, 8), (0, 0, 4),
                               (0xFFFFFFFFFFFFFFFF, 0xFFFFFFF0, 16),
                               (1234 ^ (4097 << 20), 1 << 20, 8),
                               (987654321, 123456789, 8)]:
        out = subprocess.run([exe, hex(seed), str(first), str(count)], check=True,
                             capture_output=True, text=True).stdout.split()
        cases.append({'seed': seed, 'first_counter': first,
                      'word0': [int(v) for v in out]})
    with open(os.path.join(HERE, 'philox_kat.json'), 'w') as f:
        json.dump({'source': 'project_aether/src/custom_kernels/cuda/philox.h compiled with g++',
                   'cases': cases}, f, indent=1)


def replay_fixture(ref):
    out = {}
    shapes = [(5000, 10_000), (12_345, 300), (1, 7), (2048, 1), (4096, 16_384)]
    out['shapes'] = np.array(shapes, np.int64)
    for i, (n, cells) in enumerate(shapes):
        rng = np.random.default_rng(n)
        keys = ((rng.integers(0, cells, n) << ref.SHUFFLE_BITS) |
                rng.integers(0, 1 << ref.SHUFFLE_BITS, n)).astype(np.int32)
        values = np.arange(n, dtype=np.int32)
        sk, sv = ref.onesweep_reference(keys, values, ref.num_passes(cells), rng, tile=256)
        out[f'keys_{i}'] = keys
        out[f'sorted_keys_{i}'] = sk
        out[f'sorted_values_{i}'] = sv
    status = np.zeros((4, ref.RADIX), np.int64)
    hist = np.arange(4 * ref.RADIX).reshape(4, ref.RADIX) % 5
    status[0] = hist[0] | ref.FLAG_INCLUSIVE
    status[1] = (hist[0] + hist[1]) | ref.FLAG_INCLUSIVE
    status[2] = hist[2] | ref.FLAG_AGGREGATE
    out['lookback_status'] = status
    out['lookback_exclusive'] = ref._lookback(status, 3)
    cells_list = [1, 2, 7, 128, 300, 10_000, 16_384, 262_144, 2_097_152, 1 << 24]
    out['num_passes_cells'] = np.array(cells_list, np.int64)
    out['num_passes'] = np.array([ref.num_passes(c) for c in cells_list], np.int64)
    np.savez_compressed(os.path.join(HERE, 'replay_cases.npz'), **out)


def push_fixture():
    """The move stage as the reference states it in plain PyTorch
    (fused_particle_push.py:95-108), run on CPU tensors."""
    import torch
    from src.custom_kernels.triton.fused_particle_push import reference_push
    out = {}
    specs = [
        # name, n, lo, hi, dt, velocity scale
        ('unit_box', 1024, (0.0, 0.0, 0.0), (1.0, 1.0, 1.0), 0.05, 4.0),
        ('offset_box', 1001, (0.1, -0.2, 0.0), (1.0, 1.0, 0.64), 0.02, 30.0),
        ('tiny_step', 512, (0.0, 0.0, 0.0), (1.0, 1.0, 1.0), 8.2e-5, 1.0),
    ]
    for name, n, lo, hi, dt, scale in specs:
        gen = torch.Generator().manual_seed(len(name) + n)
        pos = [(torch.rand(n, generator=gen) * (h - l) + l).to(torch.float32)
               for l, h in zip(lo, hi)]
        vel = [(torch.randn(n, generator=gen) * scale).to(torch.float32) for _ in range(3)]
        # Particles exactly on the faces, and fast ones that overshoot the opposite wall.
        for axis in range(3):
            pos[axis][axis] = lo[axis]
            pos[axis][3 + axis] = hi[axis]
            vel[axis][6 + axis] = 3.0 * (hi[axis] - lo[axis]) / dt
            vel[axis][9 + axis] = -3.0 * (hi[axis] - lo[axis]) / dt
        new_pos, new_vel = reference_push(pos, vel, dt, lo, hi)
        moved = torch.stack(new_pos)
        assert all(bool(((torch.stack(pos)[a] + torch.stack(vel)[a] * dt) < lo[a]).any()) and
                   bool(((torch.stack(pos)[a] + torch.stack(vel)[a] * dt) > hi[a]).any())
                   for a in range(3)), 'every face must be hit'
        out[name + '/pos_in'] = torch.stack(pos).numpy()
        out[name + '/vel_in'] = torch.stack(vel).numpy()
        out[name + '/scalars'] = np.array([dt, *lo, *hi], np.float64)
        out[name + '/pos_out'] = moved.numpy()
        out[name + '/vel_out'] = torch.stack(new_vel).numpy()
    np.savez_compressed(os.path.join(HERE, 'push_cases.npz'), **out)


def triton_fixture(ref_root):
    os.environ['TRITON_INTERPRET'] = '1'
    import torch
    import triton
    from src.custom_kernels.triton import fused_radix_sort as frs
    from src.custom_kernels.triton import radix_sort_reference as ref
    cases = {}
    specs = [
        ('unit', 3000, ref.CellGrid((0., 0., 0.), (1., 1., 0.64), (25, 25, 16)), 1234),
        ('offset', 2500, ref.CellGrid((0.1, -0.2, 0.), (1., 1., 0.64), (37, 25, 16)),
         0x138800007),
    ]
    for name, n, grid, seed in specs:
        gen = torch.Generator().manual_seed(7)
        pos = [torch.rand(n, generator=gen) * (h - l) * 1.1 + l - 0.05 * (h - l)
               for l, h in zip(grid.lo, grid.hi)]
        pos = [p.to(torch.float32) for p in pos]
        # A few positions exactly on the faces.
        pos[0][:4] = torch.tensor([grid.lo[0], grid.hi[0], grid.lo[0], grid.hi[0]])
        x, y, z = pos
        passes = ref.num_passes(grid.num_cells)
        keys = torch.empty(n, dtype=torch.int32)
        values = torch.empty(n, dtype=torch.int32)
        hist = torch.zeros(ref.MAX_PASSES * ref.RADIX, dtype=torch.int32)
        tiles = triton.cdiv(n, ref.TILE)
        inv = [c / (h - l) for l, h, c in zip(grid.lo, grid.hi, grid.cells)]
        frs._bin_keys_kernel[(tiles,)](
            x, y, z, keys, values, hist, n, *grid.lo, *inv, *grid.cells, seed,
            NUM_PASSES=passes, SHUFFLE=ref.SHUFFLE_BITS, PASS_PAD=ref.MAX_PASSES,
            SUB=ref.SUBTILE, SUBTILES=ref.SUBTILES_PER_TILE, RADIX_C=ref.RADIX,
            RADIX_BITS_C=ref.RADIX_BITS, num_warps=4)
        unsorted_keys = keys.clone()
        keys_alt, values_alt = torch.empty_like(keys), torch.empty_like(values)
        counts = torch.zeros(grid.num_cells, dtype=torch.int32)
        status = torch.empty(tiles * ref.RADIX, dtype=torch.int32)
        counter = torch.empty(1, dtype=torch.int32)
        for p in range(passes):
            status.zero_()
            counter.zero_()
            frs._onesweep_kernel[(tiles,)](
                keys, values, keys_alt, values_alt, hist, status, counter, counts, n, p,
                ref.SHUFFLE_BITS, IS_LAST=p == passes - 1, SUB=ref.SUBTILE,
                SUBTILES=ref.SUBTILES_PER_TILE, RADIX_C=ref.RADIX,
                RADIX_BITS_C=ref.RADIX_BITS, FLAG_AGG=ref.FLAG_AGGREGATE,
                FLAG_INC=ref.FLAG_INCLUSIVE, FLAG_BITS=ref.FLAG_MASK,
                VALUE_BITS=ref.VALUE_MASK, num_warps=8)
            keys, keys_alt = keys_alt, keys
            values, values_alt = values_alt, values
        start = torch.zeros(grid.num_cells + 1, dtype=torch.int32)
        start[1:] = torch.cumsum(counts, 0)
        cases[f'{name}_grid'] = np.array(list(grid.lo) + list(grid.hi) + list(grid.cells),
                                         np.float64)
        cases[f'{name}_seed'] = np.array([seed], np.uint64)
        for k, v in (('x', x), ('y', y), ('z', z), ('unsorted_keys', unsorted_keys),
                     ('keys', keys), ('index', values), ('counts', counts), ('start', start)):
            cases[f'{name}_{k}'] = v.numpy()
    cases['triton_version'] = np.array([triton.__version__])
    np.savez_compressed(os.path.join(HERE, 'triton_interp.npz'), **cases)


def collide_fixture():
    """Runs the reference's own inline collision functions (harness oracle/_ref/collide_ref,
    built from dsmc_collide_tma.h) on small seeded cases and stores inputs and outputs."""
    import tempfile
    sys.path.insert(0, ROOT)
    from oracle import collide_oracle
    exe = os.path.join(ROOT, 'oracle', '_ref', 'collide_ref')
    rng = np.random.default_rng(7)
    specs = {
        # Poisson occupancy with an oversized cell, as dsmc_collide_tma_test.cu:86-96 (smaller).
        # The selection factor of that test (2e-17) selects no pair at all with its majorant
        # (expected pairs per cell 2.7e-28); these cases use factors that select some.
        'poisson_300': dict(counts=np.r_[rng.poisson(300.0, 20), 3000], rng_seed=1,
                            selection_factor=2.0e12),
        # DSMC-like small cells, empty cells, single particles, odd counts; a 64-bit step and seed.
        'small_cells': dict(counts=np.r_[rng.poisson(12.0, 300), 0, 0, 1, 2, 3, 0, 5],
                            rng_seed=2, selection_factor=1.0e14, seed=0x1234567890abcdef,
                            step=(1 << 32) + 5),
        # High majorant use: most candidates are accepted; a raised majorant appears.
        'dense_accept': dict(counts=rng.poisson(40.0, 100), rng_seed=3, selection_factor=2.0e15,
                             majorant=2.0e-17),
    }
    out = {}
    for name, kw in specs.items():
        case = collide_oracle.make_case(**kw)
        with tempfile.TemporaryDirectory() as tmp:
            fin, fout = os.path.join(tmp, 'in.bin'), os.path.join(tmp, 'out.bin')
            with open(fin, 'wb') as f:
                f.write(np.array([case.sigma_g_max.size, case.velocity.shape[1]], np.int32).tobytes())
                f.write(np.array([case.selection_factor, case.coefficient, case.exponent],
                                 np.float32).tobytes())
                f.write(np.array([case.seed, case.step], np.uint64).tobytes())
                f.write(case.cell_start.tobytes())
                f.write(case.sigma_g_max.tobytes())
                f.write(case.velocity.tobytes())
            subprocess.run([exe, fin, fout], check=True)
            raw = open(fout, 'rb').read()
        nv, c = case.velocity.size, case.sigma_g_max.size
        out[name + '/velocity_in'] = case.velocity
        out[name + '/cell_start'] = case.cell_start
        out[name + '/sigma_in'] = case.sigma_g_max
        out[name + '/scalars'] = np.array([case.selection_factor, case.coefficient, case.exponent],
                                          np.float32)
        out[name + '/seed_step'] = np.array([case.seed, case.step], np.uint64)
        out[name + '/velocity_out'] = np.frombuffer(raw, np.float32, nv).reshape(3, -1)
        out[name + '/sigma_out'] = np.frombuffer(raw, np.float32, c, offset=4 * nv)
        out[name + '/collisions'] = np.frombuffer(raw, np.int32, c, offset=4 * (nv + c))
    np.savez_compressed(os.path.join(HERE, 'collide_cases.npz'), **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True,
                    help='the project_aether folder of a mounted reference tree')
    ap.add_argument('--triton', action='store_true')
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from src.custom_kernels.triton import radix_sort_reference as ref
    philox_fixture()
    replay_fixture(ref)
    collide_fixture()
    push_fixture()
    if args.triton:
        triton_fixture(args.reference)


if __name__ == '__main__':
    main()
