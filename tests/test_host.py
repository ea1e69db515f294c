"""Host-side logic and the C-ABI boundary, without a GPU: the library loads,
exports every symbol the header declares, and rejects bad arguments before it
would touch a device."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import project_aether_b200 as pa
from project_aether_b200 import _native, workloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_ERROR_INVALID_VALUE = 1


@pytest.fixture(scope='module')
def lib():
    from project_aether_b200 import build
    build.build()
    return _native.load_library()


def _declared_functions():
    text = open(os.path.join(ROOT, 'include', 'aether_sort.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(Aether[A-Za-z0-9_]+)\s*\(', text)))


def test_library_exports_every_declared_symbol(lib):
    declared = _declared_functions()
    assert declared, 'no declarations parsed from the header'
    for name in declared:
        assert hasattr(lib, name), f'{name} is declared but not exported'
    assert sorted(_native.exported_symbols()) == declared
    assert lib.AetherSortAbiVersion() >= 1


def test_workspace_query_is_pure_host_arithmetic(lib):
    small = lib.AetherSortWorkspaceBytes(1000, 10_000, 0)
    big = lib.AetherSortWorkspaceBytes(1 << 26, 1 << 22, 1)
    assert 0 < small < big
    assert big < 3 * (1 << 30)
    assert lib.AetherSortWorkspaceBytes(-1, 10, 0) == 0
    assert lib.AetherSortWorkspaceBytes(1 << 30, 10, 0) == 0
    assert lib.AetherSortWorkspaceBytes(10, 1 << 26, 0) == 0  # 33-bit keys
    assert lib.AetherSortWorkspaceBytes(10, 1 << 25, 0) > 0  # 32-bit keys fit


def test_bad_arguments_are_rejected_before_any_launch(lib):
    g = pa.particle_sort.native_grid(pa.CellGrid((0, 0, 0), (1, 1, 1), (4, 4, 4)))
    null = ctypes.c_void_p(None)
    fake = ctypes.c_void_p(256)  # never dereferenced: the checks fail first
    rc = lib.AetherSortParticlesByCell(fake, fake, fake, 8, None, 0, fake, fake, fake, fake,
                                       fake, 1 << 20, null)
    assert rc == CUDA_ERROR_INVALID_VALUE
    rc = lib.AetherSortParticlesByCell(fake, fake, fake, -5, ctypes.byref(g), 0, fake, fake,
                                       fake, fake, fake, 1 << 20, null)
    assert rc == CUDA_ERROR_INVALID_VALUE
    rc = lib.AetherSortParticlesByCell(fake, fake, fake, 8, ctypes.byref(g), 0, null, fake,
                                       fake, fake, fake, 1 << 20, null)
    assert rc == CUDA_ERROR_INVALID_VALUE
    bad = pa.particle_sort.native_grid(pa.CellGrid((0, 0, 0), (1, 1, 1), (4, 4, 4)),
                                       ix_offset=2, nx_local=4)
    rc = lib.AetherSortParticlesByCell(fake, fake, fake, 8, ctypes.byref(bad), 0, fake, fake,
                                       fake, fake, fake, 1 << 20, null)
    assert rc == CUDA_ERROR_INVALID_VALUE
    rc = lib.AetherGatherParticles(fake, 8, fake, fake, fake, fake, 4, fake, fake, fake, fake,
                                   8, null)  # padded < n
    assert rc == CUDA_ERROR_INVALID_VALUE
    rc = lib.AetherSortReadStatus(null, null, None)
    assert rc == CUDA_ERROR_INVALID_VALUE


def test_entry_point_rejects_cpu_tensors_like_the_reference():
    # fused_radix_sort.py:238-241
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (4, 4, 4))
    x = torch.zeros(8)
    with pytest.raises(ValueError, match='float32 CUDA tensors'):
        pa.sort_particles_by_cell(x, x, x, grid, 1)


def test_num_passes_and_key_width():
    assert pa.num_passes(10_000) == 3  # 14 + 7 = 21 bits -> three 8-bit digits
    assert pa.num_passes(1) == 1
    assert pa.num_passes(1 << 25) == 4  # 32-bit keys are accepted here
    with pytest.raises(ValueError):
        pa.num_passes((1 << 25) + 1)
    assert pa.key_bits(256 * 128 * 128) == 29
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 0.64), (25, 25, 16))
    assert grid.num_cells == 10_000


def test_native_grid_rounds_like_the_reference_driver():
    grid = pa.CellGrid((0.1, -0.2, 0.0), (1.0, 1.0, 0.64), (37, 25, 16))
    g = pa.particle_sort.native_grid(grid)
    assert g.inv_dx == np.float32(37 / (1.0 - 0.1))
    assert g.inv_dz == np.float32(16 / 0.64)
    assert g.x0 == np.float32(0.1)
    assert (g.nx_local, g.ix_offset) == (37, 0)


def test_workloads_are_seeded_and_shaped():
    w = workloads.WORKLOADS['c3_64m_hypersonic']
    a = workloads.make_particles(w, 'cpu', seed=3, n=50_001)
    b = workloads.make_particles(w, 'cpu', seed=3, n=50_001)
    for s, t in zip(a, b):
        assert torch.equal(s, t)
    x, y, z, v = a
    assert v.shape == (3, 50_004) and torch.all(v[:, 50_001:] == 0)
    assert float(x.min()) >= 0 and float(x.max()) < 1
    inside_body = ((x > 0.5) & (x < 0.7)).float().mean()
    assert inside_body == 0
    shock = ((x >= 0.4) & (x < 0.45)).float().mean()
    assert 0.33 < float(shock) < 0.38
    w2 = workloads.WORKLOADS['c2_16m_128']
    v2 = workloads.make_particles(w2, 'cpu', seed=0, n=20_000)[3]
    assert 4.9 < float(v2[0, :20_000].mean()) < 5.1
    assert workloads.step_seed(1234, 5000) == 1234 ^ (5000 << 20)


def test_cpu_binning_pipeline_counts_equal_the_oracle():
    """The CPU pipeline of the command-line benchmark (torch on host threads) bins particles
    into the same cells as the oracle; its shuffle bits come from another generator, so only
    the counts and the sortedness are comparable (phase2_triton_sort_benchmark.py:161-162)."""
    import numpy as np
    import torch
    from oracle import sort_oracle as so
    from project_aether_b200 import phase2_benchmark
    from project_aether_b200.cell_grid import CellGrid
    grid = CellGrid((0.0, 0.0, 0.0), (1.0, 1.0, 0.64), (25, 25, 16))
    gen = torch.Generator().manual_seed(5)
    pos = [torch.rand(20_000, generator=gen) * h for h in grid.hi]
    keys, order, counts = phase2_benchmark.cpu_binning(*pos, grid, torch.Generator().manual_seed(0))
    want = so.sort_particles(*(p.numpy() for p in pos), so.Grid(grid.lo, grid.hi, grid.cells), 3)
    np.testing.assert_array_equal(counts.numpy(), want.cell_counts)
    assert bool((keys[1:] >= keys[:-1]).all())
    np.testing.assert_array_equal(np.sort(order.numpy()), np.arange(20_000))
    np.testing.assert_array_equal((keys >> 7).numpy(), want.keys >> 7)


def test_bucket_plan_query_is_host_arithmetic(lib):
    """AetherSortBucketPlan: bucket widths and finish-group capacities of the benchmark
    configurations (a bucket never spans more cells than a group may; the small finish shape
    up to 32,768 buckets, the large one beyond)."""
    def plan(n, cells):
        shift, buckets, capacity = ctypes.c_int32(-1), ctypes.c_int64(-1), ctypes.c_int32(-1)
        rc = lib.AetherSortBucketPlan(n, cells, ctypes.byref(shift), ctypes.byref(buckets),
                                      ctypes.byref(capacity))
        return rc, shift.value, buckets.value, capacity.value

    rc, shift, buckets, capacity = plan(1 << 26, 256 * 128 * 128)   # 64 M hypersonic
    assert (rc, shift, buckets, capacity) == (0, 8, 16384, 5120)
    rc, shift, buckets, capacity = plan(1 << 24, 128 ** 3)           # 16 M
    assert (rc, shift, buckets, capacity) == (0, 7, 16384, 2560)
    rc, shift, buckets, capacity = plan(1 << 28, 512 * 256 * 256)    # 256 M
    assert (rc, shift, buckets, capacity) == (0, 9, 65536, 5120)
    rc, shift, buckets, capacity = plan(1 << 20, 64 ** 3)            # 1 M: small groups
    assert rc == 0 and buckets >= 2048 and 1024 <= capacity <= 2560
    assert n_over_capacity(lib) != 0


def n_over_capacity(lib):
    # 100,000 particles in one cell: no bucket width keeps the average load within a block.
    return lib.AetherSortBucketPlan(100_000, 1, None, None, None)


def test_scaled_workload_keeps_particles_per_cell():
    w = workloads.scaled_workload('c3_64m_hypersonic', 24)
    full = workloads.WORKLOADS['c3_64m_hypersonic']
    assert w.n == 1 << 24 and w.grid.cells[:2] == full.grid.cells[:2]
    assert w.n * full.grid.num_cells == full.n * w.grid.num_cells
    assert workloads.scaled_workload('c4_256m_512', 28) == workloads.WORKLOADS['c4_256m_512']


def test_copy_plan_tiles_every_destination_without_gaps_or_overlap():
    """The copies planned by all sources for one destination cover [0, received) exactly once,
    source by source and, within a source, slice by slice (the ordering rule of the exchange)."""
    import numpy as np
    from project_aether_b200 import slab_sort
    rng = np.random.default_rng(5)
    for world, slices in ((2, 1), (3, 4), (8, 32)):
        counts = rng.integers(0, 50, size=(world, slices, world))
        counts[rng.integers(0, world), :, :] = 0  # a source with nothing to send
        received = counts.sum(axis=(0, 1))
        for d in range(world):
            pieces = []
            for s in range(world):
                if s == d:
                    # A rank's own share is stored by the partition kernel: same rule.
                    first = counts[:s, :, d].sum()
                    pieces += [(first + counts[s, :k, d].sum(), counts[s, k, d], s, k)
                               for k in range(slices)]
                    continue
                plan = slab_sort.copy_plan(counts, s)
                assert [len(row) for row in plan] == [world - 1] * slices
                assert [row[0][0] for row in plan] == [(s + 1) % world] * slices
                for k, row in enumerate(plan):
                    pieces += [(first, count, s, k) for dest, first, count in row if dest == d]
            pieces.sort(key=lambda piece: (piece[2], piece[3]))
            at = 0
            for first, count, _, _ in pieces:
                assert first == at
                at += count
            assert at == received[d]


def test_exchange_settings_are_checked():
    from project_aether_b200 import slab_sort
    with pytest.raises(ValueError):
        slab_sort.configure(transport='carrier pigeon')
    slab_sort.configure(transport='stores', overlap=False)
    assert slab_sort.overlap_default(8) is False
    slab_sort.configure()
    assert slab_sort.overlap_default(2) is True and slab_sort.overlap_default(8) is False
    assert slab_sort.transport_default(4) == 'copies' and slab_sort.transport_default(8) == 'stores'
