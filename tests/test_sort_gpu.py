"""Parity of the CUDA path (through the C ABI) with the CPU oracle: bit-exact
keys, permutation, cell counts, cell starts and sorted payload."""

import os

import numpy as np
import pytest
import torch

import project_aether_b200 as pa
from oracle import sort_oracle as so
from project_aether_b200 import workloads

pytestmark = pytest.mark.gpu

PATHS = [pa.PATH_DIGIT_PASSES, pa.PATH_AUTO]


def _ogrid(grid):
    return so.Grid(tuple(grid.lo), tuple(grid.hi), tuple(grid.cells))


def _check_order(result, want):
    keys = result.keys.cpu().numpy().view(np.uint32)
    np.testing.assert_array_equal(keys, want.keys)
    np.testing.assert_array_equal(result.particle_index.cpu().numpy(), want.particle_index)
    np.testing.assert_array_equal(result.cell_counts.cpu().numpy(), want.cell_counts)
    np.testing.assert_array_equal(result.cell_start.cpu().numpy(), want.cell_start)


def _check_all(x, y, z, vel, grid, seed, path, big=False, **slab):
    got = pa.sort_and_gather_particles(x, y, z, vel, grid, seed, path=path, **slab)
    assert pa.last_sort_status(x.device) == 0
    xn, yn, zn, vn = (t.cpu().numpy() for t in (x, y, z, vel))
    if big:
        want, xs, ys, zs, vs = so.c_sort_particles(xn, yn, zn, vn, _ogrid(grid), seed, **slab)
    else:
        want = so.sort_particles(xn, yn, zn, _ogrid(grid), seed, **slab)
        xs, ys, zs, vs = so.gather_payload(want.particle_index, xn, yn, zn, vn)
    _check_order(got.order, want)
    for g, w in zip(got.positions, (xs, ys, zs)):
        np.testing.assert_array_equal(g.cpu().numpy(), w)
    n = x.numel()
    np.testing.assert_array_equal(got.velocity.cpu().numpy()[:, :n], vs[:, :n])
    assert torch.all(got.velocity[:, n:] == 0)
    return got


def _random_state(n, grid, device, seed=0, spill=0.0):
    gen = torch.Generator(device=device).manual_seed(seed)
    pos = []
    for l, h in zip(grid.lo, grid.hi):
        u = torch.rand(n, device=device, generator=gen)
        pos.append(((u * (1 + 2 * spill) - spill) * (h - l) + l).float())
    padded = -(-n // 4) * 4
    vel = torch.zeros((3, padded), device=device)
    vel[:, :n] = torch.randn((3, n), device=device, generator=gen)
    return pos[0], pos[1], pos[2], vel


@pytest.mark.parametrize('path', PATHS)
@pytest.mark.parametrize('name', ['unit', 'offset'])
def test_golden_cases_from_the_reference_kernels(cuda, golden_dir, name, path):
    t = np.load(os.path.join(golden_dir, 'triton_interp.npz'))
    g = t[name + '_grid']
    grid = pa.CellGrid(tuple(g[:3]), tuple(g[3:6]), tuple(int(v) for v in g[6:]))
    seed = int(t[name + '_seed'][0])
    x, y, z = (torch.from_numpy(t[f'{name}_{c}']).to(cuda) for c in 'xyz')
    res = pa.sort_particles_by_cell(x, y, z, grid, seed)
    np.testing.assert_array_equal(res.keys.cpu().numpy(), t[name + '_keys'])
    np.testing.assert_array_equal(res.particle_index.cpu().numpy(), t[name + '_index'])
    np.testing.assert_array_equal(res.cell_counts.cpu().numpy(), t[name + '_counts'])
    np.testing.assert_array_equal(res.cell_start.cpu().numpy(), t[name + '_start'])
    vel = torch.zeros((3, -(-x.numel() // 4) * 4), device=cuda)
    got = pa.sort_and_gather_particles(x, y, z, vel, grid, seed, path=path)
    np.testing.assert_array_equal(got.order.keys.cpu().numpy(), t[name + '_keys'])
    np.testing.assert_array_equal(got.order.particle_index.cpu().numpy(), t[name + '_index'])


@pytest.mark.parametrize('path', PATHS)
def test_reference_gpu_test_invariants_and_bits(cuda, path):
    """The reference's own GPU test (test_radix_sort.py:60-83), then bit parity."""
    n = 1_000_003
    grid = pa.CellGrid(lo=(0.0, 0.0, 0.0), hi=(1.0, 1.0, 1.0), cells=(25, 25, 16))
    gen = torch.Generator(device='cuda').manual_seed(0)
    x, y, z = (torch.rand(n, device='cuda', generator=gen) for _ in range(3))
    out = pa.sort_particles_by_cell(x, y, z, grid, seed=1234)
    keys = out.keys.cpu().numpy()
    assert np.all(np.diff(keys) >= 0)
    cell = keys >> pa.SHUFFLE_BITS
    index = out.particle_index.cpu().numpy().astype(np.int64)
    assert np.array_equal(np.sort(index), np.arange(n))
    expected_cell = (
        (np.clip((z.cpu().numpy() * 16).astype(int), 0, 15) * 25 +
         np.clip((y.cpu().numpy() * 25).astype(int), 0, 24)) * 25 +
        np.clip((x.cpu().numpy() * 25).astype(int), 0, 24))
    np.testing.assert_array_equal(cell, expected_cell[index])
    np.testing.assert_array_equal(out.cell_counts.cpu().numpy(),
                                  np.bincount(cell, minlength=grid.num_cells))
    vel = torch.zeros((3, n + 1), device=cuda)
    _check_all(x, y, z, vel, grid, 1234, path)


@pytest.mark.parametrize('path', PATHS)
@pytest.mark.parametrize('n,cells', [(5000, (25, 25, 16)), (12_345, (10, 6, 5)), (1, (7, 1, 1)),
                                     (2048, (1, 1, 1)), (4096, (32, 32, 16)), (0, (4, 4, 4)),
                                     (6143, (8, 8, 8)), (6144, (8, 8, 8)), (6145, (8, 8, 8)),
                                     (3 * 6144 + 17, (64, 64, 64)), (100_000, (512, 256, 256))])
def test_shapes_of_the_reference_unit_tests_and_tile_edges(cuda, n, cells, path):
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), cells)
    x, y, z, vel = _random_state(n, grid, cuda, seed=n)
    _check_all(x, y, z, vel, grid, 1234 ^ (n << 20), path)


@pytest.mark.parametrize('path', PATHS)
def test_positions_outside_the_box_nonunit_grid_and_wide_seed(cuda, path):
    grid = pa.CellGrid((0.1, -0.2, 0.0), (1.0, 1.0, 0.64), (37, 25, 16))
    x, y, z, vel = _random_state(50_000, grid, cuda, seed=11, spill=0.1)
    x[:6] = torch.tensor([0.1, 1.0, -5.0, 7.0, float('inf'), float('nan')], device=cuda)
    y[:3] = torch.tensor([-0.2, 1.0, -1e30], device=cuda)
    _check_all(x, y, z, vel, grid, 0x138800007, path)
    _check_all(x, y, z, vel, grid, (1 << 64) - 1, path)


@pytest.mark.parametrize('path', PATHS)
def test_every_particle_in_one_cell_and_empty_cells(cuda, path):
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (64, 32, 32))
    n = 40_000
    x = torch.full((n,), 0.3, device=cuda)
    y = torch.full((n,), 0.7, device=cuda)
    z = torch.full((n,), 0.999, device=cuda)
    vel = torch.zeros((3, n), device=cuda)
    vel[:, :] = torch.arange(n, device=cuda).float()
    got = _check_all(x, y, z, vel, grid, 5, path)
    assert int(got.order.cell_counts.max()) == n
    # Two far-apart cells: long runs of empty cells between and after them.
    x[: n // 2] = 0.01
    z[: n // 2] = 0.01
    _check_all(x, y, z, vel, grid, 6, path)


def test_more_than_255_equal_keys_in_a_bucket(cuda):
    """The bucketed path counts equal keys of a bucket in byte-wide counters; a
    bucket that overflows one must hand over to the digit passes, not corrupt."""
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (64, 64, 64))
    n, seed = 60_000, 4242
    x, y, z, vel = _random_state(n, grid, cuda, seed=9)
    same = torch.from_numpy(so.shuffle_bits(n, seed) == 5).to(cuda)
    assert int(same.sum()) > 300
    x[same], y[same], z[same] = 0.51, 0.52, 0.53  # one cell, one shuffle value
    got = _check_all(x, y, z, vel, grid, seed, pa.PATH_AUTO)
    assert int(got.order.cell_counts.max()) >= int(same.sum())
    assert pa.last_sort_used_digit_passes(cuda)


@pytest.mark.parametrize('n,cells,dense', [(600_000, (64, 64, 32), 0.02), (2_000_003, (128, 64, 64), 0.03),
                                           (2_400_000, (16, 16, 16), 0.05)])
def test_dense_layer_overfills_buckets_without_leaving_the_bucketed_path(cuda, n, cells, dense):
    """Bucket widths are planned from the average load.  A density contrast across rows
    (70 % of the particles in a thin y-layer) puts several times the shared-memory capacity
    into the buckets of that layer; the finish kernel cuts such a bucket into runs of cells
    that fit.  Results stay bit-exact and the digit passes are not needed."""
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), cells)
    x, y, z, vel = _random_state(n, grid, cuda, seed=13)
    layer = torch.rand(n, device=cuda, generator=torch.Generator(device=cuda).manual_seed(14)) < 0.7
    y[layer] = 0.5 + dense * (y[layer] - 0.5)
    got = _check_all(x, y, z, vel, grid, 77, pa.PATH_AUTO, big=True)
    assert not pa.last_sort_used_digit_passes(cuda)
    # The layer really overfills buckets: with the library's own bucket width some bucket holds
    # more records than a block of the finish kernel sorts at a time.
    import ctypes
    from project_aether_b200 import _native
    shift, buckets, capacity = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int32()
    assert _native.load_library().AetherSortBucketPlan(
        n, grid.num_cells, ctypes.byref(shift), ctypes.byref(buckets), ctypes.byref(capacity)) == 0
    counts = got.order.cell_counts.cpu().numpy().astype(np.int64)
    per_bucket = np.add.reduceat(counts, np.arange(0, counts.size, 1 << shift.value))
    assert per_bucket.size == buckets.value
    assert per_bucket.max() > capacity.value


def test_uniform_input_does_not_use_the_digit_passes(cuda):
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (64, 64, 64))
    x, y, z, vel = _random_state(1 << 20, grid, cuda, seed=3)
    _check_all(x, y, z, vel, grid, 1, pa.PATH_AUTO, big=True)
    assert not pa.last_sort_used_digit_passes(cuda)


@pytest.mark.parametrize('path', PATHS)
def test_unaligned_views_and_wider_velocity_padding(cuda, path):
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (16, 16, 16))
    n = 10_001
    x, y, z, vel = _random_state(n + 3, grid, cuda, seed=2)
    vel = torch.cat([vel, torch.zeros((3, 8), device=cuda)], dim=1)
    _check_all(x[1:n + 1], y[2:n + 2], z[3:n + 3], vel[:, : n + 5].contiguous(), grid, 77, path)


@pytest.mark.parametrize('path', PATHS)
def test_slab_local_cell_ids(cuda, path):
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (32, 16, 8))
    x, y, z, vel = _random_state(30_000, grid, cuda, seed=4)
    keep = (x >= 0.25) & (x < 0.5)
    xs, ys, zs = x[keep], y[keep], z[keep]
    n = xs.numel()
    v = torch.zeros((3, -(-n // 4) * 4), device=cuda)
    v[:, :n] = vel[:, : x.numel()][:, keep]
    _check_all(xs, ys, zs, v, grid, 31, path, ix_offset=8, nx_local=8)


@pytest.mark.parametrize('path', PATHS)
def test_runs_are_deterministic(cuda, path):
    w = workloads.WORKLOADS['c1_1m_64']
    x, y, z, vel = workloads.make_particles(w, cuda, seed=0)
    a = pa.sort_and_gather_particles(x, y, z, vel, w.grid, 1234, path=path)
    b = pa.sort_and_gather_particles(x, y, z, vel, w.grid, 1234, path=path)
    assert torch.equal(a.order.particle_index, b.order.particle_index)
    assert torch.equal(a.order.keys, b.order.keys)
    assert torch.equal(a.velocity, b.velocity)
    c = pa.sort_and_gather_particles(x, y, z, vel, w.grid, 1235, path=path)
    assert not torch.equal(a.order.particle_index, c.order.particle_index)
    assert torch.equal(a.order.cell_counts, c.order.cell_counts)


@pytest.mark.parametrize('path', PATHS)
@pytest.mark.parametrize('name', ['c1_1m_64', 'c2_16m_128', 'c3_64m_hypersonic'])
def test_benchmark_configurations_bit_exact(cuda, name, path):
    w = workloads.WORKLOADS[name]
    x, y, z, vel = workloads.make_particles(w, cuda, seed=0)
    _check_all(x, y, z, vel, w.grid, workloads.step_seed(1234, 1), path, big=True)


def _properties(got, x, vel, n, cells):
    keys = got.order.keys.view(torch.uint32) if hasattr(torch, 'uint32') else got.order.keys
    k64 = got.order.keys.to(torch.int64) & 0xFFFFFFFF
    assert bool(torch.all(k64[1:] >= k64[:-1]))
    idx = got.order.particle_index.long()
    seen = torch.zeros(n, dtype=torch.int32, device=x.device)
    seen.scatter_add_(0, idx, torch.ones_like(idx, dtype=torch.int32))
    assert bool(torch.all(seen == 1))
    assert torch.equal(got.positions[0], x[idx])
    assert torch.equal(got.velocity[2, :n], vel[2, :n][idx])
    counts = torch.bincount(k64 >> 7, minlength=cells).int()
    assert torch.equal(counts, got.order.cell_counts)
    start = torch.zeros(cells + 1, dtype=torch.int64, device=x.device)
    start[1:] = torch.cumsum(counts.long(), 0)
    assert torch.equal(start.int(), got.order.cell_start)


def test_largest_single_gpu_configuration_bit_exact(cuda):
    """256M particles, 33.5M cells, 32-bit keys (bit 31 in use), at full size against the C
    oracle, on both device paths; plus the size-independent properties."""
    import gc
    w = workloads.WORKLOADS['c4_256m_512']
    seed = workloads.step_seed(1234, 3)
    x, y, z, vel = workloads.make_particles(w, cuda, seed=0)
    xn, yn, zn, vn = (t.cpu().numpy() for t in (x, y, z, vel))
    want, xs, ys, zs, vs = so.c_sort_particles(xn, yn, zn, vn, _ogrid(w.grid), seed)
    del xn, yn, zn, vn
    assert want.keys[-1] >> 31 == 1  # the top key bit is really exercised
    for path in (pa.PATH_AUTO, pa.PATH_DIGIT_PASSES):
        got = pa.sort_and_gather_particles(x, y, z, vel, w.grid, seed, path=path)
        assert pa.last_sort_status(cuda) == 0
        assert not pa.last_sort_used_digit_passes(cuda)  # no hand-over on uniform input
        if path == pa.PATH_AUTO:
            _properties(got, x, vel, w.n, w.grid.num_cells)
            # Ties (same cell and shuffle bits) must keep ascending original index.
            k64 = got.order.keys.to(torch.int64) & 0xFFFFFFFF
            same = k64[1:] == k64[:-1]
            idx = got.order.particle_index
            assert bool(torch.all(idx[1:][same] > idx[:-1][same]))
            del k64, same, idx
        _check_order(got.order, want)
        for g, v in zip(got.positions, (xs, ys, zs)):
            assert np.array_equal(g.cpu().numpy(), v)
        assert np.array_equal(got.velocity.cpu().numpy(), vs)
        del got
        gc.collect()
        torch.cuda.empty_cache()


def test_steady_state_resort_loop_bit_exact(cuda):
    """The steady-state configuration at 2^24 particles: a cell-sorted state, then twenty
    consecutive (move fused into the sort) steps, each compared with the oracle stepped
    beside it (push semantics fused_particle_push.py:36-44,64-66; seeds
    dsmc_gpu_pipeline.py:106).  The sorted output of a step is the next step's input."""
    w = workloads.scaled_workload('c5_128m_256', 24)
    n, grid = w.n, w.grid
    dt = 8.2e-5
    x, y, z, vel = workloads.make_particles(w, cuda, seed=0)
    state = pa.sort_and_gather_particles(x, y, z, vel, grid, 99)
    assert pa.last_sort_status(cuda) == 0
    pos = [p.cpu().numpy() for p in state.positions]
    vel_h = [state.velocity[k, :n].cpu().numpy() for k in range(3)]
    padded = state.velocity.shape[1]
    sets = [None, None]
    crossed = []
    for step in range(20):
        seed = workloads.step_seed(1234, step)
        got = pa.sort_and_gather_particles(*state.positions, state.velocity, grid, seed,
                                           push=(dt, grid.lo, grid.hi), out=sets[step % 2])
        sets[step % 2] = got
        assert pa.last_sort_status(cuda) == 0
        assert not pa.last_sort_used_digit_passes(cuda)
        cells_before = so.cell_ids(*pos, _ogrid(grid))
        pos, vel_h = so.push_particles(pos, vel_h, dt, grid.lo, grid.hi)
        crossed.append(float((so.cell_ids(*pos, _ogrid(grid)) != cells_before).mean()))
        vn = np.zeros((3, padded), np.float32)
        vn[:, :n] = np.stack(vel_h)
        want, xs, ys, zs, vs = so.c_sort_particles(*(np.ascontiguousarray(p) for p in pos), vn,
                                                   _ogrid(grid), seed)
        _check_order(got.order, want)
        for g, v in zip(got.positions, (xs, ys, zs)):
            assert np.array_equal(g.cpu().numpy().view(np.uint32), v.view(np.uint32))
        assert np.array_equal(got.velocity.cpu().numpy().view(np.uint32), vs.view(np.uint32))
        pos, vel_h = [xs, ys, zs], [vs[k, :n] for k in range(3)]
        state = got
    assert 0.03 < np.mean(crossed) < 0.07  # about 5 % of the particles change cell per step


def test_auto_path_falls_back_to_digit_passes_in_a_small_workspace(cuda):
    """A workspace that holds the digit passes (and their payload records) but not the
    bucketed layout: `path` 0 must run the digit passes, `path` 2 must be refused."""
    import ctypes
    from project_aether_b200 import _native
    from project_aether_b200.particle_sort import native_grid
    lib = _native.load_library()
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (32, 32, 32))
    n, cells = 250_000, grid.num_cells
    x, y, z, vel = _random_state(n, grid, cuda, seed=9)
    g = native_grid(grid)
    full = lib.AetherSortWorkspaceBytes(n, cells, 1)
    # The digit passes with payload records need status words + 8 + 32 bytes per particle; the
    # bucketed layout needs its run tables on top of 32 bytes per particle.  A bare
    # 24 bytes per particle fits neither records nor buckets: digit passes + plain gather.
    for nbytes in (24 * n + (1 << 20),):
        assert nbytes < full
        ws = torch.empty(nbytes, dtype=torch.uint8, device=cuda)
        outs = dict(keys=torch.empty(n, dtype=torch.int32, device=cuda),
                    index=torch.empty(n, dtype=torch.int32, device=cuda),
                    counts=torch.empty(cells, dtype=torch.int32, device=cuda),
                    start=torch.empty(cells + 1, dtype=torch.int32, device=cuda),
                    xs=torch.empty(n, device=cuda), ys=torch.empty(n, device=cuda),
                    zs=torch.empty(n, device=cuda), vs=torch.zeros_like(vel))
        stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)

        def call(path):
            return lib.AetherSortAndGatherParticles(
                x.data_ptr(), y.data_ptr(), z.data_ptr(), vel.data_ptr(), vel.shape[1], n,
                ctypes.byref(g), 77, outs['keys'].data_ptr(), outs['index'].data_ptr(),
                outs['counts'].data_ptr(), outs['start'].data_ptr(), outs['xs'].data_ptr(),
                outs['ys'].data_ptr(), outs['zs'].data_ptr(), outs['vs'].data_ptr(), vel.shape[1],
                path, ws.data_ptr(), ws.numel(), stream)

        assert call(pa.PATH_BUCKETED) == 1  # cudaErrorInvalidValue, nothing launched
        assert call(pa.PATH_AUTO) == 0
        status = ctypes.c_int32(-1)
        _native.check(lib.AetherSortReadStatus(ws.data_ptr(), stream, ctypes.byref(status)), 'status')
        assert status.value == 0
        xn, yn, zn, vn = (t.cpu().numpy() for t in (x, y, z, vel))
        want = so.sort_particles(xn, yn, zn, _ogrid(grid), 77)
        xs, ys, zs, vs = so.gather_payload(want.particle_index, xn, yn, zn, vn)
        assert np.array_equal(outs['keys'].cpu().numpy().view(np.uint32), want.keys)
        assert np.array_equal(outs['index'].cpu().numpy(), want.particle_index)
        assert np.array_equal(outs['start'].cpu().numpy(), want.cell_start)
        assert np.array_equal(outs['zs'].cpu().numpy(), zs)
        assert np.array_equal(outs['vs'].cpu().numpy()[:, :n], vs[:, :n])


@pytest.mark.parametrize('path', PATHS)
def test_particles_outside_the_slab_are_binned_into_its_nearest_column(cuda, path):
    """The slab form's precondition broken on purpose: positions over the whole box sorted
    with the cell ids of one slab.  No table may be indexed out of range; the result follows
    the documented rule (column clamped into the slab), which the oracle applies too."""
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (32, 16, 16))
    x, y, z, vel = _random_state(120_001, grid, cuda, seed=4, spill=0.05)
    for ix_offset, nx_local in ((8, 8), (0, 4), (28, 4)):
        _check_all(x, y, z, vel, grid, 5, path, ix_offset=ix_offset, nx_local=nx_local)


def test_random_shapes_densities_and_seeds_bit_exact(cuda):
    """Forty seeded random cases (grid shape, box, particle count, density pattern, seed):
    payload sort and keys-only sort against the C oracle.  Covers bucket widths from one
    cell to 1024 cells, oversized buckets, empty regions and particles outside the box."""
    rng = np.random.default_rng(20240607)
    used_digit_passes = 0
    for case in range(40):
        cells = tuple(int(c) for c in rng.integers(1, [97, 65, 49]))
        lo = tuple(float(v) for v in rng.uniform(-2.0, 1.0, 3))
        hi = tuple(l + float(e) for l, e in zip(lo, rng.uniform(0.25, 3.0, 3)))
        grid = pa.CellGrid(lo, hi, cells)
        n = int(rng.integers(1, 400_000)) if case % 5 else int(rng.integers(1, 3000))
        seed = int(rng.integers(0, 2 ** 63 - 1)) if case % 3 else int(rng.integers(0, 2 ** 31))
        x, y, z, vel = _random_state(n, grid, cuda, seed=1000 + case,
                                     spill=0.02 if case % 4 == 0 else 0.0)
        pattern = case % 4
        if pattern == 1:      # a dense layer across rows
            sel = torch.rand(n, device=cuda) < 0.6
            mid = 0.5 * (lo[1] + hi[1])
            y[sel] = mid + 0.03 * (y[sel] - mid)
        elif pattern == 2:    # clusters: most particles in a corner of the box
            sel = torch.rand(n, device=cuda) < 0.8
            for t, l, h in zip((x, y, z), lo, hi):
                t[sel] = l + 0.2 * (t[sel] - l)
        elif pattern == 3:    # already cell-sorted input
            first = pa.sort_and_gather_particles(x, y, z, vel, grid, 1)
            x, y, z, vel = (*first.positions, first.velocity)
        _check_all(x, y, z, vel, grid, seed, pa.PATH_AUTO, big=True)
        used_digit_passes += pa.last_sort_used_digit_passes(cuda)
        keys_only = pa.sort_particles_by_cell(x, y, z, grid, seed)
        want = so.c_sort_particles(*(t.cpu().numpy() for t in (x, y, z)), None, _ogrid(grid), seed)[0]
        _check_order(keys_only, want)
    # Cells that hold more records than shared memory or 255 per counter do occur in the
    # clustered cases; most cases must stay on the bucketed path.
    assert used_digit_passes <= 20
