"""The CPU oracle against the golden vectors made from the reference itself
(tests/golden/make_golden.py).  No GPU, no reference tree needed."""

import json
import os

import numpy as np
import pytest

from oracle import sort_oracle as so


def test_philox_matches_reference_header(golden_dir):
    kat = json.load(open(os.path.join(golden_dir, 'philox_kat.json')))
    for case in kat['cases']:
        n = len(case['word0'])
        counters = np.arange(case['first_counter'], case['first_counter'] + n, dtype=np.uint64)
        got = so.philox4x32_10(counters, case['seed'])
        assert got.tolist() == case['word0']


def test_philox_known_answers_from_two_sources():
    # Word 0 for seed 1234, counters 0..7, measured both with the reference's
    # philox.h (g++) and with tl.randint under Triton's interpreter.
    want = [546353992, 2666454581, 1070188760, 3055983166, 346514135, 3391693257,
            4245463582, 3004048045]
    assert so.philox4x32_10(np.arange(8), 1234).tolist() == want
    want64 = [1505935688, 232970672, 4210063330, 3748580433]
    assert so.philox4x32_10(np.arange(4), 0x100000007).tolist() == want64


def test_c_philox_matches_numpy():
    lib = so._clib()
    if lib is None:
        pytest.skip('oracle/libsort_oracle.so not built')
    import ctypes
    c = np.arange(1000, dtype=np.uint32) * np.uint32(2654435761)
    out = np.empty_like(c)
    lib.oracle_philox_word0.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64,
                                        ctypes.c_void_p]
    for seed in (0, 1234, 0xDEADBEEFCAFEF00D):
        lib.oracle_philox_word0(c.ctypes.data, c.size, seed, out.ctypes.data)
        np.testing.assert_array_equal(out, so.philox4x32_10(c, seed))


def test_replay_matches_reference_replay(golden_dir):
    r = np.load(os.path.join(golden_dir, 'replay_cases.npz'))
    for i, (n, cells) in enumerate(r['shapes']):
        n, cells = int(n), int(cells)
        rng = np.random.default_rng(n)
        keys = ((rng.integers(0, cells, n) << so.SHUFFLE_BITS) |
                rng.integers(0, 1 << so.SHUFFLE_BITS, n)).astype(np.int32)
        np.testing.assert_array_equal(keys, r[f'keys_{i}'])
        sk, sv = so.onesweep_replay(keys, np.arange(n, dtype=np.int32),
                                    so.reference_num_passes(cells), rng, tile=256)
        np.testing.assert_array_equal(sk, r[f'sorted_keys_{i}'])
        np.testing.assert_array_equal(sv, r[f'sorted_values_{i}'])
        # The property the reference's own test pins (test_radix_sort.py:22-33).
        order = np.argsort(keys, kind='stable')
        np.testing.assert_array_equal(sk, keys[order])
        np.testing.assert_array_equal(sv, order)


def test_lookback_and_pass_counts_match_reference(golden_dir):
    r = np.load(os.path.join(golden_dir, 'replay_cases.npz'))
    np.testing.assert_array_equal(so.lookback(r['lookback_status'], 3), r['lookback_exclusive'])
    for cells, passes in zip(r['num_passes_cells'], r['num_passes']):
        assert so.reference_num_passes(int(cells)) == int(passes)
    with pytest.raises(ValueError):
        so.reference_num_passes(1 << 25)  # test_radix_sort.py:49-50


def test_lookback_raises_instead_of_waiting():
    status = np.zeros((3, so.RADIX), np.int64)
    status[0] = so.FLAG_INCLUSIVE
    with pytest.raises(RuntimeError):
        so.lookback(status, 2)  # tile 1 never published


def _grid(t, name):
    g = t[name + '_grid']
    return so.Grid(tuple(g[:3]), tuple(g[3:6]), tuple(int(v) for v in g[6:]))


@pytest.mark.parametrize('name', ['unit', 'offset'])
def test_whole_path_matches_reference_kernels(golden_dir, name):
    """Keys, permutation, counts and starts produced by the reference's Triton
    kernels (run by Triton's CPU interpreter when the fixture was made)."""
    t = np.load(os.path.join(golden_dir, 'triton_interp.npz'))
    grid, seed = _grid(t, name), int(t[name + '_seed'][0])
    x, y, z = t[name + '_x'], t[name + '_y'], t[name + '_z']
    keys = so.make_keys(x, y, z, grid, seed)
    np.testing.assert_array_equal(keys, t[name + '_unsorted_keys'].astype(np.uint32))
    out = so.sort_particles(x, y, z, grid, seed)
    np.testing.assert_array_equal(out.keys, t[name + '_keys'].astype(np.uint32))
    np.testing.assert_array_equal(out.particle_index, t[name + '_index'])
    np.testing.assert_array_equal(out.cell_counts, t[name + '_counts'])
    np.testing.assert_array_equal(out.cell_start, t[name + '_start'])


@pytest.mark.parametrize('name', ['unit', 'offset'])
def test_c_oracle_matches_numpy_oracle(golden_dir, name):
    if so._clib() is None:
        pytest.skip('oracle/libsort_oracle.so not built')
    t = np.load(os.path.join(golden_dir, 'triton_interp.npz'))
    grid, seed = _grid(t, name), int(t[name + '_seed'][0])
    x, y, z = t[name + '_x'], t[name + '_y'], t[name + '_z']
    n = x.size
    vel = np.random.default_rng(0).standard_normal((3, -(-n // 4) * 4)).astype(np.float32)
    vel[:, n:] = 0
    want = so.sort_particles(x, y, z, grid, seed)
    got, xs, ys, zs, vs = so.c_sort_particles(x, y, z, vel, grid, seed, threads=3)
    for a, b in zip(got, want):
        np.testing.assert_array_equal(a, b)
    gx, gy, gz, gv = so.gather_payload(want.particle_index, x, y, z, vel)
    np.testing.assert_array_equal(xs, gx)
    np.testing.assert_array_equal(zs, gz)
    np.testing.assert_array_equal(vs, gv)


def test_slab_local_sort_reassembles_the_global_counts():
    rng = np.random.default_rng(5)
    n, grid = 20000, so.Grid((0., 0., 0.), (1., 1., 1.), (16, 8, 4))
    pos = [rng.random(n, dtype=np.float32) for _ in range(3)]
    whole = so.sort_particles(*pos, grid, 99)
    world = 4
    nxl = grid.cells[0] // world
    dest = so.slab_of(pos[0], grid, world)
    counts = np.zeros((grid.cells[2], grid.cells[1], grid.cells[0]), np.int64)
    for r in range(world):
        sel = dest == r
        local = so.sort_particles(pos[0][sel], pos[1][sel], pos[2][sel], grid, 99,
                                  ix_offset=r * nxl, nx_local=nxl)
        counts[:, :, r * nxl:(r + 1) * nxl] = local.cell_counts.reshape(
            grid.cells[2], grid.cells[1], nxl)
    np.testing.assert_array_equal(counts.reshape(-1), whole.cell_counts)


def test_exchange_replay_keeps_source_order():
    rng = np.random.default_rng(1)
    grid = so.Grid((0., 0., 0.), (1., 1., 1.), (8, 2, 2))
    shares = [tuple(rng.random(50, dtype=np.float32) for _ in range(6)) for _ in range(2)]
    out = so.exchange_replay(shares, grid, 2)
    assert sum(o[0].size for o in out) == 100
    for d in range(2):
        assert np.all(so.slab_of(out[d][0], grid, 2) == d)
        own = shares[0][0][so.slab_of(shares[0][0], grid, 2) == d]
        np.testing.assert_array_equal(out[d][0][:own.size], own)


@pytest.mark.parametrize('name', ['unit_box', 'offset_box', 'tiny_step'])
def test_push_matches_reference_push(golden_dir, name):
    """`push_particles` against outputs of the reference's own unfused move stage
    (fused_particle_push.py:95-108, CPU tensors): particles on the faces, particles that leave
    through every face, and particles fast enough to stay outside after the one reflection."""
    g = np.load(os.path.join(golden_dir, 'push_cases.npz'))
    pos, vel = g[name + '/pos_in'], g[name + '/vel_in']
    sc = g[name + '/scalars']
    dt, lo, hi = float(sc[0]), sc[1:4], sc[4:7]
    new_pos, new_vel = so.push_particles(list(pos), list(vel), dt, lo, hi)
    want_pos, want_vel = g[name + '/pos_out'], g[name + '/vel_out']
    for axis in range(3):
        assert np.array_equal(new_pos[axis].view(np.uint32), want_pos[axis].view(np.uint32))
        assert np.array_equal(new_vel[axis].view(np.uint32), want_vel[axis].view(np.uint32))
    assert ((want_pos < lo[:, None]) | (want_pos > hi[:, None])).any()  # the overshooting ones
