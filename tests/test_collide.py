"""NTC collision stage: the C oracle against the outputs of the reference's own
inline functions (CPU), and the B200 kernel against the oracle (GPU).

The GPU checks are those of the reference's kernel test
(project_aether/src/custom_kernels/cuda/dsmc_collide_tma_test.cu:166-213): the
accept decisions of more than 99.9 % of the cells equal the CPU replay's (device
and host powf/sinf/cosf differ by a few ulps, which can flip a borderline
acceptance), momentum and energy are conserved in every cell to 1e-5 relative.
On top of that: cells whose decisions match carry velocities equal to the
replay's within 2e-6 relative to the thermal speed, the candidate-pair counts
are exact, and untouched particles are bit-identical.
"""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import collide_oracle as co  # noqa: E402

GOLDEN = os.path.join(ROOT, 'tests', 'golden', 'collide_cases.npz')


def golden_cases():
    g = np.load(GOLDEN)
    for name in sorted({k.split('/')[0] for k in g.files}):
        sc, ss = g[name + '/scalars'], g[name + '/seed_step']
        case = co.CollideCase(g[name + '/velocity_in'], g[name + '/cell_start'], g[name + '/sigma_in'],
                              float(sc[0]), float(sc[1]), float(sc[2]), int(ss[0]), int(ss[1]))
        yield name, case, g[name + '/velocity_out'], g[name + '/sigma_out'], g[name + '/collisions']


def test_oracle_equals_reference_functions_bit_for_bit():
    seen = 0
    for name, case, velocity, sigma, collisions in golden_cases():
        v, s, c = co.collide(case)
        assert np.array_equal(v.view(np.uint32), velocity.view(np.uint32)), name
        assert np.array_equal(s.view(np.uint32), sigma.view(np.uint32)), name
        assert np.array_equal(c, collisions), name
        seen += int(c.sum())
    assert seen > 1000  # the fixture does collide


def test_oracle_conserves_momentum_and_energy():
    case = co.make_case(np.random.default_rng(5).poisson(30.0, 400), rng_seed=9,
                        selection_factor=3.0e14)
    v, _, c = co.collide(case)
    assert c.sum() > 0
    check_conservation(case, v)


def check_conservation(case, after, tol=1e-5):
    """dsmc_collide_tma_test.cu:176-201."""
    before = case.velocity.astype(np.float64)
    after = after.astype(np.float64)
    start = case.cell_start
    n = int(start[-1])
    cell_of = np.repeat(np.arange(start.size - 1), np.diff(start))
    cells = start.size - 1
    e0 = np.bincount(cell_of, weights=(before[:, :n] ** 2).sum(0), minlength=cells)
    e1 = np.bincount(cell_of, weights=(after[:, :n] ** 2).sum(0), minlength=cells)
    ok = e0 > 0
    assert np.all(np.abs(e1 - e0)[ok] <= tol * e0[ok])
    for c in range(3):
        p0 = np.bincount(cell_of, weights=before[c, :n], minlength=cells)
        p1 = np.bincount(cell_of, weights=after[c, :n], minlength=cells)
        assert np.all(np.abs(p1 - p0)[ok] <= tol * np.sqrt(e0[ok]))


def run_gpu(case, cuda):
    import torch
    from project_aether_b200 import ntc_collide
    lib = ntc_collide.load_library()
    velocity = torch.as_tensor(case.velocity, device=cuda).clone()
    start = torch.as_tensor(case.cell_start, device=cuda)
    sigma = torch.as_tensor(case.sigma_g_max, device=cuda).clone()
    collisions = torch.full((sigma.numel(),), -1, dtype=torch.int32, device=cuda)
    params = ntc_collide.CollisionParams(case.selection_factor, case.coefficient, case.exponent,
                                         case.seed, case.step)
    ntc_collide.collide(lib, velocity, start, sigma, collisions, int(case.cell_start[-1]), params)
    torch.cuda.synchronize()
    return velocity.cpu().numpy(), sigma.cpu().numpy(), collisions.cpu().numpy()


def compare_with_oracle(case, got, thermal=800.0):
    v, s, c = got
    ref_v, ref_s, ref_c = co.collide(case)
    cells = ref_c.size
    same = c == ref_c
    assert same.mean() > 0.999 or (~same).sum() <= 1, f'{(~same).sum()} of {cells} cells differ'
    assert c.min() >= 0
    assert np.all(c <= co.selections(case))
    # Cells with equal accept counts: same velocities up to the ulps of powf/sinf/cosf.
    start = case.cell_start
    n = int(start[-1])
    cell_of = np.repeat(np.arange(cells), np.diff(start))
    good = same[cell_of]
    err = np.abs(v[:, :n] - ref_v[:, :n])[:, good]
    assert err.size == 0 or err.max() <= 2e-6 * thermal * 8
    assert np.all(v[:, n:] == case.velocity[:, n:])
    # The majorant never falls; where decisions match it equals the replay's to 1e-6 relative.
    assert np.all(s >= case.sigma_g_max)
    assert np.allclose(s[same], ref_s[same], rtol=1e-6, atol=0)
    # Particles that are in no candidate pair are untouched, bit for bit.
    sel = co.selections(case)
    in_pair = (np.arange(n) - start[:-1][cell_of]) < 2 * sel[cell_of]
    assert np.array_equal(v[:, :n][:, ~in_pair].view(np.uint32),
                          case.velocity[:, :n][:, ~in_pair].view(np.uint32))
    check_conservation(case, v)
    return int(c.sum())


@pytest.mark.gpu
def test_gpu_collide_golden_cases(cuda):
    total = 0
    for name, case, *_ in golden_cases():
        total += compare_with_oracle(case, run_gpu(case, cuda))
    assert total > 1000


@pytest.mark.gpu
def test_gpu_collide_reference_test_shape(cuda):
    """4096 cells of Poisson(300) particles and one cell of 3000
    (dsmc_collide_tma_test.cu:86-113), with a selection factor that selects pairs."""
    rng = np.random.default_rng(1234)
    counts = rng.poisson(300.0, 4096)
    counts[17] = 3000
    case = co.make_case(counts, rng_seed=11, selection_factor=2.0e12)
    assert compare_with_oracle(case, run_gpu(case, cuda)) > 10000


@pytest.mark.gpu
@pytest.mark.parametrize('mean,cells,factor', [(8.0, 50000, 4.0e14), (16.0, 20001, 1.0e14),
                                                (110.0, 3000, 5.0e12)])
def test_gpu_collide_dsmc_occupancies(cuda, mean, cells, factor):
    rng = np.random.default_rng(int(mean))
    counts = rng.poisson(mean, cells)
    counts[::97] = 0
    case = co.make_case(counts, rng_seed=21, selection_factor=factor, seed=0xabcdef0123456789,
                        step=(3 << 32) | 17)
    assert compare_with_oracle(case, run_gpu(case, cuda)) > 1000


@pytest.mark.gpu
def test_gpu_collide_edge_cells(cuda):
    """Cells larger than the stage (global-memory path), a cell that fills the stage exactly,
    empty runs at both ends, one and two particles, an unaligned velocity base."""
    counts = np.r_[0, 0, 1, 2, 4096, 4097, 9000, 3, 0, 0, 4095, 1, 0, 700, 0, 0]
    case = co.make_case(counts, rng_seed=31, selection_factor=5.0e10)
    assert compare_with_oracle(case, run_gpu(case, cuda)) > 100
    import torch
    from project_aether_b200 import ntc_collide
    # The same case through a view whose rows do not start on 16-byte boundaries.
    n = int(case.cell_start[-1])
    padded = case.velocity.shape[1]
    store = torch.zeros(3 * padded + 8, dtype=torch.float32, device=cuda)
    view = store[1:1 + 3 * padded].view(3, padded)
    view.copy_(torch.as_tensor(case.velocity))
    sigma = torch.as_tensor(case.sigma_g_max, device=cuda).clone()
    collisions = torch.zeros(sigma.numel(), dtype=torch.int32, device=cuda)
    params = ntc_collide.CollisionParams(case.selection_factor, case.coefficient, case.exponent,
                                         case.seed, case.step)
    ntc_collide.collide(ntc_collide.load_library(), view, torch.as_tensor(case.cell_start, device=cuda),
                        sigma, collisions, n, params)
    compare_with_oracle(case, (view.cpu().numpy(), sigma.cpu().numpy(), collisions.cpu().numpy()))
    assert float(store[0]) == 0.0 and float(store[1 + 3 * padded:].abs().sum()) == 0.0


@pytest.mark.gpu
def test_gpu_collide_no_cells_and_no_pairs(cuda):
    import torch
    from project_aether_b200 import ntc_collide
    lib = ntc_collide.load_library()
    params = ntc_collide.CollisionParams(0.0, 1.7e-18, 0.46, 1, 2)
    case = co.make_case(np.full(100, 20), rng_seed=41, selection_factor=0.0)
    v, s, c = run_gpu(case, cuda)
    assert np.array_equal(v.view(np.uint32), case.velocity.view(np.uint32))
    assert np.all(c == 0) and np.array_equal(s, case.sigma_g_max)
    empty = torch.zeros((3, 0), dtype=torch.float32, device=cuda)
    ntc_collide.collide(lib, empty, torch.zeros(1, dtype=torch.int32, device=cuda),
                        torch.zeros(0, device=cuda), torch.zeros(0, dtype=torch.int32, device=cuda),
                        0, params)
    with pytest.raises(RuntimeError):  # padded not a multiple of four
        ntc_collide.collide(lib, torch.zeros((3, 6), device=cuda),
                            torch.tensor([0, 6], dtype=torch.int32, device=cuda),
                            torch.zeros(1, device=cuda), torch.zeros(1, dtype=torch.int32, device=cuda),
                            6, params)


@pytest.mark.gpu
def test_gpu_dsmc_step_runs_the_three_stages(cuda):
    """gpu_dsmc_step (dsmc_gpu_pipeline.py:85-113): every stage against its oracle."""
    import torch
    import project_aether_b200 as pa
    from oracle import sort_oracle
    rng = np.random.default_rng(3)
    n, cells = 60001, (12, 10, 8)
    grid = pa.CellGrid((0.0, 0.0, 0.0), (1.2, 1.0, 0.8), cells)
    positions = (rng.random((n, 3)) * np.array([1.2, 1.0, 0.8])).astype(np.float32)
    velocities = (rng.standard_normal((n, 3)) * 300.0).astype(np.float32)
    sigma0 = np.full(grid.num_cells, 3.0e-16, dtype=np.float32)
    state = pa.GpuDsmcState.from_numpy(positions, velocities, sigma0, device=cuda)
    lib = pa.ntc_collide.load_library()
    dt = 2.0e-5
    px, pv = [positions[:, i].copy() for i in range(3)], [velocities[:, i].copy() for i in range(3)]
    sigma = sigma0.copy()
    for step in range(3):
        params = pa.CollisionParams(4.0e11, 1.7e-18, 0.46, 0x5eed, step)
        stats = pa.gpu_dsmc_step(state, lib, grid, params, dt)
        torch.cuda.synchronize()
        # Oracle: push, sort + gather, collide.
        px, pv = sort_oracle.push_particles(px, pv, dt, grid.lo, grid.hi)
        padded = -(-n // 4) * 4
        vel = np.zeros((3, padded), dtype=np.float32)
        vel[:, :n] = np.stack(pv)
        outputs, xs, ys, zs, vs = sort_oracle.c_sort_particles(
            np.ascontiguousarray(px[0]), np.ascontiguousarray(px[1]), np.ascontiguousarray(px[2]),
            vel, grid, params.seed ^ (step << 20))
        counts, start = outputs[2], outputs[3]
        assert np.array_equal(stats.cell_counts.cpu().numpy(), counts)
        for got, want in zip(state.positions, (xs, ys, zs)):
            assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
        case = co.CollideCase(vs, start, sigma, params.selection_factor, params.vhs_coefficient,
                              params.vhs_exponent, params.seed, params.step)
        got = (state.velocity.cpu().numpy(), state.sigma_g_max.cpu().numpy(),
               stats.collisions.cpu().numpy())
        assert compare_with_oracle(case, got, thermal=300.0) > 0
        # Continue the oracle from the device state so that ulp differences do not accumulate.
        px = [p.cpu().numpy() for p in state.positions]
        pv = [state.velocity[c, :n].cpu().numpy() for c in range(3)]
        sigma = state.sigma_g_max.cpu().numpy()


@pytest.mark.gpu
def test_phase2_benchmark_cli(cuda, capsys):
    """The command-line benchmark of the reference (scripts/phase2_triton_sort_benchmark.py)
    on a small case: counts equal the CPU pipeline's; the collision statistics it prints
    equal the CPU replay of the kernel's algorithm, which this test (not the package) runs."""
    from project_aether_b200 import phase2_benchmark
    argv = ['--particles', '400000', '--cells', '25', '25', '16', '--cpu-threads', '4',
            '--repeats', '2', '--collisions', '--fnum', '3e14']
    assert phase2_benchmark.main(argv) == 0
    out = capsys.readouterr().out
    assert 'Per-cell counts identical: True' in out
    assert 'Mean collisions per cell: GPU' in out
    report = phase2_benchmark.run(argv)
    stats = report.collisions
    assert report.counts_match and stats is not None and stats.collisions.sum() > 0
    case = co.CollideCase(stats.velocity_before, stats.cell_start, stats.sigma_g_max,
                          stats.params.selection_factor, stats.params.vhs_coefficient,
                          stats.params.vhs_exponent, stats.params.seed, stats.params.step)
    want = co.collide(case)[2]
    differing = int((stats.collisions != want).sum())
    assert differing <= max(1, stats.collisions.size // 1000)
    assert abs(float(stats.collisions.mean()) - float(want.mean())) < 1e-3 * max(1.0, want.mean())
    assert f'GPU {stats.collisions.mean():.3f}' in report.text
