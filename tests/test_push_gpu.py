"""The move stage against the oracle's restatement of the reference's unfused
push (fused_particle_push.py:95-108): bit-exact, in place."""

import numpy as np
import pytest
import torch

from oracle import sort_oracle as so
from project_aether_b200.particle_push import fused_particle_push

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('n,offset', [(100_003, 0), (4096, 0), (1, 0), (50_001, 1), (0, 0)])
def test_push_matches_the_unfused_reference(cuda, n, offset):
    gen = torch.Generator(device=cuda).manual_seed(n)
    lo, hi = (0.1, -0.2, 0.0), (1.0, 1.0, 0.64)
    state = torch.rand((6, n + offset), device=cuda, generator=gen)
    state[3:] = (state[3:] - 0.5) * 8.0           # fast particles: many wall hits, some double
    pos = [state[k, offset:] for k in range(3)]    # offset 1 -> unaligned views, scalar path
    vel = [state[3 + k, offset:] for k in range(3)]
    host_p = [p.cpu().numpy().copy() for p in pos]
    host_v = [v.cpu().numpy().copy() for v in vel]
    dt = 0.173
    fused_particle_push(pos, vel, dt, lo, hi)
    want_p, want_v = so.push_particles(host_p, host_v, dt, lo, hi)
    for got, want in zip(pos + vel, want_p + want_v):
        np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_push_rejects_bad_inputs(cuda):
    x = torch.zeros(8, device=cuda)
    with pytest.raises(ValueError):
        fused_particle_push([x, x, x], [x, x, x.double()], 0.1, (0, 0, 0), (1, 1, 1))
    with pytest.raises(ValueError):
        fused_particle_push([x.cpu()] * 3, [x.cpu()] * 3, 0.1, (0, 0, 0), (1, 1, 1))


@pytest.mark.parametrize('path', ['auto', 'digits'])
@pytest.mark.parametrize('n,cells,dt', [(300_007, (32, 24, 16), 0.05), (1_000_003, (64, 64, 64), 0.002),
                                        (5000, (8, 8, 8), 0.3)])
def test_move_stage_fused_into_the_sort(cuda, n, cells, dt, path):
    """sort_and_gather_particles(push=...) equals the oracle's push followed by its sort and
    gather, bit for bit, on both device paths; the inputs are left as they were."""
    import project_aether_b200 as pa
    lo, hi = (0.0, -0.5, 0.25), (1.0, 0.5, 1.0)
    grid = pa.CellGrid(lo, hi, cells)
    gen = torch.Generator(device=cuda).manual_seed(n)
    pos = [(torch.rand(n, device=cuda, generator=gen) * (h - l) + l).float() for l, h in zip(lo, hi)]
    padded = -(-n // 4) * 4
    vel = torch.zeros((3, padded), device=cuda)
    vel[:, :n] = torch.randn((3, n), device=cuda, generator=gen) * 2.0  # many wall hits at these dt
    before = [t.clone() for t in (*pos, vel)]
    which = pa.PATH_AUTO if path == 'auto' else pa.PATH_DIGIT_PASSES
    got = pa.sort_and_gather_particles(*pos, vel, grid, 4321, path=which, push=(dt, lo, hi))
    assert pa.last_sort_status(cuda) == 0
    for t, b in zip((*pos, vel), before):
        assert torch.equal(t, b)
    host_p = [p.cpu().numpy() for p in pos]
    host_v = [vel[k, :n].cpu().numpy() for k in range(3)]
    moved_p, moved_v = so.push_particles(host_p, host_v, dt, lo, hi)
    moved_vel = np.zeros((3, padded), dtype=np.float32)
    moved_vel[:, :n] = np.stack(moved_v)
    want, xs, ys, zs, vs = so.c_sort_particles(*[np.ascontiguousarray(p) for p in moved_p], moved_vel,
                                               so.Grid(lo, hi, cells), 4321)
    np.testing.assert_array_equal(got.order.keys.cpu().numpy().view(np.uint32), want.keys)
    np.testing.assert_array_equal(got.order.particle_index.cpu().numpy(), want.particle_index)
    np.testing.assert_array_equal(got.order.cell_counts.cpu().numpy(), want.cell_counts)
    np.testing.assert_array_equal(got.order.cell_start.cpu().numpy(), want.cell_start)
    for g, w in zip(got.positions, (xs, ys, zs)):
        np.testing.assert_array_equal(g.cpu().numpy(), w)
    np.testing.assert_array_equal(got.velocity.cpu().numpy(), vs)
