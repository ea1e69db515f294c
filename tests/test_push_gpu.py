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
