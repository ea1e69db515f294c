"""One DSMC timestep on the GPU: move, sort by cell, collide.

Mirror of project_aether/src/physics_engine/dsmc_gpu_pipeline.py (`GpuDsmcState`
:49-77, `GpuStepStats` :80-82, `gpu_dsmc_step` :85-113).  The three stages are
this library's kernels; the move stage, the sort and the payload gather of
lines 101-109 are one call, and the sorted state of one step is written into the arrays the
step before last used, so a stepping loop allocates nothing after its second
step.
"""

import dataclasses
from typing import List, NamedTuple, Optional

import numpy as np
import torch

from . import ntc_collide, particle_sort
from .cell_grid import CellGrid


@dataclasses.dataclass
class GpuDsmcState:
    """Particle state on the GPU.

    Attributes:
      positions: (x, y, z) float32 CUDA tensors (N,).
      velocity: float32 CUDA tensor (3, padded) of vx, vy, vz, padded = ceil(N / 4) * 4.
      sigma_g_max: per-cell NTC majorant, float32 (C,).
      num_particles: N.
    """
    positions: List[torch.Tensor]
    velocity: torch.Tensor
    sigma_g_max: torch.Tensor
    num_particles: int
    _spare: Optional[particle_sort.SortedParticles] = dataclasses.field(default=None, repr=False)
    _current: Optional[particle_sort.SortedParticles] = dataclasses.field(default=None, repr=False)
    _collisions: Optional[list] = dataclasses.field(default=None, repr=False)

    @classmethod
    def from_numpy(cls, positions: np.ndarray, velocities: np.ndarray,
                   sigma_g_max: np.ndarray, device='cuda') -> 'GpuDsmcState':
        """Uploads (N, 3) positions and velocities and (C,) majorants."""
        n = positions.shape[0]
        padded = -(-n // 4) * 4
        velocity = torch.zeros((3, padded), dtype=torch.float32, device=device)
        velocity[:, :n] = torch.as_tensor(np.ascontiguousarray(velocities.T), dtype=torch.float32)
        pos = [torch.as_tensor(np.ascontiguousarray(positions[:, i]), dtype=torch.float32,
                               device=device) for i in range(3)]
        return cls(pos, velocity,
                   torch.as_tensor(sigma_g_max, dtype=torch.float32, device=device), n)


class GpuStepStats(NamedTuple):
    cell_counts: torch.Tensor
    collisions: torch.Tensor


def gpu_dsmc_step(state: GpuDsmcState, library, grid: CellGrid,
                  params: ntc_collide.CollisionParams, dt: float) -> GpuStepStats:
    """Advances `state` by one DSMC timestep in place.

    Args:
      state: particle state; left in cell-sorted order.
      library: the CUDA library from `ntc_collide.load_library`.
      grid: collision-cell grid (also the reflecting box).
      params: collision parameters; `params.step` keys the Philox streams.
      dt: time step.

    Returns:
      Per-cell particle counts and accepted collisions.  The tensors belong to
      the state's buffers and are overwritten two steps later.
    """
    n = state.num_particles
    # The move stage (dsmc_gpu_pipeline.py:101-104) runs inside the sort's kernels: they read
    # x and v once, move the particle and carry the moved state into the sorted arrays.
    # The sort seed of a step (dsmc_gpu_pipeline.py:106).
    seed = params.seed ^ (params.step << 20)
    # Two sets of arrays alternate: the step writes the sorted state into the set the
    # particles left one step ago.  Arrays the caller swapped in from outside are used
    # as they are and join the rotation afterwards.
    held = state._current
    if (held is None or held.velocity is not state.velocity
            or any(a is not b for a, b in zip(held.positions, state.positions))):
        held = particle_sort.SortedParticles(None, tuple(state.positions), state.velocity)
    spare = state._spare
    if spare is not None and (spare.velocity.shape != state.velocity.shape
                              or spare.positions[0].numel() != n
                              or spare.order.cell_counts.numel() != grid.num_cells):
        spare = None
    out = particle_sort.sort_and_gather_particles(*state.positions, state.velocity, grid, seed,
                                                  out=spare, push=(dt, grid.lo, grid.hi))
    if held.order is None:
        held = particle_sort.SortedParticles(
            particle_sort.SortResult(*(torch.empty_like(t) for t in out.order)),
            held.positions, held.velocity)
    state._spare, state._current = held, out
    state.positions = list(out.positions)
    state.velocity = out.velocity
    if state._collisions is None or len(state._collisions) != 2 or \
            state._collisions[0].numel() != grid.num_cells:
        state._collisions = [torch.empty_like(out.order.cell_counts) for _ in range(2)]
    state._collisions.reverse()
    collisions = state._collisions[0]
    ntc_collide.collide(library, state.velocity, out.order.cell_start, state.sigma_g_max,
                        collisions, n, params)
    return GpuStepStats(out.order.cell_counts, collisions)
