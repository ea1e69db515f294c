"""B200-native DSMC particle sort: a drop-in for the fused particle sort of
Project AETHER (project_aether/src/custom_kernels/triton/fused_radix_sort.py)."""

from .cell_grid import SHUFFLE_BITS, CellGrid, key_bits, num_passes
from .dsmc_step import GpuDsmcState, GpuStepStats, gpu_dsmc_step
from .ntc_collide import CollisionParams, collide, vhs_parameters
from .particle_push import fused_particle_push
from .particle_sort import (PATH_AUTO, PATH_BUCKETED, PATH_DIGIT_PASSES, SortedParticles,
                            SortResult, last_sort_status, last_sort_used_digit_passes,
                            sort_and_gather_particles,
                            sort_particles_by_cell)

__all__ = [
    'SHUFFLE_BITS', 'CellGrid', 'key_bits', 'num_passes', 'PATH_AUTO', 'PATH_BUCKETED',
    'PATH_DIGIT_PASSES', 'SortedParticles', 'fused_particle_push', 'SortResult', 'last_sort_status', 'last_sort_used_digit_passes',
    'sort_and_gather_particles', 'sort_particles_by_cell', 'GpuDsmcState', 'GpuStepStats',
    'gpu_dsmc_step', 'CollisionParams', 'collide', 'vhs_parameters',
]
