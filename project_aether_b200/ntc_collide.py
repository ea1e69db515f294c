"""No-Time-Counter collisions on cell-sorted particles (B200 kernel).

This module IS the reference's ctypes binding
project_aether/src/custom_kernels/cuda/tma_collide.py restated as an interface:
`CollisionParams` has the reference's fields, `collide` its argument list and its
call into the C entry point `AetherDsmcCollideTma`, `vhs_parameters` is the
reference's six-line formula (:58-66) as it stands, and the docstrings follow the
reference's wording, so that the reference's callers can import this module in its
place.  What is this package's own: the entry point lives in libaether_sort.so
(csrc/collide.cu, a different kernel), the loader, the stride check and the 64-bit
masking of seed and step.
"""

import ctypes
import math
from typing import NamedTuple, Optional

import torch

from . import _native

BOLTZMANN = 1.380649e-23


class CollisionParams(NamedTuple):
    """Gas and timestep parameters of the collision kernel (tma_collide.py:41-55).

    Attributes:
      selection_factor: F_N * dt / V_cell.
      vhs_coefficient: sigma_T g = coefficient * g^vhs_exponent.
      vhs_exponent: 2 - 2 omega.
      seed: Philox key.
      step: timestep index (Philox counter words 2 and 3).
    """
    selection_factor: float
    vhs_coefficient: float
    vhs_exponent: float
    seed: int
    step: int


def vhs_parameters(mass: float, d_ref: float, omega: float, t_ref: float):
    """(coefficient, exponent) of sigma_T g for equal-mass variable-hard-sphere
    partners (tma_collide.py:58-66; Bird 1994)."""
    reduced_mass = 0.5 * mass
    coefficient = (math.pi * d_ref ** 2 *
                   (2.0 * BOLTZMANN * t_ref / reduced_mass) ** (omega - 0.5) /
                   math.gamma(2.5 - omega))
    return coefficient, 2.0 - 2.0 * omega


def load_library(path: Optional[str] = None) -> ctypes.CDLL:
    """The CUDA library with the C ABI declared (tma_collide.py:69-79).

    Raises:
      OSError / RuntimeError: if the library cannot be loaded.
    """
    return _native.load_library(path)


def collide(library: ctypes.CDLL, velocity: torch.Tensor, cell_start: torch.Tensor,
            sigma_g_max: torch.Tensor, collisions: torch.Tensor, num_particles: int,
            params: CollisionParams) -> None:
    """Runs the collisions in place on cell-sorted velocities (tma_collide.py:82-108).

    Args:
      library: library from `load_library`.
      velocity: float32 CUDA tensor (3, padded), padded % 4 == 0, contiguous rows;
        columns [0, num_particles) hold vx, vy, vz in cell-sorted order.
      cell_start: int32 CUDA tensor (C + 1,), exclusive prefix of the cell counts.
      sigma_g_max: float32 CUDA tensor (C,), updated in place.
      collisions: int32 CUDA tensor (C,), receives accepted pairs per cell.
      num_particles: number of real particles.
      params: collision parameters.

    Raises:
      RuntimeError: if the launch fails.
    """
    if velocity.dim() != 2 or velocity.shape[0] != 3 or (
            velocity.shape[1] > 0 and (velocity.stride(1) != 1
                                       or velocity.stride(0) != velocity.shape[1])):
        raise ValueError('Velocity must be a contiguous (3, padded) tensor.')
    with torch.cuda.device(velocity.device):
        stream = torch.cuda.current_stream().cuda_stream
        status = library.AetherDsmcCollideTma(
            velocity.data_ptr(), cell_start.data_ptr(), sigma_g_max.data_ptr(),
            collisions.data_ptr(), int(num_particles), velocity.shape[1], sigma_g_max.numel(),
            params.selection_factor, params.vhs_coefficient, params.vhs_exponent,
            int(params.seed) & 0xFFFFFFFFFFFFFFFF, int(params.step) & 0xFFFFFFFFFFFFFFFF,
            ctypes.c_void_p(stream))
    if status != 0:
        raise RuntimeError(f'AetherDsmcCollideTma failed with cudaError {status}')
