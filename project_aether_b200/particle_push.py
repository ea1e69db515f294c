"""Fused particle push with specular wall reflection on B200.

Drop-in for `fused_particle_push`
(project_aether/src/custom_kernels/triton/fused_particle_push.py:75-92): same
arguments, in-place update.  The arithmetic is that of the reference's unfused
statement `reference_push` (:95-108), so the result equals it bit for bit.
"""

import ctypes
from collections.abc import Sequence

import torch

from . import _native


def fused_particle_push(positions: Sequence[torch.Tensor], velocities: Sequence[torch.Tensor],
                        dt: float, lo: Sequence[float], hi: Sequence[float]) -> None:
    """Advances particles in place and reflects them at the box walls.

    Args:
      positions: (x, y, z) float32 CUDA tensors of shape (N,), updated in place.
      velocities: (vx, vy, vz) float32 CUDA tensors of shape (N,), updated in place (rows of
        a (3, padded) tensor are fine).
      dt: time step.
      lo: lower box corner (x, y, z).
      hi: upper box corner (x, y, z).
    """
    tensors = list(positions) + list(velocities)
    n = tensors[0].numel()
    for t in tensors:
        if (not t.is_cuda or t.dtype != torch.float32 or t.numel() != n
                or not t.is_contiguous()):
            raise ValueError('Positions and velocities must be contiguous float32 CUDA '
                             'tensors of the same length.')
    lib = _native.load_library()
    device = tensors[0].device
    lo_c = (ctypes.c_float * 3)(*[float(v) for v in lo])
    hi_c = (ctypes.c_float * 3)(*[float(v) for v in hi])
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        _native.check(lib.AetherParticlePush(
            *(ctypes.c_void_p(t.data_ptr()) for t in tensors), n, float(dt), lo_c, hi_c,
            ctypes.c_void_p(stream)), 'AetherParticlePush')
