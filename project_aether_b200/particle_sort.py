"""DSMC particle binning on B200: the host side of the CUDA particle sort.

Drop-in for the reference's `fused_radix_sort` module
(project_aether/src/custom_kernels/triton/fused_radix_sort.py:206-280):
`sort_particles_by_cell(x, y, z, grid, seed) -> SortResult` with the same
argument meaning, result fields, dtypes and errors.  `sort_and_gather_particles`
adds the payload gather that follows the sort in the DSMC step
(project_aether/src/physics_engine/dsmc_gpu_pipeline.py:105-109), so that the
caller gets cell-sorted positions and velocities from one call.

All device work is done by libaether_sort.so (hand-written sm_100a kernels)
through its C ABI; PyTorch only provides device memory and the current stream.

Typical usage example:

  result = sort_particles_by_cell(x, y, z, grid, seed=step)
  partner_order = result.particle_index  # cell-sorted, shuffled in cells
"""

import ctypes
from typing import NamedTuple, Optional, Tuple

import torch

from . import _native
from .cell_grid import CellGrid, MAX_PARTICLES, key_bits, num_passes  # noqa: F401

PATH_AUTO, PATH_DIGIT_PASSES, PATH_BUCKETED = 0, 1, 2


class SortResult(NamedTuple):
    """Output of `sort_particles_by_cell` (fused_radix_sort.py:206-218).

    Attributes:
      keys: sorted keys (cell << SHUFFLE_BITS | shuffle bits), int32 (N,).  The
        key is an unsigned 32-bit pattern; with more than 2**24 cells bit 31 may
        be set and the int32 view is then negative (use `keys.view(torch.uint32)`
        or mask after shifting).
      particle_index: original index of every sorted particle, int32 (N,).
      cell_counts: particles per cell, int32 (C,).
      cell_start: exclusive prefix sum of cell_counts, int32 (C + 1,).
    """
    keys: torch.Tensor
    particle_index: torch.Tensor
    cell_counts: torch.Tensor
    cell_start: torch.Tensor


class SortedParticles(NamedTuple):
    """Output of `sort_and_gather_particles`."""
    order: SortResult
    positions: Tuple[torch.Tensor, torch.Tensor, torch.Tensor]
    velocity: torch.Tensor


_workspaces = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """One cached scratch buffer per device and stream, grown on demand (with an eighth
    of headroom, so that a particle count that creeps up from call to call does not
    reallocate gigabytes every time)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = None
        _workspaces.pop(key, None)  # release the old buffer before asking for the new one
        buf = torch.empty(max(nbytes + nbytes // 8, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def native_grid(grid: CellGrid, ix_offset: int = 0,
                nx_local: Optional[int] = None) -> _native.AetherGrid:
    """Kernel scalars of a grid; the inverse spacing is computed in double and
    rounded to float32 exactly as the reference driver does
    (fused_radix_sort.py:250)."""
    inv = [c / (h - l) for l, h, c in zip(grid.lo, grid.hi, grid.cells)]
    nx, ny, nz = (int(c) for c in grid.cells)
    return _native.AetherGrid(float(grid.lo[0]), float(grid.lo[1]), float(grid.lo[2]),
                              inv[0], inv[1], inv[2], nx, ny, nz, int(ix_offset),
                              nx if nx_local is None else int(nx_local))


def _check_positions(x, y, z):
    for t in (x, y, z):
        if (not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.float32
                or t.numel() != x.numel()):
            raise ValueError('Positions must be float32 CUDA tensors of the '
                             'same length.')
    if x.numel() > MAX_PARTICLES:
        raise ValueError(f'At most {MAX_PARTICLES} particles per sort.')
    return tuple(t.contiguous().view(-1) for t in (x, y, z))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def sort_particles_by_cell(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor,
                           grid: CellGrid, seed: int, *, ix_offset: int = 0,
                           nx_local: Optional[int] = None) -> SortResult:
    """Bins particles by collision cell (shuffled in-cell) on the GPU.

    Args:
      x: particle x positions, float32 CUDA tensor (N,).
      y: particle y positions, float32 CUDA tensor (N,).
      z: particle z positions, float32 CUDA tensor (N,).
      grid: collision-cell grid.
      seed: Philox key (any non-negative integer below 2**64); use a different
        value every timestep.
      ix_offset, nx_local: sort over the x-slab [ix_offset, ix_offset + nx_local)
        of the grid with slab-local cell ids (multi-GPU decomposition).  The
        defaults sort over the whole grid, as the reference does.

    Returns:
      The sorted keys, permutation, and per-cell counts and offsets, as fresh
      tensors on `x.device`.  The work is enqueued on the current stream.

    Raises:
      ValueError: if the inputs are not float32 CUDA tensors of equal size, or
        the keys would need more than 32 bits.
      RuntimeError: if a kernel launch fails.
    """
    x, y, z = _check_positions(x, y, z)
    lib = _native.load_library()
    g = native_grid(grid, ix_offset, nx_local)
    cells = g.nx_local * g.ny * g.nz
    num_passes(cells)  # raises ValueError when the key does not fit
    n, device = x.numel(), x.device
    with torch.cuda.device(device):
        keys = torch.empty(n, dtype=torch.int32, device=device)
        index = torch.empty(n, dtype=torch.int32, device=device)
        counts = torch.empty(cells, dtype=torch.int32, device=device)
        start = torch.empty(cells + 1, dtype=torch.int32, device=device)
        nbytes = lib.AetherSortWorkspaceBytes(n, cells, 0)
        ws = _workspace(device, nbytes)
        stream = torch.cuda.current_stream(device).cuda_stream
        _native.check(lib.AetherSortParticlesByCell(
            _ptr(x), _ptr(y), _ptr(z), n, ctypes.byref(g), int(seed) & 0xFFFFFFFFFFFFFFFF,
            _ptr(keys), _ptr(index), _ptr(counts), _ptr(start), _ptr(ws), ws.numel(),
            ctypes.c_void_p(stream)), 'AetherSortParticlesByCell')
    return SortResult(keys, index, counts, start)


def sort_and_gather_particles(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor,
                              velocity: torch.Tensor, grid: CellGrid, seed: int, *,
                              ix_offset: int = 0, nx_local: Optional[int] = None,
                              path: int = PATH_AUTO,
                              padded_out: Optional[int] = None,
                              out: Optional[SortedParticles] = None,
                              push: Optional[tuple] = None) -> SortedParticles:
    """Sorts by cell and returns the particle payload in sorted order.

    One call for lines 105-109 of the reference's DSMC step
    (dsmc_gpu_pipeline.py): the sort, then positions and velocities gathered by
    the permutation.

    Args:
      x, y, z: float32 CUDA tensors (N,).
      velocity: float32 CUDA tensor (3, padded), rows vx, vy, vz, padded >= N
        (the reference keeps padded = ceil(N / 4) * 4, dsmc_gpu_pipeline.py:69-71).
      grid, seed, ix_offset, nx_local: as in `sort_particles_by_cell`.
      path: PATH_AUTO, PATH_DIGIT_PASSES or PATH_BUCKETED (same results).
      padded_out: row stride of the sorted velocity (default: that of the input).
      out: result tensors of an earlier call with the same sizes to write into
        instead of allocating (a stepping loop alternates between two sets).
      push: (dt, lo, hi) to fuse the move stage into the sort: particles are taken
        at x + v*dt with specular reflection at the box faces lo, hi (three floats
        each; the arithmetic of `fused_particle_push`), and the sorted payload
        carries the moved positions and reflected velocities.  The inputs are
        not modified.

    Returns:
      SortedParticles(order, (x, y, z) sorted, velocity sorted (3, padded) with
      zero padding columns).
    """
    x, y, z = _check_positions(x, y, z)
    n, device = x.numel(), x.device
    if (not isinstance(velocity, torch.Tensor) or not velocity.is_cuda
            or velocity.dtype != torch.float32 or velocity.dim() != 2
            or velocity.shape[0] != 3 or velocity.shape[1] < n):
        raise ValueError('Velocity must be a float32 CUDA tensor of shape (3, padded) '
                         'with padded >= N.')
    if velocity.stride(1) != 1:
        velocity = velocity.contiguous()
    padded = velocity.stride(0) if velocity.shape[1] > 0 else velocity.shape[1]
    lib = _native.load_library()
    g = native_grid(grid, ix_offset, nx_local)
    cells = g.nx_local * g.ny * g.nz
    num_passes(cells)
    with torch.cuda.device(device):
        padded_sorted = padded if padded_out is None else int(padded_out)
        if padded_sorted < n:
            raise ValueError('padded_out must be at least the number of particles.')
        if out is not None:
            (keys, index, counts, start), (xs, ys, zs), vs = out
            if (keys.numel() != n or index.numel() != n or counts.numel() != cells
                    or start.numel() != cells + 1 or any(t.numel() != n for t in (xs, ys, zs))
                    or tuple(vs.shape) != (3, padded_sorted) or vs.device != device):
                raise ValueError('`out` does not match the sizes of this call.')
        else:
            keys = torch.empty(n, dtype=torch.int32, device=device)
            index = torch.empty(n, dtype=torch.int32, device=device)
            counts = torch.empty(cells, dtype=torch.int32, device=device)
            start = torch.empty(cells + 1, dtype=torch.int32, device=device)
            xs, ys, zs = (torch.empty(n, dtype=torch.float32, device=device) for _ in range(3))
            vs = torch.empty((3, padded_sorted), dtype=torch.float32, device=device)
        if padded_sorted > n:
            vs[:, n:].zero_()
        nbytes = lib.AetherSortWorkspaceBytes(n, cells, 1)
        ws = _workspace(device, nbytes)
        stream = torch.cuda.current_stream(device).cuda_stream
        if push is None:
            _native.check(lib.AetherSortAndGatherParticles(
                _ptr(x), _ptr(y), _ptr(z), _ptr(velocity), padded, n, ctypes.byref(g),
                int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(keys), _ptr(index), _ptr(counts),
                _ptr(start), _ptr(xs), _ptr(ys), _ptr(zs), _ptr(vs), padded_sorted, int(path),
                _ptr(ws), ws.numel(), ctypes.c_void_p(stream)), 'AetherSortAndGatherParticles')
        else:
            dt, lo, hi = push
            _native.check(lib.AetherPushSortAndGatherParticles(
                _ptr(x), _ptr(y), _ptr(z), _ptr(velocity), padded, n, float(dt),
                (ctypes.c_float * 3)(*[float(v) for v in lo]),
                (ctypes.c_float * 3)(*[float(v) for v in hi]), ctypes.byref(g),
                int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(keys), _ptr(index), _ptr(counts),
                _ptr(start), _ptr(xs), _ptr(ys), _ptr(zs), _ptr(vs), padded_sorted, int(path),
                _ptr(ws), ws.numel(), ctypes.c_void_p(stream)),
                'AetherPushSortAndGatherParticles')
    return SortedParticles(SortResult(keys, index, counts, start), (xs, ys, zs), vs)


def last_sort_status(device=None) -> int:
    """Synchronises and returns the device status of the last sort on the
    current stream of `device`: 0 when clean, nonzero when a bounded device
    wait gave up (the results of that call are then invalid)."""
    device = torch.device('cuda', torch.cuda.current_device()) if device is None else device
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        return 0
    lib = _native.load_library()
    status = ctypes.c_int32(0)
    with torch.cuda.device(device):
        _native.check(lib.AetherSortReadStatus(_ptr(ws), ctypes.c_void_p(key[1]),
                                               ctypes.byref(status)), 'AetherSortReadStatus')
    return status.value


def last_sort_used_digit_passes(device=None) -> bool:
    """Synchronises and tells whether the last sort on the current stream of
    `device` was handed from the bucketed path to the digit passes on the device
    (same results, slower)."""
    device = torch.device('cuda', torch.cuda.current_device()) if device is None else device
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        return False
    lib = _native.load_library()
    used = ctypes.c_int32(0)
    with torch.cuda.device(device):
        _native.check(lib.AetherSortReadUsedDigitPasses(_ptr(ws), ctypes.c_void_p(key[1]),
                                                        ctypes.byref(used)),
                      'AetherSortReadUsedDigitPasses')
    return bool(used.value)
