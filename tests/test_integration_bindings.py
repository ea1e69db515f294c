"""The two reference-side bindings of INTEGRATION.md, executed as written.

Option A aliases this package's modules under the reference's module names, so that the
reference's callers run unchanged; the body of the reference's DSMC step
(project_aether/src/physics_engine/dsmc_gpu_pipeline.py:100-112) is restated here line for
line in terms of those module names and run through the aliases.  Option B is the ctypes
stub a maintainer would add beside the reference's `tma_collide.py`; it is pasted here and
called.  Both are checked against the CPU oracle.
"""

import ctypes
import sys
import types

import numpy as np
import pytest
import torch

import project_aether_b200 as pa
from oracle import sort_oracle as so

pytestmark = pytest.mark.gpu


def _install_option_a_aliases():
    """Applies the aliasing of INTEGRATION.md; returns the module names it added."""
    added = []
    # The reference's package tree (`src/custom_kernels/...`) exists where the reference is
    # installed; on a machine without it, empty packages stand in for the parents.
    for name in ('src', 'src.custom_kernels', 'src.custom_kernels.triton', 'src.custom_kernels.cuda'):
        if name not in sys.modules:
            module = types.ModuleType(name)
            module.__path__ = []
            sys.modules[name] = module
            added.append(name)
    # --- INTEGRATION.md, "The whole step" ---
    from project_aether_b200 import particle_sort, cell_grid, particle_push, ntc_collide
    sys.modules['src.custom_kernels.triton.fused_radix_sort'] = particle_sort
    sys.modules['src.custom_kernels.triton.radix_sort_reference'] = cell_grid
    sys.modules['src.custom_kernels.triton.fused_particle_push'] = particle_push
    sys.modules['src.custom_kernels.cuda.tma_collide'] = ntc_collide
    # --- end ---
    return added + ['src.custom_kernels.triton.fused_radix_sort',
                    'src.custom_kernels.triton.radix_sort_reference',
                    'src.custom_kernels.triton.fused_particle_push',
                    'src.custom_kernels.cuda.tma_collide']


def test_option_a_reference_step_body_runs_through_the_aliased_modules(cuda):
    added = _install_option_a_aliases()
    try:
        from src.custom_kernels.cuda import tma_collide
        from src.custom_kernels.triton import fused_particle_push
        from src.custom_kernels.triton import fused_radix_sort
        from src.custom_kernels.triton import radix_sort_reference
        # Names the reference's callers take from `radix_sort_reference`.
        assert radix_sort_reference.SHUFFLE_BITS == 7
        assert radix_sort_reference.num_passes(10_000) >= 1
        grid = radix_sort_reference.CellGrid((0.0, 0.0, 0.0), (1.0, 1.0, 0.64), (25, 25, 16))
        n, dt = 100_003, 1.0e-3
        rng = np.random.default_rng(11)
        pos = (rng.random((3, n)) * np.array(grid.hi)[:, None]).astype(np.float32)
        vel = rng.standard_normal((3, n)).astype(np.float32) * 20.0
        padded = -(-n // 4) * 4
        positions = [torch.as_tensor(pos[k], device=cuda) for k in range(3)]
        velocity = torch.zeros((3, padded), dtype=torch.float32, device=cuda)
        velocity[:, :n] = torch.as_tensor(vel, device=cuda)
        sigma_g_max = torch.full((grid.num_cells,), 1.0e-16, dtype=torch.float32, device=cuda)
        params = tma_collide.CollisionParams(0.0, 1.7e-18, 0.46, 0x5eed, 3)
        library = tma_collide.load_library()
        # The reference's step body, dsmc_gpu_pipeline.py:100-112.
        v = [velocity[c, :n] for c in range(3)]
        fused_particle_push.fused_particle_push(positions, v, dt, grid.lo, grid.hi)
        order = fused_radix_sort.sort_particles_by_cell(
            *positions, grid, seed=params.seed ^ (params.step << 20))
        index = order.particle_index.long()
        positions = [p.index_select(0, index) for p in positions]
        velocity[:, :n] = velocity[:, :n].index_select(1, index)
        collisions = torch.empty_like(order.cell_counts)
        tma_collide.collide(library, velocity, order.cell_start, sigma_g_max, collisions, n, params)
        torch.cuda.synchronize()
        # Oracle: push, then the sort contract; a zero selection factor selects no pairs.
        moved_p, moved_v = so.push_particles(list(pos), list(vel), dt, grid.lo, grid.hi)
        want = so.sort_particles(*moved_p, so.Grid(grid.lo, grid.hi, grid.cells),
                                 params.seed ^ (params.step << 20))
        assert np.array_equal(order.keys.cpu().numpy().view(np.uint32), want.keys)
        assert np.array_equal(order.particle_index.cpu().numpy(), want.particle_index)
        assert np.array_equal(order.cell_counts.cpu().numpy(), want.cell_counts)
        assert np.array_equal(order.cell_start.cpu().numpy(), want.cell_start)
        for k in range(3):
            assert np.array_equal(positions[k].cpu().numpy(), moved_p[k][want.particle_index])
            assert np.array_equal(velocity[k, :n].cpu().numpy(), moved_v[k][want.particle_index])
        assert int(collisions.sum()) == 0
    finally:
        for name in added:
            sys.modules.pop(name, None)


# --- INTEGRATION.md, Option B: src/custom_kernels/cuda/b200_sort.py, pasted ---

class AetherGrid(ctypes.Structure):
    _fields_ = [(n, ctypes.c_float) for n in ('x0', 'y0', 'z0', 'inv_dx', 'inv_dy', 'inv_dz')] + \
               [(n, ctypes.c_int32) for n in ('nx', 'ny', 'nz', 'ix_offset', 'nx_local')]


def load_library(path):
    lib = ctypes.CDLL(path)
    P, I64 = ctypes.c_void_p, ctypes.c_int64
    lib.AetherSortWorkspaceBytes.restype = ctypes.c_size_t
    lib.AetherSortWorkspaceBytes.argtypes = [I64, I64, ctypes.c_int]
    lib.AetherSortAndGatherParticles.restype = ctypes.c_int
    lib.AetherSortAndGatherParticles.argtypes = [P, P, P, P, I64, I64, ctypes.POINTER(AetherGrid),
        ctypes.c_uint64, P, P, P, P, P, P, P, P, I64, ctypes.c_int, P, ctypes.c_size_t, P]
    return lib


def sort_and_gather(lib, state, grid, seed, workspace):
    """Replaces dsmc_gpu_pipeline.py:105-109. `workspace` is a uint8 CUDA tensor of
    AetherSortWorkspaceBytes(n, grid.num_cells, 1) bytes kept across steps."""
    n, padded = state.num_particles, state.velocity.shape[1]
    inv = [c / (h - l) for l, h, c in zip(grid.lo, grid.hi, grid.cells)]
    g = AetherGrid(*grid.lo, *inv, *grid.cells, 0, grid.cells[0])
    dev = state.velocity.device
    keys, index = (torch.empty(n, dtype=torch.int32, device=dev) for _ in range(2))
    counts = torch.empty(grid.num_cells, dtype=torch.int32, device=dev)
    start = torch.empty(grid.num_cells + 1, dtype=torch.int32, device=dev)
    xs, ys, zs = (torch.empty_like(p) for p in state.positions)
    vs = torch.zeros_like(state.velocity)
    status = lib.AetherSortAndGatherParticles(
        *(p.data_ptr() for p in state.positions), state.velocity.data_ptr(), padded, n,
        ctypes.byref(g), seed, keys.data_ptr(), index.data_ptr(), counts.data_ptr(),
        start.data_ptr(), xs.data_ptr(), ys.data_ptr(), zs.data_ptr(), vs.data_ptr(), padded,
        0, workspace.data_ptr(), workspace.numel(), torch.cuda.current_stream().cuda_stream)
    if status != 0:
        raise RuntimeError(f'AetherSortAndGatherParticles failed with cudaError {status}')
    state.positions, state.velocity = [xs, ys, zs], vs
    return counts, start      # what tma_collide.collide and GpuStepStats need

# --- end of the pasted stub ---


def test_option_b_ctypes_stub_as_written(cuda):
    from project_aether_b200 import _native
    lib = load_library(_native.LIBRARY_PATH)
    grid = pa.CellGrid((0.1, -0.2, 0.0), (1.0, 1.0, 0.64), (37, 25, 16))
    n = 200_001
    rng = np.random.default_rng(5)
    lo, hi = np.array(grid.lo), np.array(grid.hi)
    pos = (rng.random((n, 3)) * (hi - lo) + lo).astype(np.float32)
    vel = rng.standard_normal((n, 3)).astype(np.float32)
    sigma0 = np.zeros(grid.num_cells, np.float32)
    with torch.cuda.device(cuda):
        state = pa.GpuDsmcState.from_numpy(pos, vel, sigma0, device=cuda)
        before_v = state.velocity.cpu().numpy()
        workspace = torch.empty(lib.AetherSortWorkspaceBytes(n, grid.num_cells, 1),
                                dtype=torch.uint8, device=cuda)
        seed = 0x5eed ^ (4097 << 20)  # wider than 32 bits, as steps beyond 4096 make it
        counts, start = sort_and_gather(lib, state, grid, seed, workspace)
        torch.cuda.synchronize()
    px = [np.ascontiguousarray(pos[:, k]) for k in range(3)]
    want = so.sort_particles(*px, so.Grid(grid.lo, grid.hi, grid.cells), seed)
    xs, ys, zs, vs = so.gather_payload(want.particle_index, *px, before_v)
    assert np.array_equal(counts.cpu().numpy(), want.cell_counts)
    assert np.array_equal(start.cpu().numpy(), want.cell_start)
    for got, ref in zip(state.positions, (xs, ys, zs)):
        assert np.array_equal(got.cpu().numpy(), ref)
    assert np.array_equal(state.velocity.cpu().numpy(), vs)
