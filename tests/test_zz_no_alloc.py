"""The allocation-free entry point against the ordinary one.

AetherSortParticlesByCellStatic serves callers that may not allocate device
memory (a plugin inside a host that owns the whole GPU memory pool, a real-time
step where cudaMalloc's device-wide synchronisation is banned): its scratch is
a fixed array inside the library.  Here it is called through the C ABI twice in
a row -- the second call finds the first call's leftovers in the shared scratch
-- and each result must equal, bit for bit, what AetherSortParticlesByCell
produces with a caller-provided workspace.  The file name sorts last so that a
run which stops at the first failure has already run every other test.
"""

import ctypes

import numpy as np
import pytest
import torch

import project_aether_b200 as pa
from project_aether_b200 import _native
from project_aether_b200.particle_sort import native_grid

pytestmark = pytest.mark.gpu


def _sort_with_workspace(lib, x, y, z, g, cells, seed):
    n, dev = x.numel(), x.device
    keys = torch.empty(n, dtype=torch.int32, device=dev)
    index = torch.empty(n, dtype=torch.int32, device=dev)
    counts = torch.empty(cells, dtype=torch.int32, device=dev)
    start = torch.empty(cells + 1, dtype=torch.int32, device=dev)
    ws = torch.empty(lib.AetherSortWorkspaceBytes(n, cells, 0), dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    _native.check(lib.AetherSortParticlesByCell(
        x.data_ptr(), y.data_ptr(), z.data_ptr(), n, ctypes.byref(g), seed, keys.data_ptr(),
        index.data_ptr(), counts.data_ptr(), start.data_ptr(), ws.data_ptr(), ws.numel(), stream),
        'AetherSortParticlesByCell')
    return keys, index, counts, start


def _sort_static(lib, x, y, z, g, cells, seed):
    n, dev = x.numel(), x.device
    keys = torch.empty(n, dtype=torch.int32, device=dev)
    index = torch.empty(n, dtype=torch.int32, device=dev)
    counts = torch.empty(cells, dtype=torch.int32, device=dev)
    start = torch.empty(cells + 1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    _native.check(lib.AetherSortParticlesByCellStatic(
        x.data_ptr(), y.data_ptr(), z.data_ptr(), n, ctypes.byref(g), seed, keys.data_ptr(),
        index.data_ptr(), counts.data_ptr(), start.data_ptr(), stream),
        'AetherSortParticlesByCellStatic')
    return keys, index, counts, start


def _static_status(lib, dev):
    """(device status, handed-over flag) of the last static call, read from the library's array."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    status, used = ctypes.c_int32(-1), ctypes.c_int32(-1)
    _native.check(lib.AetherSortStaticReadStatus(stream, ctypes.byref(status)),
                  'AetherSortStaticReadStatus')
    _native.check(lib.AetherSortStaticReadUsedDigitPasses(stream, ctypes.byref(used)),
                  'AetherSortStaticReadUsedDigitPasses')
    return status.value, used.value


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row(cuda):
    lib = _native.load_library()
    assert lib.AetherSortStaticMaxParticles() == 1 << 20
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (64, 64, 32))
    g = native_grid(grid)
    cells = grid.num_cells
    gen = torch.Generator(device=cuda).manual_seed(21)
    with torch.cuda.device(cuda):
        # Two different sizes and seeds, back to back on one stream: the second
        # call must not be disturbed by what the first left in the scratch.
        for n, seed in ((300_007, 11), (1 << 20, 0x1234500000007)):
            x, y, z = (torch.rand(n, device=cuda, generator=gen) for _ in range(3))
            got = _sort_static(lib, x, y, z, g, cells, seed)
            want = _sort_with_workspace(lib, x, y, z, g, cells, seed)
            assert _static_status(lib, cuda) == (0, 0)
            torch.cuda.synchronize()
            for a, b in zip(got, want):
                assert torch.equal(a, b)


def test_static_scratch_small_call_takes_the_bucketed_path_and_equals_the_oracle(cuda):
    """Below a few hundred thousand particles the bucketed record layout fits the library's
    array and that path runs; whichever path runs, the result is the CPU oracle's."""
    from oracle import sort_oracle as so
    lib = _native.load_library()
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (32, 32, 16))
    g = native_grid(grid)
    gen = torch.Generator(device=cuda).manual_seed(5)
    with torch.cuda.device(cuda):
        for n, seed in ((150_001, 3), (700_001, 4)):
            x, y, z = (torch.rand(n, device=cuda, generator=gen) for _ in range(3))
            got = _sort_static(lib, x, y, z, g, grid.num_cells, seed)
            assert _static_status(lib, cuda) == (0, 0)
            want = so.sort_particles(x.cpu().numpy(), y.cpu().numpy(), z.cpu().numpy(),
                                     so.Grid(grid.lo, grid.hi, grid.cells), seed)
            assert np.array_equal(got[0].cpu().numpy().view(np.uint32), want.keys)
            assert np.array_equal(got[1].cpu().numpy(), want.particle_index)
            assert np.array_equal(got[2].cpu().numpy(), want.cell_counts)
            assert np.array_equal(got[3].cpu().numpy(), want.cell_start)


def test_static_scratch_entry_rejects_sizes_beyond_its_limit(cuda):
    lib = _native.load_library()
    g = native_grid(pa.CellGrid((0., 0., 0.), (1., 1., 1.), (8, 8, 8)))
    x = torch.zeros(8, device=cuda)
    out = torch.empty(1024, dtype=torch.int32, device=cuda)
    rc = lib.AetherSortParticlesByCellStatic(
        x.data_ptr(), x.data_ptr(), x.data_ptr(), (1 << 20) + 1, ctypes.byref(g), 0,
        out.data_ptr(), out.data_ptr(), out.data_ptr(), out.data_ptr(), None)
    assert rc == 1  # cudaErrorInvalidValue, nothing launched
