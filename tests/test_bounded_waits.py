"""The give-up paths of the bounded device waits, exercised without hanging or faulting a GPU.

The reference's look-back spins until its predecessor publishes
(project_aether/src/custom_kernels/triton/fused_radix_sort.py:160-171); here every device
wait has a poll limit after which the kernel records a code and returns, so the context
stays usable.  These tests make a wait run out on purpose -- a status word that nothing
will ever publish, a receive buffer too small for what is sent -- and read the code back.
"""

import ctypes
import time

import numpy as np
import pytest
import torch

import project_aether_b200 as pa
from project_aether_b200 import _native
from project_aether_b200.particle_sort import native_grid

pytestmark = pytest.mark.gpu

ERR_LOOKBACK_TIMEOUT, ERR_RECEIVE_OVERFLOW = 1, 5


def test_lookback_gives_up_after_its_poll_limit_and_reports(cuda):
    lib = _native.load_library()
    with torch.cuda.device(cuda):
        nbytes = lib.AetherSortProbeLookbackWorkspaceBytes()
        ws = torch.empty(nbytes, dtype=torch.uint8, device=cuda)
        stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
        status = ctypes.c_int32(-1)
        torch.cuda.synchronize()
        for poll_limit in (0, 8):
            t0 = time.perf_counter()
            _native.check(lib.AetherSortProbeLookbackGiveUp(ws.data_ptr(), ws.numel(), poll_limit,
                                                            stream), 'AetherSortProbeLookbackGiveUp')
            _native.check(lib.AetherSortReadStatus(ws.data_ptr(), stream, ctypes.byref(status)),
                          'AetherSortReadStatus')
            elapsed = time.perf_counter() - t0
            assert status.value == ERR_LOOKBACK_TIMEOUT
            assert elapsed < 0.5, 'the wait must run out within milliseconds'
        # The context is still usable and an ordinary sort on the same workspace is clean.
        grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (16, 16, 16))
        x, y, z = (torch.rand(50_000, device=cuda) for _ in range(3))
        r = pa.sort_particles_by_cell(x, y, z, grid, 1)
        assert pa.last_sort_status(cuda) == 0
        assert int(r.cell_counts.sum()) == 50_000
        # A workspace that is too small is refused before any launch.
        assert lib.AetherSortProbeLookbackGiveUp(ws.data_ptr(), 1024, 8, stream) == 1


def test_exchange_refuses_to_overflow_a_receive_buffer(cuda):
    """world = 1: the rank's own receive buffer is the only destination.  With a capacity
    below the particle count the exchange kernel stores nothing and sets its error word."""
    lib = _native.load_library()
    n, capacity = 10_000, 4096
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (8, 8, 8))
    g = native_grid(grid)
    with torch.cuda.device(cuda):
        x, y, z = (torch.rand(n, device=cuda) for _ in range(3))
        v = torch.randn((3, n), device=cuda)
        counts = torch.zeros(1, dtype=torch.int64, device=cuda)
        ws = torch.empty(lib.AetherSlabPartitionWorkspaceBytes(n, 1), dtype=torch.uint8, device=cuda)
        stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
        _native.check(lib.AetherSlabExchangeCount(x.data_ptr(), n, ctypes.byref(g), 1,
                                                  counts.data_ptr(), ws.data_ptr(), ws.numel(),
                                                  stream), 'AetherSlabExchangeCount')
        sentinel = 12345.0
        buffer = torch.full((6 * capacity,), sentinel, device=cuda)
        error = torch.zeros(1, dtype=torch.int32, device=cuda)
        pointers = (ctypes.c_void_p * 1)(buffer.data_ptr())
        matrix = counts.clone().view(1, 1)
        _native.check(lib.AetherSlabExchangeScatter(
            x.data_ptr(), y.data_ptr(), z.data_ptr(), v.data_ptr(), n, n, ctypes.byref(g), 1, 0,
            pointers, capacity, matrix.data_ptr(), error.data_ptr(), ws.data_ptr(), ws.numel(),
            stream), 'AetherSlabExchangeScatter')
        torch.cuda.synchronize()
        assert int(counts) == n
        assert int(error) == ERR_RECEIVE_OVERFLOW
        assert bool((buffer == sentinel).all()), 'nothing may be stored past a full buffer'
        # The same call with room stores everything, in order, and leaves the error word clear.
        capacity = 10_240
        buffer = torch.full((6 * capacity,), sentinel, device=cuda)
        error.zero_()
        pointers = (ctypes.c_void_p * 1)(buffer.data_ptr())
        _native.check(lib.AetherSlabExchangeScatter(
            x.data_ptr(), y.data_ptr(), z.data_ptr(), v.data_ptr(), n, n, ctypes.byref(g), 1, 0,
            pointers, capacity, matrix.data_ptr(), error.data_ptr(), ws.data_ptr(), ws.numel(),
            stream), 'AetherSlabExchangeScatter')
        torch.cuda.synchronize()
        assert int(error) == 0
        assert torch.equal(buffer[:n], x) and torch.equal(buffer[5 * capacity:5 * capacity + n], v[2])
