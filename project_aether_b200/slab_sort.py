"""Multi-GPU particle sort: x-slab decomposition, one all-to-all, local sort.

The reference's particle path is single-device
(project_aether/src/physics_engine/dsmc_gpu_pipeline.py:85-113); this module is
the slab extension the benchmark definition asks for.  With G ranks (one per
GPU, `torch.distributed`), rank r owns the global columns
ix in [r*nx/G, (r+1)*nx/G).  One sort is

  1. a stable partition of the rank's particles by destination slab (CUDA,
     `AetherSlabPartition`);
  2. an exchange of the GxG counts and one variable-size all-to-all per payload
     array (NCCL over NVLink);
  3. the local sort with slab-local cell ids (`ix_offset`, `nx_local`).

Ordering rule, which fixes the Philox counter of every particle and so the
result: rank d's array after the exchange is the concatenation over source
ranks s = 0..G-1 of the particles s sent to d, each block in s's original order.
"""

import ctypes
from typing import List, NamedTuple, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _native
from .cell_grid import CellGrid
from .particle_sort import (PATH_AUTO, SortedParticles, SortResult, _workspace, native_grid,
                            sort_and_gather_particles)


class SlabParts(NamedTuple):
    arrays: Tuple[torch.Tensor, ...]  # x, y, z, vx, vy, vz ordered by destination
    counts: torch.Tensor              # int64 (world,), on the device


def slab_range(grid: CellGrid, world: int, rank: int) -> Tuple[int, int]:
    """(ix_offset, nx_local) of a rank's slab."""
    nx = grid.cells[0]
    if world < 1 or nx % world:
        raise ValueError(f'nx = {nx} is not divisible by {world} ranks')
    width = nx // world
    return rank * width, width


def partition_by_slab(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor,
                      velocity: torch.Tensor, grid: CellGrid, world: int) -> SlabParts:
    """Stable partition by destination rank on the GPU (no host synchronisation)."""
    n, device = x.numel(), x.device
    if not (x.is_cuda and velocity.is_cuda and velocity.dim() == 2 and velocity.shape[0] == 3
            and velocity.shape[1] >= n and x.dtype == torch.float32):
        raise ValueError('partition_by_slab needs float32 CUDA positions and a (3, padded) '
                         'float32 CUDA velocity.')
    slab_range(grid, world, 0)
    lib = _native.load_library()
    g = native_grid(grid)
    velocity = velocity.contiguous()
    with torch.cuda.device(device):
        outs = tuple(torch.empty(n, dtype=torch.float32, device=device) for _ in range(6))
        counts = torch.zeros(world, dtype=torch.int64, device=device)
        ws = _workspace(device, lib.AetherSlabPartitionWorkspaceBytes(n, world))
        stream = torch.cuda.current_stream(device).cuda_stream
        _native.check(lib.AetherSlabPartition(
            x.data_ptr(), y.data_ptr(), z.data_ptr(), velocity.data_ptr(), velocity.shape[1], n,
            ctypes.byref(g), world, *(o.data_ptr() for o in outs), counts.data_ptr(),
            ws.data_ptr(), ws.numel(), ctypes.c_void_p(stream)), 'AetherSlabPartition')
    return SlabParts(outs, counts)


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """All ranks' send counts: result[s, d] = particles rank s sends to rank d (on the host)."""
    world = dist.get_world_size(group)
    gathered = [torch.empty_like(send_counts) for _ in range(world)]
    dist.all_gather(gathered, send_counts, group=group)
    return torch.stack(gathered).cpu()


def exchange_particles(arrays: Sequence[torch.Tensor], matrix: torch.Tensor, group=None,
                       out: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
    """One variable-size all-to-all per array.  `arrays` are ordered by destination;
    `matrix[s, d]` is the host-side count matrix.  Returns the received arrays, each the
    concatenation of the blocks from source 0..G-1.  `out`, if given, are contiguous 1-D
    tensors of the right length to receive into (e.g. rows of a (3, padded) velocity)."""
    rank = dist.get_rank(group)
    send = [int(c) for c in matrix[rank]]
    recv = [int(c) for c in matrix[:, rank]]
    if sum(send) != arrays[0].numel():
        raise RuntimeError(f'rank {rank}: send counts {sum(send)} do not match the '
                           f'{arrays[0].numel()} partitioned particles')
    received = []
    for k, a in enumerate(arrays):
        r = out[k] if out is not None else torch.empty(sum(recv), dtype=a.dtype, device=a.device)
        if r.numel() != sum(recv):
            raise RuntimeError(f'rank {rank}: receive buffer holds {r.numel()}, needs {sum(recv)}')
        dist.all_to_all_single(r, a, output_split_sizes=recv, input_split_sizes=send, group=group)
        received.append(r)
    return received


class PeerBuffers:
    """Receive buffers of all ranks, mapped into every rank's address space
    (`torch.distributed._symmetric_memory`): 6 arrays of `capacity` floats per rank,
    [x | y | z | vx | vy | vz].  The fused partition + exchange kernel stores into
    them over NVLink."""

    def __init__(self, capacity: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.capacity = -(-int(capacity) // 4) * 4
        self.buffer = symm_mem.empty(6 * self.capacity, dtype=torch.float32, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, group if group is not None
                                          else dist.group.WORLD)
        self.pointers = [int(p) for p in self.handle.buffer_ptrs]
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)

    def views(self, n: int):
        """(x, y, z, velocity(3, capacity)) of the first n received particles."""
        c = self.capacity
        b = self.buffer
        return b[0:n], b[c:c + n], b[2 * c:2 * c + n], b[3 * c:6 * c].view(3, c)


_peer_buffers = {}


def _buffers_for(capacity: int, device: torch.device, group) -> PeerBuffers:
    key = (device.index, id(group))
    have = _peer_buffers.get(key)
    if have is None or have.capacity < capacity:
        # Collective: every rank takes this branch together, because the capacity asked for
        # is computed from the count matrix that all ranks hold.
        have = PeerBuffers(int(capacity * 1.25) + 1024, device, group)
        _peer_buffers[key] = have
    return have


def peer_exchange_sort(x, y, z, velocity, grid: CellGrid, seed: int, group=None,
                       path: int = PATH_AUTO, mark=lambda name: None,
                       push: Optional[tuple] = None) -> SortedParticles:
    """distributed_sort with the partition and the exchange fused: one kernel reads the
    rank's particles once and stores each into its destination GPU's receive buffer over
    NVLink.  The count all-gather before it and a one-word all-reduce after it are the only
    collectives.  The kernel reads the gathered counts on the device, so the host waits for
    them (it needs its own receive count to launch the local sort) while the exchange runs.
    With `push` = (dt, lo, hi) the count and exchange kernels take every particle as it is
    after the move stage, so the particles arrive moved and the inputs stay untouched."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    ix_offset, nx_local = slab_range(grid, world, rank)
    n, device = x.numel(), x.device
    lib = _native.load_library()
    g = native_grid(grid)
    if velocity.stride(1) != 1:
        velocity = velocity.contiguous()
    key = (device.index, id(group))
    with torch.cuda.device(device):
        current = torch.cuda.current_stream(device)
        stream = ctypes.c_void_p(current.cuda_stream)
        counts = torch.zeros(world, dtype=torch.int64, device=device)
        part_bytes = lib.AetherSlabPartitionWorkspaceBytes(n, world)
        part_ws = torch.empty(-(-part_bytes // (1 << 20)) * (1 << 20), dtype=torch.uint8,
                              device=device)
        if push is None:
            _native.check(lib.AetherSlabExchangeCount(
                x.data_ptr(), n, ctypes.byref(g), world, counts.data_ptr(), part_ws.data_ptr(),
                part_ws.numel(), stream), 'AetherSlabExchangeCount')
        else:
            dt = float(push[0])
            lo = (ctypes.c_float * 3)(*[float(c) for c in push[1]])
            hi = (ctypes.c_float * 3)(*[float(c) for c in push[2]])
            _native.check(lib.AetherSlabExchangeCountMoved(
                x.data_ptr(), velocity.data_ptr(), n, dt, lo, hi, ctypes.byref(g), world,
                counts.data_ptr(), part_ws.data_ptr(), part_ws.numel(), stream),
                'AetherSlabExchangeCountMoved')
        mark('partition')
        # The all-gather also orders this step after the peers' previous sort.
        matrix_dev = torch.empty((world, world), dtype=torch.int64, device=device)
        dist.all_gather_into_tensor(matrix_dev, counts, group=group)
        gathered = torch.cuda.Event()
        gathered.record(current)
        mark('counts')
        buffers = _peer_buffers.get(key)
        while True:
            if buffers is not None:
                pointers = (ctypes.c_void_p * world)(*buffers.pointers)
                error = torch.zeros(1, dtype=torch.int32, device=device)
                if push is None:
                    _native.check(lib.AetherSlabExchangeScatter(
                        x.data_ptr(), y.data_ptr(), z.data_ptr(), velocity.data_ptr(),
                        velocity.stride(0), n, ctypes.byref(g), world, rank, pointers,
                        buffers.capacity, matrix_dev.data_ptr(), error.data_ptr(),
                        part_ws.data_ptr(), part_ws.numel(), stream), 'AetherSlabExchangeScatter')
                else:
                    _native.check(lib.AetherSlabExchangeScatterMoved(
                        x.data_ptr(), y.data_ptr(), z.data_ptr(), velocity.data_ptr(),
                        velocity.stride(0), n, dt, lo, hi, ctypes.byref(g), world, rank, pointers,
                        buffers.capacity, matrix_dev.data_ptr(), error.data_ptr(),
                        part_ws.data_ptr(), part_ws.numel(), stream),
                        'AetherSlabExchangeScatterMoved')
                # Every rank's stores must have landed before anyone reads its buffer.
                dist.all_reduce(buffers.flag, group=group)
            # Fetch the counts on a side stream so that the copy does not queue behind the
            # exchange kernel.
            side = _side_stream(device)
            side.wait_event(gathered)
            with torch.cuda.stream(side):
                matrix = matrix_dev.to('cpu', non_blocking=True)
            side.synchronize()
            received = matrix.sum(dim=0)
            if buffers is not None and int(received.max()) <= buffers.capacity:
                break
            # First call, or a rank would receive more than the buffers hold: (re)allocate,
            # collectively, and run the exchange again.  Nobody may still be storing into
            # the buffers that are about to be dropped.
            torch.cuda.synchronize(device)
            dist.barrier(group=group)
            buffers = _buffers_for(int(received.max()), device, group)
        mark('exchange')
        m = int(received[rank])
        rx, ry, rz, rv = buffers.views(m)
        # The results are cut out of allocations of the buffers' capacity: the number of
        # particles a rank holds changes a little from step to step, and allocations whose
        # size changes every step defeat torch's caching allocator (a stall of tens of
        # milliseconds whenever it has to return its cache to the driver).
        cap, padded_out = buffers.capacity, -(-m // 4) * 4
        cells = nx_local * grid.cells[1] * grid.cells[2]

        def cut(dtype):
            return torch.empty(cap, dtype=dtype, device=device)[:m]

        order = SortResult(cut(torch.int32), cut(torch.int32),
                           torch.empty(cells, dtype=torch.int32, device=device),
                           torch.empty(cells + 1, dtype=torch.int32, device=device))
        vs = torch.empty(3 * cap, dtype=torch.float32, device=device)[:3 * padded_out].view(
            3, padded_out)
        results = SortedParticles(order, (cut(torch.float32), cut(torch.float32),
                                          cut(torch.float32)), vs)
        out = sort_and_gather_particles(rx, ry, rz, rv, grid, seed, ix_offset=ix_offset,
                                        nx_local=nx_local, path=path, padded_out=padded_out,
                                        out=results)
        mark('sort')
    return out


_side_streams = {}


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    s = _side_streams.get(device.index)
    if s is None:
        s = torch.cuda.Stream(device=device)
        _side_streams[device.index] = s
    return s


def distributed_sort(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor, velocity: torch.Tensor,
                     grid: CellGrid, seed: int, group=None, path: int = PATH_AUTO,
                     marks: Optional[list] = None, exchange: str = 'peer',
                     push: Optional[tuple] = None) -> SortedParticles:
    """Sorts the particles of all ranks by cell; every rank ends with its slab's
    particles, cell-sorted, with slab-local `cell_counts` / `cell_start`.

    `exchange`: 'peer' fuses the partition with the exchange (stores into the peers'
    receive buffers over NVLink); 'nccl' partitions locally and calls one NCCL all-to-all per
    payload array.  Same result either way.
    `marks`, if given, receives (name, cuda event) pairs recorded on the current stream
    after each phase (partition, counts, exchange, sort), for phase timing.
    `push` = (dt, lo, hi) fuses the move stage (x += v*dt, specular walls) into the step: the
    'peer' exchange moves the particles inside its count and exchange kernels; the 'nccl'
    form moves a copy first.  The inputs are not modified."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    ix_offset, nx_local = slab_range(grid, world, rank)
    if world == 1:
        return sort_and_gather_particles(x, y, z, velocity, grid, seed, path=path, push=push)

    def mark(name):
        if marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

    mark('begin')
    if exchange == 'peer':
        return peer_exchange_sort(x, y, z, velocity, grid, seed, group, path, mark, push)
    if push is not None:
        from .particle_push import fused_particle_push
        n_in = x.numel()
        x, y, z, velocity = x.clone(), y.clone(), z.clone(), velocity.clone()
        fused_particle_push([x, y, z], [velocity[k, :n_in] for k in range(3)], *push)
    parts = partition_by_slab(x, y, z, velocity, grid, world)
    mark('partition')
    matrix = exchange_counts(parts.counts, group)
    mark('counts')
    n = int(matrix[:, rank].sum())
    padded = -(-n // 4) * 4
    device = x.device
    rx, ry, rz = (torch.empty(n, dtype=torch.float32, device=device) for _ in range(3))
    rv = torch.empty((3, padded), dtype=torch.float32, device=device)
    if padded > n:
        rv[:, n:].zero_()
    exchange_particles(parts.arrays, matrix, group,
                       out=(rx, ry, rz, rv[0, :n], rv[1, :n], rv[2, :n]))
    mark('exchange')
    out = sort_and_gather_particles(rx, ry, rz, rv, grid, seed, ix_offset=ix_offset,
                                    nx_local=nx_local, path=path)
    mark('sort')
    return out
