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

import numpy as np
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


FLAG_WORDS = 1024          # words reserved in front of a receive buffer for the arrival flags
MAX_SLICES = 32            # kMaxSlices of the library
WAIT_POLLS = 1 << 22       # polls (256 ns apart: about a second) before a slice wait gives up


# How the sliced exchange shares the GPU with the local sort (set with `configure`).
_settings = {
    'overlap': None,          # None: up to four ranks
    'resident_blocks': None,  # exchange blocks per multiprocessor beside the sort; None: 0
    'sort_stream': None,      # None: a high-priority stream of its own from four ranks on
    'transport': None,        # None: 'copies' up to four ranks, 'stores' beyond
}


def configure(overlap: Optional[bool] = None, resident_blocks: Optional[int] = None,
              sort_stream: Optional[bool] = None, transport: Optional[str] = None) -> None:
    """Tuning of `distributed_sort(exchange='peer')`; None restores a default.

    transport: 'copies' (default up to four ranks) — the exchange kernel partitions into
      staging buffers in this GPU's own memory, laid out like the destinations' receive buffers
      (a rank's own share goes straight into its receive buffer), and one device-to-device
      copy per destination and slice (six rows, one per array) carries the data over NVLink on
      the copy engines, so that the multiprocessors are free for the local sort while the
      links are busy.  The host has to know the counts before it can enqueue the copies (one
      wait per step for the count all-gather).  'stores' (default beyond four ranks) — the
      exchange kernel stores every particle straight into its destination GPU's receive
      buffer over NVLink (no staging memory, no host wait), and occupies multiprocessors for
      as long as the links take.
    overlap: run the local sort's count and scatter kernels beside the exchange, slice by
      slice.  Default: up to four ranks.  Beyond, a rank's share is small, the slices' many
      short launches and copies cost more than the overlap gains, and the exchange runs in
      one piece with the ordinary local sort behind it.
    resident_blocks ('stores' only): thread blocks of the exchange kernel per multiprocessor
      while it runs beside the sort (1..4), or 0 for one block per tile, which lets the sort's
      kernels take the multiprocessors over as the exchange's blocks retire.  Default 0.
    sort_stream: run the sliced local sort on a high-priority stream of its own instead of the
      caller's stream.  Default: from four ranks on.
    Measured on the 256 M configuration, ms per step.  Two ranks: 'stores' one after the other
    8.8–9.9, overlapped 9.5; 'copies' one after the other 9.7, overlapped 8.2 (caller's stream)
    and 8.5 (own stream).  Four ranks: 'stores' overlapped 5.36–5.46, one after the other 6.32;
    'copies' overlapped 4.74 (own stream) and 4.85 (caller's), one after the other 5.42.  Eight
    ranks: 'stores' one after the other 3.01, overlapped 3.54; 'copies' overlapped 3.25, one
    after the other 3.45.  About 500 GB/s per direction cross the links while all ranks send
    and receive at once, by stores and by copies alike."""
    if transport not in (None, 'stores', 'copies'):
        raise ValueError(f'unknown transport {transport!r}')
    _settings.update(overlap=overlap, resident_blocks=resident_blocks, sort_stream=sort_stream,
                     transport=transport)
    for state in _states.values():
        state.sort_stream = None


def overlap_default(world: int) -> bool:
    """Whether the local sort runs beside the exchange (see `configure`)."""
    return world <= 4 if _settings['overlap'] is None else bool(_settings['overlap'])


def transport_default(world: int) -> str:
    """How the particles cross NVLink (see `configure`)."""
    return ('copies' if world <= 4 else 'stores') if _settings['transport'] is None \
        else _settings['transport']


class PeerBuffers:
    """Receive buffers of all ranks, mapped into every rank's address space
    (`torch.distributed._symmetric_memory`).  Per rank: FLAG_WORDS words of arrival flags
    (word [s * slices + k] = last step in which source s stored its slice k), then 6 arrays
    of `capacity` floats [x | y | z | vx | vy | vz].  The fused partition + exchange kernel
    stores into them over NVLink."""

    def __init__(self, capacity: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.capacity = -(-int(capacity) // 4) * 4
        self.buffer = symm_mem.empty(FLAG_WORDS + 6 * self.capacity, dtype=torch.float32,
                                     device=device)
        self.handle = symm_mem.rendezvous(self.buffer, group if group is not None
                                          else dist.group.WORLD)
        base = [int(p) for p in self.handle.buffer_ptrs]
        self.flag_pointers = base
        self.pointers = [p + 4 * FLAG_WORDS for p in base]
        self.buffer[:FLAG_WORDS].zero_()
        self.data = self.buffer[FLAG_WORDS:]

    def views(self, n: int):
        """(x, y, z, velocity(3, capacity)) of the first n received particles."""
        c = self.capacity
        b = self.data
        return b[0:n], b[c:c + n], b[2 * c:2 * c + n], b[3 * c:6 * c].view(3, c)


class _ExchangeState:
    """What a rank keeps from step to step for one (device, process group)."""

    def __init__(self, device: torch.device):
        self.buffers: Optional[PeerBuffers] = None
        self.epoch = 0
        self.slices = 0            # slices agreed for the next step (0: not yet known)
        self.plan_n = 0            # particle count the next local sort is planned for
        self.device = device
        self.exchange_stream = torch.cuda.Stream(device=device)
        self.sort_stream = None      # created on demand (high priority)
        self.side_stream = torch.cuda.Stream(device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)
        self.exchange_events = None  # (begin, end) of the last exchange, when timing is on
        self.time_exchange = False
        # Transport by copy engine: staging buffers (one row per destination, laid out like a
        # receive buffer), a scratch flag array for the partition kernel's own signal, one
        # stream per destination for the copies and one for the signals behind them.
        self.staging = None
        self.scratch_flags = None
        self.copy_streams = {}
        self.signal_stream = None


_states = {}


def _state_for(device: torch.device, group) -> _ExchangeState:
    key = (device.index, id(group))
    state = _states.get(key)
    if state is None:
        state = _ExchangeState(device)
        _states[key] = state
    return state


def slices_for(largest_share: int) -> int:
    """Slices every rank cuts its input into.  A slice is one chunk of the local sort's record
    layout, whose measured optimum grows with the particle count: 2^22 particles up to 64 M
    particles per rank, 2^23 up to 128 M, 2^24 beyond."""
    share = int(largest_share)
    slice_particles = 1 << (22 if share <= (1 << 26) else 23 if share <= (1 << 27) else 24)
    return max(1, min(MAX_SLICES, -(-share // slice_particles)))


def copy_plan(counts, rank: int):
    """What rank `rank` copies, from the gathered counts[source][slice][destination]: per slice
    a list of (destination, first, count) over the other ranks, starting with the next one
    (so that the ranks do not all begin with the same destination): `count` particles of the
    slice go to `destination`, where they lie from index `first` of every array on — behind
    the blocks of the sources before `rank` and behind this rank's earlier slices.  The
    staging row for a destination uses the same indices."""
    counts = np.asarray(counts)
    world, slices = counts.shape[0], counts.shape[1]
    block = counts[:rank].sum(axis=(0, 1))
    before = counts[rank].cumsum(axis=0) - counts[rank]
    peers = [(rank + step) % world for step in range(1, world)]
    return [[(d, int(block[d] + before[k, d]), int(counts[rank, k, d])) for d in peers]
            for k in range(slices)]


def _exchange_by_copies(lib, state, buffers, matrix, x, y, z, velocity, n, move, g, world, rank,
                         totals, slices, epoch, part_ws):
    """The exchange with the copy engines as transport (see `configure`): the partition kernel
    writes slice by slice into staging rows in local memory (this rank's own share goes
    straight into its receive buffer), and as soon as the host knows the counts it enqueues,
    per slice and destination, one device-to-device copy (six rows, one per array) into the
    destination's receive buffer and behind them the slice's signal.  Returns the event behind the last signal, or
    None (nothing copied) when the counts say that some rank's buffer would overflow."""
    device, capacity = state.device, buffers.capacity
    if state.staging is None or state.staging.shape[1] != 6 * capacity:
        state.staging = torch.empty((world, 6 * capacity), dtype=torch.float32, device=device)
        state.scratch_flags = torch.zeros(FLAG_WORDS, dtype=torch.int32, device=device)
    if state.signal_stream is None:
        state.signal_stream = torch.cuda.Stream(device=device)
    for d in range(world):
        if d != rank and d not in state.copy_streams:
            state.copy_streams[d] = torch.cuda.Stream(device=device)
    rows = [buffers.pointers[rank] if d == rank else state.staging[d].data_ptr()
            for d in range(world)]
    part_pointers = (ctypes.c_void_p * world)(*rows)
    part_flags = (ctypes.c_void_p * world)(*([state.scratch_flags.data_ptr()] * world))
    flag_pointers = (ctypes.c_void_p * world)(*buffers.flag_pointers)
    stream = state.exchange_stream
    part_done = []
    with torch.cuda.stream(stream):
        if state.time_exchange:
            state.exchange_events = (torch.cuda.Event(enable_timing=True),
                                     torch.cuda.Event(enable_timing=True))
            state.exchange_events[0].record(stream)
        for k in range(slices):
            _native.check(lib.AetherSlabExchangeScatterSliced(
                x.data_ptr(), y.data_ptr(), z.data_ptr(), velocity.data_ptr(), velocity.stride(0),
                n, move[0] if move else 0.0, move[1] if move else None, move[2] if move else None,
                ctypes.byref(g), world, rank, part_pointers, capacity, totals.data_ptr(),
                state.error.data_ptr(), slices, k, epoch, part_flags, part_ws.data_ptr(),
                part_ws.numel(), ctypes.c_void_p(stream.cuda_stream)),
                'AetherSlabExchangeScatterSliced')
            done = torch.cuda.Event()
            done.record(stream)
            part_done.append(done)
    # The counts: where this rank's block lies in every destination's arrays, slice by slice.
    state.side_stream.synchronize()
    counts = matrix.numpy()                       # [source][slice][destination]
    if int(counts.sum(axis=(0, 1)).max()) > capacity:
        return None
    plan = copy_plan(counts, rank)
    signal = state.signal_stream
    for k in range(slices):
        signal.wait_event(part_done[k])
        for d, first, count in plan[k]:
            copy_stream = state.copy_streams[d]
            copy_stream.wait_event(part_done[k])
            if count:
                handle = ctypes.c_void_p(copy_stream.cuda_stream)
                _native.check(lib.AetherSlabExchangeCopy(  # six rows: x, y, z, vx, vy, vz
                    ctypes.c_void_p(buffers.pointers[d] + 4 * first),
                    ctypes.c_void_p(rows[d] + 4 * first), 4 * count, 6, 4 * capacity, handle),
                    'AetherSlabExchangeCopy')
            copied = torch.cuda.Event()
            copied.record(copy_stream)
            signal.wait_event(copied)
        _native.check(lib.AetherSlabExchangeSignal(
            world, rank, slices, k, epoch, flag_pointers, ctypes.c_void_p(signal.cuda_stream)),
            'AetherSlabExchangeSignal')
    if state.time_exchange:
        state.exchange_events[1].record(signal)
    sent = torch.cuda.Event()
    sent.record(signal)
    return sent


def peer_exchange_sort(x, y, z, velocity, grid: CellGrid, seed: int, group=None,
                       path: int = PATH_AUTO, mark=lambda name: None,
                       push: Optional[tuple] = None) -> SortedParticles:
    """distributed_sort with the partition and the exchange fused, and the exchange
    overlapped with the local sort.  One kernel reads the rank's particles once, slice by
    slice, on a stream of its own, and puts each where its destination GPU's receive buffer
    wants it: in staging rows that the copy engines then carry over NVLink, or (transport
    'stores') straight into the destination's memory; behind every slice the destinations are
    told that it is complete.  Meanwhile the local sort counts and scatters, slice by slice,
    what has arrived; only its finish kernels wait for the last slice.  The count all-gather
    before the exchange is the only collective of a step.  Buffer capacity, slice count and
    bucket widths come from the previous step's counts (a step whose counts outgrow the
    buffers is repeated); with 'stores' the host therefore waits for nothing until everything
    is enqueued, with 'copies' it waits once, for the gathered counts.
    With `push` = (dt, lo, hi) the count and exchange kernels take every particle as it is
    after the move stage, so the particles arrive moved and the inputs stay untouched."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    ix_offset, nx_local = slab_range(grid, world, rank)
    n, device = x.numel(), x.device
    lib = _native.load_library()
    g = native_grid(grid)
    local_grid = native_grid(grid, ix_offset, nx_local)
    cells = nx_local * grid.cells[1] * grid.cells[2]
    if velocity.stride(1) != 1:
        velocity = velocity.contiguous()
    state = _state_for(device, group)
    move = None
    if push is not None:
        move = (float(push[0]), (ctypes.c_float * 3)(*[float(c) for c in push[1]]),
                (ctypes.c_float * 3)(*[float(c) for c in push[2]]))
    with torch.cuda.device(device):
        current = torch.cuda.current_stream(device)
        stream = ctypes.c_void_p(current.cuda_stream)
        if state.slices == 0:
            # First step: agree on the slice count from the largest share.
            largest = torch.tensor([n], dtype=torch.int64, device=device)
            dist.all_reduce(largest, op=dist.ReduceOp.MAX, group=group)
            state.slices = slices_for(int(largest))
        part_bytes = lib.AetherSlabPartitionWorkspaceBytes(n, world)
        part_ws = torch.empty(-(-part_bytes // (1 << 20)) * (1 << 20), dtype=torch.uint8,
                              device=device)
        segments = torch.empty(lib.AetherSlabSegmentsBytes(), dtype=torch.uint8, device=device)
        overlap = overlap_default(world)
        while True:
            # Without overlap the exchange is one piece and the local sort is the ordinary one.
            slices = state.slices if overlap else 1
            counts = torch.zeros(world, dtype=torch.int64, device=device)
            slice_counts = torch.zeros(slices * world, dtype=torch.int64, device=device)
            if move is None:
                _native.check(lib.AetherSlabExchangeCount(
                    x.data_ptr(), n, ctypes.byref(g), world, counts.data_ptr(), part_ws.data_ptr(),
                    part_ws.numel(), stream), 'AetherSlabExchangeCount')
            else:
                _native.check(lib.AetherSlabExchangeCountMoved(
                    x.data_ptr(), velocity.data_ptr(), n, move[0], move[1], move[2],
                    ctypes.byref(g), world, counts.data_ptr(), part_ws.data_ptr(), part_ws.numel(),
                    stream), 'AetherSlabExchangeCountMoved')
            _native.check(lib.AetherSlabExchangeSliceCounts(
                n, world, slices, slice_counts.data_ptr(), part_ws.data_ptr(), part_ws.numel(),
                stream), 'AetherSlabExchangeSliceCounts')
            mark('partition')
            # The all-gather also orders this step after the peers' previous sort: nobody
            # still reads a receive buffer when the first store of this step arrives.
            matrix_dev = torch.empty((world, slices, world), dtype=torch.int64, device=device)
            dist.all_gather_into_tensor(matrix_dev, slice_counts, group=group)
            totals = torch.empty((world, world), dtype=torch.int64, device=device)
            _native.check(lib.AetherSlabExchangePrepare(
                matrix_dev.data_ptr(), world, slices, rank, totals.data_ptr(), segments.data_ptr(),
                stream), 'AetherSlabExchangePrepare')
            gathered = torch.cuda.Event()
            gathered.record(current)
            mark('counts')
            # The counts travel to the host on a side stream; the host looks at them only
            # after everything is enqueued (or at once, when there are no buffers yet).
            state.side_stream.wait_event(gathered)
            with torch.cuda.stream(state.side_stream):
                matrix = matrix_dev.to('cpu', non_blocking=True)
            buffers = state.buffers
            if buffers is None:
                state.side_stream.synchronize()
                received = matrix.sum(dim=(0, 1))
                torch.cuda.synchronize(device)
                dist.barrier(group=group)
                buffers = state.buffers = PeerBuffers(int(int(received.max()) * 1.25) + 1024,
                                                      device, group)
                state.plan_n = max(1, int(received[rank]))
                torch.cuda.synchronize(device)
                dist.barrier(group=group)  # every rank's flags are cleared before any store
                continue  # the step starts over with buffers in place (same counts)
            capacity = buffers.capacity
            state.epoch += 1
            epoch = state.epoch
            pointers = (ctypes.c_void_p * world)(*buffers.pointers)
            flag_pointers = (ctypes.c_void_p * world)(*buffers.flag_pointers)
            resident = _settings['resident_blocks']
            _native.check(lib.AetherSlabExchangeSetResidentBlocks(0 if resident is None else resident),
                          'AetherSlabExchangeSetResidentBlocks')
            state.exchange_stream.wait_event(gathered)
            by_copies = transport_default(world) == 'copies' and world > 1
            if by_copies:
                sent = _exchange_by_copies(lib, state, buffers, matrix, x, y, z, velocity, n, move,
                                           g, world, rank, totals, slices, epoch, part_ws)
                if sent is None:  # a rank would overflow its buffer: nothing was copied
                    torch.cuda.synchronize(device)
                    state.error.zero_()
                    dist.barrier(group=group)
                    state.buffers = None
                    state.staging = None
                    continue
            else:
                with torch.cuda.stream(state.exchange_stream):
                    if state.time_exchange:
                        state.exchange_events = (torch.cuda.Event(enable_timing=True),
                                                 torch.cuda.Event(enable_timing=True))
                        state.exchange_events[0].record(state.exchange_stream)
                    for k in range(slices):
                        _native.check(lib.AetherSlabExchangeScatterSliced(
                            x.data_ptr(), y.data_ptr(), z.data_ptr(), velocity.data_ptr(),
                            velocity.stride(0), n, move[0] if move else 0.0,
                            move[1] if move else None, move[2] if move else None, ctypes.byref(g),
                            world, rank, pointers, capacity, totals.data_ptr(),
                            state.error.data_ptr(), slices, k, epoch, flag_pointers,
                            part_ws.data_ptr(), part_ws.numel(),
                            ctypes.c_void_p(state.exchange_stream.cuda_stream)),
                            'AetherSlabExchangeScatterSliced')
                    if state.time_exchange:
                        state.exchange_events[1].record(state.exchange_stream)
                    sent = torch.cuda.Event()
                    sent.record(state.exchange_stream)
            rx, ry, rz, rv = buffers.views(capacity)
            plan_n = max(1, state.plan_n)
            flags = buffers.flag_pointers[rank]
            if not overlap or lib.AetherSortBucketPlan(plan_n, cells, None, None, None) != 0:
                # No overlap wanted, or the bucketed sort cannot take this many particles per
                # cell: wait for the whole exchange and hand the received arrays to the general
                # entry point.  The host needs the particle count for that; the counts reached
                # it while the exchange was running, so the GPU does not wait for the host.
                for k in range(slices):
                    _native.check(lib.AetherSlabExchangeWait(
                        flags, world, slices, k, epoch, WAIT_POLLS, state.error.data_ptr(), stream),
                        'AetherSlabExchangeWait')
                current.wait_event(sent)
                state.side_stream.synchronize()
                received = matrix.sum(dim=(0, 1))
                if int(received.max()) > capacity:
                    torch.cuda.synchronize(device)
                    state.error.zero_()
                    dist.barrier(group=group)
                    state.buffers = None
                    continue
                m = int(received[rank])
                state.plan_n = max(1, m)
                state.slices = slices_for(int(received.max()))
                mark('exchange')
                out = sort_and_gather_particles(rx[:m], ry[:m], rz[:m], rv, grid, seed,
                                                ix_offset=ix_offset, nx_local=nx_local, path=path,
                                                padded_out=-(-m // 4) * 4)
                mark('sort')
                return out
            # The local sort, slice by slice as the slices arrive (or, without overlap, once
            # this rank's own exchange kernels are through).  It runs on a high-priority stream
            # of its own, so that its short kernels take the multiprocessors over from the
            # exchange kernel's blocks, or on the caller's stream (see `configure`).
            own_stream = ((overlap and world >= 4) if _settings['sort_stream'] is None
                          else _settings['sort_stream'])
            if own_stream and state.sort_stream is None:
                state.sort_stream = torch.cuda.Stream(device=device, priority=-1)
            sort_on = state.sort_stream if own_stream else current
            handle = ctypes.c_void_p(sort_on.cuda_stream)
            if sort_on is not current:
                sort_on.wait_event(gathered)
            with torch.cuda.stream(sort_on):
                ws_bytes = lib.AetherSortSlicedWorkspaceBytes(capacity, plan_n, cells, slices)
                ws = _workspace(device, ws_bytes)
                if not overlap:
                    sort_on.wait_event(sent)
                _native.check(lib.AetherSortSlicedBegin(
                    capacity, plan_n, ctypes.byref(local_grid), slices, ws.data_ptr(), ws.numel(),
                    handle), 'AetherSortSlicedBegin')
                for k in range(slices):
                    _native.check(lib.AetherSlabExchangeWait(
                        flags, world, slices, k, epoch, WAIT_POLLS, state.error.data_ptr(), handle),
                        'AetherSlabExchangeWait')
                    _native.check(lib.AetherSortSlicedSlice(
                        rx.data_ptr(), ry.data_ptr(), rz.data_ptr(), rv.data_ptr(), capacity,
                        capacity, plan_n, ctypes.byref(local_grid), int(seed) & 0xFFFFFFFFFFFFFFFF,
                        segments.data_ptr(), slices, k, ws.data_ptr(), ws.numel(), handle),
                        'AetherSortSlicedSlice')
                if sort_on is current:
                    mark('exchange')
                # Results are cut out of allocations of the buffers' capacity: the number of
                # particles a rank holds changes a little from step to step, and allocations
                # whose size changes every step defeat torch's caching allocator.
                keys = torch.empty(capacity, dtype=torch.int32, device=device)
                index = torch.empty(capacity, dtype=torch.int32, device=device)
                cell_counts = torch.empty(cells, dtype=torch.int32, device=device)
                cell_start = torch.empty(cells + 1, dtype=torch.int32, device=device)
                xs, ys, zs = (torch.empty(capacity, dtype=torch.float32, device=device)
                              for _ in range(3))
                vs = torch.empty((3, capacity), dtype=torch.float32, device=device)
                _native.check(lib.AetherSortSlicedFinish(
                    capacity, plan_n, ctypes.byref(local_grid), segments.data_ptr(), slices,
                    keys.data_ptr(), index.data_ptr(), cell_counts.data_ptr(),
                    cell_start.data_ptr(), xs.data_ptr(), ys.data_ptr(), zs.data_ptr(),
                    vs.data_ptr(), capacity, ws.data_ptr(), ws.numel(), handle),
                    'AetherSortSlicedFinish')
            if sort_on is not current:
                current.wait_stream(sort_on)
                for t in (keys, index, cell_counts, cell_start, xs, ys, zs, vs):
                    t.record_stream(current)
                mark('exchange')
            current.wait_event(sent)  # the inputs may be reused once this step's work is done
            mark('sort')
            # Only now does the host look at the counts.
            state.side_stream.synchronize()
            received = matrix.sum(dim=(0, 1))
            largest = int(received.max())
            state.slices = slices_for(largest)
            if largest > capacity:
                # A rank would have received more than the buffers hold: nothing was stored
                # for it.  Grow the buffers (collectively) and repeat the step.
                torch.cuda.synchronize(device)
                state.error.zero_()
                dist.barrier(group=group)
                state.buffers = None
                state.slices = slices
                continue
            break
        m = int(received[rank])
        state.plan_n = max(1, m)
        padded_out = -(-m // 4) * 4
        velocity_out = vs[:, :padded_out]
        if padded_out > m:
            velocity_out[:, m:].zero_()
        out = SortedParticles(SortResult(keys[:m], index[:m], cell_counts, cell_start),
                              (xs[:m], ys[:m], zs[:m]), velocity_out)
    return out


def time_exchange(device: torch.device, enabled: bool, group=None) -> None:
    """Turns CUDA-event timing of the exchange kernels (all slices, on their own stream) on or
    off for the following steps on `device`."""
    _state_for(device, group).time_exchange = bool(enabled)


def last_exchange_ms(device: torch.device, group=None) -> Optional[float]:
    """Synchronises and returns the duration of the last timed exchange, or None."""
    state = _states.get((device.index, id(group)))
    if state is None or state.exchange_events is None:
        return None
    state.exchange_events[1].synchronize()
    return state.exchange_events[0].elapsed_time(state.exchange_events[1])


def exchange_status(device: torch.device, group=None) -> int:
    """Synchronises and returns the device status of the last sliced exchange on `device`:
    0 when clean, 5 when a receive buffer was too small, 6 when a slice wait ran out (the
    results of that step are then invalid)."""
    state = _states.get((device.index, id(group)))
    if state is None:
        return 0
    torch.cuda.synchronize(device)
    return int(state.error.item())


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
