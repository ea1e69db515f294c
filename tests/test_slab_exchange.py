"""Multi-GPU plumbing: the exchange on CPU ranks (gloo, world size 2 and 3), the
slab partition kernel against a stable NumPy partition, and all ranks of the
multi-GPU sort emulated one after another on one GPU."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import project_aether_b200 as pa
from oracle import sort_oracle as so
from project_aether_b200 import slab_sort


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _shares(world, n, seed=0):
    rng = np.random.default_rng(seed)
    return [tuple(rng.random(n + 17 * r, dtype=np.float32) for _ in range(6)) for r in range(world)]


GRID = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (12, 4, 2))


def _gloo_worker(rank, world, port, result_dir):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        ogrid = so.Grid(GRID.lo, GRID.hi, GRID.cells)
        share = _shares(world, 500)[rank]
        dest = so.slab_of(share[0], ogrid, world)
        order = np.argsort(dest, kind='stable')          # host stand-in for the CUDA partition
        arrays = [torch.from_numpy(a[order].copy()) for a in share]
        counts = torch.from_numpy(np.bincount(dest, minlength=world).astype(np.int64))
        matrix = slab_sort.exchange_counts(counts)
        got = slab_sort.exchange_particles(arrays, matrix)
        want = so.exchange_replay(_shares(world, 500), ogrid, world)[rank]
        for g, w in zip(got, want):
            np.testing.assert_array_equal(g.numpy(), w)
        # Inconsistent counts are caught before any data moves.
        bad = matrix.clone()
        bad[rank, 0] += 1
        with pytest.raises(RuntimeError):
            slab_sort.exchange_particles(arrays, bad)
        open(os.path.join(result_dir, f'ok{rank}'), 'w').close()
    finally:
        dist.destroy_process_group()


def _steady_start(world, rank):
    """A rank's particles at the start of the stepping loop: all inside its own slab."""
    width = (GRID.hi[0] - GRID.lo[0]) / world
    share = list(_shares(world, 400, seed=5)[rank])
    share[0] = (GRID.lo[0] + (rank + share[0] * 0.999) * width).astype(np.float32)
    share[3:] = [(a - 0.5).astype(np.float32) for a in share[3:]]
    return tuple(share)


def _steady_states(world, steps, dt):
    """The steady-state loop replayed in one process: a step moves every rank's particles,
    exchanges those that left the slab and sorts every slab again.  Returns the ranks' states
    after every step."""
    ogrid = so.Grid(GRID.lo, GRID.hi, GRID.cells)
    states = [_steady_start(world, r) for r in range(world)]
    history = []
    for step in range(steps):
        moved = []
        for st in states:
            p, q = so.push_particles(list(st[:3]), list(st[3:]), dt, GRID.lo, GRID.hi)
            moved.append(tuple(p) + tuple(q))
        received = so.exchange_replay(moved, ogrid, world)
        states = []
        for r, rec in enumerate(received):
            off, wid = slab_sort.slab_range(GRID, world, r)
            order = so.sort_particles(*rec[:3], ogrid, 1234 ^ (step << 20), ix_offset=off,
                                      nx_local=wid).particle_index
            states.append(tuple(a[order] for a in rec))
        history.append(states)
    return history


def _gloo_loop_worker(rank, world, port, result_dir):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        ogrid = so.Grid(GRID.lo, GRID.hi, GRID.cells)
        steps, dt = 4, 0.08
        want = _steady_states(world, steps, dt)
        state = _steady_start(world, rank)
        crossed = 0
        for step in range(steps):
            p, q = so.push_particles(list(state[:3]), list(state[3:]), dt, GRID.lo, GRID.hi)
            arrays = tuple(p) + tuple(q)
            dest = so.slab_of(arrays[0], ogrid, world)
            crossed += int((dest != rank).sum())
            order = np.argsort(dest, kind='stable')      # host stand-in for the CUDA partition
            parts = [torch.from_numpy(a[order].copy()) for a in arrays]
            counts = torch.from_numpy(np.bincount(dest, minlength=world).astype(np.int64))
            matrix = slab_sort.exchange_counts(counts)
            got = [t.numpy() for t in slab_sort.exchange_particles(parts, matrix)]
            off, wid = slab_sort.slab_range(GRID, world, rank)
            perm = so.sort_particles(*got[:3], ogrid, 1234 ^ (step << 20), ix_offset=off,
                                     nx_local=wid).particle_index
            state = tuple(a[perm] for a in got)
            for g, w in zip(state, want[step][rank]):
                np.testing.assert_array_equal(g, w)
        assert crossed > 0  # particles really changed slab during the loop
        open(os.path.join(result_dir, f'ok{rank}'), 'w').close()
    finally:
        dist.destroy_process_group()


def test_steady_state_loop_on_cpu_ranks(tmp_path):
    """Host logic of the stepping loop on two gloo ranks: per step move, partition, count
    exchange, all-to-all, slab-local sort; every rank's state after every step equals the
    one-process replay (the per-rank particle counts drift from step to step)."""
    world = 2
    mp.spawn(_gloo_loop_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f'ok{r}' for r in range(world)]


@pytest.mark.parametrize('world', [2, 3])
def test_exchange_on_cpu_ranks_follows_the_ordering_rule(tmp_path, world):
    mp.spawn(_gloo_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f'ok{r}' for r in range(world)]


def test_slab_range_and_divisibility():
    assert slab_sort.slab_range(GRID, 4, 2) == (6, 3)
    with pytest.raises(ValueError):
        slab_sort.slab_range(GRID, 5, 0)


def _device_share(grid, n, seed, device):
    gen = torch.Generator(device=device).manual_seed(seed)
    x, y, z = (torch.rand(n, device=device, generator=gen) for _ in range(3))
    x = x * 1.2 - 0.1  # some particles outside the box on both sides
    padded = -(-n // 4) * 4
    v = torch.zeros((3, padded), device=device)
    v[:, :n] = torch.randn((3, n), device=device, generator=gen)
    return x, y, z, v


@pytest.mark.gpu
@pytest.mark.parametrize('world,n', [(2, 10_001), (8, 300_000), (4, 2048), (8, 1), (2, 0)])
def test_partition_kernel_is_a_stable_partition(cuda, world, n):
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (64, 8, 8))
    x, y, z, v = _device_share(grid, n, 5, cuda)
    parts = slab_sort.partition_by_slab(x, y, z, v, grid, world)
    ogrid = so.Grid(grid.lo, grid.hi, grid.cells)
    dest = so.slab_of(x.cpu().numpy(), ogrid, world)
    order = np.argsort(dest, kind='stable')
    np.testing.assert_array_equal(parts.counts.cpu().numpy(), np.bincount(dest, minlength=world))
    src = [x, y, z, v[0, :n], v[1, :n], v[2, :n]]
    for got, s in zip(parts.arrays, src):
        np.testing.assert_array_equal(got.cpu().numpy(), s.cpu().numpy()[order])


@pytest.mark.gpu
@pytest.mark.parametrize('world', [2, 8])
def test_all_ranks_emulated_on_one_gpu_match_the_oracle(cuda, world):
    """Partition every rank's share, exchange by concatenation in source order,
    sort every slab: per rank equal to the oracle's replay, and the slabs'
    counts reassemble the single-GPU counts."""
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (32, 16, 8))
    ogrid = so.Grid(grid.lo, grid.hi, grid.cells)
    n, seed = 40_000, 77
    shares = [_device_share(grid, n + 3 * r, 100 + r, cuda) for r in range(world)]
    parts = [slab_sort.partition_by_slab(*sh, grid, world) for sh in shares]
    host_shares = [tuple(a.cpu().numpy() for a in (sh[0], sh[1], sh[2], sh[3][0, :sh[0].numel()],
                                                   sh[3][1, :sh[0].numel()], sh[3][2, :sh[0].numel()]))
                   for sh in shares]
    replay = so.exchange_replay(host_shares, ogrid, world)
    total = np.zeros((grid.cells[2], grid.cells[1], grid.cells[0]), np.int64)
    for d in range(world):
        recv = []
        for k in range(6):
            blocks = []
            for s in range(world):
                c = parts[s].counts.cpu().numpy()
                lo = int(c[:d].sum())
                blocks.append(parts[s].arrays[k][lo:lo + int(c[d])])
            recv.append(torch.cat(blocks))
        for g, w in zip(recv, replay[d]):
            np.testing.assert_array_equal(g.cpu().numpy(), w)
        m = recv[0].numel()
        rv = torch.zeros((3, -(-m // 4) * 4), device=cuda)
        rv[0, :m], rv[1, :m], rv[2, :m] = recv[3], recv[4], recv[5]
        off, width = slab_sort.slab_range(grid, world, d)
        got = pa.sort_and_gather_particles(recv[0], recv[1], recv[2], rv, grid, seed,
                                           ix_offset=off, nx_local=width)
        want = so.sort_particles(*replay[d][:3], ogrid, seed, ix_offset=off, nx_local=width)
        np.testing.assert_array_equal(got.order.keys.cpu().numpy().view(np.uint32), want.keys)
        np.testing.assert_array_equal(got.order.particle_index.cpu().numpy(), want.particle_index)
        np.testing.assert_array_equal(got.order.cell_start.cpu().numpy(), want.cell_start)
        total[:, :, off:off + width] = want.cell_counts.reshape(grid.cells[2], grid.cells[1], width)
    allx = [np.concatenate([h[k] for h in host_shares]) for k in range(3)]
    whole = so.sort_particles(*allx, ogrid, seed)
    np.testing.assert_array_equal(total.reshape(-1), whole.cell_counts)


def _nccl_worker(rank, world, port, result_dir):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    device = torch.device('cuda', rank)
    torch.cuda.set_device(device)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    try:
        grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (32, 16, 8))
        ogrid = so.Grid(grid.lo, grid.hi, grid.cells)
        shares = [_device_share(grid, 50_000 + 3 * r, 100 + r, device) for r in range(world)]
        x, y, z, v = shares[rank]
        host = [tuple(a.cpu().numpy() for a in (sh[0], sh[1], sh[2], sh[3][0, :sh[0].numel()],
                                                sh[3][1, :sh[0].numel()], sh[3][2, :sh[0].numel()]))
                for sh in shares]
        mine = so.exchange_replay(host, ogrid, world)[rank]
        off, width = slab_sort.slab_range(grid, world, rank)
        want = so.sort_particles(*mine[:3], ogrid, 91, ix_offset=off, nx_local=width)
        # Both exchanges (NCCL all-to-all; stores into the peers' buffers), twice each: the
        # second round reuses the peer buffers of the first.
        for exchange in ('nccl', 'peer', 'peer', 'nccl'):
            got = slab_sort.distributed_sort(x, y, z, v, grid, 91, exchange=exchange)
            np.testing.assert_array_equal(got.order.keys.cpu().numpy().view(np.uint32), want.keys)
            np.testing.assert_array_equal(got.order.particle_index.cpu().numpy(),
                                          want.particle_index)
            np.testing.assert_array_equal(got.order.cell_counts.cpu().numpy(), want.cell_counts)
            np.testing.assert_array_equal(got.positions[0].cpu().numpy(),
                                          mine[0][want.particle_index])
            np.testing.assert_array_equal(got.velocity.cpu().numpy()[2, :want.keys.size],
                                          mine[5][want.particle_index])
            assert got.velocity.shape[1] == -(-want.keys.size // 4) * 4
        # The move stage fused into the step: equal to moving every share first.
        dt = 0.07
        moved = []
        for h in host:
            p, w = so.push_particles(list(h[:3]), list(h[3:]), dt, grid.lo, grid.hi)
            moved.append(tuple(p) + tuple(w))
        mine = so.exchange_replay(moved, ogrid, world)[rank]
        want = so.sort_particles(*mine[:3], ogrid, 92, ix_offset=off, nx_local=width)
        before = [t.clone() for t in (x, y, z, v)]
        for exchange in ('peer', 'nccl'):
            got = slab_sort.distributed_sort(x, y, z, v, grid, 92, exchange=exchange,
                                             push=(dt, grid.lo, grid.hi))
            np.testing.assert_array_equal(got.order.keys.cpu().numpy().view(np.uint32), want.keys)
            np.testing.assert_array_equal(got.order.particle_index.cpu().numpy(),
                                          want.particle_index)
            for k in range(3):
                np.testing.assert_array_equal(got.positions[k].cpu().numpy(),
                                              mine[k][want.particle_index])
                np.testing.assert_array_equal(got.velocity.cpu().numpy()[k, :want.keys.size],
                                              mine[3 + k][want.particle_index])
            for t, b in zip((x, y, z, v), before):
                assert torch.equal(t, b)
        assert slab_sort.exchange_status(device) == 0
        # A stepping loop over the sliced exchange: the output of a step is the next input,
        # the per-rank particle counts drift, buffers and plans come from the step before.
        state = (x, y, z, v)
        shares_now = host
        for step in range(4):
            moved = []
            for h in shares_now:
                p, w = so.push_particles(list(h[:3]), list(h[3:]), dt, grid.lo, grid.hi)
                moved.append(tuple(p) + tuple(w))
            received = so.exchange_replay(moved, ogrid, world)
            shares_now = []
            for r, rec in enumerate(received):
                o, wd = slab_sort.slab_range(grid, world, r)
                perm = so.sort_particles(*rec[:3], ogrid, 500 + step, ix_offset=o,
                                         nx_local=wd).particle_index
                shares_now.append(tuple(a[perm] for a in rec))
            got = slab_sort.distributed_sort(*state, grid, 500 + step, push=(dt, grid.lo, grid.hi))
            for k in range(3):
                np.testing.assert_array_equal(got.positions[k].cpu().numpy(), shares_now[rank][k])
                np.testing.assert_array_equal(
                    got.velocity.cpu().numpy()[k, :shares_now[rank][0].size], shares_now[rank][3 + k])
            state = (*got.positions, got.velocity)
        assert slab_sort.exchange_status(device) == 0
        # The same loop with the other transport and without overlap (the loop above ran the
        # defaults: copy engines, overlapped).
        for transport, overlap in (('stores', True), ('stores', False), ('copies', False)):
            slab_sort.configure(transport=transport, overlap=overlap)
            state = (x, y, z, v)
            shares_now = host
            for step in range(3):
                moved = []
                for h in shares_now:
                    p, w = so.push_particles(list(h[:3]), list(h[3:]), dt, grid.lo, grid.hi)
                    moved.append(tuple(p) + tuple(w))
                received = so.exchange_replay(moved, ogrid, world)
                shares_now = []
                for r, rec in enumerate(received):
                    o, wd = slab_sort.slab_range(grid, world, r)
                    perm = so.sort_particles(*rec[:3], ogrid, 700 + step, ix_offset=o,
                                             nx_local=wd).particle_index
                    shares_now.append(tuple(a[perm] for a in rec))
                got = slab_sort.distributed_sort(*state, grid, 700 + step,
                                                 push=(dt, grid.lo, grid.hi))
                for k in range(3):
                    np.testing.assert_array_equal(got.positions[k].cpu().numpy(),
                                                  shares_now[rank][k])
                    np.testing.assert_array_equal(
                        got.velocity.cpu().numpy()[k, :shares_now[rank][0].size],
                        shares_now[rank][3 + k])
                state = (*got.positions, got.velocity)
            assert slab_sort.exchange_status(device) == 0
        slab_sort.configure()
        open(os.path.join(result_dir, f'ok{rank}'), 'w').close()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_distributed_sort_over_nccl(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip('needs at least two GPUs')
    mp.spawn(_nccl_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f'ok{r}' for r in range(world)]


@pytest.mark.gpu
@pytest.mark.parametrize('world,slices,n,transport', [
    (2, 1, 30_000, 'stores'), (4, 3, 50_000, 'stores'), (8, 8, 200_000, 'stores'),
    (3, 32, 70_001, 'stores'), (2, 4, 30_000, 'copies'), (8, 3, 100_000, 'copies'),
    (3, 1, 70_001, 'copies')])
def test_sliced_exchange_and_sliced_sort_emulated_on_one_gpu(cuda, world, slices, n, transport):
    """The sliced pipeline through the C ABI with all ranks on one GPU, one after another:
    counts per (slice, destination), the gathered matrix, every rank's exchange kernel storing
    into the ranks' receive buffers and setting their arrival flags, then per rank the slice
    waits (the flags are set by then, so no wait polls twice) and the sort slice by slice.
    With transport 'copies' the exchange kernel partitions into staging rows laid out like the
    receive buffers (a rank's own share goes straight into its buffer) and device-to-device
    copies, planned by slab_sort.copy_plan, carry the rest; the signal follows the copies.
    Every rank's result equals the oracle's replay of exchange + slab-local sort."""
    import ctypes
    from project_aether_b200 import _native
    from project_aether_b200.particle_sort import native_grid
    lib = _native.load_library()
    nx = 24 if world == 3 else 32
    grid = pa.CellGrid((0., 0., 0.), (1., 1., 1.), (nx, 16, 8))
    ogrid = so.Grid(grid.lo, grid.hi, grid.cells)
    g = native_grid(grid)
    seed, dt = 0x1234500000077, 0.05
    move = (dt, (ctypes.c_float * 3)(*grid.lo), (ctypes.c_float * 3)(*grid.hi))
    shares = [_device_share(grid, n + 5 * r, 300 + r, cuda) for r in range(world)]
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
    with torch.cuda.device(cuda):
        # Counts of every rank, then the "all-gather".
        spaces, rows = [], []
        for x, y, z, v in shares:
            m = x.numel()
            ws = torch.empty(lib.AetherSlabPartitionWorkspaceBytes(m, world), dtype=torch.uint8,
                             device=cuda)
            totals = torch.zeros(world, dtype=torch.int64, device=cuda)
            per_slice = torch.zeros(slices * world, dtype=torch.int64, device=cuda)
            _native.check(lib.AetherSlabExchangeCountMoved(
                x.data_ptr(), v.data_ptr(), m, move[0], move[1], move[2], ctypes.byref(g), world,
                totals.data_ptr(), ws.data_ptr(), ws.numel(), stream), 'count')
            _native.check(lib.AetherSlabExchangeSliceCounts(
                m, world, slices, per_slice.data_ptr(), ws.data_ptr(), ws.numel(), stream), 'slices')
            assert torch.equal(per_slice.view(slices, world).sum(0), totals)
            spaces.append(ws)
            rows.append(per_slice)
        matrix = torch.stack(rows).view(world, slices, world).contiguous()
        received = matrix.sum(dim=(0, 1)).cpu()
        capacity = -(-int(received.max()) // 4) * 4 + 8
        flag_words = -(-world * slices // 4) * 4  # keeps the arrays behind the flags 16-byte aligned
        buffers = [torch.zeros(flag_words + 6 * capacity, dtype=torch.float32, device=cuda)
                   for _ in range(world)]
        flag_pointers = (ctypes.c_void_p * world)(*[b.data_ptr() for b in buffers])
        data_pointers = (ctypes.c_void_p * world)(*[b.data_ptr() + 4 * flag_words for b in buffers])
        error = torch.zeros(1, dtype=torch.int32, device=cuda)
        segments, epoch = [], 3
        for r, (x, y, z, v) in enumerate(shares):
            totals2d = torch.empty((world, world), dtype=torch.int64, device=cuda)
            seg = torch.empty(lib.AetherSlabSegmentsBytes(), dtype=torch.uint8, device=cuda)
            _native.check(lib.AetherSlabExchangePrepare(
                matrix.data_ptr(), world, slices, r, totals2d.data_ptr(), seg.data_ptr(), stream),
                'prepare')
            assert torch.equal(totals2d, matrix.sum(dim=1))
            segments.append(seg)
            if transport == 'copies':
                staging = torch.zeros((world, 6 * capacity), dtype=torch.float32, device=cuda)
                scratch = torch.zeros(flag_words, dtype=torch.int32, device=cuda)
                rows_r = [buffers[r].data_ptr() + 4 * flag_words if d == r else staging[d].data_ptr()
                          for d in range(world)]
                targets = (ctypes.c_void_p * world)(*rows_r)
                flags_r = (ctypes.c_void_p * world)(*([scratch.data_ptr()] * world))
                plan = slab_sort.copy_plan(matrix.cpu().numpy(), r)
            else:
                targets, flags_r = data_pointers, flag_pointers
            for k in range(slices):
                _native.check(lib.AetherSlabExchangeScatterSliced(
                    x.data_ptr(), y.data_ptr(), z.data_ptr(), v.data_ptr(), v.stride(0), x.numel(),
                    move[0], move[1], move[2], ctypes.byref(g), world, r, targets, capacity,
                    totals2d.data_ptr(), error.data_ptr(), slices, k, epoch, flags_r,
                    spaces[r].data_ptr(), spaces[r].numel(), stream), 'exchange')
                if transport == 'copies':
                    for d, first, count in plan[k]:
                        _native.check(lib.AetherSlabExchangeCopy(
                            ctypes.c_void_p(buffers[d].data_ptr() + 4 * (flag_words + first)),
                            ctypes.c_void_p(rows_r[d] + 4 * first), 4 * count, 6, 4 * capacity,
                            stream), 'copy')
                    _native.check(lib.AetherSlabExchangeSignal(world, r, slices, k, epoch,
                                                               flag_pointers, stream), 'signal')
            torch.cuda.synchronize()  # the staging rows of this rank go out of scope
        torch.cuda.synchronize()
        assert int(error) == 0
        for b in buffers:  # every (source, slice) flag carries the epoch
            assert torch.equal(b[:world * slices].view(torch.int32),
                               torch.full((world * slices,), epoch, dtype=torch.int32, device=cuda))
        # The oracle's replay: move every share, exchange, sort every slab.
        host = []
        for x, y, z, v in shares:
            m = x.numel()
            p, q = so.push_particles([t.cpu().numpy() for t in (x, y, z)],
                                     [v[k, :m].cpu().numpy() for k in range(3)], dt, grid.lo, grid.hi)
            host.append(tuple(p) + tuple(q))
        replay = so.exchange_replay(host, ogrid, world)
        for r in range(world):
            m = int(received[r])
            off, width = slab_sort.slab_range(grid, world, r)
            local = native_grid(grid, off, width)
            cells = width * grid.cells[1] * grid.cells[2]
            plan_n = max(1, m + (r % 2) * 1000)  # the plan may come from another step's count
            data = buffers[r][flag_words:]
            rx, ry, rz = data[0:capacity], data[capacity:2 * capacity], data[2 * capacity:3 * capacity]
            rv = data[3 * capacity:6 * capacity]
            ws = torch.empty(lib.AetherSortSlicedWorkspaceBytes(capacity, plan_n, cells, slices),
                             dtype=torch.uint8, device=cuda)
            _native.check(lib.AetherSortSlicedBegin(capacity, plan_n, ctypes.byref(local), slices,
                                                    ws.data_ptr(), ws.numel(), stream), 'begin')
            for k in range(slices):
                _native.check(lib.AetherSlabExchangeWait(buffers[r].data_ptr(), world, slices, k, epoch,
                                                         4, error.data_ptr(), stream), 'wait')
                _native.check(lib.AetherSortSlicedSlice(
                    rx.data_ptr(), ry.data_ptr(), rz.data_ptr(), rv.data_ptr(), capacity, capacity,
                    plan_n, ctypes.byref(local), seed, segments[r].data_ptr(), slices, k,
                    ws.data_ptr(), ws.numel(), stream), 'slice')
            keys = torch.empty(capacity, dtype=torch.int32, device=cuda)
            index = torch.empty(capacity, dtype=torch.int32, device=cuda)
            counts = torch.empty(cells, dtype=torch.int32, device=cuda)
            start = torch.empty(cells + 1, dtype=torch.int32, device=cuda)
            outs = [torch.empty(capacity, dtype=torch.float32, device=cuda) for _ in range(3)]
            vs = torch.empty((3, capacity), dtype=torch.float32, device=cuda)
            _native.check(lib.AetherSortSlicedFinish(
                capacity, plan_n, ctypes.byref(local), segments[r].data_ptr(), slices,
                keys.data_ptr(), index.data_ptr(), counts.data_ptr(), start.data_ptr(),
                outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), vs.data_ptr(), capacity,
                ws.data_ptr(), ws.numel(), stream), 'finish')
            status = ctypes.c_int32(-1)
            _native.check(lib.AetherSortReadStatus(ws.data_ptr(), stream, ctypes.byref(status)),
                          'status')
            assert status.value == 0 and int(error) == 0
            mine = replay[r]
            assert mine[0].size == m
            want = so.sort_particles(*mine[:3], ogrid, seed, ix_offset=off, nx_local=width)
            np.testing.assert_array_equal(keys[:m].cpu().numpy().view(np.uint32), want.keys)
            np.testing.assert_array_equal(index[:m].cpu().numpy(), want.particle_index)
            np.testing.assert_array_equal(counts.cpu().numpy(), want.cell_counts)
            np.testing.assert_array_equal(start.cpu().numpy(), want.cell_start)
            for k in range(3):
                np.testing.assert_array_equal(outs[k][:m].cpu().numpy(),
                                              mine[k][want.particle_index])
                np.testing.assert_array_equal(vs[k, :m].cpu().numpy(),
                                              mine[3 + k][want.particle_index])
        # A flag that nothing sets: the wait runs out after its few polls and reports.
        _native.check(lib.AetherSlabExchangeWait(buffers[0].data_ptr(), world, slices, 0, epoch + 1,
                                                 4, error.data_ptr(), stream), 'wait')
        torch.cuda.synchronize()
        assert int(error) == 6
