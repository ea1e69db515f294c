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
