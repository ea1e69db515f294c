"""The N > 1 leg of bench.py: one rank per GPU, x-slab decomposition.

Default workload (256 M particles): every rank starts with a random 1/G share of
all particles drawn over the whole box (generator seed 0 + rank), so (G-1)/G of
them must leave in the exchange.  One step = partition by slab, count exchange,
all-to-all, local sort.

Steady-state workload (`c5...`): every rank starts with the cell-sorted
particles of its own slab; one step = the same distributed sort with the move
stage (x += v*dt, specular walls) fused into its exchange kernels; its output
is the next step's input.  Only
the particles that crossed a slab face travel.
"""

import ctypes
import json
import os

import torch
import torch.distributed as dist


def run(args, workload: str) -> None:
    import project_aether_b200 as pa
    from project_aether_b200 import _native, slab_sort, workloads
    import bench as bench_mod  # the launcher script (repo root is on sys.path)

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', str(args.gpus)))
    local = int(os.environ.get('LOCAL_RANK', str(rank)))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29512')
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    lib = _native.load_library()
    w = workloads.WORKLOADS[workload]
    n_total = w.n
    n_local = n_total // world
    x, y, z, v = workloads.make_particles(w, device, seed=rank, n=n_local)

    exchange = os.environ.get('AETHER_EXCHANGE', 'peer')  # 'peer' (NVLink stores) or 'nccl'
    steady = workload.startswith('c5')
    steady_dt = 8.2e-5  # about 5 % of the particles change cell per step
    state = {'x': x, 'y': y, 'z': z, 'v': v}
    if steady:
        # Squeeze this rank's share into its own slab, then sort it once: the loop starts
        # from a cell-sorted state in which every particle is at home.
        lo, hi = w.grid.lo[0], w.grid.hi[0]
        width = (hi - lo) / world
        x.sub_(lo).div_(world).add_(lo + rank * width).clamp_(max=lo + (rank + 1) * width * (1 - 1e-7))
        first = slab_sort.distributed_sort(x, y, z, v, w.grid, 99, exchange=exchange)
        state = {'x': first.positions[0], 'y': first.positions[1], 'z': first.positions[2],
                 'v': first.velocity}
        del first

    move = (steady_dt, w.grid.lo, w.grid.hi) if steady else None

    def step(s):
        r = slab_sort.distributed_sort(state['x'], state['y'], state['z'], state['v'], w.grid,
                                       workloads.step_seed(1234, s), exchange=exchange, push=move)
        if steady:
            state.update(x=r.positions[0], y=r.positions[1], z=r.positions[2], v=r.velocity)
        return r

    warmup = max(3, args.warmup)
    for s in range(warmup):
        out = step(s)
    torch.cuda.synchronize()
    status = torch.tensor([pa.last_sort_status(device)], device=device)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    assert int(status) == 0

    lib.AetherSortSetStageTiming(1)
    launches0 = lib.AetherSortKernelLaunches()
    sampler = bench_mod.ClockSampler(device.index)
    if rank == 0:
        sampler.start()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    begin.record()
    ticks = []
    for s in range(args.steps):
        out = step(100 + s)
        ticks.append(torch.cuda.Event(enable_timing=True))
        ticks[-1].record()
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    step_ms = [a.elapsed_time(b) for a, b in zip([begin] + ticks[:-1], ticks)]
    clocks = sampler.stop() if rank == 0 else None
    elapsed = torch.tensor([begin.elapsed_time(end)], device=device)
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms = float(elapsed) / args.steps
    launches = int(lib.AetherSortKernelLaunches() - launches0)
    count = lib.AetherSortStageCount()
    stage_ms = (ctypes.c_float * count)()
    _native.check(lib.AetherSortReadStageTimes(stage_ms, count), 'AetherSortReadStageTimes')
    lib.AetherSortSetStageTiming(0)
    stages = {lib.AetherSortStageName(i).decode(): float(stage_ms[i]) for i in range(count)
              if stage_ms[i] >= 0}
    # Phase times of one more step (events on the stream; the count exchange includes a host wait).
    marks = []
    slab_sort.distributed_sort(state['x'], state['y'], state['z'], state['v'], w.grid,
                               workloads.step_seed(1234, 999), marks=marks, exchange=exchange,
                               push=move)
    torch.cuda.synchronize()
    phases = {marks[i][0]: marks[i - 1][1].elapsed_time(marks[i][1]) for i in range(1, len(marks))}
    received = torch.tensor([out.order.keys.numel()], device=device, dtype=torch.int64)
    dist.all_reduce(received)
    assert int(received) == n_local * world, 'particles were lost in the exchange'

    # End to end: pinned host inputs in, results back to the host, every step.
    e2e_steps = max(1, min(args.steps, 3))
    if steady:
        m = state['x'].numel()
        x, y, z = state['x'], state['y'], state['z']
        v = state['v'][:, :m].contiguous()
    hx, hy, hz, hv = (t.cpu().pin_memory() for t in (x, y, z, v))
    d2h = [0]
    pinned = {}

    def e2e_step(s):
        dx, dy, dz, dv = (t.to(device, non_blocking=True) for t in (hx, hy, hz, hv))
        r = slab_sort.distributed_sort(dx, dy, dz, dv, w.grid, workloads.step_seed(1234, s),
                                       exchange=exchange)
        outs = [r.order.keys, r.order.particle_index, r.order.cell_counts, r.order.cell_start,
                *r.positions, r.velocity]
        for i, o in enumerate(outs):  # pinned result buffers, kept across steps
            if i not in pinned or pinned[i].shape != o.shape:
                pinned[i] = torch.empty(o.shape, dtype=o.dtype, pin_memory=True)
            pinned[i].copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        d2h[0] = sum(o.numel() * o.element_size() for o in outs)

    e2e_step(0)
    dist.barrier()
    torch.cuda.synchronize()
    begin.record()
    for s in range(e2e_steps):
        e2e_step(200 + s)
    end.record()
    torch.cuda.synchronize()
    e2e_elapsed = torch.tensor([begin.elapsed_time(end)], device=device)
    dist.all_reduce(e2e_elapsed, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_elapsed) / e2e_steps
    bytes_io = torch.tensor([sum(t.numel() * t.element_size() for t in (hx, hy, hz, hv)), d2h[0]],
                            device=device, dtype=torch.int64)
    dist.all_reduce(bytes_io)

    # Strong-scaling denominator: the same workload, whole, on one GPU (rank 0 alone).
    single = None
    del hx, hy, hz, hv
    if rank == 0 and not steady:  # (the steady-state loop at one GPU is `bench.py --workload c5...`)
        ax, ay, az, av = workloads.make_particles(w, device, seed=0)
        for s in range(2):
            pa.sort_and_gather_particles(ax, ay, az, av, w.grid, workloads.step_seed(1234, s))
        torch.cuda.synchronize()
        begin.record()
        for s in range(3):
            pa.sort_and_gather_particles(ax, ay, az, av, w.grid, workloads.step_seed(1234, 50 + s))
        end.record()
        torch.cuda.synchronize()
        one_ms = begin.elapsed_time(end) / 3
        single = {'value': n_total / (one_ms * 1e-3), 'unit': 'particles/s', 'ms_per_step': one_ms,
                  'steps': 3}
        del ax, ay, az, av
    dist.barrier()

    if rank == 0:
        peak, peak_kind = bench_mod.measured_peak()
        n_rank = n_total // world
        top = max(stages, key=stages.get) if stages else None
        roofline = None
        if top:
            # The exchange kernel reads 24 B per particle and stores 24 B, (G-1)/G of them into
            # the peers' memory: NVLink bounds it, so its line also carries the crossing bytes
            # against the peer-copy bandwidth measured on this pool (770 GB/s per direction).
            per_particle = bench_mod.STAGE_BYTES_PER_PARTICLE.get(
                top, 48 if top in ('slab_partition', 'slab_exchange') else 0)
            nbytes = per_particle * n_rank
            achieved = nbytes / (stages[top] * 1e-3) / 1e9
            roofline = {'bound': 'hbm', 'kernel': top, 'achieved': achieved, 'peak': peak,
                        'unit': 'GB/s', 'frac': achieved / peak, 'peak_kind': peak_kind,
                        'traffic': (bench_mod.NCU_DRAM_BYTES_PER_PARTICLE[top] * n_rank
                                    if top in bench_mod.NCU_DRAM_BYTES_PER_PARTICLE else None),
                        'bytes_per_launch': nbytes, 'ms_per_launch': stages[top]}
            if top == 'slab_exchange' and exchange == 'peer':
                crossing = 24 * n_rank * (world - 1) / world
                link = crossing / (stages[top] * 1e-3) / 1e9
                roofline['nvlink'] = {'bytes_out_per_gpu': crossing, 'achieved': link,
                                      'peak': 770.0, 'unit': 'GB/s', 'frac': link / 770.0,
                                      'peak_kind': 'peer copy measured on this pool'}
        line = {
            'metric': 'sorted particles/s', 'value': n_total / (ms * 1e-3), 'unit': 'particles/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms,
            'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'u32',
            'data': 'synthetic',
            'config': {'workload': workload, 'particles': n_total, 'cells': list(w.grid.cells),
                       'decomposition': f'{world} x-slabs',
                       'exchange': ('partition kernel stores into the peers\' receive buffers '
                                    'over NVLink' if exchange == 'peer'
                                    else 'one NCCL all-to-all per payload array'),
                       'initial_share': ('cell-sorted particles of the rank\'s own slab; every step '
                                         'moves them (dt %g) and re-sorts' % steady_dt if steady
                                         else 'random 1/G of all particles per rank'),
                       'l2': 'inputs larger than L2 (no flush needed)'},
            'clocks': {'sm_mhz': clocks['sm_mhz'], 'sm_max_mhz': clocks['sm_max_mhz'],
                       'reasons': clocks['reasons'], 'samples': clocks['samples']},
            'e2e': {'value': n_total / (e2e_ms * 1e-3), 'unit': 'particles/s',
                    'h2d_bytes_per_step': int(bytes_io[0]), 'd2h_bytes_per_step': int(bytes_io[1]),
                    'ms_per_step': e2e_ms, 'steps': e2e_steps},
            'gpu_launches': launches, 'roofline': roofline, 'stage_ms_rank0': stages,
            'phase_ms_rank0': phases, 'step_ms_rank0': step_ms,
            'single_gpu_same_workload': single,
            'cpu_baseline': None,
        }
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
