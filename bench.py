"""Benchmark of the DSMC particle sort: sorted particles per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one full sort call on one synthetic particle state: key
generation, the sort, per-cell counts and starts, and the sorted SoA payload.
Prints ONE JSON line (rank 0).  `value` is measured with the inputs resident in
HBM; `e2e` is the same call fed from pinned host buffers with the results read
back to the host inside the timed region.  `--impl reference` times the CPU
restatement of the reference path (the C oracle, all host threads) instead.

With N > 1 (one rank per GPU under torch.distributed.run) the workload is the
256 M configuration split into x-slabs: every rank starts with a random 1/N
share of all particles, one step = partition by slab, exchange, local sort.
The steady-state workload (`c5...`) starts every rank with the cell-sorted
particles of its own slab and fuses the move stage into the step.
"""

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_HBM_GBS = 8000.0   # the benchmark definition's nominal B200 HBM peak
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used if no measured file
PEER_COPY_GBS = 770.0      # peer copy per direction measured on this pool (nominal 900)
STEADY_DT = 8.2e-5         # about 5 % of the particles change cell per step (unit thermal speed)


def algorithmic_bytes(n: int, cells: int) -> int:
    """136 B per particle + 8 B per cell + 4: read x,y,z (12); write key+index (8);
    four digit passes read and write key+index (16 each); read the permutation
    (4); gather-read and write six payload floats (24 + 24); write counts and
    starts (8 per cell)."""
    return 136 * n + 8 * cells + 4


# Algorithmic bytes per particle of each stage (what a launch must move at least).
STAGE_BYTES_PER_PARTICLE = {
    'keygen_upsweep': 12 + 4, 'digit_pass_0': 4 + 8, 'digit_pass_1': 16, 'digit_pass_2': 16,
    'digit_pass_3': 16, 'cell_tables': 4, 'payload_gather': 4 + 24 + 24,
    'bucket_count': 12, 'bucket_scan': 0, 'bucket_scatter': 24 + 32, 'bucket_finish': 32 + 32,
    'particle_push': 24 + 24, 'collide': 12 + 12, 'slab_partition': 4, 'slab_exchange': 24 + 24,
}


# DRAM bytes per particle (dram__bytes_read.sum + dram__bytes_write.sum) of each bucketed-path
# kernel, from one ncu capture at 2^24 particles of the same density; traffic grows in
# proportion to the particle count, so a launch's traffic is this figure times its particles.
NCU_DRAM_BYTES_PER_PARTICLE = {'bucket_count': 12.2, 'bucket_scatter': 52.9,
                               'bucket_finish': 62.1}


def measured_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        try:
            return float(json.load(open(path))['hbm_gbs']), 'measured'
        except Exception:
            pass
    return FALLBACK_HBM_GBS, 'fallback'


def workload_config(name, w, gpus):
    """The `config` both arms print: what the workload is, nothing about how it is run."""
    return {'workload': name, 'particles': w.n, 'cells': list(w.grid.cells),
            'decomposition': 'single GPU' if gpus == 1 else f'{gpus} x-slabs',
            'seed_per_step': 'run_seed ^ (step << 20)',
            'l2': ('inputs larger than L2 (no flush needed)' if 24 * w.n // gpus > (126 << 20)
                   else 'inputs fit L2; no flush between steps')}


def select_workload(args):
    from project_aether_b200 import workloads
    name = args.workload or ('c3_64m_hypersonic' if args.gpus == 1 else 'c4_256m_512')
    if args.log2n:
        return f'{name}@2^{args.log2n}', workloads.scaled_workload(name, args.log2n)
    return name, workloads.WORKLOADS[name]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
              'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile('w+', suffix='.csv', delete=False)
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits',
                 '-i', str(self.gpu), '-lms', '50'], stdout=self.file, stderr=subprocess.DEVNULL)
            # nvidia-smi takes a moment to start: wait for its first line so that the samples
            # that follow fall inside the measured regions.
            deadline = time.time() + 2.0
            while time.time() < deadline and os.path.getsize(self.file.name) == 0:
                time.sleep(0.01)
        except Exception:
            self.proc = None

    def stop(self):
        out = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        rows = [r.strip().split(', ') for r in open(self.file.name) if r.strip()]
        os.unlink(self.file.name)
        sm, reasons = [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                out['sm_max_mhz'] = float(r[2])
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.strip().lower().startswith('active'):
                    reasons.add(name)
        if sm:
            out['sm_mhz'] = float(np.median(sm))
        out['reasons'] = sorted(reasons)
        out['samples'] = len(sm)
        return out


# --------------------------------------------------------------------------------------
# CPU legs (the only users of oracle/ in this file: the timed baseline and the checker).
# --------------------------------------------------------------------------------------

def host_threads() -> int:
    """All host threads of the box.  Passed to the oracle explicitly: a launcher may have set
    OMP_NUM_THREADS=1 in the environment (torch.distributed.run does), which would otherwise
    cap OpenMP's default."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_reference_step(host, grid, seed, threads, **slab):
    from oracle import sort_oracle as so
    g = so.Grid(tuple(grid.lo), tuple(grid.hi), tuple(grid.cells))
    return so.c_sort_particles(host[0], host[1], host[2], host[3], g, seed, threads=threads,
                               **slab)


def torch_cpu_binning_rate(w, threads, sample_log2n=22, repeats=3):
    """The reference's own definition of the CPU baseline (cell ids, Mersenne-Twister shuffle
    bits, torch.sort(stable=True), bincount under torch.set_num_threads(T);
    scripts/phase2_triton_sort_benchmark.py:44-70) on a sample of the workload at the same
    particles per cell.  Particles per second."""
    import torch
    from project_aether_b200 import phase2_benchmark, workloads
    name = w.name
    s = workloads.scaled_workload(name, min(sample_log2n, int(np.log2(w.n))))
    x, y, z, _ = workloads.make_particles(s, 'cpu', seed=0)
    before = torch.get_num_threads()
    torch.set_num_threads(threads)
    try:
        bits = torch.Generator().manual_seed(0)
        phase2_benchmark.cpu_binning(x, y, z, s.grid, bits)
        t0 = time.perf_counter()
        for _ in range(repeats):
            phase2_benchmark.cpu_binning(x, y, z, s.grid, bits)
        seconds = (time.perf_counter() - t0) / repeats
    finally:
        torch.set_num_threads(before)
    return {'value': s.n / seconds, 'unit': 'particles/s', 'threads': threads,
            'sample': f'{s.n} particles, grid {list(s.grid.cells)}, torch {torch.__version__} '
                      f'cpu_binning (cell ids, randint, stable sort, bincount), {repeats} repeats'}


def numpy_replay_rate(sample=1 << 16):
    """The reference's NumPy replay of its Onesweep kernel (radix_sort_reference.py:93-148), as
    restated in the oracle, on a sample of configuration 1's keys.  It walks tiles and keys in
    Python loops (the reference needs 11.7 s for one million keys), so the sample is small."""
    from oracle import sort_oracle as so
    from project_aether_b200 import workloads
    w = workloads.WORKLOADS['c1_1m_64']
    x, y, z, _ = workloads.make_particles(w, 'cpu', seed=0, n=sample)
    g = so.Grid(tuple(w.grid.lo), tuple(w.grid.hi), tuple(w.grid.cells))
    keys = so.make_keys(x.numpy(), y.numpy(), z.numpy(), g, 1234).astype(np.int64)
    t0 = time.perf_counter()
    so.onesweep_replay(keys, np.arange(sample, dtype=np.int32), so.reference_num_passes(g.num_cells),
                       np.random.default_rng(0))
    seconds = time.perf_counter() - t0
    return {'value': sample / seconds, 'unit': 'particles/s', 'threads': 1,
            'sample': f'{sample} keys of c1_1m_64, NumPy replay of the Onesweep kernel'}


def run_reference(args):
    """The reference path on host cores: C restatement of keys -> stable sort ->
    counts/starts -> payload gather, on all host threads, on a bounded sample of the workload
    that keeps its particles per cell."""
    from oracle import sort_oracle as so
    from project_aether_b200 import workloads
    if int(os.environ.get('RANK', '0')) != 0:
        return
    name, w = select_workload(args)
    threads = host_threads()
    used = so.c_threads(threads)
    # A first guess of the rate from a small sample, then the largest power-of-two sample
    # (the grid's z extent shrinks with it) that keeps the whole run within a few minutes.
    probe = workloads.scaled_workload(w.name, min(22, int(np.log2(w.n))))
    px, py, pz, pv = (t.numpy() for t in workloads.make_particles(probe, 'cpu', seed=0))
    cpu_reference_step((px, py, pz, pv), probe.grid, 1, threads)
    t0 = time.perf_counter()
    cpu_reference_step((px, py, pz, pv), probe.grid, 2, threads)
    rate = probe.n / (time.perf_counter() - t0)
    budget = min(180.0, 12.0 * (args.steps + args.warmup))
    log2n = int(np.log2(w.n))
    while log2n > 20 and (1 << log2n) / rate * (args.steps + args.warmup) * 1.3 > budget:
        log2n -= 1
    s = w if (1 << log2n) == w.n else workloads.scaled_workload(w.name, log2n)
    host = [t.numpy() for t in workloads.make_particles(s, 'cpu', seed=0)]
    for k in range(args.warmup):
        cpu_reference_step(host, s.grid, workloads.step_seed(1234, k + 1), threads)
    t0 = time.perf_counter()
    for k in range(args.steps):
        cpu_reference_step(host, s.grid, workloads.step_seed(1234, k + 100), threads)
    dt = (time.perf_counter() - t0) / args.steps
    value = s.n / dt
    desc = (f'{s.n} of {w.n} particles of {name} per step on grid {list(s.grid.cells)} '
            f'(same particles per cell), C restatement of the reference path, OpenMP, '
            f'{used} threads')
    baseline = {'value': value, 'unit': 'particles/s', 'cores': used, 'kind': 'port',
                'sample': desc}
    try:
        baseline['torch_cpu_binning'] = torch_cpu_binning_rate(w, threads)
    except Exception as exc:  # a reported extra, never a reason to lose the line
        baseline['torch_cpu_binning'] = {'unavailable': repr(exc)}
    if w.name == 'c1_1m_64':
        baseline['numpy_replay'] = numpy_replay_rate()
    line = {
        'impl': 'reference', 'metric': 'sorted particles/s', 'value': value, 'unit': 'particles/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3,
        'higher_is_better': True, 'scaling': 'weak' if args.gpus == 1 else 'strong',
        'vs_baseline': None, 'dtype': 'u32', 'data': 'synthetic',
        'config': workload_config(name, w, args.gpus),
        'cpu_baseline': baseline,
        'e2e': {'value': value, 'unit': 'particles/s', 'h2d_bytes_per_step': 0,
                'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------
# One GPU.
# --------------------------------------------------------------------------------------

def stage_times(lib, _native):
    count = lib.AetherSortStageCount()
    stage_ms = (ctypes.c_float * count)()
    _native.check(lib.AetherSortReadStageTimes(stage_ms, count), 'AetherSortReadStageTimes')
    return {lib.AetherSortStageName(i).decode(): float(stage_ms[i]) for i in range(count)
            if stage_ms[i] >= 0}


def run_single(args):
    import torch
    import project_aether_b200 as pa
    from project_aether_b200 import _native, workloads
    lib = _native.load_library()  # raises if the CUDA library is missing
    if not torch.cuda.is_available():
        raise RuntimeError('bench.py needs a CUDA GPU (no CPU fallback exists)')
    if args.finish_shape == 'large':
        _native.check(lib.AetherSortSetSmallShapeBucketLimit(0), 'AetherSortSetSmallShapeBucketLimit')
    device = torch.device('cuda', int(os.environ.get('LOCAL_RANK', '0')))
    torch.cuda.set_device(device)
    workload, w = select_workload(args)
    n, cells = w.n, w.grid.num_cells
    x, y, z, v = workloads.make_particles(w, device, seed=0)
    path = {'auto': pa.PATH_AUTO, 'digits': pa.PATH_DIGIT_PASSES, 'bucketed': pa.PATH_BUCKETED}[
        args.path]

    # Steady-state re-sort (configuration 5): the state starts cell-sorted and every step
    # moves it by x += v*dt (specular walls) before sorting it again; the sorted output is
    # the next step's input.
    steady = w.name.startswith('c5')
    state = {'x': x, 'y': y, 'z': z, 'v': v}
    crossing = None
    if steady:
        from project_aether_b200.particle_push import fused_particle_push
        first = pa.sort_and_gather_particles(x, y, z, v, w.grid, 99, path=path)
        state = {'x': first.positions[0], 'y': first.positions[1], 'z': first.positions[2],
                 'v': first.velocity}
        del first

        def move(st):
            fused_particle_push([st['x'], st['y'], st['z']], [st['v'][k, :n] for k in range(3)],
                                STEADY_DT, w.grid.lo, w.grid.hi)

    if steady and args.collide:
        # Unit thermal speed: sigma*g = g^0.46 stays below the majorant 3; the selection factor
        # gives about one candidate pair per two cells of 8 particles.
        from project_aether_b200 import ntc_collide
        gas = (0.006, 1.0, 0.46)
        sigma_g_max = torch.full((cells,), 3.0, dtype=torch.float32, device=device)
        collisions = torch.zeros(cells, dtype=torch.int32, device=device)

    def step(s):
        if steady and args.separate_push:
            move(state)
        fused = (STEADY_DT, w.grid.lo, w.grid.hi) if steady and not args.separate_push else None
        r = pa.sort_and_gather_particles(state['x'], state['y'], state['z'], state['v'], w.grid,
                                         workloads.step_seed(1234, s), path=path, push=fused)
        if steady:
            state.update(x=r.positions[0], y=r.positions[1], z=r.positions[2], v=r.velocity)
            if args.collide:  # the stage after the sort, on the sorted velocities in place
                ntc_collide.collide(lib, r.velocity, r.order.cell_start, sigma_g_max, collisions,
                                    n, ntc_collide.CollisionParams(*gas, 1234, s))
        return r

    warmup = max(3, args.warmup)
    for s in range(warmup):
        out = step(s)
    torch.cuda.synchronize()
    assert pa.last_sort_status(device) == 0

    # ---- device-resident timing (inputs 1.6 GB+ per call, far larger than L2) ----
    launches0 = lib.AetherSortKernelLaunches()
    sampler = ClockSampler(device.index)
    sampler.start()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    begin.record()
    for s in range(args.steps):
        out = step(100 + s)
    end.record()
    torch.cuda.synchronize()
    launches = int(lib.AetherSortKernelLaunches() - launches0)
    ms = begin.elapsed_time(end) / args.steps
    assert pa.last_sort_status(device) == 0
    value = n / (ms * 1e-3)
    # Per-stage times from a few more steps with the library's stage events switched on (two
    # event records per stage and call: kept out of the timed steps above).
    stages = {}
    if not args.no_stage_events:
        lib.AetherSortSetStageTiming(1)
        for s in range(max(1, min(args.steps, 8))):
            out = step(300 + s)
        torch.cuda.synchronize()
        stages = stage_times(lib, _native)
        lib.AetherSortSetStageTiming(0)
        assert pa.last_sort_status(device) == 0
    if args.kernels_only:  # a short run for a profiler: no end-to-end leg, no CPU leg
        clocks = sampler.stop()
        print(json.dumps({'metric': 'sorted particles/s', 'value': value, 'ms_per_step': ms,
                          'config': workload_config(workload, w, 1), 'stage_ms': stages,
                          'gpu_launches': launches, 'kernels_only': True,
                          'used_digit_passes': bool(pa.last_sort_used_digit_passes(device))}))
        return

    peak, peak_kind = measured_peak()
    top = max(stages, key=stages.get) if stages else None
    roofline = None
    if top:
        bytes_per_launch = STAGE_BYTES_PER_PARTICLE.get(top, 0) * n
        achieved = bytes_per_launch / (stages[top] * 1e-3) / 1e9
        roofline = {'bound': 'hbm', 'kernel': top, 'achieved': achieved, 'peak': peak,
                    'unit': 'GB/s', 'frac': achieved / peak, 'peak_kind': peak_kind,
                    'traffic': (NCU_DRAM_BYTES_PER_PARTICLE[top] * n
                                if top in NCU_DRAM_BYTES_PER_PARTICLE else None),
                    'traffic_source': 'ncu capture at 2^24 particles scaled by particle count',
                    'bytes_per_launch': bytes_per_launch,
                    'ms_per_launch': stages[top]}
    b_alg = algorithmic_bytes(n, cells)
    path_gbs = b_alg / (ms * 1e-3) / 1e9

    # ---- end to end: pinned host inputs in, results back to the host, every step ----
    e2e_steps = max(1, min(args.steps, 5))
    if steady:  # feed the end-to-end leg and the parity check a moved, nearly sorted state
        before = pa.sort_particles_by_cell(state['x'], state['y'], state['z'], w.grid, 1).keys >> 7
        move(state)
        x, y, z, v = state['x'], state['y'], state['z'], state['v']
        lib_keys = torch.empty(n, dtype=torch.int32, device=device)
        g = pa.particle_sort.native_grid(w.grid)
        _native.check(lib.AetherMakeKeys(x.data_ptr(), y.data_ptr(), z.data_ptr(), n,
                                         ctypes.byref(g), 1, lib_keys.data_ptr(), None),
                      'AetherMakeKeys')
        torch.cuda.synchronize()
        # The state was sorted before the move, so position i held cell before[i].
        crossing = float(((lib_keys >> 7) != before).float().mean())
        del before, lib_keys
    hx, hy, hz, hv = (t.cpu().pin_memory() for t in (x, y, z, v))
    # Two streams: `up` carries a step's host->device copies and its sort, `down` its
    # device->host copies, so that one step's results travel back while the next step's
    # inputs travel in (PCIe is full duplex).  Every step still copies all its inputs in and
    # all its results out inside the timed region; result buffers on the host alternate.
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)
    res_sets = [None, None]
    torch.cuda.synchronize()

    def e2e_step(s, slot):
        with torch.cuda.stream(up):
            dx, dy, dz, dv = (t.to(device, non_blocking=True) for t in (hx, hy, hz, hv))
            r = pa.sort_and_gather_particles(dx, dy, dz, dv, w.grid, workloads.step_seed(1234, s),
                                             path=path)
            outs = [r.order.keys, r.order.particle_index, r.order.cell_counts,
                    r.order.cell_start, *r.positions, r.velocity]
            sorted_done = torch.cuda.Event()
            sorted_done.record(up)
        if res_sets[slot] is None:
            res_sets[slot] = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        down.wait_event(sorted_done)
        with torch.cuda.stream(down):
            for h, o in zip(res_sets[slot], outs):
                h.copy_(o, non_blocking=True)
                o.record_stream(down)

    e2e_step(0, 0)
    e2e_step(1, 1)
    torch.cuda.synchronize()
    with torch.cuda.stream(up):
        begin.record(up)
    for s in range(e2e_steps):
        e2e_step(200 + s, s % 2)
    up.wait_stream(down)
    with torch.cuda.stream(up):
        end.record(up)
    torch.cuda.synchronize()
    e2e_ms = begin.elapsed_time(end) / e2e_steps
    clocks = sampler.stop()  # samples span the device-resident and the end-to-end regions
    res_host = res_sets[(e2e_steps - 1) % 2]
    h2d = sum(t.numel() * t.element_size() for t in (hx, hy, hz, hv))
    d2h = sum(t.numel() * t.element_size() for t in res_host)
    with torch.cuda.stream(up):
        assert pa.last_sort_status(device) == 0

    # ---- CPU baseline on this box's host cores (rank 0, N = 1 only) + parity ----
    from oracle import sort_oracle as so
    threads = host_threads()
    host = [t.numpy() for t in (hx, hy, hz, hv)]
    seed = workloads.step_seed(1234, 200 + e2e_steps - 1)
    t0 = time.perf_counter()
    want, xs, ys, zs, vs = cpu_reference_step(host, w.grid, seed, threads)
    cpu_s = time.perf_counter() - t0
    parity = (np.array_equal(res_host[0].numpy().view(np.uint32), want.keys)
              and np.array_equal(res_host[1].numpy(), want.particle_index)
              and np.array_equal(res_host[2].numpy(), want.cell_counts)
              and np.array_equal(res_host[3].numpy(), want.cell_start)
              and np.array_equal(res_host[4].numpy(), xs)
              and np.array_equal(res_host[5].numpy(), ys)
              and np.array_equal(res_host[6].numpy(), zs)
              and np.array_equal(res_host[7].numpy()[:, :n], vs[:, :n]))
    baseline = {'value': n / cpu_s, 'unit': 'particles/s', 'cores': so.c_threads(threads),
                'kind': 'port',
                'sample': f'all {n} particles of {workload}, one step, C restatement of the '
                          f'reference path with OpenMP on {so.c_threads(threads)} threads'}
    try:
        baseline['torch_cpu_binning'] = torch_cpu_binning_rate(w, threads)
    except Exception as exc:
        baseline['torch_cpu_binning'] = {'unavailable': repr(exc)}
    if w.name == 'c1_1m_64':
        baseline['numpy_replay'] = numpy_replay_rate()
    line = {
        'metric': 'sorted particles/s', 'value': value, 'unit': 'particles/s', 'n_gpus': 1,
        'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'u32', 'data': 'synthetic',
        'config': workload_config(workload, w, 1),
        'details': {'path': args.path,
                    'steady_state': ({'dt': STEADY_DT, 'cell_crossing_fraction': crossing,
                                      'step': (('push kernel, then' if args.separate_push
                                                else 'push fused into the')
                                               + ' re-sort of the previous sorted state' +
                                               (' + collisions' if args.collide else ''))}
                                     if steady else None)},
        'clocks': {'sm_mhz': clocks['sm_mhz'], 'sm_max_mhz': clocks['sm_max_mhz'],
                   'reasons': clocks['reasons'], 'samples': clocks['samples']},
        'e2e': {'value': n / (e2e_ms * 1e-3), 'unit': 'particles/s', 'h2d_bytes_per_step': h2d,
                'd2h_bytes_per_step': d2h, 'ms_per_step': e2e_ms, 'steps': e2e_steps,
                'overlap': 'results of step k copied out while inputs of step k+1 are copied in'},
        'gpu_launches': launches,
        'roofline': roofline,
        'path_roofline': {'algorithmic_bytes': b_alg, 'achieved_gbs': path_gbs,
                          'frac_of_nominal_8000': path_gbs / NOMINAL_HBM_GBS,
                          'frac_of_measured': path_gbs / peak, 'peak_kind': peak_kind},
        'stage_ms': stages,
        'used_digit_passes': bool(pa.last_sort_used_digit_passes(device)),
        'cpu_baseline': baseline,
        'parity': 'bit-exact vs CPU oracle' if parity else 'MISMATCH vs CPU oracle',
    }
    print(json.dumps(line))
    if not parity:
        sys.exit(3)


def run_exchange_alone(args):
    """The multi-GPU step's kernels on ONE GPU, for profiler captures and stage timing: a
    single rank "exchanges" its whole input with itself (every particle goes through the
    fused partition + exchange kernel into the rank's own receive buffer, slice by slice,
    flags and waits included) and sorts the received arrays with the sliced local sort.  The
    result is checked against the ordinary sort of the same input."""
    import torch
    import project_aether_b200 as pa
    from project_aether_b200 import _native, slab_sort, workloads
    from project_aether_b200.particle_sort import native_grid
    lib = _native.load_library()
    device = torch.device('cuda', 0)
    torch.cuda.set_device(device)
    workload, w = select_workload(args)
    n, cells, g = w.n, w.grid.num_cells, native_grid(w.grid)
    slices = slab_sort.slices_for(n)
    x, y, z, v = workloads.make_particles(w, device, seed=0)
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    part_ws = torch.empty(lib.AetherSlabPartitionWorkspaceBytes(n, 1), dtype=torch.uint8, device=device)
    totals = torch.zeros(1, dtype=torch.int64, device=device)
    per_slice = torch.zeros(slices, dtype=torch.int64, device=device)
    capacity, flag_words = n + 8, slab_sort.FLAG_WORDS
    buffer = torch.zeros(flag_words + 6 * capacity, dtype=torch.float32, device=device)
    flags = (ctypes.c_void_p * 1)(buffer.data_ptr())
    arrays = (ctypes.c_void_p * 1)(buffer.data_ptr() + 4 * flag_words)
    data = buffer[flag_words:]
    error = torch.zeros(1, dtype=torch.int32, device=device)
    segments = torch.empty(lib.AetherSlabSegmentsBytes(), dtype=torch.uint8, device=device)
    totals2d = torch.empty((1, 1), dtype=torch.int64, device=device)
    sort_ws = torch.empty(lib.AetherSortSlicedWorkspaceBytes(capacity, n, cells, slices),
                          dtype=torch.uint8, device=device)
    keys, index = (torch.empty(capacity, dtype=torch.int32, device=device) for _ in range(2))
    counts = torch.empty(cells, dtype=torch.int32, device=device)
    start = torch.empty(cells + 1, dtype=torch.int32, device=device)
    xs, ys, zs = (torch.empty(capacity, device=device) for _ in range(3))
    vs = torch.empty((3, capacity), device=device)
    _native.check(lib.AetherSlabExchangeSetResidentBlocks(4), 'AetherSlabExchangeSetResidentBlocks')

    def step(epoch, seed):
        ck = _native.check
        ck(lib.AetherSlabExchangeCount(x.data_ptr(), n, ctypes.byref(g), 1, totals.data_ptr(),
                                       part_ws.data_ptr(), part_ws.numel(), stream), 'count')
        ck(lib.AetherSlabExchangeSliceCounts(n, 1, slices, per_slice.data_ptr(), part_ws.data_ptr(),
                                             part_ws.numel(), stream), 'slice counts')
        ck(lib.AetherSlabExchangePrepare(per_slice.data_ptr(), 1, slices, 0, totals2d.data_ptr(),
                                         segments.data_ptr(), stream), 'prepare')
        for k in range(slices):
            ck(lib.AetherSlabExchangeScatterSliced(
                x.data_ptr(), y.data_ptr(), z.data_ptr(), v.data_ptr(), v.stride(0), n, 0.0, None,
                None, ctypes.byref(g), 1, 0, arrays, capacity, totals2d.data_ptr(), error.data_ptr(),
                slices, k, epoch, flags, part_ws.data_ptr(), part_ws.numel(), stream), 'exchange')
        ck(lib.AetherSortSlicedBegin(capacity, n, ctypes.byref(g), slices, sort_ws.data_ptr(),
                                     sort_ws.numel(), stream), 'begin')
        for k in range(slices):
            ck(lib.AetherSlabExchangeWait(buffer.data_ptr(), 1, slices, k, epoch, 4,
                                          error.data_ptr(), stream), 'wait')
            ck(lib.AetherSortSlicedSlice(
                data.data_ptr(), data[capacity:].data_ptr(), data[2 * capacity:].data_ptr(),
                data[3 * capacity:].data_ptr(), capacity, capacity, n, ctypes.byref(g), seed,
                segments.data_ptr(), slices, k, sort_ws.data_ptr(), sort_ws.numel(), stream), 'slice')
        ck(lib.AetherSortSlicedFinish(
            capacity, n, ctypes.byref(g), segments.data_ptr(), slices, keys.data_ptr(),
            index.data_ptr(), counts.data_ptr(), start.data_ptr(), xs.data_ptr(), ys.data_ptr(),
            zs.data_ptr(), vs.data_ptr(), capacity, sort_ws.data_ptr(), sort_ws.numel(), stream),
            'finish')

    for s in range(max(1, args.warmup)):
        step(s + 1, workloads.step_seed(1234, s))
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for s in range(args.steps):
        step(100 + s, workloads.step_seed(1234, 100 + s))
    end.record()
    torch.cuda.synchronize()
    want = pa.sort_and_gather_particles(x, y, z, v, w.grid, workloads.step_seed(1234, 100 + args.steps - 1))
    same = (torch.equal(want.order.particle_index, index[:n]) and torch.equal(want.order.keys, keys[:n])
            and torch.equal(want.order.cell_start, start) and torch.equal(want.positions[2], zs[:n])
            and torch.equal(want.velocity[:, :n], vs[:, :n]))
    print(json.dumps({'mode': 'exchange and sliced sort of one rank on one GPU', 'slices': slices,
                      'ms_per_step': begin.elapsed_time(end) / args.steps,
                      'config': workload_config(workload, w, 1), 'device_status': int(error),
                      'equal_to_ordinary_sort': bool(same)}))
    if not same or int(error) != 0:
        sys.exit(3)


# --------------------------------------------------------------------------------------
# N > 1: one rank per GPU, x-slab decomposition.
# --------------------------------------------------------------------------------------

def distributed_parity(dist, slab_sort, share, w, seed, push, exchange, device):
    """One distributed sort of `share` (this rank's x, y, z, velocity) checked on every rank
    against the CPU oracle: the ranks' shares are gathered, the oracle replays the move, the
    exchange rule (source ranks in order, each block in source order) and the slab-local sort
    of this rank's slab.  Returns True when keys, permutation, counts, starts, positions and
    velocities all match bit for bit on this rank."""
    import torch
    from oracle import sort_oracle as so
    world, rank = dist.get_world_size(), dist.get_rank()
    x, y, z, v = share
    m = x.numel()
    got = slab_sort.distributed_sort(x, y, z, v, w.grid, seed, exchange=exchange, push=push)
    sizes = torch.zeros(world, dtype=torch.int64, device=device)
    sizes[rank] = m
    dist.all_reduce(sizes)
    longest = int(sizes.max())
    mine = torch.zeros((6, longest), dtype=torch.float32, device=device)
    for k, t in enumerate((x, y, z, v[0, :m], v[1, :m], v[2, :m])):
        mine[k, :m] = t
    everyone = torch.empty((world, 6, longest), dtype=torch.float32, device=device)
    dist.all_gather_into_tensor(everyone, mine)
    host = everyone.cpu().numpy()
    del everyone, mine
    ogrid = so.Grid(tuple(w.grid.lo), tuple(w.grid.hi), tuple(w.grid.cells))
    blocks = []
    for s in range(world):
        arrays = [host[s, k, :int(sizes[s])] for k in range(6)]
        if push is not None:
            p, q = so.push_particles(arrays[:3], arrays[3:], push[0], push[1], push[2])
            arrays = list(p) + list(q)
        here = so.slab_of(arrays[0], ogrid, world) == rank
        blocks.append([a[here] for a in arrays])
    recv = [np.ascontiguousarray(np.concatenate([b[k] for b in blocks])) for k in range(6)]
    count = recv[0].size
    padded = -(-count // 4) * 4
    vel = np.zeros((3, padded), np.float32)
    vel[:, :count] = np.stack(recv[3:])
    offset, width = slab_sort.slab_range(w.grid, world, rank)
    want, xs, ys, zs, vs = so.c_sort_particles(recv[0], recv[1], recv[2], vel, ogrid, seed,
                                               threads=max(1, host_threads() // world),
                                               ix_offset=offset, nx_local=width)
    ok = (got.order.keys.numel() == count
          and np.array_equal(got.order.keys.cpu().numpy().view(np.uint32), want.keys)
          and np.array_equal(got.order.particle_index.cpu().numpy(), want.particle_index)
          and np.array_equal(got.order.cell_counts.cpu().numpy(), want.cell_counts)
          and np.array_equal(got.order.cell_start.cpu().numpy(), want.cell_start)
          and all(np.array_equal(g.cpu().numpy(), h) for g, h in zip(got.positions, (xs, ys, zs)))
          and np.array_equal(got.velocity.cpu().numpy()[:, :count], vs[:, :count]))
    return ok, count


def run_multi(args):
    import torch
    import torch.distributed as dist
    import project_aether_b200 as pa
    from project_aether_b200 import _native, slab_sort, workloads

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', str(args.gpus)))
    local = int(os.environ.get('LOCAL_RANK', str(rank)))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29512')
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=device)
    lib = _native.load_library()
    workload, w = select_workload(args)
    n_total = w.n
    n_local = n_total // world
    x, y, z, v = workloads.make_particles(w, device, seed=rank, n=n_local)

    exchange = os.environ.get('AETHER_EXCHANGE', 'peer')  # 'peer' (NVLink stores) or 'nccl'
    # Tuning of the sliced exchange from the environment (for sweeps): overlap 0/1, resident
    # exchange blocks per multiprocessor 0..4, local sort on a stream of its own 0/1, transport
    # 'stores' or 'copies'.
    knobs = {key: os.environ.get(name) for key, name in (
        ('overlap', 'AETHER_EXCHANGE_OVERLAP'), ('resident_blocks', 'AETHER_EXCHANGE_BLOCKS'),
        ('sort_stream', 'AETHER_EXCHANGE_SORT_STREAM'))}
    slab_sort.configure(**{key: (None if value is None else int(value))
                           for key, value in knobs.items()},
                        transport=os.environ.get('AETHER_EXCHANGE_TRANSPORT'))
    steady = w.name.startswith('c5')
    state = {'x': x, 'y': y, 'z': z, 'v': v}

    def squeeze_into_own_slab(px, grid):
        lo, hi = grid.lo[0], grid.hi[0]
        width = (hi - lo) / world
        px.sub_(lo).div_(world).add_(lo + rank * width).clamp_(
            max=lo + (rank + 1) * width * (1 - 1e-7))

    if steady:
        # Squeeze this rank's share into its own slab, then sort it once: the loop starts
        # from a cell-sorted state in which every particle is at home.
        squeeze_into_own_slab(x, w.grid)
        first = slab_sort.distributed_sort(x, y, z, v, w.grid, 99, exchange=exchange)
        state = {'x': first.positions[0], 'y': first.positions[1], 'z': first.positions[2],
                 'v': first.velocity}
        del first

    move = (STEADY_DT, w.grid.lo, w.grid.hi) if steady else None

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

    def device_status():
        worst = max(pa.last_sort_status(device), slab_sort.exchange_status(device))
        status = torch.tensor([worst], device=device)
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
        return int(status)

    assert device_status() == 0

    launches0 = lib.AetherSortKernelLaunches()
    sampler = ClockSampler(device.index)
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
    # Stage and phase times of one more step, kept out of the timed steps: the library's stage
    # events, phase events on the caller's stream, and the exchange kernels (all slices) on the
    # stream of their own on which they run beside the local sort's count and scatter kernels.
    # With the sliced exchange a stage's figure is that of the last slice's launch.
    lib.AetherSortSetStageTiming(1)
    marks = []
    if exchange == 'peer':
        slab_sort.time_exchange(device, True)
    slab_sort.distributed_sort(state['x'], state['y'], state['z'], state['v'], w.grid,
                               workloads.step_seed(1234, 999), marks=marks, exchange=exchange,
                               push=move)
    torch.cuda.synchronize()
    stages = stage_times(lib, _native)
    lib.AetherSortSetStageTiming(0)
    phases = {marks[i][0]: marks[i - 1][1].elapsed_time(marks[i][1]) for i in range(1, len(marks))}
    exchange_ms = slab_sort.last_exchange_ms(device) if exchange == 'peer' else None
    slab_sort.time_exchange(device, False)
    if args.kernels_only:  # a short run for sweeps: no parity, end-to-end or one-GPU leg
        if rank == 0:
            print(json.dumps({'metric': 'sorted particles/s', 'value': n_total / (ms * 1e-3),
                              'n_gpus': world, 'ms_per_step': ms,
                              'config': workload_config(workload, w, world),
                              'stage_ms_rank0': stages, 'phase_ms_rank0': phases,
                              'exchange_ms_rank0': exchange_ms, 'step_ms_rank0': step_ms,
                              'kernels_only': True}))
        dist.barrier()
        dist.destroy_process_group()
        return
    received = torch.tensor([out.order.keys.numel()], device=device, dtype=torch.int64)
    dist.all_reduce(received)
    assert int(received) == n_local * world, 'particles were lost in the exchange'
    assert device_status() == 0, 'a bounded device wait gave up during the timed steps'

    # Parity where the numbers are made: one step's results on every rank against the CPU
    # oracle's replay of move + exchange + slab-local sort.  At the full size on up to two
    # ranks; with more ranks (host memory: every rank holds all shares) on a case of 2^24
    # particles per rank at the same particles per cell.
    if world <= 2 or n_local <= (1 << 24):
        check_w, share = w, (state['x'], state['y'], state['z'], state['v'])
        if not steady:
            share = (x, y, z, v)
    else:
        check_w = workloads.scaled_workload(w.name, 24 + int(np.log2(world)))
        share = workloads.make_particles(check_w, device, seed=rank, n=1 << 24)
        if steady:
            squeeze_into_own_slab(share[0], check_w.grid)
            first = slab_sort.distributed_sort(*share, check_w.grid, 99, exchange=exchange)
            share = (*first.positions, first.velocity)
    ok, checked = distributed_parity(dist, slab_sort, share, check_w, workloads.step_seed(1234, 7),
                                     move, exchange, device)
    verdict = torch.tensor([0 if ok else 1, checked], device=device, dtype=torch.int64)
    dist.all_reduce(verdict)
    parity_ok = int(verdict[0]) == 0
    del share

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

    # Strong-scaling denominator: the same workload, whole, on one GPU (rank 0 alone), over
    # as many steps as the distributed run.
    single = None
    del hx, hy, hz, hv, pinned
    if rank == 0:
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        ax, ay, az, av = workloads.make_particles(w, device, seed=0)
        one = {'x': ax, 'y': ay, 'z': az, 'v': av}
        if steady:
            first = pa.sort_and_gather_particles(ax, ay, az, av, w.grid, 99)
            one = {'x': first.positions[0], 'y': first.positions[1], 'z': first.positions[2],
                   'v': first.velocity}
            del first

        def one_step(s):
            r = pa.sort_and_gather_particles(one['x'], one['y'], one['z'], one['v'], w.grid,
                                             workloads.step_seed(1234, s), push=move)
            if steady:
                one.update(x=r.positions[0], y=r.positions[1], z=r.positions[2], v=r.velocity)

        for s in range(3):
            one_step(s)
        torch.cuda.synchronize()
        begin.record()
        for s in range(args.steps):
            one_step(50 + s)
        end.record()
        torch.cuda.synchronize()
        one_ms = begin.elapsed_time(end) / args.steps
        single = {'value': n_total / (one_ms * 1e-3), 'unit': 'particles/s', 'ms_per_step': one_ms,
                  'steps': args.steps}
        del ax, ay, az, av, one
    dist.barrier()

    if rank == 0:
        peak, peak_kind = measured_peak()
        n_rank = n_total // world
        top = max(stages, key=stages.get) if stages else None
        roofline = None
        if top:
            per_particle = STAGE_BYTES_PER_PARTICLE.get(top, 0)
            nbytes = per_particle * n_rank
            achieved = nbytes / (stages[top] * 1e-3) / 1e9
            roofline = {'bound': 'hbm', 'kernel': top, 'achieved': achieved, 'peak': peak,
                        'unit': 'GB/s', 'frac': achieved / peak, 'peak_kind': peak_kind,
                        'traffic': (NCU_DRAM_BYTES_PER_PARTICLE[top] * n_rank
                                    if top in NCU_DRAM_BYTES_PER_PARTICLE else None),
                        'bytes_per_launch': nbytes, 'ms_per_launch': stages[top]}
        nvlink = None
        if exchange_ms and not steady:
            # 24 B per particle, (G-1)/G of them, cross NVLink: by device-to-device copies out
            # of the staging rows the partition kernel fills, or by the kernel's own stores.
            # Timed from the first slice's partition to the last slice's signal of one step,
            # while the local sort's kernels run beside the exchange.
            crossing = 24 * n_rank * (world - 1) / world
            link = crossing / (exchange_ms * 1e-3) / 1e9
            by_stores = slab_sort.transport_default(world) == 'stores'
            nvlink = {'kernel': ('slab_scatter_kernel (all slices)' if by_stores else
                                 'slab_scatter_kernel into staging rows + copy engines (all slices)'),
                      'bytes_out_per_gpu': crossing,
                      'achieved': link, 'peak': PEER_COPY_GBS, 'unit': 'GB/s',
                      'frac': link / PEER_COPY_GBS, 'ms': exchange_ms,
                      'peak_kind': 'peer copy measured on this pool'}
        line = {
            'metric': 'sorted particles/s', 'value': n_total / (ms * 1e-3), 'unit': 'particles/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms,
            'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'u32',
            'data': 'synthetic',
            'config': workload_config(workload, w, world),
            'details': {'exchange': ('one NCCL all-to-all per payload array' if exchange != 'peer'
                                     else 'partition kernel stores into the peers\' receive buffers '
                                          'over NVLink'
                                     if slab_sort.transport_default(world) == 'stores'
                                     else 'partition kernel fills staging rows, copy engines carry '
                                          'them into the peers\' receive buffers over NVLink'),
                        'overlap_with_local_sort': bool(exchange == 'peer' and
                                                        slab_sort.overlap_default(world)),
                        'initial_share': ('cell-sorted particles of the rank\'s own slab; every '
                                          'step moves them (dt %g) and re-sorts' % STEADY_DT
                                          if steady else 'random 1/G of all particles per rank')},
            'clocks': {'sm_mhz': clocks['sm_mhz'], 'sm_max_mhz': clocks['sm_max_mhz'],
                       'reasons': clocks['reasons'], 'samples': clocks['samples']},
            'e2e': {'value': n_total / (e2e_ms * 1e-3), 'unit': 'particles/s',
                    'h2d_bytes_per_step': int(bytes_io[0]), 'd2h_bytes_per_step': int(bytes_io[1]),
                    'ms_per_step': e2e_ms, 'steps': e2e_steps},
            'gpu_launches': launches, 'roofline': roofline, 'nvlink': nvlink,
            'stage_ms_rank0': stages, 'phase_ms_rank0': phases, 'step_ms_rank0': step_ms,
            'single_gpu_same_workload': single,
            'scaling_efficiency_same_workload': (single['ms_per_step'] / ms / world
                                                 if single else None),
            'cpu_baseline': None,
            'parity': (('bit-exact vs CPU oracle' if parity_ok else 'MISMATCH vs CPU oracle') +
                       f' (every rank; {int(verdict[1])} particles of '
                       f'{check_w.name} on grid {list(check_w.grid.cells)})'),
        }
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
    if not parity_ok:
        sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default=None)
    ap.add_argument('--log2n', type=int, default=0,
                    help='scale the workload to 2^LOG2N particles at the same particles per cell '
                         '(the grid\'s z extent follows); for profiler captures and quick runs')
    ap.add_argument('--kernels-only', action='store_true',
                    help='stop after the device-resident timing (no end-to-end leg, no CPU '
                         'baseline, no parity check); for profiler captures and sweeps')
    ap.add_argument('--no-stage-events', action='store_true',
                    help='single GPU: skip the extra steps that collect per-stage event times')
    ap.add_argument('--separate-push', action='store_true',
                    help='steady-state workload only: run the move stage as its own kernel '
                         'instead of inside the sort kernels')
    ap.add_argument('--collide', action='store_true',
                    help='steady-state workload only: run the collision stage after every sort')
    ap.add_argument('--exchange-alone', action='store_true',
                    help='one GPU: run the multi-GPU step\'s kernels (partition + exchange into the '
                         'rank\'s own buffer, sliced local sort) for one rank; for profiler captures')
    ap.add_argument('--path', default='auto', choices=['auto', 'digits', 'bucketed'])
    ap.add_argument('--finish-shape', default='auto', choices=['auto', 'large'],
                    help='single GPU: plan the large shape of the finish kernel whatever the size '
                         '(to capture the 64 M configuration\'s kernel on a scaled-down case)')
    args = ap.parse_args()
    if args.impl == 'reference':
        run_reference(args)
    elif args.exchange_alone:
        run_exchange_alone(args)
    elif args.gpus == 1:
        run_single(args)
    else:
        run_multi(args)


if __name__ == '__main__':
    main()
