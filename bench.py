"""Benchmark of the DSMC particle sort: sorted particles per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one full sort call on one synthetic particle state: key
generation, the sort, per-cell counts and starts, and the sorted SoA payload.
Prints ONE JSON line (rank 0).  `value` is measured with the inputs resident in
HBM; `e2e` is the same call fed from pinned host buffers with the results read
back to the host inside the timed region.  `--impl reference` times the CPU
restatement of the reference path (the C oracle, all host threads) instead.
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
    'particle_push': 24 + 24, 'collide': 12 + 12,
}


# DRAM bytes per particle (dram__bytes_read.sum + dram__bytes_write.sum) of each bucketed-path
# kernel, from one ncu capture at 2^24 particles of the same density
# (profiles/bucketed_kernels_c3_hypersonic_16m.md); traffic grows in proportion to the
# particle count, so a launch's traffic is this figure times its particles.
NCU_DRAM_BYTES_PER_PARTICLE = {'bucket_count': 12.2, 'bucket_scatter': 52.9,
                               'bucket_finish': 61.5}


def measured_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        try:
            return float(json.load(open(path))['hbm_gbs']), 'measured'
        except Exception:
            pass
    return FALLBACK_HBM_GBS, 'fallback'


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


def cpu_reference_step(host, grid, seed, threads=0):
    from oracle import sort_oracle as so
    g = so.Grid(tuple(grid.lo), tuple(grid.hi), tuple(grid.cells))
    return so.c_sort_particles(host[0], host[1], host[2], host[3], g, seed, threads=threads)


def run_reference(args, workload):
    """The reference path on host cores: C restatement of keys -> stable sort ->
    counts/starts -> payload gather, all threads."""
    import torch
    from project_aether_b200 import workloads
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    w = workloads.WORKLOADS[workload]
    n = w.n
    cores = os.cpu_count() or 1
    x, y, z, v = workloads.make_particles(w, 'cpu', seed=0, n=n)
    host = [t.numpy() for t in (x, y, z, v)]
    t0 = time.perf_counter()
    cpu_reference_step(host, w.grid, workloads.step_seed(1234, 0))
    first = time.perf_counter() - t0
    sample = n
    budget = min(240.0, 15.0 * (args.steps + args.warmup))  # seconds for the whole run
    if first * (args.steps + args.warmup) > budget:  # keep the run within a few minutes
        sample = max(1 << 20, int(n * budget / (first * (args.steps + args.warmup))))
        x, y, z, v = workloads.make_particles(w, 'cpu', seed=0, n=sample)
        host = [t.numpy() for t in (x, y, z, v)]
    for s in range(max(0, args.warmup - 1)):
        cpu_reference_step(host, w.grid, workloads.step_seed(1234, s + 1))
    t0 = time.perf_counter()
    for s in range(args.steps):
        cpu_reference_step(host, w.grid, workloads.step_seed(1234, s + 100))
    dt = (time.perf_counter() - t0) / args.steps
    value = sample / dt
    desc = (f'{sample} of {n} particles of {workload} per step, '
            f'C restatement of the reference path, OpenMP, {cores} threads')
    line = {
        'impl': 'reference', 'metric': 'sorted particles/s', 'value': value, 'unit': 'particles/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'u32',
        'data': 'synthetic', 'config': {'workload': workload, 'particles': n,
                                        'cells': list(w.grid.cells)},
        'cpu_baseline': {'value': value, 'unit': 'particles/s', 'cores': cores, 'kind': 'port',
                         'sample': desc},
        'e2e': {'value': value, 'unit': 'particles/s', 'h2d_bytes_per_step': 0,
                'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


def run_single(args, workload):
    import torch
    import project_aether_b200 as pa
    from project_aether_b200 import _native, workloads
    lib = _native.load_library()  # raises if the CUDA library is missing
    if not torch.cuda.is_available():
        raise RuntimeError('bench.py needs a CUDA GPU (no CPU fallback exists)')
    device = torch.device('cuda', int(os.environ.get('LOCAL_RANK', '0')))
    torch.cuda.set_device(device)
    w = workloads.WORKLOADS[workload]
    n, cells = w.n, w.grid.num_cells
    x, y, z, v = workloads.make_particles(w, device, seed=0)
    path = {'auto': pa.PATH_AUTO, 'digits': pa.PATH_DIGIT_PASSES, 'bucketed': pa.PATH_BUCKETED}[
        args.path]

    # Steady-state re-sort (configuration 5): the state starts cell-sorted and every step
    # moves it by x += v*dt (specular walls) before sorting it again; the sorted output is
    # the next step's input.  dt is the value at which about 5 % of the particles cross a
    # cell boundary for unit thermal speed and 1/256 cells.
    steady = workload.startswith('c5')
    steady_dt = 8.2e-5
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
                                steady_dt, w.grid.lo, w.grid.hi)

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
        fused = (steady_dt, w.grid.lo, w.grid.hi) if steady and not args.separate_push else None
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
    lib.AetherSortSetStageTiming(1)
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
    stage_count = lib.AetherSortStageCount()
    stage_ms = (ctypes.c_float * stage_count)()
    _native.check(lib.AetherSortReadStageTimes(stage_ms, stage_count), 'AetherSortReadStageTimes')
    lib.AetherSortSetStageTiming(0)
    stages = {lib.AetherSortStageName(i).decode(): float(stage_ms[i]) for i in range(stage_count)
              if stage_ms[i] >= 0}
    assert pa.last_sort_status(device) == 0
    value = n / (ms * 1e-3)

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
    cores = os.cpu_count() or 1
    host = [t.numpy() for t in (hx, hy, hz, hv)]
    seed = workloads.step_seed(1234, 200 + e2e_steps - 1)
    t0 = time.perf_counter()
    want, xs, ys, zs, vs = cpu_reference_step(host, w.grid, seed)
    cpu_s = time.perf_counter() - t0
    parity = (np.array_equal(res_host[0].numpy().view(np.uint32), want.keys)
              and np.array_equal(res_host[1].numpy(), want.particle_index)
              and np.array_equal(res_host[2].numpy(), want.cell_counts)
              and np.array_equal(res_host[3].numpy(), want.cell_start)
              and np.array_equal(res_host[4].numpy(), xs)
              and np.array_equal(res_host[7].numpy()[:, :n], vs[:, :n]))
    line = {
        'metric': 'sorted particles/s', 'value': value, 'unit': 'particles/s', 'n_gpus': 1,
        'steps': args.steps, 'warmup': warmup, 'ms_per_step': ms, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'u32', 'data': 'synthetic',
        'config': {'workload': workload, 'particles': n, 'cells': list(w.grid.cells),
                   'path': args.path, 'l2': 'inputs larger than L2 (no flush needed)',
                   'steady_state': ({'dt': steady_dt, 'cell_crossing_fraction': crossing,
                                     'step': (('push kernel, then' if args.separate_push else 'push fused into the')
                                              + ' re-sort of the previous sorted state' +
                                              (' + collisions' if args.collide else ''))}
                                    if steady else None),
                   'seed_per_step': 'run_seed ^ (step << 20)'},
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
        'cpu_baseline': {'value': n / cpu_s, 'unit': 'particles/s', 'cores': cores,
                         'kind': 'port',
                         'sample': f'all {n} particles of {workload}, one step, C restatement '
                                   f'of the reference path with OpenMP on {cores} threads'},
        'parity': 'bit-exact vs CPU oracle' if parity else 'MISMATCH vs CPU oracle',
    }
    print(json.dumps(line))
    if not parity:
        sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default=None)
    ap.add_argument('--separate-push', action='store_true',
                    help='steady-state workload only: run the move stage as its own kernel '
                         'instead of inside the sort kernels')
    ap.add_argument('--collide', action='store_true',
                    help='steady-state workload only: run the collision stage after every sort')
    ap.add_argument('--path', default='auto', choices=['auto', 'digits', 'bucketed'])
    args = ap.parse_args()
    workload = args.workload or ('c3_64m_hypersonic' if args.gpus == 1 else 'c4_256m_512')
    if args.impl == 'reference':
        run_reference(args, workload)
    elif args.gpus == 1:
        run_single(args, workload)
    else:
        from project_aether_b200 import multi_gpu_bench
        multi_gpu_bench.run(args, workload)


if __name__ == '__main__':
    main()
