"""Benchmark of the point-neuron hot path on the V1-scale synthetic network.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload ("c3"): 230 924 GLIF-3 neurons in 17 types, ~70 M synapses from a Gaussian distance
rule, 17 400 Poisson virtual cells, dt = 0.25 ms (bmtk_b200.workloads.c3; synthetic, seeded).
One bench STEP simulates 1000 ms of biological time = 4000 update steps. Metric: synaptic events
delivered per wall second (whole job), with sim-ms per wall-ms beside it.

  value  device-resident: Poisson cells generated on the GPU (Philox), spikes logged on the GPU;
         timed with CUDA events on the engine's stream, max over ranks.
  e2e    through the public Engine API with HOST buffers: every step hands that second's virtual
         spikes over from pinned host memory (set_input_spikes), runs, and reads the spike
         list back (fetch_spikes); wall clock between barriers.
  roofline  per-launch CUDA-event time of the dominant kernel in a profiled pass of the same
         workload, against algorithmic bytes (128 B per neuron-step, 16 B per synaptic event).
  cpu_baseline  the fp64 CPU oracle (OpenMP port; the reference's own engine, NEST, is not
         available) on a bounded slice of the same network, rank 0, N = 1 only.

With N > 1 the neurons are split into N contiguous blocks (strong scaling: the network is fixed);
each rank owns the CSR rows of its targets and the ranks exchange the spike ids of every phase
inside the stepping kernel over peer memory (NVLink; --exchange nccl: one NCCL all-gather per
min-delay window around the per-step kernels).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BYTES_PER_NEURON_STEP = 128.0
BYTES_PER_EVENT = 16.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu (see profiles/); None until captured
# per update step for the persistent kernel (profiles/persistent_kernel_c3_phases.md), per launch for the others
# (profiles/glif_update_2M_neurons_ncu_full.md scaled to this network, profiles/propagate_atomic_c2like_100k_ncu_full.md
# at 12.4 B per event)
NCU_TRAFFIC_BYTES = {'glif_update': 102.8 * 230924, 'propagate': None, 'persistent_per_step': 5.97e6,
                     'pipelined_per_step': 3.81e6}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='b200', choices=['b200', 'reference'])
    ap.add_argument('--scale', type=float, default=1.0, help='shrink the network (testing only)')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-cpu', action='store_true')
    ap.add_argument('--cpu-slice-ms', type=float, default=250.0)
    ap.add_argument('--step-ms', type=float, default=1000.0, help='simulated ms per bench step (1000 = the configuration)')
    ap.add_argument('--workload', default='c3', choices=['c0', 'c1', 'c2', 'c3', 'c4'],
                    help='c3: the V1-scale network (the headline line). c4: trial sweep, the 50 000-neuron E/I network as 64 '
                         'independent trials over one CSR, trials sharded over the ranks, one step = 500 ms. c0 / c1 / c2: the '
                         'small network (3000 ms), the current-clamp sweep (1500 ms) and the mid-scale E/I network (1000 ms; '
                         'neurons in contiguous blocks with several ranks), one step = the whole configured run')
    ap.add_argument('--trials', type=int, default=64)
    ap.add_argument('--engine-option', action='append', default=[], metavar='KEY=VALUE',
                    help='extra engine option (bmtk_engine_set_option), e.g. pipeline=0 for the two-phase persistent kernel')
    ap.add_argument('--exchange', default='p2p', choices=['p2p', 'nccl'],
                    help='several ranks: spike exchange inside the persistent kernel over peer memory, or one NCCL '
                         'all-gather per window around the per-step kernels')
    return ap.parse_args()


def extra_options(args):
    out = {}
    for kv in args.engine_option:
        k, _, v = kv.partition('=')
        out[k] = int(v)
    return out


def make_network(scale, lo_hi=None, poisson_online=True):
    from bmtk_b200 import workloads as W
    n = int(round(230924 * scale))
    nv = max(8, int(round(17400 * scale)))
    radius = 845.0 * np.sqrt(scale)
    lo, hi = lo_hi if lo_hi else (0, n)
    return W.c3(n=n, n_virtual=nv, radius_um=radius, lo=lo, hi=hi, poisson_online=poisson_online)


def peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        return float(json.load(open(p))['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


class ClockSampler(object):
    """nvidia-smi clocks and throttle reasons sampled every 20 ms. The sampler is started (and has printed its first
    line) before the timed region begins; begin() / stop() bracket the region and only the samples whose time
    stamp lies inside it are reported (`window`: "timed region"). A region too short to hold a sample reports the
    samples nearest to it instead and says so."""
    Q = ('timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
         'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile('w+', suffix='.csv', delete=False)
        self.p = None
        self.t0 = self.t1 = None
        try:
            self.p = subprocess.Popen(['nvidia-smi', '-i', str(gpu_index), '--query-gpu=' + self.Q,
                                       '--format=csv,noheader,nounits', '-lms', '20'], stdout=self.f,
                                      stderr=subprocess.DEVNULL)
        except OSError:
            return
        t = time.time()
        while time.time() - t < 2.0 and os.path.getsize(self.f.name) == 0:    # until the first sample is there
            time.sleep(0.01)

    def begin(self):
        self.t0 = time.time()

    def stop(self):
        self.t1 = time.time()
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.p is None:
            return out
        time.sleep(0.03)   # one more sample, in case the region was shorter than the period
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        import datetime
        rows = []
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(',')]
            if len(c) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(c[0], '%Y/%m/%d %H:%M:%S.%f').timestamp()
                rows.append((ts, float(c[1]), float(c[2]), float(c[3]),
                             [nm for nm, v in zip(names, c[5:9]) if v.lower().startswith('active')]))
            except ValueError:
                continue
        self.f.close()
        os.unlink(self.f.name)
        t0 = self.t0 if self.t0 is not None else 0.0
        inside = [r for r in rows if t0 <= r[0] <= self.t1]
        window = 'timed region'
        if not inside and rows:
            mid = 0.5 * (t0 + self.t1)
            inside = sorted(rows, key=lambda r: abs(r[0] - mid))[:2]
            window = 'nearest samples (the timed region was shorter than the sampling period)'
        if inside:
            out.update(sm_mhz=float(np.median([r[1] for r in inside])), sm_max_mhz=float(max(r[2] for r in inside)),
                       reasons=sorted(set(x for r in inside for x in r[4])), samples=len(inside),
                       power_w_max=float(max(r[3] for r in inside)), window=window)
        return out


def poisson_chunk(rng, rates_hz, dt, step0, n_steps):
    """Virtual spikes of one chunk for the replayed (host-buffer) mode: a superposition of Poisson
    processes has a Poisson total count, sources drawn in proportion to their rate, times uniform."""
    lam = rates_hz.sum() * n_steps * dt * 1e-3
    n = rng.poisson(lam)
    src = rng.choice(len(rates_hz), size=n, p=rates_hz / rates_hz.sum()).astype(np.uint32)
    stamp = (step0 + 1 + rng.integers(0, n_steps, size=n)).astype(np.uint32)
    return src, stamp


def run_cpu(net, slice_ms, threads, n_slices=1):
    """Oracle (OpenMP port of the engine contract) prepared for `n_slices` runs of `slice_ms`."""
    from oracle import glif_oracle as O
    O.build()
    n_steps = int(round(slice_ms / net.dt))
    t0 = time.time()
    sim = O.OracleSim(net.types, net.type_index, net.dt, n_virtual=net.n_virtual, src=net.src, trg=net.trg,
                      weight=net.weight, delay_steps=net.delay_steps, port=net.port, n_threads=threads,
                      canonical_csr=False)
    steps, srcs = O.poisson_spikes(net.poisson_rate_hz, net.dt, net.poisson_seed, 0, n_steps * n_slices)
    sim.set_input_spikes(steps, srcs)
    t_setup = time.time() - t0
    return sim, n_steps, t_setup


def parity_check(full_net, st, ids, n_steps, threads, stream=0):
    """Checker, outside every timed region: the fp64 oracle runs the same network from rest on the same
    Philox input for `n_steps`, and the engine's recorded spikes of those steps are compared with it:
    first differing step, every spike of the first 25 ms within one step, share of the first 100 ms's
    spikes in trains that differ by more, per-type firing rates over the whole span."""
    from oracle import compare as K
    from oracle import glif_oracle as O
    O.build()
    t0 = time.time()
    sim = O.OracleSim(full_net.types, full_net.type_index, full_net.dt, n_virtual=full_net.n_virtual, src=full_net.src,
                      trg=full_net.trg, weight=full_net.weight, delay_steps=full_net.delay_steps, port=full_net.port,
                      n_threads=threads, canonical_csr=False)
    steps, srcs = O.poisson_spikes(full_net.poisson_rate_hz, full_net.dt, full_net.poisson_seed, 0, n_steps, stream=stream)
    sim.set_input_spikes(steps, srcs)
    t_setup = time.time() - t0
    r = sim.run(n_steps, spike_cap=max(1 << 20, full_net.n_neurons * 16))
    t_run = time.time() - t0 - t_setup
    ost, oid = r['spike_step'], r['spike_id'].astype(np.int64)
    st, ids = np.asarray(st, dtype=np.int64), np.asarray(ids, dtype=np.int64)
    o = np.lexsort((ids, st))
    st, ids = st[o], ids[o]
    s25, s100 = int(round(25.0 / full_net.dt)), int(round(100.0 / full_net.dt))
    strict = K.within_one_step(st, ids, ost, oid, s25, full_net.n_neurons)
    wide = K.within_one_step(st, ids, ost, oid, s100, full_net.n_neurons)
    ra = K.rate_agreement(full_net.type_index, len(full_net.types), ids, oid, n_steps * full_net.dt)
    return {
        'against': 'fp64 CPU oracle (%d threads), same network and Philox input, from rest, %g ms' % (threads, n_steps * full_net.dt),
        'spikes_gpu': int(len(st)), 'spikes_oracle': int(len(ost)),
        'first_divergence_step': K.first_divergence(st, ids, ost, oid),
        'first_25ms_within_one_step': strict['ok'], 'first_25ms_spikes': strict['n_b'],
        'first_100ms': {'spikes': wide['n_b'], 'neurons_with_other_count': wide['neurons_with_other_count'],
                        'spikes_beyond_one_step': wide['spikes_beyond_one_step'],
                        'share_beyond': (wide['neurons_with_other_count'] + wide['spikes_beyond_one_step']) / max(1, wide['n_b'])},
        'max_type_rate_rel_err': ra['max_rel_err'], 'rates_within_2pct': ra['within_rel_only'],
        'ok': bool(strict['ok'] and ra['within_rel_only']),
        'oracle_wall_s': {'setup': t_setup, 'run': t_run, 'compare': time.time() - t0 - t_setup - t_run},
    }


def gather_spikes(st, ids, world, rank, dist):
    """All ranks' recorded spikes on rank 0 (None elsewhere)."""
    if world == 1:
        return st, ids
    parts = [None] * world
    dist.all_gather_object(parts, (np.asarray(st), np.asarray(ids)))
    if rank != 0:
        return None, None
    return np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts])


def reference_arm(args):
    """Times the CPU implementation of the path on the host cores. The reference's own engine is
    NEST (third-party C++, not in the reference tree, not installed), so this is the repo's fp64
    oracle port with all host threads; each step is a bounded slice of the same workload."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    net = make_network(args.scale)
    slice_ms = 100.0
    sim, n_steps, _ = run_cpu(net, slice_ms, threads, args.warmup + args.steps)
    for _ in range(args.warmup):
        sim.run(n_steps, record_spikes=False)
    ev = 0
    t0 = time.time()
    for _ in range(args.steps):
        ev += sim.run(n_steps, record_spikes=False)['n_events']
    wall = time.time() - t0
    val = ev / wall
    line = {
        'impl': 'reference', 'metric': 'synaptic_events_per_sec', 'value': val, 'unit': 'events/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': 1e3 * wall / args.steps,
        'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f64', 'data': 'synthetic',
        'sim_ms_per_wall_ms': slice_ms * args.steps / (wall * 1e3),
        'config': {'workload': 'c3: %d GLIF-3 neurons, %d synapses, %d Poisson cells, dt 0.25 ms'
                               % (net.n_neurons, net.n_edges, net.n_virtual),
                   'step': '%g ms of simulated time per step (bounded slice of the 1000 ms bench step)' % slice_ms},
        'cpu_baseline': {'value': val, 'unit': 'events/s', 'cores': threads, 'kind': 'port',
                         'sample': '%d consecutive %g ms slices after %d warm-up slices, fp64 oracle, OpenMP'
                                   % (args.steps, slice_ms, args.warmup)},
        'e2e': {'value': val, 'unit': 'events/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


def main():
    args = parse_args()
    STEP_MS = args.step_ms
    if args.impl == 'reference':
        return reference_arm(args)
    # Only the JSON line may reach stdout: libraries (NCCL prints its version there) write to fd 1,
    # so fd 1 is pointed at stderr for the duration and the line goes to the saved descriptor.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist
    from bmtk_b200 import workloads as W
    from bmtk_b200.engine import nccl_unique_id

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: bmtk_b200 has no CPU path')
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    libnccl = None
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=dev)
        libnccl = os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), 'nvidia', 'nccl', 'lib', 'libnccl.so.2')
        if not os.path.exists(libnccl):
            libnccl = None

    def fresh_uid():
        """A new ncclUniqueId for every engine (an id serves one communicator), made on rank 0."""
        if world == 1:
            return None
        buf = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            buf.copy_(torch.frombuffer(bytearray(nccl_unique_id(libnccl)), dtype=torch.uint8))
        dist.broadcast(buf, 0)
        return bytes(buf.cpu().numpy().tobytes())

    def barrier():
        if world > 1:
            dist.barrier()

    def reduce(x, op):
        if world == 1:
            return x
        t = torch.tensor([float(x)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return float(t.item())

    if args.workload == 'c4':
        trial_sweep(args, torch, dist, W, world, rank, local_rank, dev, barrier, reduce, json_fd)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload in ('c0', 'c1', 'c2'):
        small_config(args, torch, dist, W, world, rank, local_rank, dev, barrier, reduce, json_fd, fresh_uid, libnccl)
        if world > 1:
            dist.destroy_process_group()
        return
    n_total = int(round(230924 * args.scale))
    bounds = np.linspace(0, n_total, world + 1).astype(np.int64)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    t0 = time.time()
    net = make_network(args.scale, (lo, hi))
    t_gen = time.time() - t0
    steps_per_bench_step = int(round(STEP_MS / net.dt))

    # ---------------- device-resident run
    t0 = time.time()
    eng = W.build_engine(net, device=local_rank, record_spikes=True, record_vm=False,
                         options=dict(chunk_steps=steps_per_bench_step, **extra_options(args)), rank=rank, n_ranks=world, nccl_uid=fresh_uid(),
                         libnccl=libnccl, p2p=args.exchange == 'p2p')
    t_build = time.time() - t0
    n_warm = 0
    first_spikes = None
    for _ in range(args.warmup):
        eng.run(steps_per_bench_step)
        sp = eng.fetch_spikes()
        if first_spikes is None:
            first_spikes = (sp[0].copy(), sp[1].copy())     # the first step starts from rest: what the parity check compares
        n_warm = max(n_warm, len(sp[0]))
    # the timed launches leave their spikes in the host store: pin it before the clock starts
    eng.set_option('spike_store_reserve', int(n_warm * 1.25 + 1e5) * args.steps)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    torch.cuda.synchronize()
    barrier()
    if sampler:
        sampler.begin()
    ev0, sp0, l0 = eng.counter('events'), eng.counter('spikes'), eng.counter('launches')
    eng.mark(0)
    w0 = time.time()
    for _ in range(args.steps):
        eng.run(steps_per_bench_step)
    eng.mark(1)
    dev_ms = eng.elapsed_ms(0, 1)
    torch.cuda.synchronize()
    wall_ms = (time.time() - w0) * 1e3
    barrier()
    clocks = sampler.stop() if sampler else None
    eng.fetch_spikes()
    dev_ms = reduce(dev_ms, dist.ReduceOp.MAX if world > 1 else None)
    wall_ms = reduce(wall_ms, dist.ReduceOp.MAX if world > 1 else None)
    local_events = eng.counter('events') - ev0
    events = reduce(local_events, dist.ReduceOp.SUM if world > 1 else None)
    spikes = reduce(eng.counter('spikes') - sp0, dist.ReduceOp.SUM if world > 1 else None)
    launches = reduce(eng.counter('launches') - l0, dist.ReduceOp.SUM if world > 1 else None)
    value = events / (dev_ms * 1e-3)

    # ---------------- phase timers of the persistent kernel (device %globaltimer, thread 0)
    phases = None
    if eng.counter('persistent_blocks') > 0 and (world == 1 or args.exchange == 'p2p'):
        eng.set_option('phase_timers', 1)
        e0 = eng.counter('events')
        eng.run(steps_per_bench_step)
        eng.set_option('phase_timers', 0)
        eng.fetch_spikes()
        nw = max(1, eng.counter('phase_windows'))
        pu, pp = eng.counter('phase_update_ns') / nw, eng.counter('phase_propagate_ns') / nw
        ev_w = (eng.counter('events') - e0) / nw
        win = eng.counter('window')
        pipelined = bool(eng.counter('pipelined'))
        steps_w = steps_per_bench_step / nw          # steps between two grid barriers
        s1, s2 = eng.counter('phase_sync1_ns') / nw, eng.counter('phase_sync2_ns') / nw
        phases = {
            'kernel': 'pipelined (update and delivery warps side by side, per-side hand-over each phase)' if pipelined
                      else 'two-phase (update, barrier, delivery, barrier per window)',
            'timing': 'in-kernel %globaltimer, block 0, summed in registers over one cooperative launch (= one bench step)',
            'windows': nw, 'steps_per_window': steps_w,
            'update_phase_us': pu * 1e-3, 'propagate_phase_us': pp * 1e-3,
            'of_which_barrier_wait_us': [s1 * 1e-3, s2 * 1e-3],
            'update_gbs': BYTES_PER_NEURON_STEP * eng.counter('n_pad') * steps_w / (pu - s1 if pipelined else pu),
            'propagate_gbs': BYTES_PER_EVENT * ev_w / (pp - s2 if pipelined else pp), 'events_per_window': ev_w,
            'resident_state': bool(eng.counter('persistent_resident')), 'pipelined': pipelined,
        }
        if pipelined:
            phases['phase_us'] = pu * 1e-3           # both sides span the whole phase
            phases['row_streaming_us'] = eng.counter('phase_rows_ns') / nw * 1e-3
            if world > 1:
                # of the row streaming time of block 0's first chunk warp: waiting for the other ranks' count words of
                # the phase, then fetching their spikes and streaming those rows (the rest is this rank's own chunks)
                phases['remote_count_wait_us'] = eng.counter('phase_remote_wait_ns') / nw * 1e-3
                phases['remote_rows_us'] = eng.counter('phase_remote_rows_ns') / nw * 1e-3
                phases['local_rows_us'] = phases['row_streaming_us'] - phases['remote_count_wait_us'] - phases['remote_rows_us']

    # ---------------- delivery against the device's rate of scattered fp32 reductions into a buffer of the ring's size
    if phases is not None and rank == 0:
        from bmtk_b200.engine import scatter_reduction_rate
        cells = eng.csr_info()['ring_slots'] * 4 * eng.counter('n_pad')
        ceiling = scatter_reduction_rate(cells, 8 * 1024 * 1024, device=local_rank)
        busy_ns = (eng.counter('phase_rows_ns') / max(1, eng.counter('phase_windows'))) or 1.0
        phases['scatter_red_ceiling_per_s'] = ceiling
        phases['delivery_events_per_s_while_streaming'] = phases['events_per_window'] / (busy_ns * 1e-9)
        phases['delivery_frac_of_scatter_ceiling'] = phases['delivery_events_per_s_while_streaming'] / ceiling
        phases['delivery_note'] = ('one fp32 reduction per synaptic event into a random ring cell: the ceiling is what the device '
                                   'sustains for such reductions alone (bmtk_probe_scatter_reductions); delivery runs beside the '
                                   'update warps and is latency-bound per chunk, not throughput-bound')

    # ---------------- latency of the exchange primitive between ranks 0 and 1 (what a phase cannot go below)
    if world > 1 and args.exchange == 'p2p' and phases is not None:
        barrier()
        if rank < 2:
            lat = eng.p2p_pingpong(1 - rank, rank == 0, 2000)
            if rank == 0:
                phases['peer_word_one_way_us'] = lat * 1e-3
        barrier()

    # ---------------- profiled pass: per-launch CUDA events around both kernels
    prof_steps = min(steps_per_bench_step, 800)
    eng.set_option('profile', 1)
    e0 = eng.counter('events')
    eng.run(prof_steps)
    eng.set_option('profile', 0)
    eng.fetch_spikes()
    up_ns, up_n = eng.counter('update_ns'), max(1, eng.counter('update_launches'))
    pr_ns, pr_n = eng.counter('propagate_ns'), max(1, eng.counter('propagate_launches'))
    prof_events = eng.counter('events') - e0
    n_pad = eng.counter('n_pad')
    peak, peak_kind = peaks()
    up_bytes = BYTES_PER_NEURON_STEP * n_pad
    pr_bytes = BYTES_PER_EVENT * prof_events / pr_n
    kernels = {
        'glif_update': {'launches': up_n, 'avg_us': up_ns / up_n * 1e-3, 'bytes_per_launch': up_bytes,
                        'achieved_gbs': up_bytes / (up_ns / up_n), 'traffic': 102.8 * n_pad},
        'propagate': {'launches': pr_n, 'avg_us': pr_ns / pr_n * 1e-3, 'bytes_per_launch': pr_bytes,
                      'achieved_gbs': pr_bytes / (pr_ns / pr_n), 'traffic': NCU_TRAFFIC_BYTES['propagate']},
    }
    if phases:
        # The timed region is ONE cooperative launch per bench step: that launch is the dominant kernel.
        # Algorithmic bytes of this rank's launch over its CUDA-event duration (engine marks on the stream).
        alg_bytes = BYTES_PER_NEURON_STEP * n_pad * steps_per_bench_step + BYTES_PER_EVENT * local_events / args.steps
        launch_ns = dev_ms / args.steps * 1e6
        roofline = {
            'kernel': 'pipelined_kernel' if phases['pipelined'] else 'persistent_kernel', 'bound': 'hbm',
            'achieved': alg_bytes / launch_ns, 'peak': peak, 'unit': 'GB/s', 'frac': alg_bytes / launch_ns / peak,
            'traffic': NCU_TRAFFIC_BYTES['pipelined_per_step' if phases['pipelined'] else 'persistent_per_step'] * steps_per_bench_step,
            'peak_kind': peak_kind,
            'traffic_note': 'dram bytes of one cooperative launch (= one bench step), ncu on a 100-step launch scaled by steps',
            'timing': 'CUDA events on the launching stream around the %d timed launches (one per bench step)' % args.steps,
            'bytes_per_launch': alg_bytes,
            'note': 'algorithmic bytes = 128 B per neuron-step + 16 B per synaptic event; the kernel keeps the 96 B of '
                    'neuron state in registers, so what actually moves per neuron-step is the 32 B of ring traffic: the '
                    'launch is bound by L2 / barrier latency per step, not by HBM',
            'persistent_phases': phases,
            'per_step_kernels': dict(kernels, timing='CUDA events around every launch of the per-step kernels '
                                                     '(engine option profile; the path used without cooperative launch)'),
        }
    else:
        dom = 'glif_update' if up_ns >= pr_ns else 'propagate'
        roofline = {'kernel': dom, 'bound': 'hbm', 'achieved': kernels[dom]['achieved_gbs'], 'peak': peak, 'unit': 'GB/s',
                    'frac': kernels[dom]['achieved_gbs'] / peak, 'traffic': kernels[dom]['traffic'], 'peak_kind': peak_kind,
                    'timing': 'CUDA events around every launch of the per-step kernels (engine option profile)',
                    'kernels': kernels}
    window = eng.counter('window')
    eng.close()

    # ---------------- end to end with host buffers (replayed virtual spikes)
    e2e = None
    if not args.no_e2e:
        net.poisson_rate_hz, rates = None, net.poisson_rate_hz.astype(np.float64)
        eng = W.build_engine(net, device=local_rank, record_spikes=True, record_vm=False,
                             options=dict(chunk_steps=steps_per_bench_step, **extra_options(args)), rank=rank, n_ranks=world, nccl_uid=fresh_uid(),
                             libnccl=libnccl, p2p=args.exchange == 'p2p')
        rng = np.random.default_rng(99)   # same seed on every rank: virtual cells are replicated
        n_chunks = 1 + args.steps
        cap = int(rates.sum() * STEP_MS * 1e-3 * 1.2) + 4096
        pin_src = torch.empty((n_chunks, cap), dtype=torch.int32).pin_memory()
        pin_stamp = torch.empty((n_chunks, cap), dtype=torch.int32).pin_memory()
        counts = []
        for c in range(n_chunks):
            s, st = poisson_chunk(rng, rates, net.dt, c * steps_per_bench_step, steps_per_bench_step)
            k = min(len(s), cap)
            pin_src[c, :k] = torch.from_numpy(s[:k].astype(np.int32))
            pin_stamp[c, :k] = torch.from_numpy(st[:k].astype(np.int32))
            counts.append(k)
        h2d = d2h = 0
        ev_start = 0
        for c in range(n_chunks):
            if c == 1:
                torch.cuda.synchronize()
                barrier()
                ev_start = eng.counter('events')
                t_start = time.time()
            k = counts[c]
            eng.set_input_spikes(pin_src[c, :k].numpy().view(np.uint32), pin_stamp[c, :k].numpy().view(np.uint32))
            eng.run(steps_per_bench_step)
            st, ids = eng.fetch_spikes()
            if c >= 1:
                h2d += 8 * k
                d2h += 8 * len(st)
        torch.cuda.synchronize()
        barrier()
        e2e_wall = reduce(time.time() - t_start, dist.ReduceOp.MAX if world > 1 else None)
        e2e_events = reduce(eng.counter('events') - ev_start, dist.ReduceOp.SUM if world > 1 else None)
        e2e = {'value': e2e_events / e2e_wall, 'unit': 'events/s',
               'h2d_bytes_per_step': int(reduce(h2d, dist.ReduceOp.SUM if world > 1 else None) / args.steps),
               'd2h_bytes_per_step': int(reduce(d2h, dist.ReduceOp.SUM if world > 1 else None) / args.steps),
               'sim_ms_per_wall_ms': STEP_MS * args.steps / (e2e_wall * 1e3),
               'timing': 'wall clock between barriers, includes host-side packing and sorting of spikes'}
        eng.close()
        net.poisson_rate_hz = rates.astype(np.float32)

    # ---------------- parity of the first bench step (from rest) with the oracle, every N, rank 0
    parity = None
    if not args.no_cpu and first_spikes is not None:
        g_st, g_ids = gather_spikes(first_spikes[0], first_spikes[1], world, rank, dist)
        if rank == 0:
            full = net if world == 1 else make_network(args.scale)
            parity = parity_check(full, g_st, g_ids, steps_per_bench_step, len(os.sched_getaffinity(0)) or 1)
            del full

    # ---------------- CPU baseline (rank 0, N = 1 only)
    cpu = None
    if world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        sim, n_steps, t_setup = run_cpu(net, args.cpu_slice_ms, threads, 2)
        sim.run(n_steps, record_spikes=False)      # untimed: lets the onset transient pass
        t0 = time.time()
        r = sim.run(n_steps, record_spikes=False)
        t_cpu = time.time() - t0
        cpu = {'value': r['n_events'] / t_cpu, 'unit': 'events/s', 'cores': threads, 'kind': 'port',
               'sim_ms_per_wall_ms': args.cpu_slice_ms / (t_cpu * 1e3),
               'sample': '%g ms of the same network after a %g ms untimed lead-in from rest (%d events, %d spikes, %.1f s), fp64 oracle, OpenMP'
                         % (args.cpu_slice_ms, args.cpu_slice_ms, r['n_events'], r['n_spikes'], t_cpu)}

    if rank == 0:
        line = {
            'metric': 'synaptic_events_per_sec', 'value': value, 'unit': 'events/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dev_ms / args.steps,
            'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
            'sim_ms_per_wall_ms': STEP_MS * args.steps / dev_ms,
            'config': {'workload': 'c3: %d GLIF-3 neurons in 17 types, %d synapses%s, %d Poisson cells, dt 0.25 ms'
                                   % (n_total, int(reduce_edges(net, world, dist, dev)), '' if world == 1 else ' (all ranks)',
                                      net.n_virtual),
                       'step': '%g ms of simulated time = %d update steps' % (STEP_MS, steps_per_bench_step),
                       'partition': ('neurons in %d contiguous blocks, spike ids of every %d-step window exchanged %s'
                                     % (world, window, 'inside the stepping kernel over peer memory (NVLink)'
                                        if args.exchange == 'p2p' else 'with one NCCL all-gather'))
                       if world > 1 else 'single GPU',
                       'l2': 'state + ring (~80 MB) are re-read every step; the 560 MB CSR exceeds L2',
                       'mean_rate_hz': spikes / n_total / (STEP_MS * 1e-3 * args.steps)},
            'clocks': clocks, 'e2e': e2e, 'gpu_launches': int(launches), 'roofline': roofline, 'cpu_baseline': cpu,
            'parity': parity, 'wall_ms_per_step': wall_ms / args.steps, 'setup_s': {'generate': t_gen, 'build_engine': t_build},
        }
        os.write(json_fd, (json.dumps(line) + '\n').encode())
    else:
        reduce_edges(net, world, dist, dev)
    if world > 1:
        dist.destroy_process_group()


def trial_sweep(args, torch, dist, W, world, rank, local_rank, dev, barrier, reduce, json_fd):
    """Workload c4. Every rank holds the whole CSR and runs trials [rank*T/N, (rank+1)*T/N) of the sweep:
    independent replicas, no collective on the data path (strong scaling: the sweep is fixed)."""
    T = args.trials
    if T % world:
        raise SystemExit('--trials must be a multiple of the number of ranks')
    t_loc = T // world
    step_ms = 500.0 if args.step_ms == 1000.0 else args.step_ms
    n = int(round(50000 * args.scale))
    net = W.c4(n=n, in_degree=min(1000, n // 4), n_virtual=max(8, int(round(2000 * args.scale))), t_stop_ms=step_ms)
    n_steps = int(round(step_ms / net.dt))
    eng = W.build_engine(net, device=local_rank, record_spikes=True, record_vm=False,
                         options={**dict(trials=t_loc, trial_base=rank * t_loc, chunk_steps=1000), **extra_options(args)})
    MAX, SUM = (dist.ReduceOp.MAX, dist.ReduceOp.SUM) if world > 1 else (None, None)
    n_warm = 0
    first_trial = None
    for _ in range(args.warmup):
        eng.run(n_steps)
        sp = eng.fetch_spikes()
        if first_trial is None and rank == 0:
            n_pad1 = eng.counter('n_pad1')
            m = sp[1] < n_pad1                  # local trial 0 of rank 0 = Philox stream 0, from rest
            first_trial = (sp[0][m].copy(), sp[1][m].copy())
        n_warm = max(n_warm, len(sp[0]))
    eng.set_option('spike_store_reserve', int(n_warm * 1.25 + 1e5) * args.steps)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    torch.cuda.synchronize()
    barrier()
    if sampler:
        sampler.begin()
    ev0, sp0, l0 = eng.counter('events'), eng.counter('spikes'), eng.counter('launches')
    eng.mark(0)
    for _ in range(args.steps):
        eng.run(n_steps)
    eng.mark(1)
    dev_ms = eng.elapsed_ms(0, 1)
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop() if sampler else None
    eng.fetch_spikes()
    dev_ms = reduce(dev_ms, MAX)
    events = reduce(eng.counter('events') - ev0, SUM)
    spikes = reduce(eng.counter('spikes') - sp0, SUM)
    launches = reduce(eng.counter('launches') - l0, SUM)
    # end to end: the Poisson cells live on the device, so a step's host traffic is its spike list
    torch.cuda.synchronize()
    barrier()
    e0, d2h = eng.counter('events'), 0
    t0 = time.time()
    for _ in range(args.steps):
        eng.run(n_steps)
        st, ids = eng.fetch_spikes()
        d2h += 8 * len(st)
    torch.cuda.synchronize()
    barrier()
    wall = reduce(time.time() - t0, MAX)
    e2e_events = reduce(eng.counter('events') - e0, SUM)
    n_pad, window = eng.counter('n_pad'), eng.counter('window')
    per_launch = eng.counter('pipeline_trials') if eng.counter('pipelined') else 0
    eng.close()
    peak, peak_kind = peaks()
    alg_bytes = BYTES_PER_NEURON_STEP * n_pad * world * n_steps * args.steps + BYTES_PER_EVENT * events
    parity = None
    if rank == 0 and not args.no_cpu and first_trial is not None:
        parity = parity_check(net, first_trial[0], first_trial[1], n_steps, os.cpu_count() or 1, stream=0)
        parity['trial'] = 'trial 0 of %d (Philox stream 0)' % T
    if rank == 0:
        line = {
            'metric': 'synaptic_events_per_sec', 'value': events / (dev_ms * 1e-3), 'unit': 'events/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dev_ms / args.steps, 'higher_is_better': True,
            'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
            'sim_ms_per_wall_ms': step_ms * T * args.steps / dev_ms,
            'config': {'workload': 'c4: %d trials of the %d-neuron E/I network (%d synapses, one CSR per GPU), %d Poisson '
                                   'cells per trial on their own Philox streams, dt 0.1 ms' % (T, n, net.n_edges, net.n_virtual),
                       'step': '%g ms of simulated time in every trial = %d update steps' % (step_ms, n_steps),
                       'partition': '%d trials per GPU, no exchange between GPUs' % t_loc,
                       'l2': ('state + ring of %d trials exceed L2; a launch steps %d trials, whose ring slots fit'
                              % (t_loc, per_launch)) if per_launch else 'state + ring of %d trials exceed L2' % t_loc,
                       'kernel': 'pipelined, %d trials per launch' % per_launch if per_launch else 'two-phase persistent',
                       'window_steps': window,
                       'mean_rate_hz': spikes / (n * T) / (step_ms * 1e-3 * args.steps)},
            'clocks': clocks,
            'e2e': {'value': e2e_events / wall, 'unit': 'events/s', 'h2d_bytes_per_step': 0,
                    'd2h_bytes_per_step': int(reduce(d2h, SUM) / args.steps),
                    'timing': 'wall clock; inputs are device-generated Poisson cells, every step reads its spike list back'},
            'gpu_launches': int(launches),
            'roofline': {'kernel': 'pipelined_kernel' if per_launch else 'persistent_kernel (update + delivery)', 'bound': 'hbm',
                         'achieved': alg_bytes / world / (dev_ms * 1e6), 'peak': peak, 'unit': 'GB/s',
                         'frac': alg_bytes / world / (dev_ms * 1e6) / peak, 'traffic': None, 'peak_kind': peak_kind,
                         'note': 'algorithmic bytes per GPU = 128 B per neuron-step + 16 B per event, over the whole timed region'},
            'cpu_baseline': None, 'parity': parity,
        }
        os.write(json_fd, (json.dumps(line) + '\n').encode())
    else:
        reduce(d2h, SUM)


def small_config(args, torch, dist, W, world, rank, local_rank, dev, barrier, reduce, json_fd, fresh_uid, libnccl):
    """Workloads c0, c1, c2 at their configured size: one bench step = one whole run from rest (a fresh state
    is loaded from a checkpoint before every step, outside the timed region), so every step does the same
    work. CPU baseline = the oracle's full run of the same configuration."""
    import tempfile as _tf
    name = args.workload
    make = {'c0': lambda **kw: W.c0(poisson_online=True), 'c1': lambda **kw: W.c1(), 'c2': lambda **kw: W.c2(**kw)}[name]
    full = make()
    n_total = full.n_neurons
    if world > 1 and name != 'c2':
        raise SystemExit('%s runs on one GPU (its windows are too small to be worth an exchange); use c2, c3 or c4 with --gpus' % name)
    bounds = np.linspace(0, n_total, world + 1).astype(np.int64)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    net = full if world == 1 else make(lo=lo, hi=hi)
    n_steps = net.n_steps
    MAX, SUM = (dist.ReduceOp.MAX, dist.ReduceOp.SUM) if world > 1 else (None, None)
    eng = W.build_engine(net, device=local_rank, record_spikes=True, record_vm=False,
                         options=dict(chunk_steps=n_steps, **extra_options(args)), rank=rank, n_ranks=world,
                         nccl_uid=fresh_uid(), libnccl=libnccl, p2p=args.exchange == 'p2p')
    ck = os.path.join(_tf.mkdtemp(), 'rest_%d.ck' % rank)
    eng.save_state(ck)
    first = None
    for _ in range(max(1, args.warmup)):
        eng.load_state(ck)
        eng.run(n_steps)
        sp = eng.fetch_spikes()
        if first is None:
            first = (sp[0].copy(), sp[1].copy())
    eng.set_option('spike_store_reserve', int(len(first[0]) * 1.25 + 1e5))
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.begin()   # (the region of these legs includes the reload of the rest state before every step)
    dev_ms, wall_ms, events, spikes, launches, d2h = 0.0, 0.0, 0, 0, 0, 0
    for _ in range(args.steps):
        eng.load_state(ck)
        torch.cuda.synchronize()
        barrier()
        ev0, sp0, l0 = eng.counter('events'), eng.counter('spikes'), eng.counter('launches')
        eng.mark(0)
        t0 = time.time()
        eng.run(n_steps)
        eng.mark(1)
        dev_ms += reduce(eng.elapsed_ms(0, 1), MAX)
        st, _ids = eng.fetch_spikes()               # end to end: the run plus its spike list on the host
        wall_ms += reduce((time.time() - t0) * 1e3, MAX)
        d2h += 8 * len(st)
        events += eng.counter('events') - ev0
        spikes += eng.counter('spikes') - sp0
        launches += eng.counter('launches') - l0
    clocks = sampler.stop() if sampler else None
    events, spikes, launches = reduce(events, SUM), reduce(spikes, SUM), reduce(launches, SUM)
    n_pad, pipelined, window = eng.counter('n_pad'), bool(eng.counter('pipelined')), eng.counter('window')
    eng.close()
    os.unlink(ck)
    peak, peak_kind = peaks()
    g_st, g_ids = gather_spikes(first[0], first[1], world, rank, dist)
    if rank != 0:
        return
    neuron_steps = float(n_total) * n_steps * args.steps
    # c1 has no synapses: its unit of work is the neuron-step
    metric, unit, value = ('synaptic_events_per_sec', 'events/s', events / (dev_ms * 1e-3)) if name != 'c1' else \
                          ('neuron_steps_per_sec', 'neuron-steps/s', neuron_steps / (dev_ms * 1e-3))
    e2e_value = (events if name != 'c1' else neuron_steps) / (wall_ms * 1e-3)
    alg = BYTES_PER_NEURON_STEP * n_pad * world * n_steps * args.steps + BYTES_PER_EVENT * events
    cpu = parity = None
    if not args.no_cpu:
        from oracle import glif_oracle as O
        threads = os.cpu_count() or 1
        sim = O.OracleSim(full.types, full.type_index, full.dt, n_virtual=full.n_virtual, src=full.src, trg=full.trg,
                          weight=full.weight, delay_steps=full.delay_steps, port=full.port, n_threads=threads, canonical_csr=False)
        if full.poisson_rate_hz is not None:
            sim.set_input_spikes(*O.poisson_spikes(full.poisson_rate_hz, full.dt, full.poisson_seed, 0, n_steps))
        if len(full.clamp_step):
            sim.set_clamp_events(full.clamp_step, full.clamp_target, full.clamp_delta.astype(np.float64))
        t0 = time.time()
        r = sim.run(n_steps, spike_cap=max(1 << 20, n_total * 400))
        t_cpu = time.time() - t0
        cpu = {'value': (r['n_events'] if name != 'c1' else float(n_total) * n_steps) / t_cpu, 'unit': unit, 'cores': threads,
               'kind': 'port', 'sim_ms_per_wall_ms': n_steps * full.dt / (t_cpu * 1e3),
               'sample': 'the whole configured run (%g ms, %d spikes, %.2f s), fp64 oracle, OpenMP' % (n_steps * full.dt, r['n_spikes'], t_cpu)}
        from oracle import compare as K
        o = np.lexsort((np.asarray(g_ids, dtype=np.int64), np.asarray(g_st, dtype=np.int64)))
        gst, gid = np.asarray(g_st, dtype=np.int64)[o], np.asarray(g_ids, dtype=np.int64)[o]
        ost, oid = r['spike_step'], r['spike_id'].astype(np.int64)
        s100 = int(round((200.0 if name == 'c1' else 100.0) / full.dt))    # c1: the first 100 ms of the current step
        w1 = K.within_one_step(gst, gid, ost, oid, s100, n_total)
        strict = K.within_one_step(gst, gid, ost, oid, int(round(25.0 / full.dt)), n_total)
        ra = K.rate_agreement(full.type_index, len(full.types), gid, oid, n_steps * full.dt)
        parity = {'against': 'fp64 CPU oracle, whole run', 'spikes_gpu': int(len(gst)), 'spikes_oracle': int(len(ost)),
                  'first_divergence_step': K.first_divergence(gst, gid, ost, oid),
                  'first_25ms_within_one_step': strict['ok'], 'first_25ms_spikes': strict['n_b'],
                  'first_100ms': dict(w1, share_beyond=(w1['neurons_with_other_count'] + w1['spikes_beyond_one_step']) / max(1, w1['n_b'])),
                  'max_type_rate_rel_err': ra['max_rel_err'], 'rates_within_2pct': ra['within_rel_only'],
                  'ok': bool(strict['ok'] and ra['within_rel_only'])}
    line = {
        'metric': metric, 'value': value, 'unit': unit, 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': dev_ms / args.steps, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32',
        'data': 'synthetic', 'sim_ms_per_wall_ms': n_steps * full.dt * args.steps / dev_ms,
        'config': {'workload': '%s: %d neurons, %d synapses, %d virtual cells, dt %g ms' % (name, n_total, full.n_edges if world == 1 else -1, full.n_virtual, full.dt),
                   'step': 'the whole configured run from rest: %g ms = %d update steps' % (n_steps * full.dt, n_steps),
                   'partition': 'single GPU' if world == 1 else 'neurons in %d contiguous blocks, exchange inside the stepping kernel' % world,
                   'l2': 'the working set fits L2; every step starts from a reloaded state', 'window_steps': window,
                   'kernel': 'pipelined' if pipelined else 'two-phase persistent',
                   'mean_rate_hz': spikes / n_total / (n_steps * full.dt * 1e-3 * args.steps)},
        'clocks': clocks,
        'e2e': {'value': e2e_value, 'unit': unit, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': int(d2h / args.steps),
                'timing': 'wall clock around run + fetch_spikes; inputs are device-generated (Poisson cells / clamp table)'},
        'gpu_launches': int(launches),
        'roofline': {'kernel': 'pipelined_kernel' if pipelined else 'persistent_kernel', 'bound': 'hbm',
                     'achieved': alg / world / (dev_ms * 1e6), 'peak': peak, 'unit': 'GB/s', 'frac': alg / world / (dev_ms * 1e6) / peak,
                     'traffic': None, 'peak_kind': peak_kind,
                     'note': 'algorithmic bytes per GPU = 128 B per neuron-step + 16 B per event over the timed launches; at this '
                             'size the launch is bound by the per-phase hand-over, not by HBM'},
        'cpu_baseline': cpu, 'parity': parity,
    }
    os.write(json_fd, (json.dumps(line, default=lambda x: x.tolist() if hasattr(x, 'tolist') else str(x)) + '\n').encode())


def reduce_edges(net, world, dist, dev):
    if world == 1:
        return net.n_edges
    import torch
    t = torch.tensor([float(net.n_edges)], dtype=torch.float64, device=dev)
    dist.all_reduce(t)
    return t.item()


if __name__ == '__main__':
    main()
