"""PointSimulator: runs a PointNetwork on the B200 engine.

Same surface as bmtk.simulator.pointnet.PointSimulator (bmtk/simulator/pointnet/pointsimulator.py:
39-284): from_config reads run / inputs / reports, instantiates the modules, builds nodes and
recurrent edges; run() initialises the modules (virtual cells, clamps, recorders), creates the
engine, simulates `tstop` and lets the modules write their files.
With several ranks (torchrun: RANK / WORLD_SIZE / LOCAL_RANK) every rank owns a contiguous block of
engine ids and the engines exchange the spike ids of every min-delay window, by default inside the
stepping kernel over peer memory (NVLink), with NCCL all-gathers in deterministic mode; spikes and
traces are merged on rank 0.
"""
import glob
import os

import numpy as np

from . import modules as mods
from .config import Config
from .io_tools import io
from .pointnetwork import BadDelay
from .sim_settings import inputs_from_config, reports_from_config


class PointSimulator(object):
    def __init__(self, graph, dt=0.001, overwrite=True, print_time=False, n_thread=1):
        self._graph = graph
        self._dt = float(dt)
        self._tstop = 0.0
        self._overwrite = overwrite
        self._print_time = print_time
        self._n_thread = n_thread
        self._output_dir = './output/'
        self._block_run = False
        self._block_size = -1
        self._mods = []
        self._sg_params = {'precise_times': True}
        self._record_spikes = False
        self._clamps = []            # (times, values, gids)
        self._vm_recorders = []      # (gids, interval_steps, variable names)
        self._engine = None
        self._engine_options = {}
        self._spikes = (np.zeros(0, dtype=np.int64), np.zeros(0, dtype=np.int64))
        self._traces = {}
        graph.dt = self._dt          # the resolution is known to the network from here on

    # ---- properties (pointsimulator.py:76-110)
    @property
    def tstart(self):
        return 0.0

    @property
    def dt(self):
        return self._dt

    @property
    def tstop(self):
        return self._tstop

    @tstop.setter
    def tstop(self, val):
        self._tstop = val

    def simulation_time(self, units='ms'):
        t = self.tstop - self.tstart
        return t if units.lower() == 'ms' else t / 1000.0

    @property
    def n_steps(self):
        return int(round((self.tstop - self.tstart) / self.dt))

    @property
    def net(self):
        return self._graph

    @property
    def gid_map(self):
        return self._graph.gid_pool

    @property
    def engine(self):
        return self._engine

    def set_spike_generator_params(self, **params):
        self._sg_params.update(params)

    def get_spike_generator_params(self):
        return self._sg_params

    def add_mod(self, mod):
        self._mods.append(mod)

    def set_engine_options(self, **options):
        """Options of the C ABI (deterministic, window, spike_capacity, use_graph, ...)."""
        self._engine_options.update(options)

    # ---- requests the modules make
    def enable_spike_recording(self):
        self._record_spikes = True

    def add_current_clamp(self, times, values, gids):
        self._clamps.append((list(times), list(values), np.asarray(list(gids), dtype=np.int64)))

    def add_vm_recorder(self, gids, interval_steps, variables=('V_m',)):
        self._vm_recorders.append((np.asarray(gids, dtype=np.int64), int(interval_steps), list(variables)))
        return len(self._vm_recorders) - 1

    def recorded_spikes(self):
        return self._spikes

    def recorded_vm(self, handle):
        return self._traces[handle]

    # ---- running
    def _clamp_events(self):
        """(step, target, delta) triples: an amplitude listed at time T acts from step round(T/dt)+1
        (the generator is connected with delay = dt, modules/iclamp.py:54)."""
        steps, targets, deltas = [], [], []
        for times, values, gids in self._clamps:
            prev = 0.0
            for t, v in sorted(zip(times, values), key=lambda tv: tv[0]):
                s = int(round(t / self._dt)) + 1
                steps.append(np.full(len(gids), s, dtype=np.uint64))
                targets.append(gids.astype(np.uint32))
                deltas.append(np.full(len(gids), v - prev, dtype=np.float32))
                prev = v
        if not steps:
            return None
        return np.concatenate(steps), np.concatenate(targets), np.concatenate(deltas)

    def _build_engine(self):
        import ctypes  # noqa: F401
        from ..engine import Engine, time_to_stamp
        from .._cabi import BadDelay as EngineBadDelay
        net = self._graph
        n = len(net.gid_pool)
        rank, world = io.mpi_rank, io.mpi_size
        if world > 1:
            # blocks balanced by in-degree; the network has expanded only this rank's incoming edges
            if net.target_block is None:
                io.log_exception('the network was built before the ranks were known: call PointNetwork.partition(rank, '
                                 'world) before build() or let build_recurrent_edges do it (RANK / WORLD_SIZE set)')
            lo, hi = net.target_block
        else:
            lo, hi = 0, n
        self._block = (lo, hi)
        device = int(os.environ.get('LOCAL_RANK', '0'))
        eng = Engine(self._dt, device=device)
        if not net.types:
            io.log_exception('the network has no point neurons to simulate')
        eng.set_nodes(net.types, net.type_index[lo:hi], n_global=n, lo=lo)
        eng.set_virtual(net.n_virtual)
        src, trg, w, d_ms, port = net.edge_arrays()
        d_steps = np.round(d_ms / self._dt).astype(np.int64)
        keep = (trg >= lo) & (trg < hi)
        try:
            eng.add_edges(src[keep], trg[keep], w[keep], d_steps[keep], port[keep])
        except EngineBadDelay as e:
            io.log_error(str(e))
            raise BadDelay(str(e))
        if net.input_spikes:
            v = np.concatenate([x[0] for x in net.input_spikes])
            t = np.concatenate([x[1] for x in net.input_spikes])
            eng.set_input_spikes(v, time_to_stamp(t, self._dt))
        ce = self._clamp_events()
        if ce is not None:
            m = (ce[1] >= lo) & (ce[1] < hi)
            eng.set_clamp_events(ce[0][m], ce[1][m], ce[2][m])
        eng.record_spikes(self._record_spikes)
        # one device recorder serves all membrane reports: union of cells at the finest interval
        self._probe_gids = np.zeros(0, dtype=np.int64)
        if self._vm_recorders:
            allg = np.unique(np.concatenate([g for g, _, _ in self._vm_recorders]))
            self._probe_interval = int(np.gcd.reduce([s for _, s, _ in self._vm_recorders]))
            self._probe_vars = []
            for _, _, names in self._vm_recorders:
                self._probe_vars.extend(v for v in names if v not in self._probe_vars)
            self._probe_gids = allg[(allg >= lo) & (allg < hi)]
            if len(self._probe_gids):
                eng.record_state(self._probe_gids, self._probe_interval, self._probe_vars)
        for k, v in self._engine_options.items():
            eng.set_option(k, v)
        if world > 1:
            import torch
            import torch.distributed as dist
            from ..engine import nccl_unique_id
            if not dist.is_initialized():
                dist.init_process_group('gloo')
            io.set_barrier(dist.barrier)
            lib = os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), 'nvidia', 'nccl', 'lib', 'libnccl.so.2')
            lib = lib if os.path.exists(lib) else None
            uid = [nccl_unique_id(lib) if rank == 0 else None]
            dist.broadcast_object_list(uid, 0)
            eng.comm_init(uid[0], rank, world, lib)
            eng.agree_layout()       # exchange window, spike capacity and buffer offsets: the same on every rank
        eng.finalize()
        if world > 1 and not self._engine_options.get('deterministic', 0) and self._engine_options.get('persistent', 1):
            eng.connect_peers()      # spike exchange inside the stepping kernel over peer memory
        self._engine = eng

    def _collect(self):
        eng = self._engine
        stamps, gids = (np.zeros(0, np.int64), np.zeros(0, np.int64))
        if self._record_spikes:
            s, g = eng.fetch_spikes()
            stamps, gids = s.astype(np.int64), g.astype(np.int64)
        n_vars = len(getattr(self, '_probe_vars', [])) or 1
        trace = eng.fetch_trace() if len(self._probe_gids) else np.zeros((0, n_vars, 0), dtype=np.float32)
        if trace.ndim == 2:
            trace = trace[:, None, :]           # [samples, variables, cells]
        probe = self._probe_gids
        if io.mpi_size > 1:
            import torch.distributed as dist
            parts = [None] * io.mpi_size
            dist.gather_object((stamps, gids, probe, trace), parts if io.mpi_rank == 0 else None, 0)
            if io.mpi_rank == 0:
                stamps = np.concatenate([p[0] for p in parts])
                gids = np.concatenate([p[1] for p in parts])
                o = np.lexsort((gids, stamps))
                stamps, gids = stamps[o], gids[o]
                have = [p for p in parts if len(p[2])]
                probe = np.concatenate([p[2] for p in have]) if have else probe
                trace = np.concatenate([p[3] for p in have], axis=2) if have else trace
        self._spikes = (stamps, gids)
        for h, (g, steps, names) in enumerate(self._vm_recorders):
            if len(probe) == 0:
                self._traces[h] = (g, {v: np.zeros((0, len(g))) for v in names})
                continue
            cols = np.searchsorted(probe, g)
            stride = steps // self._probe_interval
            sub = trace[stride - 1::stride]
            self._traces[h] = (g, {v: sub[:, self._probe_vars.index(v)][:, cols].astype(np.float64) for v in names})

    def run(self, tstop=None):
        """pointsimulator.py:144-174."""
        if tstop is None:
            tstop = self._tstop
        self._tstop = tstop
        for mod in self._mods:
            mod.initialize(self)
        io.barrier()
        self._build_engine()
        io.log_info('Starting Simulation')
        import time
        t0 = time.time()
        self._engine.run(self.n_steps)
        io.barrier()
        wall = time.time() - t0
        io.log_info('Simulation finished, finalizing results.')
        self._collect()
        for mod in self._mods:
            mod.finalize(self)
        self._write_metrics(wall)
        io.barrier()
        io.log_info('Done.')

    def _write_metrics(self, wall_s):
        """<output_dir>/metrics.json on rank 0: what ran and how fast (this rank's counters)."""
        import json
        eng = self._engine
        m = {
            'n_neurons': len(self._graph.gid_pool), 'n_virtual': self._graph.n_virtual, 'dt_ms': self._dt,
            'n_steps': self.n_steps, 'sim_ms': self.n_steps * self._dt, 'wall_s': wall_s,
            'sim_ms_per_wall_ms': self.n_steps * self._dt / max(wall_s * 1e3, 1e-9),
            'ranks': io.mpi_size, 'rank_block': list(self._block),
            'spikes': eng.counter('spikes'), 'synaptic_events': eng.counter('events'),
            'events_per_s': eng.counter('events') / max(wall_s, 1e-9), 'kernel_launches': eng.counter('launches'),
            'window_steps': eng.counter('window'), 'persistent_kernel': bool(eng.counter('persistent_blocks')) and
            io.mpi_size == 1 and not self._engine_options.get('deterministic', 0),
        }
        self.metrics = m
        if io.mpi_rank == 0 and os.path.isdir(self._output_dir):
            with open(os.path.join(self._output_dir, 'metrics.json'), 'w') as f:
                json.dump(m, f, indent=1)

    @classmethod
    def from_config(cls, configure, graph, n_thread=None):
        """pointsimulator.py:176-284."""
        if isinstance(configure, str):
            config = Config.from_json(configure, validate=True)
        elif isinstance(configure, dict):
            config = configure
        else:
            raise Exception('Could not convert {} (type "{}") to json.'.format(configure, type(configure)))
        if 'run' not in config:
            raise Exception('Json file is missing "run" entry. Unable to build PointNetwork.')
        run = config['run']
        n_thread = run.get('n_thread', n_thread if n_thread is not None else 1)
        overwrite = run.get('overwrite_output_dir', True)
        print_time = run.get('print_time', False)
        network = cls(graph, dt=run['dt'], overwrite=overwrite, print_time=print_time, n_thread=n_thread)
        out = config.get('output', {})
        if 'output_dir' in out:
            network._output_dir = out['output_dir']
        if run.get('block_run'):
            if 'block_size' not in run:
                raise Exception('"block_run" is set to True but "block_size" not found.')
            network._block_size = run['block_size']
        if 'duration' in run:
            network.tstop = run['duration']
        elif 'tstop' in run:
            network.tstop = run['tstop']
        if 'precise_times' in run:
            network.set_spike_generator_params(precise_times=run['precise_times'])
        if run.get('allow_offgrid_spikes', False):
            network.set_spike_generator_params(allow_offgrid_spikes=True)
        if isinstance(config.get('engine'), dict):
            network.set_engine_options(**config['engine'])
        graph.io.log_info('Setting up output directory')
        if 'output_dir' in out:
            if not os.path.exists(out['output_dir']):
                if io.mpi_rank == 0:
                    os.makedirs(out['output_dir'])
            elif overwrite and io.mpi_rank == 0:
                for f in glob.glob(os.path.join(out['output_dir'], '*.gdf')):
                    os.remove(f)
        for sim_input in inputs_from_config(config):
            if sim_input.input_type == 'spikes' and sim_input.module in ('nwb', 'csv', 'sonata', 'h5', 'hdf5'):
                network.add_mod(mods.SpikesInputsMod(name=sim_input.name, input_type=sim_input.input_type,
                                                     module=sim_input.module, **sim_input.params))
            elif sim_input.module == 'IClamp':
                network.add_mod(mods.IClampMod(input_type=sim_input.input_type, **sim_input.params))
            else:
                graph.io.log_warning('Unknown input type {}'.format(sim_input.input_type))
        for report in reports_from_config(config):
            if report.module == 'spikes_report':
                mod = mods.SpikesMod(**report.params)
            elif report.module in ('membrane_report', 'multimeter_report', 'multimeter'):
                mod = mods.MultimeterMod(**report.params)
            else:
                graph.io.log_exception('Unknown report type {}'.format(report.module))
            mod.preload(graph)
            network.add_mod(mod)
        graph.io.log_info('Building cells.')
        graph.build_nodes()
        graph.io.log_info('Building recurrent connections')
        graph.build_recurrent_edges()
        io.log_info('Network created.')
        return network
