"""Simulation modules: inputs and recorders with the preload / initialize / finalize protocol.

Counterparts of bmtk/simulator/pointnet/modules/{spikes_inputs,iclamp,record_spikes,
multimeter_reporter}.py. Where the reference creates a NEST device and later parses the device's
text output, these modules register the request with the simulator and read arrays back from the
engine.
"""
import os

import numpy as np
import pandas as pd

from . import reports
from .io_tools import io
from .spike_trains import SpikeTrains


class SimulatorMod(object):
    """bmtk/simulator/pointnet/modules/sim_module.py:23-79 (only preload, initialize and finalize
    are ever called by the simulator)."""

    def preload(self, sim):
        pass

    def initialize(self, sim):
        pass

    def step(self, sim, tstep):
        pass

    def block(self, sim, block_interval):
        pass

    def finalize(self, sim):
        pass


class SpikesInputsMod(SimulatorMod):
    """inputs of input_type "spikes" (modules/spikes_inputs.py:29-46)."""

    def __init__(self, name, input_type, module, input_file=None, node_set=None, spikes=None, **opts):
        self._name = name
        self._module = module
        self._input_file = input_file
        self._node_set = node_set
        self._spikes = spikes
        self._opts = opts

    def initialize(self, sim):
        st = self._spikes if self._spikes is not None else SpikeTrains.load(self._input_file, file_type=self._module)
        node_set = sim.net.get_node_set(self._node_set if self._node_set is not None else 'all')
        sim.net.add_spike_trains(st, node_set, sim.get_spike_generator_params())


class IClampMod(SimulatorMod):
    """Current clamp (modules/iclamp.py:7-54 + core/modules/iclamp.py:9-61): amp / delay / duration
    as scalars or equal-length lists, or a csv `file` of (timestamps, amps). Onsets <= dt are
    skipped with a warning; an "off" entry is added at delay + duration."""

    def __init__(self, input_type, node_set, amp=None, delay=None, duration=None, file=None, module='IClamp', **opts):
        self._node_set = node_set
        self._has_durations = True
        if file is not None:
            df = pd.read_csv(file, sep=opts.get('separator', ' '))
            tcol, acol = opts.get('timestamps_column', 'timestamps'), opts.get('amplitudes_column', 'amps')
            if len(df) < 2:
                io.log_exception('IClampMod: csv file must be row oriented and contain two or more values.')
            for c in (tcol, acol):
                if c not in df.columns:
                    io.log_exception('IClampMod: csv file missing column "{}".'.format(c))
            self.amps, self.delays, self.durations = df[acol].values, df[tcol].values, None
            self._has_durations = False
        else:
            if amp is None or delay is None or duration is None:
                io.log_exception('IClampMod: missing current-clamp parameter (amp, delay, duration).')
            as_list = lambda v: list(v) if isinstance(v, (list, tuple, np.ndarray)) else [v]  # noqa: E731
            self.amps, self.delays, self.durations = as_list(amp), as_list(delay), as_list(duration)
            if not len(self.amps) == len(self.delays) == len(self.durations):
                io.log_exception('IClampMod: current clamp parameters amp, delay, duration must be same length '
                                 'when using list.')

    def amplitude_table(self, dt):
        times, vals = [], []
        n = len(self.delays)
        for i in range(n):
            start = self.delays[i]
            if start <= dt:
                io.log_warning('IClamp Stimulus has onset ("delay") skipping values that occur before "dt"',
                               display_once=True)
                continue
            times.append(float(start))
            vals.append(float(self.amps[i]))
            if self._has_durations:
                stop = start + self.durations[i]
                if i + 1 == n or stop <= self.delays[i + 1]:
                    times.append(float(stop))
                    vals.append(0.0)
        return times, vals

    def initialize(self, sim):
        times, vals = self.amplitude_table(sim.dt)
        gids = sim.net.get_node_set(self._node_set).gids()
        sim.add_current_clamp(times, vals, gids)


class SpikesMod(SimulatorMod):
    """Spike recorder on every non-virtual cell -> spikes .h5 / .csv (modules/record_spikes.py:95-166)."""

    def __init__(self, tmp_dir='.', spikes_file_csv=None, spikes_file=None, spikes_file_nwb=None, spikes_sort_order=None,
                 cache_to_disk=True, compression='gzip', **opts):
        def path(f):
            if f is None:
                return None
            if os.path.isabs(f):
                return f
            return f if os.path.abspath(f).startswith(os.path.abspath(tmp_dir)) else os.path.join(tmp_dir, f)
        self._csv, self._h5, self._nwb = path(spikes_file_csv), path(spikes_file), path(spikes_file_nwb)
        self._sort = spikes_sort_order or 'none'
        self._compression = compression
        self.spike_trains = None

    def initialize(self, sim):
        sim.enable_spike_recording()

    def finalize(self, sim):
        stamps, gids = sim.recorded_spikes()       # gathered on rank 0 when there are several ranks
        if io.mpi_rank == 0:
            st = SpikeTrains()
            if len(gids):
                node_ids, pops = sim.net.gid_pool.get_node_ids(gids)
                # the decimal value of stamp x dt (NEST writes spike times as decimal text, which the reference reads
                # back: 215 x 0.1 is 21.5 there, not 21.500000000000004)
                t = np.round(stamps.astype(np.float64) * sim.dt, 6)
                for p in pd.unique(pops):
                    m = pops == p
                    st.add_spikes(node_ids[m], t[m], p)
            else:
                for p in sim.net.gid_pool.populations:
                    st.add_spikes(np.zeros(0, dtype=np.int64), np.zeros(0), p)
            self.spike_trains = st
            if self._csv is not None:
                st.to_csv(self._csv, sort_order=self._sort)
            if self._h5 is not None:
                st.to_sonata(self._h5, sort_order=self._sort, compression=self._compression)
            if self._nwb is not None:
                io.log_warning('spikes_file_nwb is not supported; {} was not written'.format(self._nwb))
        io.barrier()


class MultimeterMod(SimulatorMod):
    """Report of a node set (modules/multimeter_reporter.py:68-167): `variable_name` (V_m, I_syn, ASCurrents_sum,
    threshold, threshold_spike, threshold_voltage, I) every `interval` (default dt); sample k is the state at
    k*interval, k >= 1; one element per node."""

    def __init__(self, tmp_dir, file_name, variable_name, cells, tstart=None, tstop=None, interval=None, to_h5=True,
                 delete_dat=True, **opts):
        self._file = file_name if os.path.isabs(file_name) else os.path.join(tmp_dir, file_name)
        self._variables = variable_name if isinstance(variable_name, (list, tuple)) else [variable_name]
        self._node_set = cells
        self._tstart, self._tstop, self._interval = tstart, tstop, interval
        self._to_h5 = to_h5
        self._gids = None
        self._population = None

    def initialize(self, sim):
        from .._cabi import RECORDABLES
        for v in self._variables:
            if v not in RECORDABLES:
                io.log_exception('MultimeterMod: variable "{}" cannot be recorded (available: {})'.format(
                    v, ', '.join(sorted(RECORDABLES))))
        node_set = sim.net.get_node_set(self._node_set)
        self._gids = sorted(set(node_set.gids()))
        self._population = node_set.population_names()[0] if node_set.population_names() else None
        self._tstart = self._tstart or sim.tstart
        self._tstop = self._tstop or sim.tstop
        self._interval = self._interval or sim.dt
        steps = int(round(self._interval / sim.dt))
        if steps < 1 or abs(steps * sim.dt - self._interval) > 1e-9 * max(1.0, self._interval):
            io.log_exception('MultimeterMod: interval {} is not a multiple of dt {}'.format(self._interval, sim.dt))
        self._handle = sim.add_vm_recorder(self._gids, steps, self._variables)

    def finalize(self, sim):
        gids, by_var = sim.recorded_vm(self._handle)       # per variable [samples, n_gids], rank 0 has all columns
        # The reference creates ONE report named after the first variable and writes every listed variable's values
        # into the same block, one after the other (multimeter_reporter.py:130-157): what stays in the file are the
        # values of the LAST variable under the name of the first. Reproduced as it is.
        data = by_var[self._variables[-1]]
        if io.mpi_rank == 0 and self._to_h5:
            k0 = int(np.floor(self._tstart / self._interval + 1e-9))          # samples with t <= tstart are dropped
            k1 = int(np.floor(self._tstop / self._interval + 1e-9))
            data = data[k0:k1]
            node_ids, pops = sim.net.gid_pool.get_node_ids(gids) if len(gids) else (np.zeros(0, np.int64), np.zeros(0, object))
            out = {}
            for p in pd.unique(pops):
                m = pops == p
                out[p] = (node_ids[m], data[:, m])
            reports.write_membrane_report(self._file, out, self._tstart, self._tstart + data.shape[0] * self._interval,
                                          self._interval, variable=self._variables[0],
                                          units='mV' if self._variables[0] in ('V_m', 'threshold', 'threshold_spike', 'threshold_voltage') else 'pA')
        io.barrier()
