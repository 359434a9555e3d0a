"""Spike trains: readers, writers and the Poisson generator used around the simulator.

On-disk formats are the reference's:
  * SONATA spikes .h5: /spikes/<population>/{timestamps f64 [@units], node_ids} with group attribute
    `sorting` in {none, by_id, by_time}, root attributes magic / version
    (bmtk/utils/reports/spike_trains/spikes_file_writers.py:35-73, utils/sonata/utils.py:103-108);
    the legacy layout /spikes/{gids,timestamps} is read too (spike_train_readers.py:368-391);
  * spikes .csv: header `timestamps population node_ids`, space separated
    (spikes_file_writers.py:115-126).
`PoissonSpikeGenerator` keeps the reference's construction: exponential inter-spike intervals
drawn from numpy's global RandomState, seconds -> ms (spike_trains.py:131-206).
"""
import os

import numpy as np
import pandas as pd

from .. import h5io

SORT_ORDERS = ('none', 'by_id', 'by_time', 'unknown')


def _norm_sort(order):
    if order is None:
        return 'none'
    o = getattr(order, 'value', order)
    o = str(o).lower()
    o = {'time': 'by_time', 'id': 'by_id', 'gid': 'by_id', 'node_id': 'by_id'}.get(o, o)
    if o not in SORT_ORDERS:
        raise ValueError('unknown sort order {}'.format(order))
    return o


class SpikeTrains(object):
    """In-memory spike store with the reading/writing calls the simulator modules use
    (bmtk/utils/reports/spike_trains/spike_trains.py:33-108)."""

    def __init__(self, population=None, units='ms', **kw):
        self._default_pop = population
        self._units = units
        self._ts = {}       # population -> list of arrays
        self._ids = {}

    # ---- filling
    def add_spike(self, node_id, timestamp, population=None, **kw):
        self.add_spikes([node_id], [timestamp], population)

    def add_spikes(self, node_ids, timestamps, population=None, **kw):
        pop = population or self._default_pop or 'unknown'
        ts = np.atleast_1d(np.asarray(timestamps, dtype=np.float64))
        ids = np.asarray(node_ids)
        ids = np.full(len(ts), int(ids), dtype=np.int64) if ids.ndim == 0 else ids.astype(np.int64)
        if len(ids) != len(ts):
            raise ValueError('node_ids and timestamps differ in length')
        self._ts.setdefault(pop, []).append(ts)
        self._ids.setdefault(pop, []).append(ids)

    def _flat(self, pop):
        if pop not in self._ts:
            return np.zeros(0), np.zeros(0, dtype=np.int64)
        if len(self._ts[pop]) > 1:
            self._ts[pop] = [np.concatenate(self._ts[pop])]
            self._ids[pop] = [np.concatenate(self._ids[pop])]
        return self._ts[pop][0], self._ids[pop][0]

    # ---- queries
    @property
    def populations(self):
        return list(self._ts.keys())

    def units(self, population=None):
        return self._units

    def n_spikes(self, population=None):
        pops = [population] if population else self.populations
        return int(sum(len(self._flat(p)[0]) for p in pops))

    def node_ids(self, population=None):
        pops = [population] if population else self.populations
        ids = [self._flat(p)[1] for p in pops]
        return np.unique(np.concatenate(ids)) if ids else np.zeros(0, dtype=np.int64)

    def get_times(self, node_id, population=None, time_window=None, **kw):
        pop = population or self._default_pop or (self.populations[0] if self.populations else None)
        ts, ids = self._flat(pop)
        out = ts[ids == node_id]
        if time_window is not None:
            out = out[(out >= time_window[0]) & (out <= time_window[1])]
        return out

    def to_dataframe(self, populations=None, sort_order='none', with_population_col=True, **kw):
        pops = [populations] if isinstance(populations, str) else (populations or self.populations)
        frames = []
        for p in pops:
            ts, ids = self._flat(p)
            d = {'timestamps': ts, 'population': np.full(len(ts), p, dtype=object), 'node_ids': ids}
            frames.append(pd.DataFrame(d))
        df = pd.concat(frames, ignore_index=True) if frames else \
            pd.DataFrame({'timestamps': np.zeros(0), 'population': np.zeros(0, dtype=object), 'node_ids': np.zeros(0, dtype=np.int64)})
        so = _norm_sort(sort_order)
        if so == 'by_time':
            df = df.sort_values(['timestamps', 'node_ids'], kind='stable')
        elif so == 'by_id':
            df = df.sort_values(['node_ids', 'timestamps'], kind='stable')
        if not with_population_col:
            df = df.drop(columns=['population'])
        return df.reset_index(drop=True)

    # ---- reading
    @classmethod
    def load(cls, path, file_type=None, population=None, **kw):
        ft = (file_type or '').lower()
        if ft in ('h5', 'sonata', 'hdf5') or (not ft and path.endswith(('.h5', '.hdf5', '.sonata'))):
            return cls.from_sonata(path, population=population, **kw)
        if ft == 'csv' or (not ft and path.endswith('.csv')):
            return cls.from_csv(path, population=population, **kw)
        if ft == 'nwb' or path.endswith('.nwb'):
            raise NotImplementedError('NWB spike files are not supported')
        raise ValueError('Unable to determine the type of spikes file {}'.format(path))

    @classmethod
    def from_sonata(cls, path, population=None, **kw):
        st = cls(population=population)
        with h5io.File(path, 'r') as h:
            root = h['spikes']
            keys = list(root.keys())
            if 'timestamps' in keys and ('gids' in keys or 'node_ids' in keys):      # legacy layout
                ids = root['gids' if 'gids' in keys else 'node_ids'][()]
                st.add_spikes(ids, root['timestamps'][()], population or 'unknown')
                return st
            for pop in keys:
                if population and pop != population:
                    continue
                g = root[pop]
                ts = g['timestamps']
                units = ts.attrs.get('units', 'ms') if hasattr(ts.attrs, 'get') else 'ms'
                t = np.asarray(ts[()], dtype=np.float64)
                if str(units) in ('s', 'seconds'):
                    t = t * 1000.0
                st.add_spikes(np.asarray(g['node_ids'][()]), t, pop)
        if st._default_pop is None and len(st.populations) == 1:
            st._default_pop = st.populations[0]
        return st

    @classmethod
    def from_csv(cls, path, population=None, sep=' ', **kw):
        df = pd.read_csv(path, sep=sep)
        st = cls(population=population)
        if 'population' in df.columns:
            for pop, g in df.groupby('population', sort=False):
                if population and pop != population:
                    continue
                st.add_spikes(g['node_ids'].values, g['timestamps'].values, pop)
        else:
            st.add_spikes(df['node_ids'].values, df['timestamps'].values, population or 'unknown')
        if st._default_pop is None and len(st.populations) == 1:
            st._default_pop = st.populations[0]
        return st

    # ---- writing
    def to_sonata(self, path, mode='w', sort_order='none', compression='gzip', **kw):
        write_sonata(path, self, mode=mode, sort_order=sort_order, compression=compression)

    def to_csv(self, path, mode='w', sort_order='none', **kw):
        write_csv(path, self, sort_order=sort_order)

    def flush(self):
        pass

    def close(self):
        pass


def write_sonata(path, spike_trains, mode='w', sort_order='none', units='ms', compression='gzip', **kw):
    if isinstance(compression, str) and compression.lower() == 'none':
        compression = None
    d = os.path.dirname(path)
    if d and not os.path.exists(d):
        os.makedirs(d)
    so = _norm_sort(sort_order)
    with h5io.File(path, 'w') as h:
        h.attrs['magic'] = np.uint32(0x0A7A)
        h.attrs['version'] = np.array([0, 1], dtype=np.uint32)
        root = h.create_group('/spikes')
        for pop in spike_trains.populations:
            df = spike_trains.to_dataframe(populations=pop, with_population_col=False, sort_order=so)
            g = root.create_group(pop)
            if so != 'unknown':
                g.attrs['sorting'] = so
            ts = g.create_dataset('timestamps', data=df['timestamps'].values.astype(np.float64), compression=compression)
            ts.attrs['units'] = spike_trains.units()
            g.create_dataset('node_ids', data=df['node_ids'].values.astype(np.int64), compression=compression)


def write_csv(path, spike_trains, sort_order='none', include_header=True, **kw):
    d = os.path.dirname(path)
    if d and not os.path.exists(d):
        os.makedirs(d)
    df = spike_trains.to_dataframe(sort_order=sort_order)
    # the reference's CSV buffer orders by population first and stores integer node ids
    df = df.sort_values('population', kind='stable') if _norm_sort(sort_order) == 'none' else df
    df[['timestamps', 'population', 'node_ids']].to_csv(path, header=include_header, index=False, sep=' ')


class PoissonSpikeGenerator(SpikeTrains):
    """Homogeneous (constant rate) or inhomogeneous (rate array + times) Poisson trains
    (bmtk/utils/reports/spike_trains/spike_trains.py:131-251). Rates in Hz, times in seconds,
    output in ms. Uses numpy's global RandomState like the reference; `seed` seeds it."""
    max_spikes_per_node = 10000000

    def __init__(self, population=None, seed=None, output_units='ms', **kw):
        super().__init__(population=population, units=output_units)
        if seed is not None:
            np.random.seed(seed)
        self._conv = 1000.0 if output_units.lower() in ('ms', 'millisecond', 'milliseconds') else 1.0

    def add(self, node_ids, firing_rate, population=None, times=(0.0, 1.0)):
        node_ids = [node_ids] if np.isscalar(node_ids) else list(node_ids)
        if np.isscalar(firing_rate):
            if firing_rate < 0:
                raise Exception('Firing rates must not be negative')
            tstart, tstop = (times[0], times[-1]) if not np.isscalar(times) else (0.0, times)
            if tstart >= tstop:
                raise ValueError('Poisson generator: times must be increasing')
            for nid in node_ids:
                c_time = tstart
                out = []
                while True:
                    if firing_rate <= 0:
                        break
                    interval = -np.log(1.0 - np.random.uniform()) / float(firing_rate)
                    c_time += interval
                    if c_time > tstop or len(out) >= self.max_spikes_per_node:
                        break
                    out.append(c_time * self._conv)
                self.add_spikes(nid, np.array(out), population)
        else:
            rates = np.asarray(firing_rate, dtype=float)
            t = np.asarray(times, dtype=float)
            if len(t) != len(rates):
                raise Exception('Poisson generator: firing_rate and times differ in length')
            if np.any(rates < 0):
                raise Exception('Firing rates must not be negative')
            rmax = rates.max()
            for nid in node_ids:
                c_time, out = t[0], []
                while rmax > 0:
                    c_time += -np.log(1.0 - np.random.uniform()) / rmax
                    if c_time > t[-1] or len(out) >= self.max_spikes_per_node:
                        break
                    if np.random.uniform() < np.interp(c_time, t, rates) / rmax:      # thinning
                        out.append(c_time * self._conv)
                self.add_spikes(nid, np.array(out), population)
