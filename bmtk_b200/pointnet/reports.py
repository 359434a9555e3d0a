"""Membrane (compartment) report files.

Layout of the reference's PopulationWriterv01 for point cells — one element per node
(bmtk/utils/reports/compartment/compartment_writer.py:162-229,261-275):
  /report/<population>/data  f64 [n_steps, n_nodes]  (@variable, @units)
  /report/<population>/mapping/{node_ids u64, element_ids u64 (=0), element_pos f64 (=0.0),
                                index_pointer u64 [n_nodes+1], time f64 [tstart, tstop, dt]}
"""
import os

import numpy as np

from .. import h5io


def write_membrane_report(path, populations, tstart, tstop, dt, variable='V_m', units='mV', compression=None):
    """populations: {name: (node_ids int[n], data float[n_steps, n])}."""
    d = os.path.dirname(path)
    if d and not os.path.exists(d):
        os.makedirs(d)
    with h5io.File(path, 'w') as h:
        h.attrs['magic'] = np.uint32(0x0A7A)
        h.attrs['version'] = np.array([0, 1], dtype=np.uint32)
        for pop, (node_ids, data) in populations.items():
            n = len(node_ids)
            g = h.create_group('/report/{}'.format(pop))
            ds = g.create_dataset('data', data=np.asarray(data, dtype=np.float64).reshape(-1, n), compression=compression)
            ds.attrs['variable'] = variable
            ds.attrs['units'] = units
            m = g.create_group('mapping')
            m.create_dataset('node_ids', data=np.asarray(node_ids, dtype=np.uint64))
            m.create_dataset('element_ids', data=np.zeros(n, dtype=np.uint64))
            m.create_dataset('element_pos', data=np.zeros(n, dtype=np.float64))
            m.create_dataset('index_pointer', data=np.arange(n + 1, dtype=np.uint64))
            m.create_dataset('time', data=np.array([tstart, tstop, dt], dtype=np.float64))


def read_membrane_report(path, population=None):
    """-> {population: dict(node_ids, data, time)}."""
    out = {}
    with h5io.File(path, 'r') as h:
        root = h['report']
        for pop in root.keys():
            if population and pop != population:
                continue
            g = root[pop]
            out[pop] = dict(node_ids=g['mapping/node_ids'][()], data=g['data'][()], time=g['mapping/time'][()],
                            variable=g['data'].attrs.get('variable'), units=g['data'].attrs.get('units'))
    return out
