"""Generates tests/golden/point_450glifs_network.npz and point_120cells_network.npz from the reference's
example networks.

    python tests/golden/make_point450_fixture.py /path/to/reference

Reads examples/point_450glifs (nodes/edges .h5, type tables, cell and synapse JSON, input spikes)
through bmtk_b200.pointnet and stores what the engine is built from: the per-type NEST parameter
dicts (five glif_psc types, two iaf_psc_alpha types), the engine type index, the expanded edge list
(source, target, weight = nsyns*syn_weight, delay ms, port) and the virtual-cell spike times. The
GPU parity test then runs this very network (the reference's own example) against the oracle
without needing the reference tree on the GPU box. examples/point_120cells (120 iaf_psc_delta cells
driven by 'thalamus' virtual cells) is stored the same way.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def one(ref, example, input_name, node_set, out_name):
    from bmtk_b200 import pointnet
    ex = os.path.join(ref, 'examples', example)
    cwd = os.getcwd()
    os.chdir(ex)
    try:
        conf = pointnet.Config.from_json('config.simulation.json')
        g = pointnet.PointNetwork.from_config(conf)
        g.dt = 0.1
        g.build()
        g.add_spike_trains(pointnet.SpikeTrains.load(conf.inputs[input_name]['input_file']), node_set)
    finally:
        os.chdir(cwd)
    src, trg, w, d, port = g.edge_arrays()
    node_ids, _ = g.gid_pool.get_node_ids(np.arange(len(g.gid_pool)))
    v = np.concatenate([x[0] for x in g.input_spikes])
    t = np.concatenate([x[1] for x in g.input_spikes])
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), out_name)
    np.savez_compressed(dst, types_json=np.array(json.dumps(g.types)), type_labels=np.array(json.dumps(g.type_labels)),
                        type_index=g.type_index, node_ids=node_ids, src=src, trg=trg, weight=w, delay_ms=d, port=port,
                        n_virtual=np.int64(g.n_virtual), in_virt=v.astype(np.uint32), in_time_ms=t)
    print('wrote', dst, os.path.getsize(dst), 'bytes;', len(src), 'edges,', len(v), 'input spikes')


def main(ref):
    one(ref, 'point_450glifs', 'LGN_spikes', 'lgn', 'point_450glifs_network.npz')
    one(ref, 'point_120cells', 'thalamus_spikes', 'thalamus', 'point_120cells_network.npz')


if __name__ == '__main__':
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get('BMTK_REFERENCE', '/root/reference'))
