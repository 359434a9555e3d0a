"""Writes a workloads.Network as a SONATA project (nodes/edges .h5, type tables, cell and synapse
JSON files, input spikes, config) so that the drop-in surface - or any other SONATA tool - can be
driven from files, the way examples/point_450glifs is laid out. Stands in for bmtk.builder on this
path: the on-disk layout follows what the builder writes (groups /nodes/<pop>, /edges/<pop> with
node_id / node_type_id / node_group_id / node_group_index, source_node_id / target_node_id with their
node_population attribute, edge_type_id, edge_group_id / edge_group_index and a property group "0";
builder/network_adaptors/dm_network.py:103-121,305-351) including the lookup indices
indices/{source_to_target, target_to_source}/{node_id_to_range, range_to_edge_id}
(builder/index_builders.py:50-96) that every builder-written edges file carries.

Everything is written with vectorised numpy through bmtk_b200.h5io (contiguous datasets), so the
V1-scale workload (70 M edges, about 3.2 GB of edge columns) is a matter of disk bandwidth."""
import json
import os

import numpy as np

from . import h5io
from .pointnet.spike_trains import SpikeTrains


def edge_index_tables(ids):
    """The two tables of a SONATA edge lookup index over the column `ids` (source_node_id or target_node_id), as
    builder/index_builders.py:50-96 builds them: runs of equal consecutive ids become rows (begin, end) of
    range_to_edge_id, ordered by id (runs of one id in file order); row i of node_id_to_range is the block of
    range_to_edge_id rows of node id i, (0, 0) for an id without edges, up to the largest id present.
    Returns (node_id_to_range uint64[max_id + 1, 2], range_to_edge_id uint64[runs, 2])."""
    ids = np.asarray(ids)
    total = len(ids)
    if total == 0:
        return np.zeros((0, 2), dtype=np.uint64), np.zeros((0, 2), dtype=np.uint64)
    cut = np.nonzero(np.diff(ids))[0] + 1
    beg = np.concatenate(([0], cut))
    end = np.concatenate((cut, [total]))
    run_id = ids[beg]
    order = np.argsort(run_id, kind='stable')      # pandas sort_values (quicksort) leaves ties in no defined order;
    r2e = np.stack([beg[order], end[order]], axis=1).astype(np.uint64)   # file order is the natural choice
    sorted_ids = run_id[order].astype(np.int64)
    cut2 = np.nonzero(np.diff(sorted_ids))[0] + 1
    b2 = np.concatenate(([0], cut2))
    e2 = np.concatenate((cut2, [len(sorted_ids)]))
    i2r = np.zeros((int(sorted_ids.max()) + 1, 2), dtype=np.uint64)
    i2r[sorted_ids[b2], 0] = b2
    i2r[sorted_ids[b2], 1] = e2
    return i2r, r2e


def write_edge_indices(pop_group, source_ids, target_ids):
    """Adds indices/source_to_target and indices/target_to_source to an /edges/<population> group."""
    for name, ids in (('source_to_target', source_ids), ('target_to_source', target_ids)):
        i2r, r2e = edge_index_tables(ids)
        g = pop_group.create_group('indices/' + name)
        g.create_dataset('node_id_to_range', data=i2r)
        g.create_dataset('range_to_edge_id', data=r2e)


def write_project(net, root, with_report=True, iclamp=None, tstop=None, extra_output=None):
    os.makedirs(os.path.join(root, 'network'), exist_ok=True)
    os.makedirs(os.path.join(root, 'components', 'cell_models'), exist_ok=True)
    os.makedirs(os.path.join(root, 'components', 'synaptic_models'), exist_ok=True)
    os.makedirs(os.path.join(root, 'inputs'), exist_ok=True)
    n = net.n_neurons
    rng = np.random.default_rng(7)
    # ---- nodes: SONATA node ids are a permutation-free 0..n-1 here but types are interleaved on disk so that the
    # façade's batching by node type (and its id map) is exercised
    disk_order = rng.permutation(n)                    # disk row -> engine-order neuron
    node_id = np.arange(n, dtype=np.uint64)            # node_id of disk row r
    type_of_row = net.type_index[disk_order]
    with h5io.File(os.path.join(root, 'network', 'v1_nodes.h5'), 'w') as h:
        h.attrs['magic'] = np.uint32(0x0A7A)
        h.attrs['version'] = np.array([0, 1], dtype=np.uint32)
        g = h.create_group('/nodes/v1')
        g.create_dataset('node_id', data=node_id)
        g.create_dataset('node_type_id', data=(100 + type_of_row).astype(np.uint64))
        g.create_dataset('node_group_id', data=np.zeros(n, dtype=np.uint32))
        g.create_dataset('node_group_index', data=np.arange(n, dtype=np.uint64))
        g.create_dataset('0/x', data=rng.normal(size=n))
    with open(os.path.join(root, 'network', 'v1_node_types.csv'), 'w') as f:
        f.write('node_type_id model_type model_template model_name ei dynamics_params\n')
        for t, p in enumerate(net.types):
            fn = 'type_%d_glif_lif_asc_psc.json' % t
            with open(os.path.join(root, 'components', 'cell_models', fn), 'w') as jf:
                json.dump({k: (list(v) if isinstance(v, tuple) else v) for k, v in p.items()}, jf)
            f.write('%d point_neuron nest:glif_psc %s %s %s\n' % (100 + t, net.type_names[t],
                                                                 'i' if net.type_is_inh[t] else 'e', fn))
    # engine-order neuron k lives at disk row inv[k] and has node_id inv[k]
    inv = np.empty(n, dtype=np.int64)
    inv[disk_order] = np.arange(n)
    # ---- virtual nodes
    nv = net.n_virtual
    with h5io.File(os.path.join(root, 'network', 'lgn_nodes.h5'), 'w') as h:
        g = h.create_group('/nodes/lgn')
        g.create_dataset('node_id', data=np.arange(nv, dtype=np.uint64))
        g.create_dataset('node_type_id', data=np.full(nv, 100, dtype=np.uint64))
        g.create_dataset('node_group_id', data=np.zeros(nv, dtype=np.uint32))
        g.create_dataset('node_group_index', data=np.arange(nv, dtype=np.uint64))
        h.create_group('/nodes/lgn/0')
    with open(os.path.join(root, 'network', 'lgn_node_types.csv'), 'w') as f:
        f.write('node_type_id model_type ei\n100 virtual e\n')
    # ---- edges: one edge type per port; weight = nsyns(1) * syn_weight column, delay column in ms
    for k in range(4):
        with open(os.path.join(root, 'components', 'synaptic_models', 'port%d.json' % (k + 1)), 'w') as jf:
            json.dump({'receptor_type': k + 1}, jf)

    def write_edges(fname, pop, src_pop, m, src_ids, types_fname):
        with h5io.File(os.path.join(root, 'network', fname), 'w') as h:
            g = h.create_group('/edges/' + pop)
            s = g.create_dataset('source_node_id', data=src_ids.astype(np.uint64))
            s.attrs['node_population'] = src_pop
            t = g.create_dataset('target_node_id', data=inv[net.trg[m]].astype(np.uint64))
            t.attrs['node_population'] = 'v1'
            g.create_dataset('edge_type_id', data=(100 + net.port[m]).astype(np.uint32))
            g.create_dataset('edge_group_id', data=np.zeros(int(m.sum()), dtype=np.uint16))
            g.create_dataset('edge_group_index', data=np.arange(int(m.sum()), dtype=np.uint32))
            g.create_dataset('0/syn_weight', data=net.weight[m].astype(np.float64))
            g.create_dataset('0/delay', data=net.delay_steps[m].astype(np.float64) * net.dt)
            g.create_dataset('0/nsyns', data=np.ones(int(m.sum()), dtype=np.uint32))
            write_edge_indices(g, src_ids, inv[net.trg[m]])
        with open(os.path.join(root, 'network', types_fname), 'w') as f:
            f.write('edge_type_id target_query source_query model_template dynamics_params\n')
            for k in range(4):
                f.write("%d * * static_synapse port%d.json\n" % (100 + k, k + 1))

    rec = net.src < n
    write_edges('v1_v1_edges.h5', 'v1_to_v1', 'v1', rec, inv[net.src[rec]], 'v1_v1_edge_types.csv')
    write_edges('lgn_v1_edges.h5', 'lgn_to_v1', 'lgn', ~rec, net.src[~rec].astype(np.int64) - n, 'lgn_v1_edge_types.csv')
    # ---- input spikes: times on the dt grid so that stamps are reproduced exactly
    st = SpikeTrains(population='lgn')
    st.add_spikes(net.in_virt, net.in_stamp.astype(np.float64) * net.dt, 'lgn')
    st.to_sonata(os.path.join(root, 'inputs', 'lgn_spikes.h5'), sort_order='by_id')
    # ---- configuration (split circuit / simulation files like the example)
    circuit = {
        'manifest': {'$BASE_DIR': '${configdir}', '$NETWORK_DIR': '$BASE_DIR/network', '$MODELS_DIR': '$BASE_DIR/components'},
        'components': {'point_neuron_models_dir': '$MODELS_DIR/cell_models', 'synaptic_models_dir': '$MODELS_DIR/synaptic_models'},
        'networks': {
            'nodes': [{'nodes_file': '$NETWORK_DIR/v1_nodes.h5', 'node_types_file': '$NETWORK_DIR/v1_node_types.csv'},
                      {'nodes_file': '$NETWORK_DIR/lgn_nodes.h5', 'node_types_file': '$NETWORK_DIR/lgn_node_types.csv'}],
            'edges': [{'edges_file': '$NETWORK_DIR/v1_v1_edges.h5', 'edge_types_file': '$NETWORK_DIR/v1_v1_edge_types.csv'},
                      {'edges_file': '$NETWORK_DIR/lgn_v1_edges.h5', 'edge_types_file': '$NETWORK_DIR/lgn_v1_edge_types.csv'}]}}
    sim = {
        'manifest': {'$BASE_DIR': '${configdir}', '$OUTPUT_DIR': '$BASE_DIR/output', '$INPUT_DIR': '$BASE_DIR/inputs'},
        'run': {'tstop': float(tstop if tstop is not None else net.n_steps * net.dt), 'dt': net.dt},
        'inputs': {'LGN_spikes': {'input_type': 'spikes', 'module': 'sonata', 'input_file': '$INPUT_DIR/lgn_spikes.h5',
                                  'node_set': 'lgn'}},
        'output': {'log_file': 'log.txt', 'output_dir': '$OUTPUT_DIR', 'spikes_file': 'spikes.h5',
                   'spikes_file_csv': 'spikes.csv', 'spikes_sort_order': 'time', 'overwrite_output_dir': True,
                   'log_to_console': False},
        'reports': {},
        'engine': {'deterministic': 1},
        'network': 'config.circuit.json',
    }
    if extra_output:
        sim['output'].update(extra_output)
    if with_report:
        sim['reports']['membrane_potential'] = {'module': 'multimeter_report', 'cells': {'population': 'v1', 'node_id':
                                                [int(inv[i]) for i in net.probe_ids]}, 'variable_name': 'V_m'}
    if iclamp:
        sim['inputs']['clamp'] = dict(input_type='current_clamp', module='IClamp', **iclamp)
    with open(os.path.join(root, 'config.circuit.json'), 'w') as f:
        json.dump(circuit, f, indent=1)
    with open(os.path.join(root, 'config.simulation.json'), 'w') as f:
        json.dump(sim, f, indent=1)
    return dict(config=os.path.join(root, 'config.simulation.json'), node_id_of_engine=inv, disk_order=disk_order)
