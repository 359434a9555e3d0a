"""Host side of the drop-in surface (no GPU): configuration, settings, SONATA loading, node
batching, edge expansion, id bookkeeping, virtual cells, clamps — against independent numpy
statements and, where the reference tree is mounted, against the reference's own pure-Python code."""
import importlib.util
import json
import os

import numpy as np
import pytest

from bmtk_b200 import pointnet, workloads as W
from bmtk_b200.pointnet import sim_settings
from bmtk_b200.pointnet.glif_utils import convert_aibs2nest
from bmtk_b200.pointnet.modules import IClampMod
from bmtk_b200.sonata_writer import write_project

REF = os.environ.get('BMTK_REFERENCE', '/root/reference')
needs_ref = pytest.mark.skipif(not os.path.isdir(REF), reason='reference tree not mounted')


def _ref_module(rel, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def _scrub(o):
    return json.loads(json.dumps(o, sort_keys=True, default=str))


@needs_ref
def test_config_parser_equals_reference_on_example_configs():
    import glob
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        ref = _ref_module('bmtk/utils/sonata/config/sonata_config.py', 'ref_sonata_config')
    n = 0
    for f in sorted(glob.glob(REF + '/examples/point_*/config*.json')):
        a = ref.SonataConfig.from_json(f)
        b = pointnet.Config.from_json(f)
        drop = ('time', 'date', 'datetime')
        assert _scrub({k: v for k, v in a.items() if k != 'manifest'}) == _scrub({k: v for k, v in b.items() if k != 'manifest'}), f
        assert _scrub({k: v for k, v in a['manifest'].items() if k not in drop}) == \
            _scrub({k: v for k, v in b['manifest'].items() if k not in drop}), f
        n += 1
    assert n >= 10


def test_config_variables_and_output_paths(tmp_path):
    """Cases of bmtk/tests/utils/sonata/test_config.py: chained manifest variables, ${VAR} inside a
    string, typed user variables, output-path prefixing, split network file, node_sets_file."""
    (tmp_path / 'ns.json').write_text(json.dumps({'sel': {'population': 'v1', 'ei': 'e'}}))
    (tmp_path / 'circuit.json').write_text(json.dumps({
        'manifest': {'$NET': '${configdir}/network'},
        'networks': {'nodes': [{'nodes_file': '$NET/n.h5', 'node_types_file': '$NET/n.csv'}]}}))
    cfg = {
        'manifest': {'$BASE': '${configdir}', '$OUT': '$BASE/out_${tag}', '$DEEP': '$OUT/deeper'},
        'run': {'tstop': '${tstop}', 'dt': 0.1, 'flag': '$flag', 'lst': '${lst}'},
        'output': {'output_dir': '$OUT', 'log_file': 'log.txt', 'spikes_file': '$OUT/spikes.h5', 'spikes_file_csv': '/abs/s.csv'},
        'node_sets_file': '$BASE/ns.json', 'network': 'circuit.json', 'other': ['$DEEP/x', 5, {'k': '${undefined}/y'}]}
    p = tmp_path / 'config.json'
    p.write_text(json.dumps(cfg))
    c = pointnet.Config.from_json(str(p), tag='run7', tstop=250.0, flag=True, lst=[1, 2])
    base = str(tmp_path)
    assert c.output_dir == base + '/out_run7'
    assert c.output['log_file'] == base + '/out_run7/log.txt'
    assert c.output['spikes_file'] == base + '/out_run7/spikes.h5' and c.output['spikes_file_csv'] == '/abs/s.csv'
    assert c.run['tstop'] == 250.0 and c.run['flag'] is True and c.run['lst'] == [1, 2]
    assert c['other'] == [base + '/out_run7/deeper/x', 5, {'k': '${undefined}/y'}]
    assert c.networks['nodes'][0]['nodes_file'] == base + '/network/n.h5'
    assert c.node_sets == {'sel': {'population': 'v1', 'ei': 'e'}}
    assert c.tstop == 250.0 and c.dt == 0.1 and c['config_path'] == str(p)
    with pytest.raises(Exception):
        pointnet.Config.from_dict({'manifest': {'$A': '$B/x', '$B': '$A/y'}})


@needs_ref
def test_inputs_and_reports_sections_equal_reference():
    ref_in = _ref_module('bmtk/simulator/utils/simulation_inputs.py', 'ref_sim_inputs')
    ref_rp = _ref_module('bmtk/simulator/utils/simulation_reports.py', 'ref_sim_reports')
    conf = pointnet.Config.from_json(REF + '/examples/point_450glifs/config.simulation.json')
    conf['reports'] = {'vm': {'module': 'multimeter_report', 'cells': 'v1', 'variable_name': 'V_m'},
                       'off': {'module': 'multimeter_report', 'cells': 'v1', 'variable_name': 'V_m', 'enabled': False}}
    conf._set_props()
    a, b = ref_in.from_config(conf), sim_settings.inputs_from_config(conf)
    assert [(x.name, x.input_type, x.module, x.params) for x in a] == [(x.name, x.input_type, x.module, x.params) for x in b]
    ra, rb = ref_rp.from_config(conf), sim_settings.reports_from_config(conf)
    assert [r.module for r in ra] == [r.module for r in rb]
    sa = [r for r in ra if r.module == 'spikes_report'][0].params
    sb = [r for r in rb if r.module == 'spikes_report'][0].params
    assert sa == sb
    ma = [r for r in ra if r.module == 'multimeter_report'][0].params
    mb = [r for r in rb if r.module == 'multimeter_report'][0].params
    for k in ('cells', 'variable_name', 'file_name', 'tmp_dir'):
        va = ma[k][0] if k == 'variable_name' else ma[k]
        assert va == mb[k], k


def test_glif_converter_matches_golden():
    g = json.load(open(os.path.join(os.path.dirname(__file__), 'golden', 'glif_known_answers.json')))
    for case in g['cases']:
        model, p = convert_aibs2nest(case['model_template'], case['aibs_params'])
        assert model == case['nest_model']
        exp = case['nest_params']
        assert set(p) == set(exp), case['model_template']
        for k, v in exp.items():
            assert np.allclose(np.asarray(p[k], dtype=float), np.asarray(v, dtype=float), rtol=0, atol=0), (case['model_template'], k)
    assert convert_aibs2nest('nest:iaf_psc_alpha', {'a': 1}) == ('nest:iaf_psc_alpha', {'a': 1})


@pytest.fixture(scope='module')
def project(tmp_path_factory):
    net = W.c0(t_stop_ms=300.0)
    root = str(tmp_path_factory.mktemp('proj'))
    info = write_project(net, root, iclamp=dict(node_set={'population': 'v1', 'node_id': [3, 4]}, amp=[120.0, 80.0],
                                                delay=[50.0, 150.0], duration=[100.0, 30.0]))
    return net, info


def test_network_build_reproduces_the_edge_list(project):
    net, info = project
    conf = pointnet.Config.from_json(info['config'])
    g = pointnet.PointNetwork.from_config(conf)
    sim = pointnet.PointSimulator.from_config(conf, g)
    for m in sim._mods:
        m.initialize(sim)
    n = net.n_neurons
    assert len(g.gid_pool) == n and g.n_virtual == net.n_virtual
    node_ids, pops = g.gid_pool.get_node_ids(np.arange(n))
    assert set(pops) == {'v1'}
    # batches: one per node type, in order of first appearance on disk, ids contiguous per batch
    first_types = []
    for t in (100 + net.type_index[info['disk_order']]):
        if t not in first_types:
            first_types.append(int(t))
    assert [lab[1] for lab in g.type_labels] == first_types
    assert np.all(np.diff(g.type_index.astype(int)) >= 0)
    wl_of_node = np.empty(n, dtype=np.int64)
    wl_of_node[info['node_id_of_engine']] = np.arange(n)
    wl_of_gid = wl_of_node[node_ids]
    assert np.array_equal(np.array([g.type_labels[k][1] - 100 for k in g.type_index]), net.type_index[wl_of_gid])
    for k, (pop, tid) in enumerate(g.type_labels):
        exp = net.types[tid - 100]
        for key, v in exp.items():
            assert np.allclose(np.asarray(g.types[k][key], dtype=float), np.asarray(v, dtype=float)), key
    # id map round trip
    assert np.array_equal(g.gid_pool.get_nestids('v1', node_ids), np.arange(n))
    assert g.gid_pool.get_pool_id(5) == ('v1', int(node_ids[5]))
    # edges: bit-exact against the workload's edge list (weight = nsyns * syn_weight, fp32)
    src, trg, w, d_ms, port = g.edge_arrays()
    s2 = np.where(src < n, wl_of_gid[np.minimum(src, n - 1)], src)
    t2 = wl_of_gid[trg]
    d = np.round(d_ms / net.dt).astype(np.int64)
    a = np.lexsort((w, port, d, t2, s2))
    b = np.lexsort((net.weight, net.port, net.delay_steps, net.trg, net.src))
    assert np.array_equal(s2[a], net.src[b]) and np.array_equal(t2[a], net.trg[b])
    assert np.array_equal(w[a].view(np.uint32), net.weight[b].view(np.uint32))
    assert np.array_equal(d[a], net.delay_steps[b]) and np.array_equal(port[a], net.port[b])
    # virtual cells
    v = np.concatenate([x[0] for x in g.input_spikes])
    t = np.concatenate([x[1] for x in g.input_spikes])
    from bmtk_b200.engine import time_to_stamp
    got = sorted(zip(v.tolist(), time_to_stamp(t, net.dt).tolist()))
    assert got == sorted(zip(net.in_virt.tolist(), net.in_stamp.tolist()))
    # clamp: off entry after delay+duration unless the next onset comes first; events act one step late
    ce = sim._clamp_events()
    gid3, gid4 = g.gid_pool.get_gid('v1', 3), g.gid_pool.get_gid('v1', 4)
    ev = sorted((int(s), int(tg), float(dl)) for s, tg, dl in zip(*ce))
    exp = []
    for gid in (gid3, gid4):
        exp += [(501, gid, 120.0), (1501, gid, -120.0), (1501, gid, 80.0), (1801, gid, -80.0)]
    assert ev == sorted(exp)
    # node sets
    assert sorted(g.get_node_set('v1').gids()) == list(range(n))
    assert g.get_node_set([1, 2, 3]).gids() == [1, 2, 3]
    sel = g.get_node_set({'population': 'v1', 'ei': 'i'}).gids()
    assert len(sel) == int(net.type_is_inh[net.type_index].sum())
    assert g.get_node_set('lgn').gids() == []


def test_iclamp_table_rules():
    m = IClampMod('current_clamp', 'all', amp=[100.0, 50.0, 20.0], delay=[0.05, 10.0, 15.0], duration=[3.0, 5.0, 2.0])
    # onset <= dt skipped; second stops exactly when the third starts -> off entry kept (stop <= next onset)
    t, v = m.amplitude_table(0.1)
    assert t == [10.0, 15.0, 15.0, 17.0] and v == [50.0, 0.0, 20.0, 0.0]
    m = IClampMod('current_clamp', 'all', amp=[100.0, 50.0], delay=[10.0, 12.0], duration=[5.0, 5.0])
    t, v = m.amplitude_table(0.1)
    assert t == [10.0, 12.0, 17.0] and v == [100.0, 50.0, 0.0]          # overlapped: no off entry in between
    with pytest.raises(Exception):
        IClampMod('current_clamp', 'all', amp=[1.0, 2.0], delay=[1.0], duration=[1.0])


def test_delay_below_resolution_and_bad_spike_times(project):
    """bmtk/tests/simulator/pointnet/test_pointnetwork.py:46-57 and :59-100."""
    net, info = project
    conf = pointnet.Config.from_json(info['config'])
    conf['run']['dt'] = 5.0          # every delay (1-2 ms) is now shorter than the resolution
    g = pointnet.PointNetwork.from_config(conf)
    with pytest.raises(pointnet.BadDelay):
        pointnet.PointSimulator.from_config(conf, g)
    conf = pointnet.Config.from_json(info['config'])
    g = pointnet.PointNetwork.from_config(conf)
    g.build_nodes()

    class Spikes(object):
        def __init__(self, times):
            self.times = times

        def get_times(self, node_id):
            return self.times
    for ok in ([], None, [3.0, 1.0, 2.0], np.array([0.5, 0.1])):
        g2 = pointnet.PointNetwork.from_config(conf)
        g2.build_nodes()
        g2.add_spike_trains(Spikes(ok), 'lgn')
    for bad in ([0.0, 1.0], [-1.0], np.array([1.0, 2.0, -0.5])):
        g2 = pointnet.PointNetwork.from_config(conf)
        g2.build_nodes()
        with pytest.raises(Exception):
            g2.add_spike_trains(Spikes(bad), 'lgn')


def test_spike_train_files_round_trip(tmp_path):
    """Layout per bmtk/tests/utils/reports/spike_trains/test_sonata_adaptor.py:31-53."""
    from bmtk_b200 import h5io
    st = pointnet.SpikeTrains()
    st.add_spikes([3, 1, 2, 1], [4.0, 1.5, 0.5, 3.0], 'v1')
    st.add_spike(7, 2.0, 'lgn')
    p = str(tmp_path / 'sp.h5')
    st.to_sonata(p, sort_order='by_time')
    with h5io.File(p, 'r') as h:
        assert int(h.attrs['magic']) == 0x0A7A
        g = h['/spikes/v1']
        assert g.attrs['sorting'] == 'by_time' and g['timestamps'].attrs['units'] == 'ms'
        assert g['timestamps'][()].tolist() == [0.5, 1.5, 3.0, 4.0] and g['node_ids'][()].tolist() == [2, 1, 1, 3]
        assert h['/spikes/lgn/node_ids'][()].tolist() == [7]
    back = pointnet.SpikeTrains.load(p)
    assert sorted(back.populations) == ['lgn', 'v1'] and back.get_times(1, 'v1').tolist() == [1.5, 3.0]
    c = str(tmp_path / 'sp.csv')
    st.to_csv(c, sort_order='by_id')
    lines = open(c).read().splitlines()
    assert lines[0] == 'timestamps population node_ids' and len(lines) == 6
    assert pointnet.SpikeTrains.load(c).n_spikes() == 5


def test_poisson_generator_rate_and_units():
    psg = pointnet.PoissonSpikeGenerator(population='lgn', seed=10)
    psg.add(node_ids=range(50), firing_rate=15.0, times=(0.0, 3.0))
    assert psg.n_spikes() == pytest.approx(50 * 15 * 3, rel=0.1)
    t = psg.to_dataframe()['timestamps'].values
    assert t.min() > 0 and 2500 < t.max() <= 3000.0
    psg2 = pointnet.PoissonSpikeGenerator(population='lgn', seed=10)
    psg2.add(node_ids=range(50), firing_rate=15.0, times=(0.0, 3.0))
    assert np.array_equal(psg2.to_dataframe()['timestamps'].values, t)          # seeded
    psg3 = pointnet.PoissonSpikeGenerator(population='lgn', seed=1)
    psg3.add(node_ids=[0], firing_rate=np.array([0.0, 50.0, 0.0]), times=np.array([0.0, 1.0, 2.0]))
    assert 20 < psg3.n_spikes() < 90


@needs_ref
def test_stock_example_network_expands_to_the_expected_edge_list():
    """examples/point_450glifs read from the reference tree: per edge weight = nsyns * syn_weight,
    delay 2.0 ms, port from the synapse JSON (e2e 1, i2e 2, e2i 3, i2i 4, LGN 1; iaf_psc_alpha
    targets by weight sign) — computed here independently from the raw files."""
    import pandas as pd
    from bmtk_b200 import h5io
    ex = REF + '/examples/point_450glifs'
    cwd = os.getcwd()
    os.chdir(ex)
    try:
        conf = pointnet.Config.from_json('config.simulation.json')
        g = pointnet.PointNetwork.from_config(conf)
        g.dt = conf.run['dt']
        g.build()
        g.add_spike_trains(pointnet.SpikeTrains.load(conf.inputs['LGN_spikes']['input_file']), 'lgn')
    finally:
        os.chdir(cwd)
    assert len(g.gid_pool) == 450 and g.n_virtual == 100
    src, trg, w, d, port = g.edge_arrays()
    assert len(src) == 28555 + 36035 and np.all(d == 2.0)
    node_types = pd.read_csv(ex + '/network/v1_node_types.csv', sep=' ').set_index('node_type_id')
    with h5io.File(ex + '/network/v1_nodes.h5', 'r') as h:
        ntid = h['/nodes/v1/node_type_id'][()].astype(int)
    is_iaf_node = np.array([node_types.loc[t, 'model_template'] == 'nest:iaf_psc_alpha' for t in ntid])
    gid_of_node = g.gid_pool.get_nestids('v1', np.arange(450))
    exp = []
    for fname, pop, types_csv, virtual in (('v1_v1_edges.h5', 'v1_to_v1', 'v1_v1_edge_types.csv', False),
                                           ('lgn_v1_edges.h5', 'lgn_to_v1', 'lgn_v1_edge_types.csv', True)):
        et = pd.read_csv(ex + '/network/' + types_csv, sep=' ').set_index('edge_type_id')
        with h5io.File(ex + '/network/' + fname, 'r') as h:
            p = h['/edges/' + pop]
            s, t = p['source_node_id'][()].astype(int), p['target_node_id'][()].astype(int)
            etid, ns = p['edge_type_id'][()].astype(int), p['0/nsyns'][()].astype(float)
        for k in range(len(s)):
            row = et.loc[etid[k]]
            weight = np.float32(ns[k] * row['syn_weight'])
            dyn = json.load(open(ex + '/../point_components/synaptic_models/' + row['dynamics_params']))
            prt = int(weight < 0) if is_iaf_node[t[k]] else dyn.get('receptor_type', 1) - 1
            exp.append((450 + s[k] if virtual else int(gid_of_node[s[k]]), int(gid_of_node[t[k]]), float(weight), prt))
    got = sorted(zip(src.tolist(), trg.tolist(), w.tolist(), port.tolist()))
    assert got == sorted(exp)
    n_in = sum(len(x[0]) for x in g.input_spikes)
    assert n_in == 3044
    # the two iaf_psc_alpha types became engine types with that model tag
    assert sum(t.get('model') == 'iaf_psc_alpha' for t in g.types) == 2


def test_weight_function_is_called_per_edge_type(project, tmp_path):
    """sonata_adaptors.py:319-335: a `weight_function` column replaces nsyns*syn_weight; the function
    gets (edges, source nodes, target nodes) data frames of one edge type and returns one weight per edge."""
    import shutil
    net, info = project
    root = tmp_path / 'proj'
    shutil.copytree(os.path.dirname(info['config']), str(root))
    tf = root / 'network' / 'v1_v1_edge_types.csv'
    lines = tf.read_text().splitlines()
    lines[0] += ' weight_function'
    lines[1:] = [ln + (' scaled_by_target' if ln.startswith('100 ') else ' NONE') for ln in lines[1:]]
    tf.write_text('\n'.join(lines) + '\n')
    calls = []

    @pointnet.synaptic_weight
    def scaled_by_target(edges, src_nodes, trg_nodes):
        calls.append((len(edges), len(src_nodes), len(trg_nodes), sorted(set(edges['edge_type_id']))))
        assert list(trg_nodes['node_id'].values) == list(edges['target_node_id'].values)
        return edges['syn_weight'].values * edges['nsyns'].values * np.where(trg_nodes['ei'].values == 'i', 2.0, 0.5)

    conf = pointnet.Config.from_json(str(root / 'config.simulation.json'))
    g = pointnet.PointNetwork.from_config(conf)
    g.build()
    assert len(calls) == 1 and calls[0][0] == calls[0][1] == calls[0][2] and calls[0][3] == [100]
    g0 = pointnet.PointNetwork.from_config(pointnet.Config.from_json(info['config']))
    g0.build()
    b1 = [b for b in g.edge_batches if b['edge_type_id'] == 100][0]
    b0 = [b for b in g0.edge_batches if b['edge_type_id'] == 100][0]
    inh = np.array([t.get('V_th') is not None for t in g.types])   # placeholder to keep shapes explicit
    node_ids, _ = g.gid_pool.get_node_ids(b1['trg'])
    ei = g.get_node_population('v1').to_dataframe().loc[node_ids, 'ei'].values
    assert np.allclose(b1['weight'], b0['weight'] * np.where(ei == 'i', 2.0, 0.5))
    others1 = [b for b in g.edge_batches if b['edge_type_id'] != 100]
    others0 = [b for b in g0.edge_batches if b['edge_type_id'] != 100]
    assert all(np.array_equal(x['weight'], y['weight']) for x, y in zip(others1, others0))
    with pytest.raises(Exception):
        lines[1] = lines[1].replace('scaled_by_target', 'not_registered')
        tf.write_text('\n'.join(lines) + '\n')
        pointnet.PointNetwork.from_config(conf).build()


def test_partition_by_in_degree_expands_only_the_local_edges(project):
    """Several ranks: blocks of engine ids are cut where the running in-degree sum passes k/N of the total, and
    a rank expands only the edges that end in its block; the ranks' edge lists together are the whole list."""
    from bmtk_b200.pointnet.pointnetwork import balanced_bounds
    net, info = project
    conf = pointnet.Config.from_json(info['config'])
    whole = pointnet.PointNetwork.from_config(conf)
    whole.dt = 0.1
    whole.build()
    whole.add_spike_trains(pointnet.SpikeTrains.load(conf.inputs[list(conf.inputs)[0]]['input_file']), 'lgn'
                           if 'lgn' in [p.name for p in whole.node_populations] else [p.name for p in whole.node_populations if p.is_virtual][0])
    src, trg, w, d, port = whole.edge_arrays()
    n = len(whole.gid_pool)
    indeg = np.bincount(trg, minlength=n)
    world = 3
    parts, bounds = [], None
    for rank in range(world):
        g = pointnet.PointNetwork.from_config(conf)
        g.dt = 0.1
        b = g.partition(rank, world)
        assert bounds is None or np.array_equal(b, bounds)
        bounds = b
        g.build()
        g.add_spike_trains(pointnet.SpikeTrains.load(conf.inputs[list(conf.inputs)[0]]['input_file']),
                           [p.name for p in g.node_populations if p.is_virtual][0])
        s2, t2, w2, d2, p2 = g.edge_arrays()
        lo, hi = g.target_block
        assert len(t2) and t2.min() >= lo and t2.max() < hi
        m = (trg >= lo) & (trg < hi)
        assert np.array_equal(s2, src[m]) and np.array_equal(t2, trg[m]) and np.array_equal(w2, w[m])
        assert np.array_equal(d2, d[m]) and np.array_equal(p2, port[m])
        parts.append(len(t2))
    assert sum(parts) == len(src) and bounds[0] == 0 and bounds[-1] == n and np.all(np.diff(bounds) > 0)
    # balanced by in-degree: every block within one neuron's in-degree of the ideal share
    share = np.array([indeg[bounds[k]:bounds[k + 1]].sum() for k in range(world)])
    assert np.abs(share - len(src) / world).max() <= indeg.max() + 1
    # the helper on its own: unconnected items still spread, more parts than items does not crash
    assert balanced_bounds(np.zeros(10), 2).tolist() == [0, 5, 10]
    assert balanced_bounds(np.array([5, 1, 1, 1, 1, 1]), 2).tolist() == [0, 1, 6]
    assert balanced_bounds(np.ones(2), 4)[-1] == 2
