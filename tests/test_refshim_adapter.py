"""The unmodified reference adapter (bmtk.simulator.pointnet of the reference tree) and
bmtk_b200.pointnet, run side by side on the reference's own example projects.

tests/refshim puts a recording `nest` module and an h5py stand-in under the reference package, so the
reference's own node batching, GidPool, edge expansion, add_spike_trains, IClampMod, SpikesMod and
MultimeterMod code runs as it is. Both adapters drive the same engine class (the fp64 oracle behind the
Engine API, so that this runs without a GPU): what differs between the two runs is only the adapter.
Compared bit for bit: neurons and their parameters, the edge list handed to the engine (source, target,
weight, delay, receptor port, in order), virtual-cell spike times, clamp tables, and the spikes / membrane
report files the modules write. Needs the reference tree (environment variable BMTK_REFERENCE); skipped without it."""
import gc
import json
import os
import shutil
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get('BMTK_REFERENCE', '/root/reference')
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, 'bmtk')), reason='reference tree not present')


def _copy_example(tmp_path, example, config, tstop, dt, tag, report=None):
    root = tmp_path / tag
    shutil.copytree(os.path.join(REF, 'examples', example), str(root / example))
    shutil.copytree(os.path.join(REF, 'examples', 'point_components'), str(root / 'point_components'))
    ex = str(root / example)
    conf = json.load(open(os.path.join(ex, config)))
    conf['run']['tstop'] = tstop
    conf['run']['dt'] = dt
    for inp in conf.get('inputs', {}).values():
        if inp.get('input_type') == 'current_clamp':
            # the stock example injects 0.15-0.2 pA from 500 ms on, which moves no cell; scaled so that the clamped
            # cells fire inside the shortened run (the same change in both copies)
            inp['amp'] = inp['amp'] * 3000.0
            inp['delay'] = inp['delay'] / 10.0
            inp['duration'] = inp['duration'] / 10.0
    if report:
        conf.setdefault('reports', {})['membrane_potential'] = {
            'cells': {'population': 'v1', 'node_id': [0, 100, 200, 300, 400]}, 'variable_name': report,
            'module': 'multimeter_report', 'file_name': 'membrane_potential.h5'}
    json.dump(conf, open(os.path.join(ex, 'config.short.json'), 'w'))
    return ex


def _run_reference(ex):
    """examples/<example>/run_pointnet.py, statement for statement, on the stand-in modules."""
    import refshim
    from refshim.oracle_engine import OracleEngine
    nest = refshim.install(REF, lambda dt: OracleEngine(dt))
    cwd = os.getcwd()
    os.chdir(ex)
    try:
        from bmtk.simulator import pointnet
        configure = pointnet.Config.from_json('config.short.json')
        configure.build_env()
        network = pointnet.PointNetwork.from_config(configure)
        sim = pointnet.PointSimulator.from_config(configure, network)
        sim.run()
        gc.collect()        # write_sonata leaves its file to the garbage collector
        net = nest.network()
        gid_map = network.gid_map
        node_ids, pops = gid_map.get_node_ids(net['neurons'])
        net['node_ids'], net['populations'] = np.asarray(node_ids), np.asarray(pops)
        net['clamps'] = [(nest._K.nodes[g]['params'], posts) for g, posts, _ in nest._K.clamp_links]
        net['n_calls'] = len(nest._K.calls)
    finally:
        os.chdir(cwd)
        import logging
        logging.shutdown()
        refshim.uninstall(REF)
    return net


def _run_facade(ex, monkeypatch):
    from refshim.oracle_engine import OracleEngine
    import bmtk_b200.engine as engine_mod
    from bmtk_b200 import pointnet
    monkeypatch.setattr(engine_mod, 'Engine', OracleEngine)
    cwd = os.getcwd()
    os.chdir(ex)
    try:
        conf = pointnet.Config.from_json('config.short.json')
        conf.build_env()
        graph = pointnet.PointNetwork.from_config(conf)
        sim = pointnet.PointSimulator.from_config(conf, graph)
        sim.run()
    finally:
        os.chdir(cwd)
    return graph, sim


def _params_bytes(d):
    from bmtk_b200.engine import glif_params
    return bytes(glif_params(d))


def _read_outputs(ex):
    from bmtk_b200 import h5io
    from bmtk_b200.pointnet.reports import read_membrane_report
    out = {}
    sp = os.path.join(ex, 'output', 'spikes.h5')
    with h5io.File(sp, 'r') as h:
        for pop in h['/spikes'].keys():
            g = h['/spikes'][pop]
            t, n = g['timestamps'][()], g['node_ids'][()]
            o = np.lexsort((n, t))
            out['spikes/' + pop] = (t[o], n[o].astype(np.int64), g['timestamps'].attrs.get('units'))
    rep = os.path.join(ex, 'output', 'membrane_potential.h5')
    if os.path.exists(rep):
        out['report'] = read_membrane_report(rep)
    csv = os.path.join(ex, 'output', 'spikes.csv')
    if os.path.exists(csv):
        rows = [ln.split() for ln in open(csv).read().splitlines()[1:]]
        out['csv'] = sorted((float(r[0]), r[1], int(r[2])) for r in rows)
        out['csv_header'] = open(csv).readline().strip()
    return out


@pytest.mark.parametrize('example,config,report', [
    ('point_450glifs', 'config.simulation.json', None),
    ('point_120cells', 'config.simulation.json', None),
    ('point_120cells', 'config.simulation_iclamp.json', None),
    # a multimeter on another recordable, and on two at once (the reference then leaves the LAST variable's values
    # in the file under the FIRST one's name)
    ('point_450glifs', 'config.simulation.json', ['I_syn']),
    ('point_450glifs', 'config.simulation.json', ['V_m', 'ASCurrents_sum'])])
def test_reference_adapter_and_facade_build_the_same_network_and_files(tmp_path, monkeypatch, example, config, report):
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    dt, tstop = 0.1, 300.0
    ex_ref = _copy_example(tmp_path, example, config, tstop, dt, 'ref', report)
    ex_fac = _copy_example(tmp_path, example, config, tstop, dt, 'facade', report)
    ref = _run_reference(ex_ref)
    graph, sim = _run_facade(ex_fac, monkeypatch)

    # a2 / a3: neurons in creation order, their parameters, and the id bookkeeping
    assert len(ref['neurons']) == len(graph.gid_pool)
    f_ids, f_pops = graph.gid_pool.get_node_ids(np.arange(len(graph.gid_pool)))
    assert np.array_equal(ref['node_ids'], f_ids) and np.array_equal(ref['populations'], f_pops)
    ref_p = [_params_bytes(t) for t in ref['types']]
    fac_p = [_params_bytes(t) for t in graph.types]
    assert [ref_p[k] for k in ref['type_index']] == [fac_p[k] for k in graph.type_index]
    # a4 / a5: the edge list, in the order it reaches the engine
    src, trg, w, d, port = graph.edge_arrays()
    assert len(src) == len(ref['src']) > 1000
    assert np.array_equal(src, ref['src']) and np.array_equal(trg, ref['trg'])
    w64 = np.concatenate([np.asarray(b['weight'], dtype=np.float64) for b in graph.edge_batches + graph.virtual_edge_batches])
    assert np.array_equal(w64, ref['weight'])                                   # nsyns x syn_weight as the adapter computes it (fp64)
    assert np.array_equal(w, ref['weight'].astype(np.float32))                  # and as the engine receives it (fp32)
    assert np.array_equal(np.asarray(d, dtype=np.float64), ref['delay_ms'])
    assert np.array_equal(np.asarray(port, dtype=np.uint8), ref['port'])
    # a6: virtual cells and their spike times
    assert graph.n_virtual == len(ref['virtual'])
    if graph.input_spikes:
        v = np.concatenate([x[0] for x in graph.input_spikes])
        t = np.concatenate([x[1] for x in graph.input_spikes])
        o1, o2 = np.lexsort((t, v)), np.lexsort((ref['in_time_ms'], ref['in_virt']))
        assert np.array_equal(v[o1], ref['in_virt'][o2]) and np.array_equal(t[o1], ref['in_time_ms'][o2])
    else:
        assert len(ref['in_virt']) == 0
    # a12: clamp tables
    if 'iclamp' in config:
        assert len(ref['clamps']) >= 1 and len(sim._clamps) == len(ref['clamps'])
        for (p, posts), (times, vals, gids) in zip(ref['clamps'], sim._clamps):
            assert list(p['amplitude_times']) == list(times) and list(p['amplitude_values']) == list(vals)
            assert sorted(np.asarray(gids).tolist()) == sorted(i - 1 for i in posts)      # NEST ids count from 1
    # a10 / a11: the files the modules wrote
    a, b = _read_outputs(ex_ref), _read_outputs(ex_fac)
    assert set(a) == set(b)
    n_spikes = 0
    for k in a:
        if k.startswith('spikes/'):
            assert np.array_equal(a[k][0], b[k][0]) and np.array_equal(a[k][1], b[k][1]) and a[k][2] == b[k][2]
            n_spikes += len(a[k][0])
    assert n_spikes > 50
    if 'csv' in a:
        assert a['csv'] == b['csv'] and a['csv_header'] == b['csv_header']
    if report:
        assert 'report' in a and float(np.ptp(a['report']['v1']['data'])) > 0.0
        assert a['report']['v1']['variable'] == b['report']['v1']['variable'] == report[0]
    if 'report' in a:
        for pop in a['report']:
            ra, rb = a['report'][pop], b['report'][pop]
            oa, ob = np.argsort(ra['node_ids']), np.argsort(rb['node_ids'])
            assert np.array_equal(ra['node_ids'][oa], rb['node_ids'][ob])
            # the reference reads the recorder's text file back with pandas' default float parser, which is allowed to be
            # one unit in the last place off; nothing else separates the two files' values
            assert ra['data'].shape == rb['data'].shape
            assert np.allclose(ra['data'][:, oa], rb['data'][:, ob], rtol=4e-16, atol=0.0)
            # time = [first, last, step]: the reference takes the first and last RECORDED time (dt and tstop), the façade
            # writes the recording window's start (tstart = 0); the same samples either way
            assert ra['time'][1] == rb['time'][1] and ra['time'][2] == rb['time'][2]
            assert ra['time'][0] == pytest.approx(rb['time'][0] + rb['time'][2])


def test_delay_below_resolution_is_refused_by_both_adapters(tmp_path, monkeypatch):
    """dt = 2 ms against the example's 1.5 ms delays: the reference logs and re-raises NEST's BadDelay
    (pointnetwork.py:229-243), bmtk_b200.pointnet raises its BadDelay at the same place (building the edges)."""
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    ex = _copy_example(tmp_path, 'point_120cells', 'config.simulation.json', 100.0, 2.0, 'ref')
    with pytest.raises(Exception) as ei:
        _run_reference(ex)
    assert type(ei.value).__name__ == '_BadDelay' and ei.value.errorname == 'BadDelay'
    ex2 = _copy_example(tmp_path, 'point_120cells', 'config.simulation.json', 100.0, 2.0, 'facade')
    from bmtk_b200.pointnet.pointnetwork import BadDelay
    with pytest.raises(BadDelay):
        _run_facade(ex2, monkeypatch)
