"""End to end through the drop-in surface on the GPU: a SONATA project on disk is run with
Config -> PointNetwork.from_config -> PointSimulator.from_config(...).run(), and the spikes / report
files it writes must contain exactly what a directly driven engine (and, within tolerance, the
oracle) produces for the same network."""
import numpy as np
import pytest

from bmtk_b200 import h5io, pointnet, workloads as W
from bmtk_b200.pointnet.reports import read_membrane_report
from netutil import oracle_from_network
from bmtk_b200.sonata_writer import write_project

pytestmark = pytest.mark.gpu


def test_run_from_files_equals_direct_engine(cabi, tmp_path):
    net = W.c0(t_stop_ms=300.0)
    info = write_project(net, str(tmp_path))
    conf = pointnet.Config.from_json(info['config'])
    conf.build_env()
    graph = pointnet.PointNetwork.from_config(conf)
    sim = pointnet.PointSimulator.from_config(conf, graph)
    sim.run()
    # direct run
    eng = W.build_engine(net, deterministic=True)
    eng.run(net.n_steps)
    st, ids = eng.fetch_spikes()
    tr = eng.fetch_trace()
    node_of = info['node_id_of_engine']
    # spikes.h5: sorted by time, times = stamp*dt, node ids = SONATA ids
    with h5io.File(conf.output['spikes_file'], 'r') as h:
        g = h['/spikes/v1']
        assert g.attrs['sorting'] == 'by_time'
        ts, nid = g['timestamps'][()], g['node_ids'][()]
    assert len(ts) == len(st) > 100
    exp = sorted(zip((st * net.dt).round(6).tolist(), node_of[ids].tolist()))
    assert sorted(zip(ts.round(6).tolist(), nid.tolist())) == exp
    assert np.all(np.diff(ts) >= 0)
    # spikes.csv
    lines = open(conf.output['spikes_file_csv']).read().splitlines()
    assert lines[0] == 'timestamps population node_ids' and len(lines) == len(st) + 1
    # membrane report: one column per requested node, V_m every dt, first sample at t = dt
    rep = read_membrane_report(str(tmp_path / 'output' / 'membrane_potential.h5'))['v1']
    assert rep['time'].tolist() == [0.0, 300.0, net.dt] and rep['variable'] == 'V_m'
    want = node_of[net.probe_ids]
    assert sorted(rep['node_ids'].tolist()) == sorted(want.tolist())
    col = {int(n): k for k, n in enumerate(rep['node_ids'])}
    data = rep['data'][:, [col[int(n)] for n in want]]
    assert data.shape == tr.shape
    assert np.array_equal(data.astype(np.float32).view(np.uint32), tr.view(np.uint32))
    # and against the oracle
    r = oracle_from_network(net).run(net.n_steps)
    n = min(len(st), len(r['spike_step']))
    same = (st[:n] == r['spike_step'][:n]) & (ids[:n] == r['spike_id'][:n])
    assert same[:50].all()
    assert (tmp_path / 'output' / 'log.txt').exists() and (tmp_path / 'output' / 'config.simulation.json').exists()


def test_iclamp_through_the_modules(cabi, tmp_path):
    """IClamp module -> clamp events -> update kernel, against the oracle driven with the same table."""
    net = W.c0(t_stop_ms=200.0)
    net.src, net.trg = net.src[:0], net.trg[:0]
    net.weight, net.delay_steps, net.port = net.weight[:0], net.delay_steps[:0], net.port[:0]
    net.in_virt, net.in_stamp = net.in_virt[:0], net.in_stamp[:0]
    clamp = dict(node_set='v1', amp=[250.0, 400.0], delay=[20.0, 100.0], duration=[50.0, 60.0])
    info = write_project(net, str(tmp_path), iclamp=clamp)
    conf = pointnet.Config.from_json(info['config'])
    conf.build_env()
    graph = pointnet.PointNetwork.from_config(conf)
    sim = pointnet.PointSimulator.from_config(conf, graph)
    sim.run()
    stamps, gids = sim.recorded_spikes()
    assert len(stamps) > 200
    node_ids, _ = graph.gid_pool.get_node_ids(gids)
    wl_of_node = np.empty(net.n_neurons, dtype=np.int64)
    wl_of_node[info['node_id_of_engine']] = np.arange(net.n_neurons)
    # oracle with the same table: on at round(T/dt)+1, off likewise
    n = net.n_neurons
    allids = np.arange(n, dtype=np.uint32)
    steps = [201, 701, 1001, 1601]
    deltas = [250.0, -250.0, 400.0, -400.0]
    net.clamp_step = np.repeat(np.array(steps, dtype=np.uint64), n)
    net.clamp_target = np.tile(allids, 4)
    net.clamp_delta = np.repeat(np.array(deltas, dtype=np.float32), n)
    r = oracle_from_network(net).run(net.n_steps)
    got = sorted(zip(wl_of_node[node_ids].tolist(), stamps.tolist()))
    exp = sorted(zip(r['spike_id'].tolist(), r['spike_step'].tolist()))
    assert len(got) == len(exp)
    d = np.abs(np.array([g[1] for g in got]) - np.array([e[1] for e in exp]))
    assert [g[0] for g in got] == [e[0] for e in exp]
    assert d.max() <= 1 and np.mean(d == 0) > 0.9
