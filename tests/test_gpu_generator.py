"""Device-side network generator (bmtk_generate_distance_edges) against its CPU restatement, and the V1-scale
network it samples: written as a SONATA project, read back through the drop-in surface, built and run."""
import os
import time

import numpy as np
import pytest

from bmtk_b200 import generator as G
from bmtk_b200 import workloads as W
from oracle import glif_oracle as O

pytestmark = pytest.mark.gpu


def _small_spec(seed=3, n=20000, nt=5, R=250.0):
    rng = np.random.default_rng(seed)
    inh = np.array([0, 0, 0, 1, 1], dtype=bool)
    ti = np.sort(rng.integers(0, nt, n)).astype(np.uint16)
    rad = R * np.sqrt(rng.random(n))
    ang = rng.uniform(0, 2 * np.pi, n)
    return G.distance_spec(ti, inh, rad * np.cos(ang), rad * np.sin(ang), rng.uniform(100, 200, (2, nt)),
                           np.log(rng.uniform(0.8, 2.5, (nt, nt))), R, 330.0, 0.25, 99), inh, ti


def test_device_generator_equals_its_cpu_restatement_bit_for_bit(cabi, oracle):
    spec, inh, ti = _small_spec()
    cpu = O.generate_distance_edges(spec)
    gpu = G.generate_edges(spec)
    assert len(cpu[0]) > 3e6
    for a, b, name in zip(gpu, cpu, ('source', 'target', 'weight', 'delay', 'port')):
        assert a.dtype == b.dtype and np.array_equal(a.view(np.uint8), b.view(np.uint8)), name
    # any partition of the targets gives the same edges
    parts = [G.generate_edges(spec, lo, hi) for lo, hi in ((0, 1), (1, 7001), (7001, 20000))]
    for k in range(5):
        assert np.array_equal(np.concatenate([p[k] for p in parts]), gpu[k])
    src, trg, w, d, port = gpu
    # what the rule promises: no self loops, targets in order, sign by the source's class, port by the class pair,
    # delays 0.5-4 ms on the 0.25 ms grid
    assert np.all(src != trg) and np.all(np.diff(trg.astype(np.int64)) >= 0)
    s_inh, t_inh = inh[ti[src]], inh[ti[trg]]
    assert np.all((w < 0) == s_inh) and np.array_equal(port, s_inh.astype(np.uint8) + 2 * t_inh.astype(np.uint8))
    assert d.min() == 2 and d.max() == 16
    # distance dependence: connected pairs are much closer than random pairs
    x, y = spec['x'], spec['y']
    dist = np.hypot(x[src] - x[trg], y[src] - y[trg])
    rnd = np.random.default_rng(0).integers(0, len(x), (200000, 2))
    assert np.median(dist) < 0.75 * np.median(np.hypot(x[rnd[:, 0]] - x[rnd[:, 1]], y[rnd[:, 0]] - y[rnd[:, 1]]))


def test_v1_scale_network_from_the_device_generator(cabi, tmp_path):
    """230 924 neurons, ~70 M synapses sampled on the GPU; the project is written with the SONATA writer (lookup
    indices included), read back through PointNetwork, and the engine built from the files runs 100 ms."""
    from bmtk_b200 import h5io, pointnet
    from bmtk_b200.sonata_writer import write_project
    t0 = time.time()
    net = G.c3_device()
    t_gen = time.time() - t0
    n = net.n_neurons
    rec = net.src < n
    assert n == 230924 and 68e6 < rec.sum() < 72e6
    indeg = np.bincount(net.trg[rec], minlength=n)
    assert 280 < indeg.mean() < 320 and indeg.min() > 20
    # a sample of targets against the CPU restatement
    for lo in (0, 100000, n - 50):
        cpu = O.generate_distance_edges(net.meta['spec'], lo, lo + 50)
        m = rec & (net.trg >= lo) & (net.trg < lo + 50)
        assert np.array_equal(net.src[m], cpu[0]) and np.array_equal(net.weight[m].view(np.uint32), cpu[2].view(np.uint32))
    net.in_virt, net.in_stamp = W._poisson_trains(np.random.default_rng(5), np.full(net.n_virtual, 8.0), 100.0, net.dt)
    rates, net.poisson_rate_hz = net.poisson_rate_hz, None
    t0 = time.time()
    info = write_project(net, str(tmp_path), with_report=False, tstop=100.0)
    t_write = time.time() - t0
    with h5io.File(str(tmp_path / 'network' / 'v1_v1_edges.h5'), 'r') as h:
        g = h['/edges/v1_to_v1']
        assert len(g['source_node_id']) == rec.sum()
        i2r = g['indices/target_to_source/node_id_to_range'][()]
        r2e = g['indices/target_to_source/range_to_edge_id'][()]
        assert i2r.shape == (n, 2) and int((r2e[:, 1] - r2e[:, 0]).sum()) == rec.sum()
    t0 = time.time()
    conf = pointnet.Config.from_json(info['config'])
    graph = pointnet.PointNetwork.from_config(conf)
    sim = pointnet.PointSimulator.from_config(conf, graph)
    t_read = time.time() - t0
    sim.run()                                             # the input module adds the virtual cells' edges
    src, trg, w, d, port = graph.edge_arrays()
    assert len(src) == net.n_edges
    # same multiset of edges after the node-id permutation of the files: compare invariant sums
    assert float(w.astype(np.float64).sum()) == pytest.approx(float(net.weight.astype(np.float64).sum()), rel=1e-9)
    assert np.array_equal(np.bincount(port, minlength=4), np.bincount(net.port, minlength=4))
    assert np.array_equal(np.bincount(np.round(d / net.dt).astype(np.int64)), np.bincount(net.delay_steps))
    st = sim.recorded_spikes()
    rate = len(st[0]) / n / 0.1
    print('generate %.1f s, write %.1f s, read+expand %.1f s, %d spikes in 100 ms (%.2f Hz)' % (t_gen, t_write, t_read, len(st[0]), rate))
    assert 0.5 < rate < 20.0
    net.poisson_rate_hz = rates
