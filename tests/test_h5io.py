"""The built-in HDF5 subset: known answers read out of library-written SONATA files (committed
as facts, the files themselves stay in the reference tree), and writer -> reader round trips."""
import os

import numpy as np
import pytest

from bmtk_b200 import h5io

REF_ROOT = os.environ.get('BMTK_REFERENCE', '/root/reference')
REF = REF_ROOT + '/examples/point_450glifs'
needs_ref = pytest.mark.skipif(not os.path.isdir(REF), reason='reference tree not mounted')


@needs_ref
def test_reads_library_written_nodes_file():
    with h5io.File(os.path.join(REF, 'network/v1_nodes.h5'), 'r') as h:
        assert int(h.attrs['magic']) == 0x0A7A and list(h.attrs['version']) == [0, 1]
        pop = h['/nodes/v1']
        assert sorted(pop.keys()) == ['0', '1', 'node_group_id', 'node_group_index', 'node_id', 'node_type_id']
        nid = pop['node_id'][()]
        assert nid.dtype == np.uint64 and np.array_equal(nid, np.arange(450))
        t, c = np.unique(pop['node_type_id'][()], return_counts=True)
        assert dict(zip(t.tolist(), c.tolist())) == {100: 80, 101: 80, 102: 80, 103: 30, 104: 30, 105: 75, 106: 75}
        g, c = np.unique(pop['node_group_id'][()], return_counts=True)
        assert pop['node_group_id'].dtype == np.uint32 and dict(zip(g.tolist(), c.tolist())) == {0: 300, 1: 150}
        assert sorted(pop['0'].keys()) == ['rotation_angle_yaxis', 'rotation_angle_zaxis', 'x', 'y', 'z']
        assert pop['0/x'].shape == (300,) and pop['1/z'].shape == (150,) and pop['0/x'].dtype == np.float64


@needs_ref
def test_reads_library_written_edges_file():
    with h5io.File(os.path.join(REF, 'network/v1_v1_edges.h5'), 'r') as h:
        pop = h['edges']['v1_to_v1']
        src, trg = pop['source_node_id'], pop['target_node_id']
        assert src.shape == (28555,) and src.dtype == np.uint64
        assert src.attrs['node_population'] == 'v1' and trg.attrs['node_population'] == 'v1'
        assert np.all(np.diff(trg[()].astype(np.int64)) >= 0)
        t, c = np.unique(pop['edge_type_id'][()], return_counts=True)
        assert dict(zip(t.tolist(), c.tolist())) == {100: 15149, 101: 1860, 102: 3224, 103: 1584, 104: 4709, 105: 2029}
        assert np.array_equal(pop['edge_group_index'][()], np.arange(28555))
        ns = pop['0/nsyns'][()]
        assert int(ns.sum()) == 71572
        first = list(zip(src[:5].tolist(), trg[:5].tolist(), ns[:5].tolist()))
        assert first == [(232, 0, 4), (39, 0, 1), (159, 0, 1), (113, 0, 3), (408, 0, 1)]
        idx = pop['indices/target_to_source/range_to_edge_id'][()]
        assert idx.shape == (450, 2) and idx[:3].tolist() == [[0, 83], [83, 159], [159, 231]]
    with h5io.File(os.path.join(REF, 'network/lgn_v1_edges.h5'), 'r') as h:
        pop = h['edges/lgn_to_v1']
        assert len(pop['source_node_id']) == 36035
        t, c = np.unique(pop['edge_type_id'][()], return_counts=True)
        assert dict(zip(t.tolist(), c.tolist())) == {100: 19202, 101: 4834, 102: 11999}


@needs_ref
def test_reads_library_written_spikes_file():
    with h5io.File(os.path.join(REF, 'inputs/lgn_spikes.h5'), 'r') as h:
        g = h['spikes/lgn']
        assert g.attrs['sorting'] == 'none'
        ts, ids = g['timestamps'], g['node_ids']
        assert ts.attrs['units'] == 'ms' and ts.shape == (3044,) and ids.dtype == np.uint32
        assert len(np.unique(ids[()])) == 100
        assert np.allclose(ts[:4], [445.539, 859.83, 897.245, 906.315])
        assert ts[()].min() == pytest.approx(1.176, abs=1e-3) and ts[()].max() == pytest.approx(2998.693, abs=1e-3)


@needs_ref
def test_reads_chunked_deflate_datasets():
    """examples/bio_1cell/output_iclamp holds gzip-compressed, chunked datasets written by h5py."""
    p = REF_ROOT + '/examples/bio_1cell/output_iclamp/spikes.h5'
    with h5io.File(p, 'r') as h:
        pops = h['spikes'].keys()
        g = h['spikes'][pops[0]]
        ts = g['timestamps'][()]
        assert ts.ndim == 1 and len(ts) == len(g['node_ids']) and np.all(np.isfinite(ts))
    p = REF_ROOT + '/examples/bio_1cell/output_iclamp/membrane_potential.h5'
    with h5io.File(p, 'r') as h:
        pop = h['report'][h['report'].keys()[0]]
        data = pop['data']
        assert data.ndim == 2 and data.shape[1] == len(pop['mapping/node_ids'])
        t0, t1, dt = pop['mapping/time'][()]
        assert data.shape[0] == int(round((t1 - t0) / dt))


@pytest.mark.skipif(h5io.HAVE_H5PY, reason='round trip of the built-in writer')
@pytest.mark.parametrize('compression', [None, 'gzip'])
def test_round_trip(tmp_path, compression):
    rng = np.random.default_rng(0)
    p = str(tmp_path / 'x.h5')
    ts = np.sort(rng.uniform(0, 1000, 5000))
    ids = rng.integers(0, 450, 5000).astype(np.uint64)
    with h5io.File(p, 'w') as h:
        h.attrs['magic'] = np.uint32(0x0A7A)
        h.attrs['version'] = np.array([0, 1], dtype=np.uint32)
        g = h.create_group('/spikes/v1')
        g.attrs['sorting'] = 'by_time'
        d = g.create_dataset('timestamps', data=ts, compression=compression)
        d.attrs['units'] = 'ms'
        g.create_dataset('node_ids', data=ids, compression=compression)
        rep = h.create_group('report/v1')
        rep.create_dataset('data', data=rng.normal(size=(300, 7)).astype(np.float64), compression=compression)
        rep.create_dataset('mapping/time', data=np.array([0.0, 30.0, 0.1]))
        rep.create_dataset('mapping/empty', data=np.zeros(0, dtype=np.uint64))
        many = h.create_group('many')
        for i in range(150):                       # more members than one symbol-table node holds
            many.create_dataset('d%03d' % i, data=np.arange(i, dtype=np.int32))
        h.create_dataset('flags', data=np.array([True, False, True]))
        h.create_dataset('f32', data=np.arange(6, dtype=np.float32).reshape(2, 3))
    with h5io.File(p, 'r') as h:
        assert int(h.attrs['magic']) == 0x0A7A and list(h.attrs['version']) == [0, 1]
        g = h['spikes/v1']
        assert g.attrs['sorting'] == 'by_time' and g['timestamps'].attrs['units'] == 'ms'
        assert np.array_equal(g['timestamps'][()], ts) and g['timestamps'].dtype == np.float64
        assert np.array_equal(g['node_ids'][()], ids) and g['node_ids'].dtype == np.uint64
        assert h['report/v1/data'].shape == (300, 7)
        assert np.array_equal(h['/report/v1/mapping/time'][()], [0.0, 30.0, 0.1])
        assert h['report/v1/mapping/empty'].shape == (0,)
        assert len(h['many']) == 150 and np.array_equal(h['many/d149'][()], np.arange(149))
        assert h['many'].keys() == sorted(h['many'].keys())
        assert h['f32'][1, 2] == 5.0 and h['f32'].dtype == np.float32
        assert h['flags'][()].tolist() == [1, 0, 1]
        assert 'spikes' in h and 'nope' not in h and 'spikes/v1/timestamps' in h


def test_rejects_foreign_files(tmp_path):
    if h5io.HAVE_H5PY:
        pytest.skip('h5py present')
    p = tmp_path / 'bad.h5'
    p.write_bytes(b'not hdf5 at all')
    with pytest.raises(IOError):
        h5io.File(str(p), 'r')


def test_edge_lookup_indices_equal_the_builders(tmp_path):
    """The index tables written next to the edges (indices/source_to_target, indices/target_to_source) re-derived
    from the id columns of the reference's own builder-written files must equal the tables stored in those files."""
    import glob
    from bmtk_b200.sonata_writer import edge_index_tables, write_edge_indices
    ref = os.environ.get('BMTK_REFERENCE', '/root/reference')
    files = sorted(glob.glob(os.path.join(ref, 'examples', 'point_450glifs', 'network', '*_edges.h5')) +
                   glob.glob(os.path.join(ref, 'examples', 'point_120cells', 'network', '*_edges.h5')))
    if not files:
        pytest.skip('reference tree not present')
    checked = 0
    for path in files:
        with h5io.File(path, 'r') as h:
            for pop in h['/edges'].keys():
                g = h['/edges'][pop]
                if 'indices' not in g:
                    continue
                for name, col in (('source_to_target', 'source_node_id'), ('target_to_source', 'target_node_id')):
                    i2r, r2e = edge_index_tables(g[col][()])
                    want_i2r = g['indices'][name]['node_id_to_range'][()]
                    want_r2e = g['indices'][name]['range_to_edge_id'][()]
                    assert np.array_equal(i2r, want_i2r) and i2r.dtype == want_i2r.dtype
                    # rows of one node id hold the same set of ranges (the builder's sort leaves their order open)
                    assert r2e.shape == want_r2e.shape
                    for b, e in i2r[:200]:
                        assert sorted(map(tuple, r2e[int(b):int(e)])) == sorted(map(tuple, want_r2e[int(b):int(e)]))
                    checked += 1
    assert checked >= 4
    # and through the writer: the groups exist and describe the columns
    src = np.array([3, 3, 0, 0, 0, 3, 5], dtype=np.uint64)
    trg = np.array([1, 1, 1, 2, 2, 2, 0], dtype=np.uint64)
    p = str(tmp_path / 'e.h5')
    with h5io.File(p, 'w') as h:
        g = h.create_group('/edges/a_to_b')
        g.create_dataset('source_node_id', data=src)
        g.create_dataset('target_node_id', data=trg)
        write_edge_indices(g, src, trg)
    with h5io.File(p, 'r') as h:
        s2t = h['/edges/a_to_b/indices/source_to_target']
        assert s2t['node_id_to_range'][()].tolist() == [[0, 1], [0, 0], [0, 0], [1, 3], [0, 0], [3, 4]]
        assert s2t['range_to_edge_id'][()].tolist() == [[2, 5], [0, 2], [5, 6], [6, 7]]
        t2s = h['/edges/a_to_b/indices/target_to_source']
        assert t2s['node_id_to_range'][()].tolist() == [[0, 1], [1, 2], [2, 3]]
        assert t2s['range_to_edge_id'][()].tolist() == [[6, 7], [0, 3], [3, 6]]
