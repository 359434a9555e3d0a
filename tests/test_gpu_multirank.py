"""Two ranks on two GPUs: neuron blocks + one exchange of spike ids per min-delay window must
reproduce the single-GPU result — bit for bit with deterministic delivery over NCCL ('replay',
'poisson'), and with exact event bookkeeping for the persistent kernel that exchanges over peer
memory ('p2p'). Skipped on a box with
one GPU; the CPU side of the partition logic is covered by test_partition_gloo.py."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize('mode', ['replay', 'poisson', 'p2p', 'uneven', 'clamp'])
def test_two_ranks_equal_one(cabi, tmp_path, mode):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    out = tmp_path / 'result.json'
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2', '--master-addr',
           '127.0.0.1', '--master-port', '29617', os.path.join(ROOT, 'tests', 'multirank_worker.py'), str(out), mode]
    p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:]
    r = json.load(open(out))
    assert r['ok'], r['msg']


def test_pointnet_surface_with_two_ranks(cabi, tmp_path):
    """The same SONATA project run by one rank and by two ranks (deterministic delivery) must write
    identical spikes and membrane-report files."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    import numpy as np
    from bmtk_b200 import h5io, pointnet, workloads as W
    from bmtk_b200.pointnet.reports import read_membrane_report
    sys.path.insert(0, os.path.join(ROOT, 'tests'))
    from bmtk_b200.sonata_writer import write_project
    net = W.c0(t_stop_ms=200.0)
    out = {}
    for tag, nproc in (('one', 1), ('two', 2)):
        root = tmp_path / tag
        info = write_project(net, str(root))
        env = dict(os.environ, NCCL_NVLS_ENABLE='0')
        cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', str(nproc),
               '--master-addr', '127.0.0.1', '--master-port', str(29630 + nproc),
               os.path.join(ROOT, 'tests', 'pointnet_worker.py'), info['config']]
        p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
        assert p.returncode == 0, p.stdout[-3000:]
        with h5io.File(str(root / 'output' / 'spikes.h5'), 'r') as h:
            g = h['/spikes/v1']
            out[tag] = (g['timestamps'][()], g['node_ids'][()], read_membrane_report(str(root / 'output' / 'membrane_potential.h5'))['v1'])
    a, b = out['one'], out['two']
    assert len(a[0]) > 100
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    oa, ob = np.argsort(a[2]['node_ids']), np.argsort(b[2]['node_ids'])
    assert np.array_equal(a[2]['node_ids'][oa], b[2]['node_ids'][ob])
    assert np.array_equal(a[2]['data'][:, oa], b[2]['data'][:, ob])
