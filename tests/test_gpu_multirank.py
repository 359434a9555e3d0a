"""Two ranks on two GPUs: neuron blocks + one NCCL all-gather of spike ids per min-delay window
must reproduce the single-GPU result bit for bit (deterministic delivery). Skipped on a box with
one GPU; the CPU side of the partition logic is covered by test_partition_gloo.py."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize('mode', ['replay', 'poisson'])
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
