"""Host side of the multi-rank path on CPU: two gloo ranks each generate their own block of a
network; together the blocks must be exactly the network a single rank generates (same edges, same
order inside a block), and rank 0's merge of per-rank spike records must be (stamp, id)-sorted."""
import os
import sys

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from bmtk_b200 import workloads as W
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    n = 20000
    bounds = np.linspace(0, n, world + 1).astype(int)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    part = W.c3(n=n, n_virtual=500, radius_um=250.0, lo=lo, hi=hi)
    # fake per-rank spike records: (stamp, id) of the rank's own neurons
    rng = np.random.default_rng(rank)
    st = np.sort(rng.integers(1, 100, 50)); ids = rng.integers(lo, hi, 50)
    gathered = [None] * world
    dist.gather_object(dict(src=part.src, trg=part.trg, w=part.weight, d=part.delay_steps, p=part.port, st=st, ids=ids,
                            types=part.types, rates=part.poisson_rate_hz), gathered if rank == 0 else None, 0)
    if rank == 0:
        whole = W.c3(n=n, n_virtual=500, radius_um=250.0)
        ok = True
        for r, g in enumerate(gathered):
            b0, b1 = int(bounds[r]), int(bounds[r + 1])
            m = (whole.trg >= b0) & (whole.trg < b1)
            ok &= np.array_equal(whole.src[m], g['src']) and np.array_equal(whole.trg[m], g['trg'])
            ok &= np.array_equal(whole.weight[m].view(np.uint32), g['w'].view(np.uint32))
            ok &= np.array_equal(whole.delay_steps[m], g['d']) and np.array_equal(whole.port[m], g['p'])
            ok &= g['types'] == whole.types and np.array_equal(g['rates'], whole.poisson_rate_hz)
        total = sum(len(g['src']) for g in gathered)
        ok &= total == whole.n_edges
        ast = np.concatenate([g['st'] for g in gathered]); aids = np.concatenate([g['ids'] for g in gathered])
        o = np.lexsort((aids, ast))
        ok &= bool(np.all(np.diff(ast[o]) >= 0))
        q.put(bool(ok))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_generate_the_same_network():
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 400)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
    assert ok
    assert all(p.exitcode == 0 for p in procs)
