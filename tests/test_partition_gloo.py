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


def _layout_worker(rank, world, port, q):
    """Each rank describes the exchange layout it would use (window, spike capacity, offsets follow from
    the minimum delay and the block size it knows), the ranks gather the descriptions over gloo and
    compare them with the library's own comparison: local values disagree, network-wide values agree."""
    sys.path.insert(0, ROOT)
    import ctypes as C
    from bmtk_b200 import _cabi
    lib = _cabi.load()
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    n = 100001
    bounds = np.linspace(0, n, world + 1).astype(int)
    n_local = int(bounds[rank + 1] - bounds[rank])
    min_delay = 8 if rank == 0 else 9           # rank 1 happens to hold no 8-step edge

    def describe(window, block):
        # the engine's rule: capacity = max(4096, block * window / 8) rounded up to 4; 2*16 + 2*ranks*cap words before the
        # pipelined area
        cap = (max(4096, block * window // 8) + 3) // 4 * 4
        d = np.zeros(16, dtype=np.uint64)
        d[0] = 0x424d544b58444553
        d[1:7] = [world, window, cap, 2 * 16 + 2 * world * cap, 148, 148]
        d[9], d[10] = n, 100
        return d

    import torch
    out = {}
    for tag, (w, blk) in (('local', (min_delay, n_local)), ('global', (None, None))):
        if tag == 'global':
            t = torch.tensor([-min_delay, n_local], dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            w, blk = int(-t[0]), int(t[1])
        mine = describe(w, blk)
        all_d = [None] * world
        dist.all_gather_object(all_d, mine)
        other = all_d[1 - rank]
        rc = lib.bmtk_exchange_layout_compare(mine.ctypes.data_as(C.c_void_p), other.ctypes.data_as(C.c_void_p), 1 - rank)
        out[tag] = (rc, lib.bmtk_last_error().decode() if rc else '')
    res = [None] * world
    dist.gather_object(out, res if rank == 0 else None, 0)
    if rank == 0:
        q.put(res)
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_with_different_exchange_layouts_are_refused():
    from bmtk_b200 import _cabi
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = 29100 + (os.getpid() % 400)
    procs = [ctx.Process(target=_layout_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
    assert all(p.exitcode == 0 for p in procs)
    for r in res:
        assert r['local'][0] == _cabi.E_INVALID and 'set_global_layout' in r['local'][1]
        assert 'exchange window' in r['local'][1]      # the first differing quantity is named
        assert r['global'][0] == _cabi.OK
