"""Worker for the 2-GPU parity test (launched with torch.distributed.run): every rank owns one
contiguous block of the c0 network, the ranks exchange each window's spike ids with NCCL, and the
merged spike list is compared on rank 0 with a single-engine run of the whole network.
Deterministic delivery makes the comparison bit-exact."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    from bmtk_b200 import workloads as W
    from bmtk_b200.engine import nccl_unique_id
    rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
    local = int(os.environ.get('LOCAL_RANK', rank))
    torch.cuda.set_device(local)
    dist.init_process_group('gloo')
    libnccl = os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), 'nvidia', 'nccl', 'lib', 'libnccl.so.2')
    libnccl = libnccl if os.path.exists(libnccl) else None
    uid = [nccl_unique_id(libnccl) if rank == 0 else None]
    dist.broadcast_object_list(uid, 0)
    mode = sys.argv[2] if len(sys.argv) > 2 else 'replay'
    poisson = mode in ('poisson', 'p2p')
    p2p = mode in ('p2p', 'uneven', 'clamp')
    exact = mode in ('uneven', 'clamp')   # weights on a 0.25 pA grid: every fp32 sum is exact, whatever the order

    def make():
        if mode == 'uneven':
            # blocks of 5000 and 5001 neurons, window 8: the automatic spike capacity (block * window / 8) would be 5000
            # on one rank and 5004 on the other if each rank sized its own exchange buffer
            net = W.c2(n=10001, in_degree=100, n_virtual=200, t_stop_ms=150.0, input_weight=90.0)
        elif mode == 'clamp':
            # current steps into neurons of rank 0 only: the ranks must still pick the same stepping kernel
            net = W.c0(t_stop_ms=200.0, poisson_online=False)
            ids = np.arange(0, 100, dtype=np.uint32)
            net.clamp_step = np.concatenate([np.full(100, 301), np.full(100, 1501)]).astype(np.uint64)
            net.clamp_target = np.concatenate([ids, ids])
            net.clamp_delta = np.concatenate([np.full(100, 80.0), np.full(100, -80.0)]).astype(np.float32)
        else:
            net = W.c0(t_stop_ms=300.0, poisson_online=poisson)
        if exact:
            net.weight = (np.round(net.weight * 4.0) / 4.0).astype(np.float32)
        return net

    net = make()
    n = net.n_neurons
    bounds = np.linspace(0, n, world + 1).astype(int)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    m = (net.trg >= lo) & (net.trg < hi)
    part = make()
    part.lo, part.hi = lo, hi
    for k in ('src', 'trg', 'weight', 'delay_steps', 'port'):
        setattr(part, k, getattr(net, k)[m])
    eng = W.build_engine(part, device=local, deterministic=not p2p, rank=rank, n_ranks=world, nccl_uid=uid[0],
                         libnccl=libnccl, p2p=p2p, options=dict(chunk_steps=700) if p2p else None)
    if mode == 'uneven':
        assert eng.counter('pipelined') == 1 and eng.counter('spike_capacity') == 5004, eng.counter('spike_capacity')
    if mode == 'clamp':
        assert eng.counter('pipelined') == 0      # the rank without clamp targets follows the others
    eng.run(net.n_steps)
    st, ids = eng.fetch_spikes()
    tr = eng.fetch_trace()
    probes = part.probe_ids[(part.probe_ids >= lo) & (part.probe_ids < hi)]
    gathered = [None] * world
    dist.gather_object((st, ids, tr, probes, eng.counter('events')), gathered if rank == 0 else None, 0)
    ok = True
    msg = ''
    if rank == 0:
        ref = W.build_engine(net, device=local, deterministic=not p2p)
        ref.run(net.n_steps)
        rst, rids = ref.fetch_spikes()
        rtr = ref.fetch_trace()
        ast = np.concatenate([g[0] for g in gathered]); aids = np.concatenate([g[1] for g in gathered])
        o = np.lexsort((aids, ast))
        ast, aids = ast[o], aids[o]
        atr = np.concatenate([g[2] for g in gathered], axis=1)
        aprobe = np.concatenate([g[3] for g in gathered])
        ok &= bool(np.array_equal(aprobe, net.probe_ids))
        events = sum(g[4] for g in gathered)
        if not p2p or exact:
            ok &= bool(np.array_equal(ast, rst) and np.array_equal(aids, rids))
            ok &= bool(np.array_equal(atr.view(np.uint32), rtr.view(np.uint32)))
            ok &= events == ref.counter('events')
            ok &= len(ast) > 300
        else:
            # atomic sums: identical spikes until fp32 summation order makes the runs part, and exact
            # integer bookkeeping: every spike of every rank was delivered exactly once on every rank
            k = min(len(ast), len(rst))
            neq = np.nonzero((ast[:k] != rst[:k]) | (aids[:k] != rids[:k]))[0]
            div = int(ast[neq[0]]) if len(neq) else net.n_steps
            ok &= div > 800 and abs(len(ast) - len(rst)) <= 0.03 * len(rst) and eng.counter('launches') < 40   # 5 cooperative launches + log sorts, not 300 windows x 2
            rowptr = ref.csr()[0].astype(np.int64)
            outdeg = np.diff(rowptr)
            sys.path.insert(0, os.path.join(ROOT, 'tests'))
            from oracle import glif_oracle as O
            steps, srcs = O.poisson_spikes(net.poisson_rate_hz, net.dt, net.poisson_seed, 0, net.n_steps)
            expect = int(outdeg[aids].sum() + outdeg[n + srcs].sum())
            ok &= events == expect
            msg = 'p2p: first divergence %d, events %d expected %d; ' % (div, events, expect)
        msg += 'spikes %d ref %d events %d ref %d' % (len(ast), len(rst), events, ref.counter('events'))
        with open(sys.argv[1], 'w') as f:
            json.dump(dict(ok=bool(ok), msg=msg), f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
