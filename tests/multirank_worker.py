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
    poisson = len(sys.argv) > 2 and sys.argv[2] == 'poisson'
    net = W.c0(t_stop_ms=300.0, poisson_online=poisson)
    n = net.n_neurons
    bounds = np.linspace(0, n, world + 1).astype(int)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    m = (net.trg >= lo) & (net.trg < hi)
    part = W.c0(t_stop_ms=300.0, poisson_online=poisson)
    part.lo, part.hi = lo, hi
    for k in ('src', 'trg', 'weight', 'delay_steps', 'port'):
        setattr(part, k, getattr(net, k)[m])
    eng = W.build_engine(part, device=local, deterministic=True, rank=rank, n_ranks=world, nccl_uid=uid[0],
                         libnccl=libnccl)
    eng.run(net.n_steps)
    st, ids = eng.fetch_spikes()
    tr = eng.fetch_trace()
    probes = part.probe_ids[(part.probe_ids >= lo) & (part.probe_ids < hi)]
    gathered = [None] * world
    dist.gather_object((st, ids, tr, probes, eng.counter('events')), gathered if rank == 0 else None, 0)
    ok = True
    msg = ''
    if rank == 0:
        ref = W.build_engine(net, device=local, deterministic=True)
        ref.run(net.n_steps)
        rst, rids = ref.fetch_spikes()
        rtr = ref.fetch_trace()
        ast = np.concatenate([g[0] for g in gathered]); aids = np.concatenate([g[1] for g in gathered])
        o = np.lexsort((aids, ast))
        ok &= bool(np.array_equal(ast[o], rst) and np.array_equal(aids[o], rids))
        atr = np.concatenate([g[2] for g in gathered], axis=1)
        aprobe = np.concatenate([g[3] for g in gathered])
        ok &= bool(np.array_equal(aprobe, net.probe_ids))
        ok &= bool(np.array_equal(atr.view(np.uint32), rtr.view(np.uint32)))
        ok &= sum(g[4] for g in gathered) == ref.counter('events')
        msg = 'spikes %d ref %d events %d ref %d' % (len(ast), len(rst), sum(g[4] for g in gathered), ref.counter('events'))
        with open(sys.argv[1], 'w') as f:
            json.dump(dict(ok=bool(ok), msg=msg), f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
