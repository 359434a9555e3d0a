"""Per-kernel roofline probe: runs one kernel family of the engine on an input larger than L2
and prints achieved GB/s against algorithmic bytes.

    python -m bmtk_b200.microbench --kernel update    --neurons 4000000 --steps 64
    python -m bmtk_b200.microbench --kernel propagate --neurons 100000 --in-degree 1000 --steps 200

`update`    unconnected GLIF-3 neurons (the shape of the current-clamp configuration): only the
            fused state-update kernel does work; 128 B per neuron-step.
`propagate` an E/I network with fixed in-degree whose neurons are all held in tonic firing by a
            constant current (recurrent weights scaled down so they do not matter), so that every
            window delivers millions of synaptic events; 16 B per event.
Times come from CUDA events recorded around every launch (engine option "profile").
"""
import argparse
import json
import os

import numpy as np

from . import workloads as W


def _peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        return float(json.load(open(p))['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--kernel', choices=['update', 'propagate'], required=True)
    ap.add_argument('--neurons', type=int, default=4000000)
    ap.add_argument('--in-degree', type=int, default=1000)
    ap.add_argument('--steps', type=int, default=64)
    ap.add_argument('--warmup', type=int, default=16)
    ap.add_argument('--input-weight', type=float, default=60.0)
    ap.add_argument('--drive-pa', type=float, default=600.0, help='propagate: mean tonic current per neuron')
    ap.add_argument('--profile', type=int, default=1, help='0: plain launches only (for ncu captures)')
    a = ap.parse_args()
    if a.kernel == 'update':
        net = W.c1(n=a.neurons, t_stop_ms=1.0)
        net.clamp_step = net.clamp_step[:0]
        net.clamp_target = net.clamp_target[:0]
        net.clamp_delta = net.clamp_delta[:0]
        eng = W.build_engine(net, record_spikes=False, record_vm=False, options=dict(use_graph=0, window=8, persistent=0))
    else:
        net = W.c2(n=a.neurons, in_degree=a.in_degree, input_weight=a.input_weight, n_virtual=64, w_scale=0.01)
        rng = np.random.default_rng(5)
        ids = np.arange(a.neurons, dtype=np.uint32)
        net.clamp_step = np.ones(a.neurons, dtype=np.uint64)
        net.clamp_target = ids
        net.clamp_delta = rng.uniform(a.drive_pa * 0.6, a.drive_pa * 1.4, size=a.neurons).astype(np.float32)
        eng = W.build_engine(net, record_spikes=False, record_vm=False,
                             options=dict(use_graph=0, persistent=0, spike_capacity=a.neurons * 2))
    eng.run(a.warmup)
    eng.set_option('profile', a.profile)
    e0, s0 = eng.counter('events'), eng.counter('spikes')
    eng.run(a.steps)
    eng.set_option('profile', 0)
    ev, sp = eng.counter('events') - e0, eng.counter('spikes') - s0
    peak, kind = _peak()
    out = dict(kernel=a.kernel, neurons=a.neurons, steps=a.steps, events=ev, spikes=sp, peak_gbs=peak, peak_kind=kind)
    if a.kernel == 'propagate':
        from .engine import scatter_reduction_rate
        cells = eng.csr_info()['ring_slots'] * 4 * eng.counter('n_pad')
        out['scatter_red_ceiling_per_s'] = scatter_reduction_rate(cells, 8 * 1024 * 1024)
        out['ring_cells'] = cells
    if a.profile:
        un, pn = max(1, eng.counter('update_launches')), max(1, eng.counter('propagate_launches'))
        ut, pt = eng.counter('update_ns') / un, eng.counter('propagate_ns') / pn
        ub = 128.0 * eng.counter('n_pad')
        pb = 16.0 * ev / pn
        out.update(update=dict(launches=un, avg_us=ut * 1e-3, bytes_per_launch=ub, gbs=ub / ut, frac=ub / ut / peak),
                   propagate=dict(launches=pn, avg_us=pt * 1e-3, bytes_per_launch=pb, gbs=pb / max(pt, 1e-9),
                                  frac=pb / max(pt, 1e-9) / peak, events_per_launch=ev / pn,
                                  events_per_s=ev / pn / max(pt, 1e-9) * 1e9))
        if 'scatter_red_ceiling_per_s' in out:
            out['propagate']['frac_of_scatter_red_ceiling'] = out['propagate']['events_per_s'] / out['scatter_red_ceiling_per_s']
    print(json.dumps(out))


if __name__ == '__main__':
    main()
