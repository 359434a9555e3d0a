"""The benchmark configurations at their real size on the GPU against the fp64 oracle.

c3 (230 924 neurons, ~70 M synapses, 1000 ms), c2 (50 000 neurons, in-degree 1000, 1000 ms), c1
(10 000 clamped neurons, dt 0.05 ms, 1500 ms) and c4 (64 trials of the c2 network, 500 ms), each on
the engine's default path, compared with the oracle run of the same seeded network:

* the (stamp, id)-sorted spike lists are identical up to a first divergence, which is printed;
* every neuron's spikes agree within one step over an initial span, in both directions. fp32 state
  against an fp64 reference moves an occasional threshold crossing by one step, and in a recurrent
  network of this size that difference spreads: measured on these networks, every spike of the
  first 25 ms (c3) / 50 ms (c2) agrees within one step, and over the first 100 ms fewer than 0.2 % of
  the spikes belong to a train that differs by more (c3: 297 + 61 neurons of 216 905 spikes). The
  tests assert exactly that: strict agreement over the short span, the 0.2 % bound over 100 ms;
* firing rates per node type (spikes / neurons / seconds) agree within 2 % over the full run, with
  no absolute allowance;
* the integer count of delivered synaptic events equals the oracle's at every checkpoint that lies
  before the first divergence.
"""
import os

import numpy as np
import pytest

from bmtk_b200 import workloads as W
from oracle import compare as K
from oracle import glif_oracle as O

pytestmark = pytest.mark.gpu
THREADS = os.cpu_count() or 1


def _oracle(net, stream=0):
    sim = O.OracleSim(net.types, net.type_index, net.dt, n_virtual=net.n_virtual, src=net.src, trg=net.trg,
                      weight=net.weight, delay_steps=net.delay_steps, port=net.port, n_threads=THREADS,
                      canonical_csr=False)
    if net.poisson_rate_hz is not None:
        steps, srcs = O.poisson_spikes(net.poisson_rate_hz, net.dt, net.poisson_seed, 0, net.n_steps, stream=stream)
        sim.set_input_spikes(steps, srcs)
    if len(net.clamp_step):
        sim.set_clamp_events(net.clamp_step, net.clamp_target, net.clamp_delta.astype(np.float64))
    if len(net.probe_ids):
        sim.set_probes(net.probe_ids, 1)
    return sim


def _connected(net, strict_steps, span_steps, pieces):
    eng = W.build_engine(net, record_vm=False)
    assert eng.counter('pipelined') == 1          # the kernel bench.py times
    ev_g, done = [], 0
    for k in pieces:
        eng.run(k)
        done += k
        ev_g.append(eng.counter('events'))
    eng.run(net.n_steps - done)
    st, ids = eng.fetch_spikes()
    st, ids = st.astype(np.int64), ids.astype(np.int64)
    sim = _oracle(net)
    ev_o, rs, ri, tot = [], [], [], 0
    for k in pieces + [net.n_steps - done]:
        r = sim.run(k, spike_cap=max(1 << 20, net.n_neurons * 16))
        tot += r['n_events']
        ev_o.append(tot)
        rs.append(r['spike_step'])
        ri.append(r['spike_id'].astype(np.int64))
    ost, oid = np.concatenate(rs), np.concatenate(ri)
    div = K.first_divergence(st, ids, ost, oid)
    print('%s: %d GPU spikes, %d oracle spikes, first divergence at step %s' % (net.name, len(st), len(ost), div))
    assert div is None or div > 50
    strict = K.within_one_step(st, ids, ost, oid, strict_steps, net.n_neurons)
    assert strict['ok'] and strict['n_a'] > 1000, strict
    wide = K.within_one_step(st, ids, ost, oid, span_steps, net.n_neurons)
    print('%s: first %d steps: %s' % (net.name, span_steps, wide))
    assert wide['neurons_with_other_count'] + wide['spikes_beyond_one_step'] <= 0.002 * wide['n_b'], wide
    # per-type rates over the full run: 2 %, nothing added
    ra = K.rate_agreement(net.type_index, len(net.types), ids, oid, net.n_steps * net.dt)
    print('%s: largest rate error %.3f %% (type %d)' % (net.name, 100 * ra['max_rel_err'], ra['worst_type']))
    assert ra['within_rel_only'], (ra['rates_a'], ra['rates_b'])
    assert abs(len(st) - len(ost)) <= 0.005 * len(ost)
    # integer bookkeeping: delivered events equal the oracle's wherever the lists still agree
    done = 0
    checked = 0
    for k, g, o in zip(pieces, ev_g, ev_o):
        done += k
        if div is None or done < div:
            assert g == o, (done, g, o)
            checked += 1
    assert checked >= 1
    eng.close()


def test_c3_full_size_against_oracle(cabi, oracle):
    net = W.c3()
    assert net.n_neurons == 230924 and 69e6 < net.n_edges < 71.5e6 and net.n_steps == 4000
    _connected(net, strict_steps=100, span_steps=400, pieces=[50, 50, 100, 200])


def test_c2_full_size_against_oracle(cabi, oracle):
    net = W.c2()
    assert net.n_neurons == 50000 and net.n_edges == 50000 * 1000 + 2000 * 200 and net.n_steps == 10000
    _connected(net, strict_steps=500, span_steps=1000, pieces=[100, 150, 250, 500])


def test_c1_full_size_against_oracle(cabi, oracle):
    """10 000 unconnected neurons, current steps 0..300 pA from 100 to 1100 ms, dt 0.05 ms, 1500 ms: the state
    update alone. Every neuron fires regularly for a second, so one threshold crossing that fp32 puts a step
    later shifts all later spikes of that neuron; compared are therefore the spikes of the first 100 ms of the
    current step (all within one step, counts equal), the per-neuron counts over the run (equal or one apart),
    and the V_m traces of the probed neurons up to the neuron's first differing spike."""
    net = W.c1()
    assert net.n_neurons == 10000 and net.n_steps == 30000 and net.dt == 0.05
    eng = W.build_engine(net)
    assert eng.counter('pipelined') == 1
    eng.run(net.n_steps)
    st, ids = eng.fetch_spikes()
    st, ids = st.astype(np.int64), ids.astype(np.int64)
    tr = eng.fetch_trace()
    r = _oracle(net).run(net.n_steps, spike_cap=net.n_neurons * 400)
    ost, oid = r['spike_step'], r['spike_id'].astype(np.int64)
    assert len(ost) > 50000
    first = K.within_one_step(st, ids, ost, oid, int(round(200.0 / net.dt)), net.n_neurons)
    assert first['ok'] and first['n_a'] > 10000, first
    cg, co = np.bincount(ids, minlength=net.n_neurons), np.bincount(oid, minlength=net.n_neurons)
    assert np.abs(cg - co).max() <= 1 and np.count_nonzero(cg != co) <= 0.002 * net.n_neurons
    n_checked = 0
    for q, i in enumerate(net.probe_ids.astype(np.int64)):
        a, b = st[ids == i], ost[oid == i]
        m = min(len(a), len(b))
        neq = np.nonzero(a[:m] != b[:m])[0]
        if len(neq):
            upto = int(min(a[neq[0]], b[neq[0]])) - 1
        elif len(a) != len(b):
            upto = int((a if len(a) > m else b)[m]) - 1
        else:
            upto = net.n_steps
        err = np.abs(tr[:upto, q].astype(np.float64) - r['trace'][:upto, q])
        assert np.all(err <= 1e-4 * np.abs(r['trace'][:upto, q]) + 2e-4), (i, float(err.max()))
        n_checked += upto
    assert n_checked > 0.5 * net.n_steps * len(net.probe_ids)
    eng.close()


def test_c4_full_size_trials_against_oracle(cabi, oracle):
    """64 trials of the 50 000-neuron network over one CSR, 500 ms; trials 0, 21, 42 and 63 against the oracle
    run of that trial's Philox stream (strict agreement over the first 40 ms; over 100 ms the trains that differ by
    more than a step stay below 0.6 % of the spikes: measured 0.1-0.53 % on the four trials); input spikes and
    delivered events add up exactly over all 64."""
    T = 64
    net = W.c4()
    assert net.n_neurons == 50000 and net.n_steps == 5000
    eng = W.build_engine(net, record_vm=False, options=dict(trials=T, chunk_steps=1000))
    eng.run(net.n_steps)
    st, ids = eng.fetch_spikes()
    st, ids = st.astype(np.int64), ids.astype(np.int64)
    n_pad1 = eng.counter('n_pad1')
    trial, cell = ids // n_pad1, ids % n_pad1
    assert cell.max() < net.n_neurons and len(np.unique(trial)) == T
    rowptr = eng.csr()[0].astype(np.int64)
    outdeg = np.diff(rowptr)
    n_in, ev_in = 0, 0
    for t in range(T):
        steps, srcs = O.poisson_spikes(net.poisson_rate_hz, net.dt, net.poisson_seed, 0, net.n_steps, stream=t)
        n_in += len(steps)
        ev_in += int(outdeg[net.n_neurons + srcs].sum())
    assert eng.counter('input_spikes') == n_in
    assert eng.counter('events') == ev_in + int(outdeg[cell].sum())
    for t in (0, 21, 42, 63):
        m = trial == t
        r = _oracle(net, stream=t).run(net.n_steps, spike_cap=net.n_neurons * 32)
        ost, oid = r['spike_step'], r['spike_id'].astype(np.int64)
        div = K.first_divergence(st[m], cell[m], ost, oid)
        print('c4 trial %d: %d GPU spikes, %d oracle spikes, first divergence at step %s' % (t, m.sum(), len(ost), div))
        assert div > 100
        strict = K.within_one_step(st[m], cell[m], ost, oid, 400, net.n_neurons)
        assert strict['ok'] and strict['n_a'] > 1000, (t, strict)
        wide = K.within_one_step(st[m], cell[m], ost, oid, 1000, net.n_neurons)
        assert wide['neurons_with_other_count'] + wide['spikes_beyond_one_step'] <= 0.006 * wide['n_b'], (t, wide)
        ra = K.rate_agreement(net.type_index, len(net.types), cell[m], oid, net.n_steps * net.dt)
        assert ra['within_rel_only'], (t, ra['rates_a'], ra['rates_b'])
    eng.close()
