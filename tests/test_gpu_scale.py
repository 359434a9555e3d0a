"""Full-size and mid-size workloads on the GPU, checked through properties that do not need the
CPU oracle to simulate them: exact integer bookkeeping of synaptic events, CSR invariants,
agreement of the deterministic and the atomic delivery, plus a reduced E/I network against the
oracle."""
import numpy as np
import pytest

from bmtk_b200 import workloads as W
from netutil import oracle_from_network, rates_by_type

pytestmark = pytest.mark.gpu


def _first_divergence(st_a, id_a, st_b, id_b):
    n = min(len(st_a), len(st_b))
    neq = np.nonzero((st_a[:n] != st_b[:n]) | (id_a[:n] != id_b[:n]))[0]
    if len(neq):
        return int(min(st_a[neq[0]], st_b[neq[0]]))
    return np.inf if len(st_a) == len(st_b) else int((st_a if len(st_a) > n else st_b)[n])


def test_c3_full_size_bookkeeping_and_mode_agreement(cabi, oracle):
    """The benchmark network itself (230 924 neurons, ~70 M synapses, Philox Poisson cells), 100 ms."""
    net = W.c3()
    n_steps = 400
    n = net.n_neurons
    assert n == 230924 and 69e6 < net.n_edges < 71.5e6
    eng = W.build_engine(net, record_vm=False)
    # CSR invariants against the edge list (integer work: exact)
    rowptr, packed, weight = eng.csr()
    info = eng.csr_info()
    tb = info['target_bits']
    rowptr = rowptr.astype(np.int64)
    assert rowptr[0] == 0 and rowptr[-1] == net.n_edges and np.all(np.diff(rowptr) >= 0)
    assert np.array_equal(np.diff(rowptr), np.bincount(net.src, minlength=n + net.n_virtual))
    row_of = np.repeat(np.arange(n + net.n_virtual), np.diff(rowptr))
    key = (row_of.astype(np.int64) << 32) | packed
    assert np.all(np.diff(key) >= 0)                       # rows by source, entries by (delay, port, target)
    assert np.array_equal(np.bincount(packed & ((1 << tb) - 1), minlength=n), np.bincount(net.trg, minlength=n))
    assert np.array_equal(np.bincount(packed >> (tb + 2)), np.bincount(net.delay_steps))
    assert float(weight.astype(np.float64).sum()) == pytest.approx(float(net.weight.astype(np.float64).sum()), rel=1e-12)
    assert info['min_delay'] == 2 and info['max_delay'] == 16 and eng.counter('window') == 2
    # atomic delivery (persistent kernel) and deterministic delivery (per-step kernels)
    eng.run(n_steps)
    st, ids = eng.fetch_spikes()
    det = W.build_engine(net, record_vm=False, deterministic=True)
    det.run(n_steps)
    st_d, ids_d = det.fetch_spikes()
    assert len(st) > 50000
    div = _first_divergence(st.astype(np.int64), ids.astype(np.int64), st_d.astype(np.int64), ids_d.astype(np.int64))
    assert div > 100                                       # identical spikes until fp32 summation order matters
    assert abs(len(st) - len(st_d)) <= 0.01 * len(st_d)
    ra, rd = rates_by_type(net, ids, 100.0), rates_by_type(net, ids_d, 100.0)
    # two deliveries of the same network over 100 ms: 2 % of the rate plus three standard deviations of the counting
    # noise of two runs that have parted (oracle/compare.py:rate_agreement)
    from oracle import compare as K
    assert K.rate_agreement(net.type_index, len(net.types), ids, ids_d, 100.0)['ok'], (ra, rd)
    # events delivered = sum of the row lengths of every spike emitted (neurons and Poisson cells)
    steps, srcs = oracle.poisson_spikes(net.poisson_rate_hz, net.dt, net.poisson_seed, 0, n_steps)
    outdeg = np.diff(rowptr)
    for e, i in ((eng, ids), (det, ids_d)):
        assert e.counter('input_spikes') == len(steps)
        assert e.counter('events') == int(outdeg[i].sum() + outdeg[n + srcs].sum())
        assert e.counter('spikes') == len(i)


@pytest.mark.parametrize('deterministic', [True, False])
def test_c2_reduced_against_oracle(cabi, deterministic):
    """The mid-scale E/I configuration at 1/10 size (5000 neurons, in-degree 200, 4 ports, delays
    0.8-3.0 ms -> window 8) for 400 ms against the fp64 oracle."""
    net = W.c2(n=5000, in_degree=200, n_virtual=200, t_stop_ms=400.0, input_weight=90.0)
    eng = W.build_engine(net, deterministic=deterministic)
    assert eng.counter('window') == 8
    eng.run(net.n_steps)
    st, ids = eng.fetch_spikes()
    st, ids = st.astype(np.int64), ids.astype(np.int64)
    r = oracle_from_network(net).run(net.n_steps)
    assert r['n_spikes'] > 2000
    div = _first_divergence(st, ids, r['spike_step'], r['spike_id'])
    assert div > 300
    m_g, m_c = st <= 1000, r['spike_step'] <= 1000
    a = sorted(zip(ids[m_g].tolist(), st[m_g].tolist()))
    b = sorted(zip(r['spike_id'][m_c].tolist(), r['spike_step'][m_c].tolist()))
    assert len(a) == len(b)
    assert all(x[0] == y[0] and abs(x[1] - y[1]) <= 1 for x, y in zip(a, b))
    rg, rc = rates_by_type(net, ids, 400.0), rates_by_type(net, r['spike_id'], 400.0)
    from oracle import compare as K       # 2 % plus 3 sigma of the counting noise (5000 neurons, 400 ms)
    assert K.rate_agreement(net.type_index, len(net.types), ids, r['spike_id'], 400.0)['ok'], (rg, rc)


@pytest.mark.parametrize('mode', ['pipelined_one_launch', 'pipelined_groups_of_2', 'two_phase'])
def test_trial_batching_shares_the_csr(cabi, oracle, mode):
    """Option "trials": T independent copies of a network over ONE CSR, each with its own Philox stream
    (counter word 3 = trial). Every trial must reproduce the oracle run of that trial's input stream
    (spikes within one step over the first 100 ms, then until the first divergence), the trials must
    differ from each other, and events / input spikes must add up exactly over the trials. The pipelined
    kernel steps all trials in one launch or, group by group, two at a time (the last group has one);
    the two-phase kernel is the third way."""
    T = 5
    net = W.c2(n=3000, in_degree=150, n_virtual=150, t_stop_ms=300.0, input_weight=90.0)
    opts = dict(pipelined_one_launch=dict(), pipelined_groups_of_2=dict(pipeline_trials=2, chunk_steps=1100),
                two_phase=dict(pipeline=0))[mode]
    eng = W.build_engine(net, record_vm=False, options=dict(trials=T, **opts))
    assert eng.counter('trials') == T and eng.csr_info()['n_edges'] == net.n_edges
    eng.run(net.n_steps)
    assert eng.counter('pipelined') == (0 if mode == 'two_phase' else 1)
    if mode != 'two_phase':
        assert eng.counter('pipeline_trials') == (5 if mode == 'pipelined_one_launch' else 2)
    st, ids = eng.fetch_spikes()
    st, ids = st.astype(np.int64), ids.astype(np.int64)
    n_pad1 = eng.counter('n_pad1')
    trial, cell = ids // n_pad1, ids % n_pad1
    assert cell.max() < net.n_neurons and set(np.unique(trial)) == set(range(T))
    rowptr = eng.csr()[0].astype(np.int64)
    outdeg = np.diff(rowptr)
    n_inputs, events = 0, 0
    trains = []
    for t in range(T):
        steps, srcs = oracle.poisson_spikes(net.poisson_rate_hz, net.dt, net.poisson_seed, 0, net.n_steps, stream=t)
        n_inputs += len(steps)
        m = trial == t
        events += int(outdeg[cell[m]].sum() + outdeg[net.n_neurons + srcs].sum())
        sim = oracle_from_network(net)
        sim.set_input_spikes(steps, srcs)
        r = sim.run(net.n_steps)
        div = _first_divergence(st[m], cell[m], r['spike_step'], r['spike_id'])
        assert div > 300, (t, div)
        a = sorted(zip(cell[m][st[m] <= 1000].tolist(), st[m][st[m] <= 1000].tolist()))
        b = sorted(zip(r['spike_id'][r['spike_step'] <= 1000].tolist(), r['spike_step'][r['spike_step'] <= 1000].tolist()))
        assert len(a) == len(b) and all(x[0] == y[0] and abs(x[1] - y[1]) <= 1 for x, y in zip(a, b))
        trains.append((st[m], cell[m]))
    assert eng.counter('input_spikes') == n_inputs
    assert eng.counter('events') == events
    assert not (len(trains[0][0]) == len(trains[1][0]) and np.array_equal(trains[0][0], trains[1][0]))
    # per-step kernels give the same early spikes as the persistent kernel
    e2 = W.build_engine(net, record_vm=False, options=dict(trials=T, persistent=0))
    e2.run(1200)
    s2, i2 = e2.fetch_spikes()
    m = st <= 1200
    assert _first_divergence(st[m], ids[m], s2.astype(np.int64), i2.astype(np.int64)) > 300
    U = eng.state('U')
    assert U.shape == (T * n_pad1,)


def test_trial_groups_replay_after_an_overflow(cabi):
    """Trial batches stepped two trials per launch with a spike log far too small: the chunk in which the log
    overflowed (in whichever group) starts again from its first step with the log doubled, all groups over; the
    result is, bit for bit, that of a run with ample lists (weights on a 0.25 pA grid)."""
    T = 5
    net = W.c2(n=3000, in_degree=150, n_virtual=150, t_stop_ms=120.0, input_weight=90.0)
    net.weight = (np.round(net.weight * 4.0) / 4.0).astype(np.float32)
    roomy = W.build_engine(net, record_vm=False, options=dict(trials=T, pipeline_trials=2, chunk_steps=500))
    roomy.run(net.n_steps)
    tight = W.build_engine(net, record_vm=False, options=dict(trials=T, pipeline_trials=2, chunk_steps=500, log_capacity=1024))
    tight.run(net.n_steps)
    assert roomy.counter('pipelined') == 1 and tight.counter('pipelined') == 1
    assert roomy.counter('replays') == 0 and tight.counter('replays') >= 1
    a, b = roomy.fetch_spikes(), tight.fetch_spikes()
    assert len(a[0]) > 3000
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    for c in ('events', 'spikes', 'input_spikes', 'steps'):
        assert roomy.counter(c) == tight.counter(c), c
    for var in ('U', 'asc0', 'y1_0', 'refr'):
        assert np.array_equal(roomy.state(var).view(np.uint32), tight.state(var).view(np.uint32)), var
