"""GPU tests of the pipelined persistent kernel (update and delivery warps side by side).

With weights on a 0.25 pA grid every synaptic sum is exact in fp32 whatever the order of the
reductions, so the per-step kernels, the two-phase persistent kernel and the pipelined kernel
must agree BIT FOR BIT on connected networks: spikes, traces, final state and counters."""
import numpy as np
import pytest

from bmtk_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _grid_weights(net):
    net.weight = (np.round(net.weight * 4.0) / 4.0).astype(np.float32)
    return net


def _run(net, pieces=None, **options):
    eng = W.build_engine(net, options=options)
    for k in (pieces or [net.n_steps]):
        eng.run(k)
    st, ids = eng.fetch_spikes()
    return eng, st.astype(np.int64), ids.astype(np.int64), eng.fetch_trace()


def _same(a, b, state=True):
    assert np.array_equal(a[1], b[1]) and np.array_equal(a[2], b[2])
    assert np.array_equal(a[3].view(np.uint32), b[3].view(np.uint32))
    for c in ('events', 'spikes', 'input_spikes'):
        assert a[0].counter(c) == b[0].counter(c), c
    if state:
        for var in ('U', 'asc0', 'asc1', 'refr'):
            assert np.array_equal(a[0].state(var).view(np.uint32), b[0].state(var).view(np.uint32)), var


def _c3_small(**kw):
    n = 6000
    return W.c3(n=n, n_virtual=400, radius_um=845.0 * np.sqrt(n / 230924.0), t_stop_ms=150.0, **kw)


@pytest.mark.parametrize('poisson', [True, False])
def test_pipelined_equals_other_paths_min_delay_2(cabi, poisson):
    """c3-like network: min delay 2 steps, so a phase is ONE step; Poisson cells drawn in the kernel
    or replayed virtual spikes."""
    net = _grid_weights(_c3_small(poisson_online=poisson))
    a = _run(net, persistent=1, pipeline=1, chunk_steps=250)
    b = _run(net, persistent=1, pipeline=0, chunk_steps=250)
    c = _run(net, persistent=0)
    assert a[0].counter('pipelined') == 1 and b[0].counter('pipelined') == 0
    assert a[0].counter('window') == 2
    assert len(a[1]) > 500 and a[0].counter('events') > 100000
    _same(a, b)
    _same(a, c)


def test_pipelined_phases_of_several_steps_and_split_runs(cabi):
    """c2-like network: min delay 8 steps, a phase is 4 steps; runs cut at odd step counts (partial
    phases, spikes of the last phase delivered before the launch ends) equal one long run."""
    net = _grid_weights(W.c2(n=4000, in_degree=100, n_virtual=100, t_stop_ms=200.0, input_weight=90.0))
    a = _run(net, pipeline=1)
    b = _run(net, persistent=0)
    c = _run(net, pieces=[1, 2, 3, 5, 7, 1001, 333, 648], pipeline=1, chunk_steps=97)
    assert a[0].counter('pipelined') == 1 and a[0].counter('window') == 8
    assert len(a[1]) > 500
    _same(a, b)
    _same(a, c)


def test_pipelined_clamps_and_probes(cabi):
    """Current steps that begin inside a phase cut the phase short; probes sample on their grid."""
    net = W.c1(n=5000, t_stop_ms=160.0)
    a = _run(net, pipeline=1, chunk_steps=901)
    b = _run(net, persistent=0)
    assert a[0].counter('pipelined') == 1
    assert len(a[1]) > 100 and a[3].size > 0
    _same(a, b)
    assert np.array_equal(a[0].state('i_ext').view(np.uint32), b[0].state('i_ext').view(np.uint32))
    # launches that end exactly on the step a current changes (2001 = round(100 ms / dt) + 1): the change
    # must be applied once, by the launch that runs that step
    for kw in (dict(chunk_steps=2001), dict(chunk_steps=4096, pieces=[2001, 1199]), dict(chunk_steps=667)):
        c = _run(net, pipeline=1, **kw)
        _same(c, b)
        assert np.array_equal(c[0].state('i_ext').view(np.uint32), b[0].state('i_ext').view(np.uint32)), kw


def test_pipelined_log_overflow_is_reported_and_reserve_is_harmless(cabi):
    """The spike log of the pipelined kernel lives in per-block segments: a log that is too small is
    reported as an error (nothing traps), and pinning the host store ahead changes no result."""
    from bmtk_b200._cabi import EngineError
    net = _grid_weights(W.c2(n=4000, in_degree=100, n_virtual=100, t_stop_ms=100.0, input_weight=90.0))
    eng = W.build_engine(net, options=dict(pipeline=1, log_capacity=2048, replay_on_overflow=0))
    assert eng.counter('pipelined') == 1
    with pytest.raises(EngineError) as ei:
        eng.run(net.n_steps)
    assert 'spike log full' in str(ei.value)
    a = _run(net, pipeline=1)
    e2 = W.build_engine(net, options=dict(pipeline=1))
    e2.set_option('spike_store_reserve', 5000000)
    e2.run(net.n_steps)
    st, ids = e2.fetch_spikes()
    assert np.array_equal(st.astype(np.int64), a[1]) and np.array_equal(ids.astype(np.int64), a[2])
