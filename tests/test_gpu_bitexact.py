"""Bit-level comparison of the CUDA path with the CPU restatement of its own single-precision arithmetic.

The fp64 oracle is the reference for results (tests/test_gpu_parity.py, tests/test_gpu_fullsize_parity.py, within the
stated tolerances). These tests pin the device arithmetic itself: one neuron step is a fixed sequence of IEEE-754
single-precision operations (bmtk_b200/csrc/glif_math.cuh), and deterministic delivery adds the weights that meet in
a ring cell in a fixed order, so oracle/glif_oracle.c:orc_f32_run - plain C with fmaf() - must give the SAME BITS:
every spike (step and id), every trace sample, the final state. Where no synaptic sum depends on an order (no
synapses, or weights on a 0.25 pA grid) the default pipelined kernel with atomic delivery must give them too."""
import os

import numpy as np
import pytest

from bmtk_b200 import workloads as W
from netutil import oracle_f32_from_network

pytestmark = pytest.mark.gpu


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _compare(net, eng, r, sim, state=True):
    st, ids = eng.fetch_spikes()
    assert len(r['spike_step']) > 100
    assert np.array_equal(st.astype(np.int64), r['spike_step']) and np.array_equal(ids.astype(np.int64), r['spike_id'])
    if len(net.probe_ids):
        assert np.array_equal(_bits(eng.fetch_trace()), _bits(r['trace']))
    assert eng.counter('events') == r['n_events'] and eng.counter('spikes') == r['n_spikes']
    if state:
        n = net.n_neurons
        for var, ref in (('U', sim.U), ('asc0', sim.asc0), ('asc1', sim.asc1), ('y1_0', sim.y1[:n]), ('y2_3', sim.y2[3 * n:4 * n]),
                         ('th_spike', sim.th_spike), ('th_voltage', sim.th_voltage)):
            assert np.array_equal(_bits(eng.state(var)), _bits(ref)), var
        assert np.array_equal(eng.state('refr').astype(np.int32), sim.refr)


@pytest.mark.parametrize('poisson', [False, True])
def test_c0_whole_run_deterministic_delivery(cabi, oracle, poisson):
    """450 neurons, 3000 ms (30 000 steps), replayed or on-line Poisson input: ~7000 spikes, every bit."""
    net = W.c0(poisson_online=poisson)
    eng = W.build_engine(net, deterministic=True)
    eng.run(net.n_steps)
    sim = oracle_f32_from_network(net, eng.counter('window'))
    r = sim.run(net.n_steps)
    assert len(r['spike_step']) > 5000
    _compare(net, eng, r, sim)


def test_c1_full_size_every_spike_time(cabi, oracle):
    """The current-clamp sweep at its configured size (10 000 neurons, dt 0.05 ms, 1500 ms): no synapses, so the
    default pipelined kernel and the deterministic per-step path must both reproduce all ~80 000 spike times."""
    net = W.c1()
    sim = oracle_f32_from_network(net, 32)
    r = sim.run(net.n_steps, spike_cap=net.n_neurons * 400)
    assert len(r['spike_step']) > 50000
    for det in (False, True):
        eng = W.build_engine(net, deterministic=det)
        assert det or eng.counter('pipelined') == 1
        eng.run(net.n_steps)
        _compare(net, eng, r, sim)


def test_c2_reduced_and_split_runs(cabi, oracle):
    """E/I network (5000 neurons, in-degree 200, window 8, Poisson cells), 200 ms, deterministic delivery; run in one
    piece and in pieces (a piece ends a window early, which the restatement follows through chunk_steps)."""
    net = W.c2(n=5000, in_degree=200, n_virtual=200, t_stop_ms=200.0, input_weight=90.0)
    eng = W.build_engine(net, deterministic=True, options=dict(chunk_steps=500))
    eng.run(net.n_steps)
    sim = oracle_f32_from_network(net, eng.counter('window'), 500)
    r = sim.run(net.n_steps)
    assert len(r['spike_step']) > 1500
    _compare(net, eng, r, sim)


def test_threshold_dynamics_iaf_and_delta_cells(cabi, oracle):
    """All model variants in one network: glif_psc with spike-dependent and adapting thresholds, iaf_psc_alpha and
    iaf_psc_delta cells, current steps, replayed input."""
    rng = np.random.default_rng(41)
    n, nv = 500, 50
    net = W.Network('mixed', 0.1, 4000)
    g = W._glif3_type(np.random.default_rng(1), False)
    net.types = [g,
                 dict(g, spike_dependent_threshold=True, th_spike_add=0.5, th_spike_decay=0.01, voltage_reset_fraction=0.3, voltage_reset_add=3.0),
                 dict(g, spike_dependent_threshold=True, adapting_threshold=True, th_spike_add=0.4, th_spike_decay=0.02,
                      voltage_reset_fraction=0.2, voltage_reset_add=2.0, th_voltage_index=0.004, th_voltage_decay=0.08),
                 dict(model='iaf_psc_alpha', I_e=100.0, tau_m=12.0, C_m=100.0, t_ref=2.0, E_L=-70.0, V_th=-50.0, V_reset=-65.0),
                 dict(model='iaf_psc_delta', I_e=300.0, tau_m=10.0, C_m=250.0, t_ref=1.5)]
    net.type_names = ['lif_asc', 'lif_r_asc', 'lif_r_asc_a', 'iaf_alpha', 'iaf_delta']
    net.type_is_inh = np.zeros(5, dtype=bool)
    net.type_index = np.repeat(np.arange(5), n // 5).astype(np.uint16)
    net.lo, net.hi = 0, n
    net.n_virtual = nv
    k = 20000
    net.src = rng.integers(0, n + nv, k).astype(np.uint32)
    net.trg = rng.integers(0, n, k).astype(np.uint32)
    is_delta = net.type_index[net.trg] == 4
    net.weight = np.where(is_delta, rng.normal(0.3, 0.8, k), rng.normal(20.0, 40.0, k)).astype(np.float32)
    is_alpha = net.type_index[net.trg] == 3
    net.port = np.where(is_alpha, (net.weight < 0).astype(np.uint8), np.where(is_delta, 0, rng.integers(0, 4, k))).astype(np.uint8)
    net.delay_steps = rng.integers(3, 25, k).astype(np.uint16)
    net.in_virt, net.in_stamp = W._poisson_trains(np.random.default_rng(42), np.full(nv, 50.0), 400.0, net.dt)
    ids = np.arange(n, dtype=np.uint32)
    amp = rng.uniform(50.0, 250.0, n).astype(np.float32)
    net.clamp_step = np.concatenate([np.full(n, 501), np.full(n, 3001)]).astype(np.uint64)
    net.clamp_target = np.concatenate([ids, ids])
    net.clamp_delta = np.concatenate([amp, -amp])
    net.probe_ids = np.array([0, 99, 100, 199, 200, 299, 300, 399, 400, 499], dtype=np.uint32)
    eng = W.build_engine(net, deterministic=True)
    eng.run(net.n_steps)
    sim = oracle_f32_from_network(net, eng.counter('window'))
    r = sim.run(net.n_steps)
    for t in range(5):
        assert np.count_nonzero(net.type_index[r['spike_id']] == t) > 20, t     # every variant fires
    _compare(net, eng, r, sim)
    # the same network with weights on a 1/64 grid (sums exact in any order): the threshold, clamp and probe code of
    # the pipelined kernel in both block sizes, scalar and packed arithmetic, and of the two-phase kernel
    net.weight = (np.round(net.weight * 64.0) / 64.0).astype(np.float32)
    sim = oracle_f32_from_network(net, eng.counter('window'))
    r = sim.run(net.n_steps)
    for opts in (dict(), dict(pipeline_warps=20), dict(pipeline_warps=20, tune=2), dict(tune=1), dict(pipeline=0)):
        eng = W.build_engine(net, options=opts)
        eng.run(net.n_steps)
        assert eng.counter('pipelined') == (0 if 'pipeline' in opts else 1)
        _compare(net, eng, r, sim)


def test_grid_weights_make_the_atomic_kernels_exact_too(cabi, oracle):
    """Weights that are multiples of 0.25 pA add exactly in any order: the pipelined kernel and the two-phase kernel
    (atomic delivery) then reproduce the restatement as well, on the c3-like network with its 2-step windows."""
    n = 6000
    net = W.c3(n=n, n_virtual=400, radius_um=845.0 * np.sqrt(n / 230924.0), t_stop_ms=150.0)
    net.weight = (np.round(net.weight * 4.0) / 4.0).astype(np.float32)
    sim = oracle_f32_from_network(net, 2)
    r = sim.run(net.n_steps)
    # default: the 12-warp block with packed arithmetic; then the 20-warp block (scalar arithmetic, what the full-size
    # network runs), each block size with the other arithmetic, and the two-phase kernel
    for opts in (dict(), dict(pipeline_warps=20), dict(pipeline_warps=20, tune=2), dict(pipeline_warps=12, tune=1), dict(pipeline=0)):
        eng = W.build_engine(net, options=opts)
        eng.run(net.n_steps)
        _compare(net, eng, r, sim)


def test_phases_of_four_steps_with_staged_ring_cells(cabi, oracle):
    """E/I network with minimum delay 8 steps: the pipelined kernel runs phases of 4 steps and copies the ring cells of
    the next step to shared memory while a step computes (option ring_stage). Weights on the 0.25 pA grid: with and
    without the staging, and in the two-phase kernel, every bit must be the restatement's."""
    net = W.c2(n=5000, in_degree=200, n_virtual=200, t_stop_ms=200.0, input_weight=90.0)
    net.weight = (np.round(net.weight * 4.0) / 4.0).astype(np.float32)
    sim = oracle_f32_from_network(net, 8, 700)
    r = sim.run(net.n_steps)
    assert len(r['spike_step']) > 1500
    for opts in (dict(), dict(ring_stage=0), dict(pipeline_warps=20), dict(pipeline=0)):
        eng = W.build_engine(net, options=dict(chunk_steps=700, **opts))
        assert eng.counter('window') == 8
        eng.run(net.n_steps)
        assert eng.counter('pipelined') == (0 if 'pipeline' in opts else 1)
        _compare(net, eng, r, sim)


@pytest.mark.parametrize('per_launch', [0, 2])
def test_trial_batches_every_trial_every_bit(cabi, oracle, per_launch):
    """Three trials over one CSR in the pipelined kernel - all in one launch, or two per launch and then the third -
    with weights on the 0.25 pA grid: each trial must be, bit for bit, the restatement's run of that trial's Poisson
    stream (spikes, events, final membrane state)."""
    T = 3
    net = W.c2(n=4000, in_degree=150, n_virtual=200, t_stop_ms=150.0, input_weight=90.0)
    net.weight = (np.round(net.weight * 4.0) / 4.0).astype(np.float32)
    eng = W.build_engine(net, record_vm=False, options=dict(trials=T, pipeline_trials=per_launch, chunk_steps=700))
    eng.run(net.n_steps)
    assert eng.counter('pipelined') == 1 and eng.counter('pipeline_trials') == (per_launch or T)
    st, ids = eng.fetch_spikes()
    st, ids = st.astype(np.int64), ids.astype(np.int64)
    n_pad1, n = eng.counter('n_pad1'), net.n_neurons
    U = eng.state('U')
    events = 0
    for t in range(T):
        sim = oracle_f32_from_network(net, 8, 700)
        sim.set_poisson(net.poisson_rate_hz, net.poisson_seed, stream=t)
        r = sim.run(net.n_steps)
        assert len(r['spike_step']) > 500
        m = ids // n_pad1 == t
        assert np.array_equal(st[m], r['spike_step']) and np.array_equal(ids[m] - t * n_pad1, r['spike_id']), t
        assert np.array_equal(_bits(U[t * n_pad1:t * n_pad1 + n]), _bits(sim.U)), t
        events += r['n_events']
    assert eng.counter('events') == events
