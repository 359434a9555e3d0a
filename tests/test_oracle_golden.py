"""Pins the CPU oracle: the reference's known-answer vectors, an independent matrix exponential,
Philox known answers, and the CSR construction. No GPU."""
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')


def _known_answers():
    with open(os.path.join(GOLDEN, 'glif_known_answers.json')) as f:
        return json.load(f)


def run_known_answer(case, g, make_sim):
    dt = g['resolution_ms']
    st = g['stimulus']
    stamps = np.ceil(np.array(st['spike_times_ms']) / dt - 1e-9).astype(np.int64)
    return make_sim(case['nest_params'], dt, stamps, st['spike_weight_pA'], int(round(st['delay_ms'] / dt)),
                    st['receptor_type'] - 1, int(round(g['tstop_ms'] / dt)))


@pytest.mark.parametrize('idx', range(5))
def test_known_answer_spikes(oracle, idx):
    """bmtk/tests/simulator/pointnet/test_glif_utils.py:16-44: spike count exact, times atol 1 ms.
    NEST reports step*dt - offset, so the grid stamp must be the first grid point at or after the
    expected time; for the graded model (glif_lif_asc_psc) and for every first spike of the
    non-adapting variants this holds to the step."""
    g = _known_answers()
    case = g['cases'][idx]

    def make_sim(params, dt, stamps, w, d, port, n_steps):
        sim = oracle.OracleSim([params], [0], dt, n_virtual=1, src=[1], trg=[0], weight=[w], delay_steps=[d],
                               port=[port])
        sim.set_input_spikes(stamps - 1, np.zeros(len(stamps), dtype=np.int32))
        return sim.run(n_steps)

    r = run_known_answer(case, g, make_sim)
    t = r['spike_step'] * g['resolution_ms']
    exp = np.array(case['expected_spike_times_ms'])
    assert len(t) == len(exp)
    assert np.allclose(t, exp, atol=g['atol_ms'])
    # first spike: exact grid step for the four variants without voltage-dependent threshold
    if not case['nest_params']['adapting_threshold']:
        assert abs(t[0] - np.ceil(exp[0] / g['resolution_ms']) * g['resolution_ms']) < 1e-9
    else:
        assert abs(t[0] - exp[0]) < 0.005


def test_converted_parameters_match_hand_computed_values():
    """Values the reference converter (glif_utils.py:259-418) yields for the fixtures."""
    g = _known_answers()
    by = {c['model_template']: c['nest_params'] for c in g['cases']}
    p = by['nest:glif_lif_asc_psc']
    assert p['E_L'] == pytest.approx(-71.399902, abs=1e-6)
    assert p['V_reset'] == pytest.approx(-71.399902, abs=1e-6)
    assert p['C_m'] == pytest.approx(85.870098, abs=1e-6)
    assert p['t_ref'] == pytest.approx(6.7)
    assert p['V_th'] == pytest.approx(-48.972984, abs=1e-6)
    assert p['g'] == pytest.approx(2.940785, abs=1e-6)
    assert p['asc_decay'] == pytest.approx([0.03, 0.3])
    assert p['asc_amps'] == pytest.approx([-73.834644, -449.682854], abs=1e-6)
    assert by['nest:glif_lif_psc']['V_th'] == pytest.approx(-47.818993, abs=1e-6)
    assert by['nest:glif_lif_r_asc_a_psc']['V_th'] == pytest.approx(-53.391180, abs=1e-6)


@pytest.mark.parametrize('h', [0.001, 0.05, 0.1, 0.25, 1.0])
@pytest.mark.parametrize('tau_syn', [(5.5, 8.5, 2.8, 5.8), (10.0, 10.0 + 1e-9, 9.999, 2.0)])
def test_propagators_against_matrix_exponential(oracle, h, tau_syn):
    """Exact-integration constants equal expm(A h) of the linear system
    (y1' = -y1/ts, y2' = y1 - y2/ts, U' = -U/tau + y2/C), also next to the tau_syn = tau_m
    singularity (C_m/g = 10 ms here)."""
    from scipy.linalg import expm
    p = dict(C_m=100.0, g=10.0, E_L=-70.0, V_th=-50.0, V_reset=-70.0, V_m=-70.0, t_ref=2.0, tau_syn=tau_syn,
             asc_decay=(0.003, 0.1), asc_amps=(-10.0, -100.0), after_spike_currents=True)
    c = oracle.glif_consts(p, h)
    tau = p['C_m'] / p['g']
    for k, ts in enumerate(tau_syn):
        A = np.array([[-1 / ts, 0, 0], [1, -1 / ts, 0], [0, 1 / p['C_m'], -1 / tau]])
        E = expm(A * h)
        assert c.P11[k] == pytest.approx(E[0, 0], rel=1e-12)
        assert c.P21[k] == pytest.approx(E[1, 0], rel=1e-12)
        assert c.P31[k] == pytest.approx(E[2, 0], rel=1e-9, abs=1e-300)
        assert c.P32[k] == pytest.approx(E[2, 1], rel=1e-9)
        assert c.P33 == pytest.approx(E[2, 2], rel=1e-12)
        assert c.psc_init[k] == pytest.approx(np.e / ts)
    assert c.P30 == pytest.approx(-np.expm1(-h / tau) / p['g'], rel=1e-12)
    for j, kk in enumerate(p['asc_decay']):
        # mean of exp(-k t) over [0, h]
        assert c.asc_stable_coeff[j] == pytest.approx(-np.expm1(-kk * h) / (kk * h), rel=1e-12)
        assert c.asc_refr_rate[j] == pytest.approx(np.exp(-kk * p['t_ref']), rel=1e-12)


def test_refractory_count_follows_double_countdown(oracle):
    """NEST sets a double countdown to t_ref at the spike and subtracts h per step until it is
    <= 0; the count must be that loop's, not round(t_ref/h)."""
    def countdown(t_ref, h):
        r, n = t_ref, 0
        while True:
            r -= h
            n += 1
            if r <= 0.0:
                return n
    for t_ref, h in [(2.0, 0.1), (2.0, 0.25), (6.7, 0.001), (0.05, 0.1), (2.6000000000000005, 0.1), (1.7, 0.05),
                     (3.1, 0.1), (2.3, 0.1)]:
        assert oracle.glif_consts(dict(t_ref=t_ref), h).n_ref == countdown(t_ref, h)
    assert oracle.glif_consts(dict(t_ref=2.0), 0.25).n_ref == 8
    assert oracle.glif_consts(dict(t_ref=0.05), 0.1).n_ref == 1


def test_single_psc_peaks_at_weight(oracle):
    """A spike of weight w makes an alpha PSC that peaks at w pA, tau_syn after arrival
    (glif_psc normalisation e/tau)."""
    dt, tau = 0.01, 5.5
    p = dict(V_th=1e9, tau_syn=(tau,), E_L=-70.0, V_m=-70.0, V_reset=-70.0)
    sim = oracle.OracleSim([p], [0], dt, n_virtual=1, src=[1], trg=[0], weight=[37.0], delay_steps=[100], port=[0])
    sim.set_input_spikes([0], [0])
    peak, at = 0.0, 0
    for n in range(2000):
        sim.run(1)
        if sim.y2[0] > peak:
            peak, at = sim.y2[0], n + 1
    assert peak == pytest.approx(37.0, rel=1e-5)
    # emitted in step 0 (stamp 1), delay 100 -> y1 jumps at the end of step 100 = t 101*dt
    assert at * dt == pytest.approx(101 * dt + tau, abs=2 * dt)


def test_philox_known_answers(oracle):
    """Known-answer vectors of Philox4x32-10 from the Random123 distribution's kat_vectors."""
    assert oracle.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert oracle.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert oracle.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_poisson_thresholds_and_rate(oracle):
    thr = oracle.poisson_thresholds(0.0)
    assert list(thr) == [0xFFFFFFFF] * 4
    lam = 0.004
    thr = oracle.poisson_thresholds(lam)
    assert thr[0] == int(np.floor(np.exp(-lam) * 2 ** 32))
    assert np.all(np.diff(thr.astype(np.int64)) >= 0)
    steps, srcs = oracle.poisson_spikes([16.0] * 50, 0.25, 7, 0, 4000)   # 50 cells, 1 s
    assert len(steps) == pytest.approx(50 * 16, rel=0.15)
    assert np.all(np.diff(steps) >= 0)
    # counter based: the same (source, step) gives the same draw whatever the window asked for
    s2, v2 = oracle.poisson_spikes([16.0] * 50, 0.25, 7, 1000, 500)
    m = (steps >= 1000) & (steps < 1500)
    assert np.array_equal(steps[m], s2) and np.array_equal(srcs[m], v2)


def test_csr_build_orders_rows_by_delay_port_target(oracle):
    rng = np.random.default_rng(0)
    n_rows, E = 37, 5000
    src = rng.integers(0, n_rows, E)
    src[src == 5] = 6                      # an empty row
    trg = rng.integers(0, 20, E)
    d = rng.integers(1, 9, E)
    port = rng.integers(0, 4, E)
    w = rng.normal(size=E)
    rowptr, order = oracle.build_csr(n_rows, src, trg, w, d, port)
    assert rowptr[0] == 0 and rowptr[-1] == E and rowptr[6] == rowptr[5]
    assert sorted(order.tolist()) == list(range(E))
    for r in range(n_rows):
        sl = order[rowptr[r]:rowptr[r + 1]]
        assert np.all(src[sl] == r)
        key = (d[sl] * 4 + port[sl]) * 1000 + trg[sl]
        assert np.all(np.diff(key) >= 0)
        # ties keep edge-list order
        same = np.diff(key) == 0
        assert np.all(np.diff(sl)[same] > 0)


def test_empty_and_input_only_networks(oracle):
    p = dict(tau_syn=(5.5, 8.5, 2.8, 5.8), after_spike_currents=True)
    sim = oracle.OracleSim([p], np.zeros(10, dtype=int), 0.1)
    r = sim.run(100)
    assert r['n_spikes'] == 0 and r['n_events'] == 0
    assert np.allclose(sim.v_m(), -78.85)
    sim = oracle.OracleSim([p], np.zeros(0, dtype=int), 0.1)
    assert sim.run(10)['n_spikes'] == 0


def test_iaf_psc_delta_oracle_against_closed_forms(oracle):
    """iaf_psc_delta restatement: (1) under a constant current the first threshold crossing is the first grid
    point at which E_L + I R (1 - exp(-t/tau)) >= V_th, and the neuron then repeats with period
    crossing + t_ref (reset in the spike step, t_ref/dt refractory steps); (2) a weight arriving through a
    synapse of d steps from a spike emitted in step n is a jump of exactly that many mV in step n + d;
    (3) a jump that arrives while the neuron is refractory is dropped."""
    dt = 0.1
    p = dict(model='iaf_psc_delta', I_e=400.0, tau_m=10.0, C_m=250.0, t_ref=2.0, E_L=-70.0, V_th=-55.0, V_reset=-70.0)
    sim = oracle.OracleSim([p], np.zeros(1, dtype=np.uint16), dt)
    sim.set_probes([0], 1)
    r = sim.run(1000)
    R = p['tau_m'] / p['C_m'] * 1e3          # MOhm * pA = uV -> mV: tau/C in ms/pF = GOhm
    vinf = p['I_e'] * p['tau_m'] / p['C_m']   # mV above E_L
    k = np.arange(1, 2000)
    first = int(k[vinf * (1.0 - np.exp(-k * dt / p['tau_m'])) >= p['V_th'] - p['E_L']][0])
    assert r['spike_step'][0] == first
    period = first + int(round(p['t_ref'] / dt))
    assert np.all(np.diff(r['spike_step']) == period) and len(r['spike_step']) == (1000 - first) // period + 1
    del R
    # (2), (3): one virtual cell -> neuron, weight 3.25 mV, delay 7 steps; no current
    q = dict(p, I_e=0.0)
    sim = oracle.OracleSim([q], np.zeros(1, dtype=np.uint16), dt, n_virtual=1, src=[1], trg=[0], weight=[3.25],
                           delay_steps=[7], port=[2])
    sim.set_probes([0], 1)
    sim.set_input_spikes([10], [0])           # emitted in step 10 -> jump in step 17
    tr = sim.run(40)['trace'][:, 0]
    assert np.all(tr[:17] == -70.0) and tr[17] == -70.0 + 3.25
    assert tr[18] == pytest.approx(-70.0 + 3.25 * np.exp(-dt / 10.0), abs=1e-12)
    big = dict(q)
    sim = oracle.OracleSim([big], np.zeros(1, dtype=np.uint16), dt, n_virtual=1, src=[1], trg=[0], weight=[16.0],
                           delay_steps=[1], port=[0])
    sim.set_probes([0], 1)
    sim.set_input_spikes([5, 10, 40], [0, 0, 0])   # 16 mV > 15 mV: fires in step 6; the jump of step 11 falls in the refractory period
    r = sim.run(60)
    assert r['spike_step'].tolist() == [7, 42]
    assert np.all(r['trace'][6:26, 0] == -70.0)
