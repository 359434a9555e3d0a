"""ctypes front end of the CPU oracle (test infrastructure, not product).

Wraps oracle/glif_oracle.c, the fp64 restatement of the NEST glif_psc / static_synapse /
spike_generator / step_current_generator behaviour that BMTK PointNet drives through
nest.Simulate (bmtk/simulator/pointnet/pointsimulator.py:166). Also holds the independent
numpy construction of the delay-bucketed CSR (np.lexsort) that the device build is compared
with bit for bit.

Only tests/, __graft_entry__.smoke() and bench.py's cpu-baseline legs may import this module.
"""
import ctypes as C
import hashlib
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, 'libglif_oracle.so')
MAX_PORTS = 4


class GlifParams(C.Structure):
    """NEST glif_psc parameters, fp64 (field order = orc_glif_params)."""
    _fields_ = [
        ('V_m', C.c_double), ('V_th', C.c_double), ('g', C.c_double), ('E_L', C.c_double),
        ('C_m', C.c_double), ('t_ref', C.c_double), ('V_reset', C.c_double),
        ('asc_init', C.c_double * 2), ('asc_decay', C.c_double * 2), ('asc_amps', C.c_double * 2),
        ('asc_r', C.c_double * 2), ('tau_syn', C.c_double * MAX_PORTS),
        ('th_spike_add', C.c_double), ('th_spike_decay', C.c_double),
        ('voltage_reset_fraction', C.c_double), ('voltage_reset_add', C.c_double),
        ('th_voltage_index', C.c_double), ('th_voltage_decay', C.c_double),
        ('n_ports', C.c_int32), ('spike_dependent_threshold', C.c_int32),
        ('after_spike_currents', C.c_int32), ('adapting_threshold', C.c_int32),
        ('I_e', C.c_double), ('model', C.c_int32), ('reserved', C.c_int32),
    ]


class GlifConsts(C.Structure):
    _fields_ = [
        ('P33', C.c_double), ('P30', C.c_double),
        ('P11', C.c_double * MAX_PORTS), ('P21', C.c_double * MAX_PORTS),
        ('P31', C.c_double * MAX_PORTS), ('P32', C.c_double * MAX_PORTS),
        ('psc_init', C.c_double * MAX_PORTS),
        ('asc_decay_rate', C.c_double * 2), ('asc_stable_coeff', C.c_double * 2),
        ('asc_refr_rate', C.c_double * 2), ('asc_amps', C.c_double * 2),
        ('th_inf', C.c_double), ('v_reset', C.c_double),
        ('theta_spike_decay', C.c_double), ('theta_spike_refr_decay', C.c_double),
        ('th_spike_add', C.c_double), ('reset_fraction', C.c_double), ('reset_add', C.c_double),
        ('phi', C.c_double), ('abpara', C.c_double), ('theta_voltage_decay', C.c_double),
        ('G', C.c_double), ('E_L', C.c_double),
        ('n_ref', C.c_int32), ('n_ports', C.c_int32), ('has_theta_spike', C.c_int32),
        ('has_asc', C.c_int32), ('has_theta_voltage', C.c_int32),
        ('I_e', C.c_double), ('iaf', C.c_int32), ('pad', C.c_int32),
    ]


_p = C.c_void_p


class RunArgs(C.Structure):
    _fields_ = [
        ('n_neurons', C.c_int64), ('n_virtual', C.c_int64), ('type_index', _p),
        ('n_types', C.c_int32), ('types', _p),
        ('rowptr', _p), ('target', _p), ('port', _p), ('delay', _p), ('weight', _p),
        ('max_delay', C.c_int32),
        ('in_step_ptr', _p), ('in_src', _p),
        ('n_clamp', C.c_int64), ('ce_step', _p), ('ce_target', _p), ('ce_delta', _p),
        ('dt', C.c_double), ('step0', C.c_int64), ('n_steps', C.c_int64), ('n_threads', C.c_int32),
        ('U', _p), ('asc', _p), ('y1', _p), ('y2', _p), ('th_spike', _p), ('th_voltage', _p),
        ('i_ext', _p), ('ring', _p), ('refr', _p),
        ('spike_cap', C.c_int64), ('n_spikes', _p), ('spike_step', _p), ('spike_id', _p),
        ('n_probe', C.c_int32), ('probe_ids', _p), ('probe_interval', C.c_int32),
        ('trace', _p), ('n_samples', _p), ('n_events', _p),
        ('n_probe_vars', C.c_int32), ('probe_vars', C.c_uint32),
    ]


# NEST's glif_psc defaults for the keys a dynamics_params file may omit.
_DEFAULTS = dict(
    V_m=-78.85, V_th=-51.68, g=9.43, E_L=-78.85, C_m=58.72, t_ref=3.75, V_reset=-78.85,
    asc_init=(0.0, 0.0), asc_decay=(0.003, 0.1), asc_amps=(-9.18, -198.94), asc_r=(1.0, 1.0),
    tau_syn=(2.0,), th_spike_add=0.37, th_spike_decay=0.009, voltage_reset_fraction=0.20,
    voltage_reset_add=18.51, th_voltage_index=0.005, th_voltage_decay=0.09,
    spike_dependent_threshold=False, after_spike_currents=False, adapting_threshold=False, I_e=0.0)

_IAF_DEFAULTS = dict(V_m=-70.0, E_L=-70.0, C_m=250.0, tau_m=10.0, t_ref=2.0, V_th=-55.0, V_reset=-70.0,
                     tau_syn_ex=2.0, tau_syn_in=2.0, I_e=0.0)


def make_params(d):
    """dict with NEST glif_psc key names -> GlifParams; {'model': 'iaf_psc_alpha', ...} with NEST
    iaf_psc_alpha names is mapped to g = C_m/tau_m, tau_syn = (tau_syn_ex, tau_syn_in), model = 1;
    {'model': 'iaf_psc_delta', ...} likewise with model = 2 (no synaptic time constants)."""
    if d.get('model') == 'iaf_psc_alpha':
        q = dict(_IAF_DEFAULTS)
        q.update({k: v for k, v in d.items() if k in _IAF_DEFAULTS})
        p = make_params(dict(V_m=q['V_m'], E_L=q['E_L'], C_m=q['C_m'], g=q['C_m'] / q['tau_m'], t_ref=q['t_ref'],
                             V_th=q['V_th'], V_reset=q['V_reset'], tau_syn=(q['tau_syn_ex'], q['tau_syn_in']),
                             I_e=q['I_e']))
        p.model = 1
        return p
    if d.get('model') == 'iaf_psc_delta':
        q = dict(_IAF_DEFAULTS)
        q.update({k: v for k, v in d.items() if k in _IAF_DEFAULTS})
        p = make_params(dict(V_m=q['V_m'], E_L=q['E_L'], C_m=q['C_m'], g=q['C_m'] / q['tau_m'], t_ref=q['t_ref'],
                             V_th=q['V_th'], V_reset=q['V_reset'], tau_syn=(1.0,), I_e=q['I_e']))
        p.model = 2
        return p
    q = dict(_DEFAULTS)
    q.update({k: v for k, v in d.items() if k in _DEFAULTS})
    p = GlifParams()
    for k in ('V_m', 'V_th', 'g', 'E_L', 'C_m', 't_ref', 'V_reset', 'th_spike_add', 'th_spike_decay',
              'voltage_reset_fraction', 'voltage_reset_add', 'th_voltage_index', 'th_voltage_decay', 'I_e'):
        setattr(p, k, float(q[k]))
    for k in ('asc_init', 'asc_decay', 'asc_amps', 'asc_r'):
        v = [float(x) for x in q[k]]
        if len(v) != 2:
            raise ValueError('%s must have 2 entries' % k)
        setattr(p, k, (C.c_double * 2)(*v))
    ts = [float(x) for x in np.atleast_1d(q['tau_syn'])]
    if not 1 <= len(ts) <= MAX_PORTS:
        raise ValueError('tau_syn must have 1..%d entries' % MAX_PORTS)
    p.n_ports = len(ts)
    p.tau_syn = (C.c_double * MAX_PORTS)(*(ts + [1.0] * (MAX_PORTS - len(ts))))
    p.spike_dependent_threshold = int(bool(q['spike_dependent_threshold']))
    p.after_spike_currents = int(bool(q['after_spike_currents']))
    p.adapting_threshold = int(bool(q['adapting_threshold']))
    return p


def _host_tag():
    """Identifies the CPU the library was compiled for: the recipe uses -march=native, and the built file
    travels with the tree, so a machine with another instruction set must compile its own."""
    try:
        with open('/proc/cpuinfo') as f:
            for line in f:
                if line.startswith('flags'):
                    return hashlib.sha1(line.encode()).hexdigest()
    except OSError:
        pass
    return 'unknown'


def build(force=False):
    """Compile oracle/glif_oracle.c with the recipe in oracle/Makefile (again whenever the source is newer
    or the library was compiled on a CPU with different features)."""
    src = os.path.join(_HERE, 'glif_oracle.c')
    stamp = _LIB_PATH + '.host'
    tag = _host_tag()
    try:
        same_host = open(stamp).read().strip() == tag
    except OSError:
        same_host = False
    if (force or not same_host or not os.path.exists(_LIB_PATH)
            or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(os.path.join(_HERE, 'Makefile')))):
        subprocess.check_call(['make', '-C', _HERE, '-B', 'libglif_oracle.so'],
                              stdout=subprocess.DEVNULL)
        with open(stamp, 'w') as f:
            f.write(tag)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_run.argtypes = [C.POINTER(RunArgs)]
        _lib.orc_run.restype = C.c_int
        _lib.orc_init_state.argtypes = [C.POINTER(RunArgs)]
        _lib.orc_glif_consts_init.argtypes = [C.POINTER(GlifParams), C.c_double, C.POINTER(GlifConsts)]
        _lib.orc_philox4x32_10.argtypes = [C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        _lib.orc_poisson_thresholds.argtypes = [C.c_double, C.POINTER(C.c_uint32)]
        _lib.orc_poisson_count.argtypes = [C.c_uint32, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint32)]
        _lib.orc_poisson_count.restype = C.c_int32
        _lib.orc_poisson_fill.argtypes = [C.c_int64, C.c_void_p, C.c_uint64, C.c_int64, C.c_int64, C.c_int64,
                                          C.c_void_p, C.c_void_p]
        _lib.orc_poisson_fill.restype = C.c_int64
        _lib.orc_poisson_fill_stream.argtypes = [C.c_int64, C.c_void_p, C.c_uint64, C.c_uint32, C.c_int64, C.c_int64,
                                                 C.c_int64, C.c_void_p, C.c_void_p]
        _lib.orc_poisson_fill_stream.restype = C.c_int64
        _lib.orc_csr_by_source.argtypes = [C.c_int64, C.c_int64] + [C.c_void_p] * 10
        _lib.orc_csr_by_source.restype = None
    return _lib


def glif_consts(params, dt):
    c = GlifConsts()
    p = params if isinstance(params, GlifParams) else make_params(params)
    lib().orc_glif_consts_init(C.byref(p), float(dt), C.byref(c))
    return c


def philox4x32_10(ctr, key):
    c = (C.c_uint32 * 4)(*[int(x) & 0xFFFFFFFF for x in ctr])
    k = (C.c_uint32 * 2)(*[int(x) & 0xFFFFFFFF for x in key])
    o = (C.c_uint32 * 4)()
    lib().orc_philox4x32_10(c, k, o)
    return [int(x) for x in o]


def poisson_thresholds(lam):
    o = (C.c_uint32 * 4)()
    lib().orc_poisson_thresholds(float(lam), o)
    return np.array(list(o), dtype=np.uint32)


def poisson_spikes(rates_hz, dt, seed, step0, n_steps, stream=0):
    """Host statement of the on-line Poisson sources: for every step n in [step0, step0+n_steps)
    and every source v, count = poisson_count(v, n, seed, thresholds(rate_v*dt/1000)); a source with
    count k contributes k entries. `stream` is the fourth word of the Philox counter (the trial of a
    trial-batched run; 0 otherwise). Returns (emit_step int64[], source int32[]) ordered by (step, source)."""
    L = lib()
    rates_hz = np.asarray(rates_hz, dtype=np.float64)
    thr = np.ascontiguousarray(np.concatenate([poisson_thresholds(r * dt * 1e-3) for r in rates_hz])
                               if len(rates_hz) else np.zeros(0, dtype=np.uint32), dtype=np.uint32)
    cap = int(rates_hz.sum() * dt * 1e-3 * n_steps * 1.5 + 1000)
    while True:
        steps = np.zeros(cap, dtype=np.int64)
        srcs = np.zeros(cap, dtype=np.int32)
        n = L.orc_poisson_fill_stream(len(rates_hz), _ptr(thr), int(seed), int(stream), int(step0), int(n_steps), cap,
                                      _ptr(steps), _ptr(srcs))
        if n <= cap:
            return steps[:n].copy(), srcs[:n].copy()
        cap = int(n)


def build_csr(n_rows, src, trg, weight, delay_steps, port):
    """Delay-bucketed CSR by source, stated independently with np.lexsort.

    Rows are sources; inside a row entries are ordered by (delay, port, target) and ties keep
    their order of appearance in the edge list (lexsort is stable). Returns
    (rowptr int64[n_rows+1], order int64[E]) where `order` is the permutation of the input edges.
    """
    src = np.asarray(src, dtype=np.int64)
    order = np.lexsort((np.asarray(trg, dtype=np.int64), np.asarray(port, dtype=np.int64),
                        np.asarray(delay_steps, dtype=np.int64), src))
    counts = np.bincount(src, minlength=n_rows).astype(np.int64)
    rowptr = np.zeros(n_rows + 1, dtype=np.int64)
    np.cumsum(counts, out=rowptr[1:])
    return rowptr, order


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class OracleSim:
    """One network + its fp64 state; run() may be called repeatedly (state persists).

    Arguments mirror what the engine's C-ABI takes: `type_index[n]` into `types` (dicts with
    NEST glif_psc keys), an edge list with sources >= n_neurons meaning virtual cells, delays in
    steps (>= 1), 0-based ports, weights in pA (converted to fp64 as given).
    """

    def __init__(self, types, type_index, dt, n_virtual=0, src=None, trg=None, weight=None,
                 delay_steps=None, port=None, n_threads=1, canonical_csr=True):
        self.L = lib()
        self.dt = float(dt)
        self.N = int(len(type_index))
        self.n_virtual = int(n_virtual)
        self.type_index = np.ascontiguousarray(type_index, dtype=np.int32)
        self.types = (GlifParams * len(types))(*[t if isinstance(t, GlifParams) else make_params(t) for t in types])
        self.n_types = len(types)
        n_rows = self.N + self.n_virtual
        if src is None or len(src) == 0:
            src = trg = delay_steps = port = np.zeros(0, dtype=np.int64)
            weight = np.zeros(0, dtype=np.float64)
        delay_steps = np.asarray(delay_steps, dtype=np.int64)
        if delay_steps.size and delay_steps.min() < 1:
            raise ValueError('delay below one step')
        if canonical_csr:
            self.rowptr, order = build_csr(n_rows, src, trg, weight, delay_steps, port)
            self.order = order
            self.target = np.ascontiguousarray(np.asarray(trg)[order], dtype=np.int32)
            self.port = np.ascontiguousarray(np.asarray(port)[order], dtype=np.int32)
            self.delay = np.ascontiguousarray(delay_steps[order], dtype=np.int32)
            self.weight = np.ascontiguousarray(np.asarray(weight)[order], dtype=np.float64)
        else:
            # large networks: stable counting sort by source in C (row order = edge-list order)
            E = len(src)
            s32 = np.ascontiguousarray(src, dtype=np.uint32); t32 = np.ascontiguousarray(trg, dtype=np.uint32)
            w32 = np.ascontiguousarray(weight, dtype=np.float32); d16 = np.ascontiguousarray(delay_steps, dtype=np.uint16)
            p8 = np.ascontiguousarray(port, dtype=np.uint8)
            self.rowptr = np.zeros(n_rows + 1, dtype=np.int64)
            self.target = np.zeros(E, dtype=np.int32); self.port = np.zeros(E, dtype=np.int32)
            self.delay = np.zeros(E, dtype=np.int32); self.weight = np.zeros(E, dtype=np.float64)
            self.L.orc_csr_by_source(n_rows, E, _ptr(s32), _ptr(t32), _ptr(w32), _ptr(d16), _ptr(p8), _ptr(self.rowptr),
                                     _ptr(self.target), _ptr(self.port), _ptr(self.delay), _ptr(self.weight))
            self.order = None
        self.max_delay = int(self.delay.max()) if self.delay.size else 1
        N, S = self.N, self.max_delay + 1
        self.U = np.zeros(N); self.asc = np.zeros(2 * N)
        self.y1 = np.zeros(MAX_PORTS * N); self.y2 = np.zeros(MAX_PORTS * N)
        self.th_spike = np.zeros(N); self.th_voltage = np.zeros(N); self.i_ext = np.zeros(N)
        self.ring = np.zeros(S * MAX_PORTS * N); self.refr = np.zeros(N, dtype=np.int32)
        self.step = 0
        self.n_threads = int(n_threads)
        self.in_step = np.zeros(0, dtype=np.int64); self.in_src = np.zeros(0, dtype=np.int32)
        self.ce_step = np.zeros(0, dtype=np.int64); self.ce_target = np.zeros(0, dtype=np.int32)
        self.ce_delta = np.zeros(0, dtype=np.float64)
        self.probe_ids = np.zeros(0, dtype=np.int32); self.probe_interval = 1
        self.probe_vars = [0]
        self.n_events = np.zeros(1, dtype=np.int64)
        a = self._args(0)
        self.L.orc_init_state(C.byref(a))

    def set_input_spikes(self, emit_step, virt_index):
        """Virtual spikes as (emitting step = stamp-1, virtual index 0..n_virtual-1)."""
        emit_step = np.asarray(emit_step, dtype=np.int64)
        o = np.lexsort((np.asarray(virt_index), emit_step))
        self.in_step = np.ascontiguousarray(emit_step[o])
        self.in_src = np.ascontiguousarray(np.asarray(virt_index)[o], dtype=np.int32)

    def set_clamp_events(self, step, target, delta):
        step = np.asarray(step, dtype=np.int64)
        o = np.argsort(step, kind='stable')
        self.ce_step = np.ascontiguousarray(step[o])
        self.ce_target = np.ascontiguousarray(np.asarray(target)[o], dtype=np.int32)
        self.ce_delta = np.ascontiguousarray(np.asarray(delta)[o], dtype=np.float64)

    def set_probes(self, ids, interval_steps=1, variables=None):
        """Recorded cells; `variables` are recorder codes (0 V_m, 1 I_syn, 2 ASCurrents_sum, 3 threshold,
        4 threshold_spike, 5 threshold_voltage, 6 I). With more than one the trace is [sample, variable, cell]."""
        self.probe_ids = np.ascontiguousarray(ids, dtype=np.int32)
        self.probe_interval = int(interval_steps)
        self.probe_vars = [int(v) for v in (variables or [0])]

    def _args(self, n_steps):
        a = RunArgs()
        a.n_neurons = self.N; a.n_virtual = self.n_virtual
        a.type_index = _ptr(self.type_index); a.n_types = self.n_types
        a.types = C.cast(self.types, C.c_void_p)
        a.rowptr = _ptr(self.rowptr); a.target = _ptr(self.target); a.port = _ptr(self.port)
        a.delay = _ptr(self.delay); a.weight = _ptr(self.weight); a.max_delay = self.max_delay
        a.dt = self.dt; a.step0 = self.step; a.n_steps = n_steps; a.n_threads = self.n_threads
        a.U = _ptr(self.U); a.asc = _ptr(self.asc); a.y1 = _ptr(self.y1); a.y2 = _ptr(self.y2)
        a.th_spike = _ptr(self.th_spike); a.th_voltage = _ptr(self.th_voltage)
        a.i_ext = _ptr(self.i_ext); a.ring = _ptr(self.ring); a.refr = _ptr(self.refr)
        return a

    def run(self, n_steps, spike_cap=None, record_spikes=True):
        """Advance n_steps. Returns dict(spike_step, spike_id, trace, n_spikes, n_events)."""
        n_steps = int(n_steps)
        a = self._args(n_steps)
        end = self.step + n_steps
        # per-step pointer into the replayed virtual spikes
        self._in_ptr = np.searchsorted(self.in_step, np.arange(end + 1), side='left').astype(np.int64)
        a.in_step_ptr = _ptr(self._in_ptr) if self.in_step.size else None
        a.in_src = _ptr(self.in_src)
        a.n_clamp = len(self.ce_step); a.ce_step = _ptr(self.ce_step)
        a.ce_target = _ptr(self.ce_target); a.ce_delta = _ptr(self.ce_delta)
        if spike_cap is None:
            spike_cap = max(1024, self.N * 64)
        n_spikes = np.zeros(1, dtype=np.int64)
        sp_step = np.zeros(spike_cap if record_spikes else 1, dtype=np.int64)
        sp_id = np.zeros(spike_cap if record_spikes else 1, dtype=np.int32)
        a.spike_cap = spike_cap; a.n_spikes = _ptr(n_spikes)
        a.spike_step = _ptr(sp_step) if record_spikes else None
        a.spike_id = _ptr(sp_id)
        n_samp_max = n_steps // max(1, self.probe_interval) + 1
        nv = len(self.probe_vars)
        trace = np.zeros((n_samp_max, nv, max(1, len(self.probe_ids))))
        a.n_probe_vars = nv
        a.probe_vars = sum(v << (4 * k) for k, v in enumerate(self.probe_vars))
        n_samples = np.zeros(1, dtype=np.int64)
        a.n_probe = len(self.probe_ids); a.probe_ids = _ptr(self.probe_ids)
        a.probe_interval = self.probe_interval; a.trace = _ptr(trace); a.n_samples = _ptr(n_samples)
        ev0 = int(self.n_events[0])
        a.n_events = _ptr(self.n_events)
        rc = self.L.orc_run(C.byref(a))
        if rc < 0:
            raise MemoryError('oracle allocation failed')
        if rc == 1:
            raise RuntimeError('oracle spike log full (cap %d)' % spike_cap)
        self.step = end
        k = int(n_spikes[0]) if record_spikes else 0
        return dict(spike_step=sp_step[:k].copy(), spike_id=sp_id[:k].copy(),
                    trace=(trace[:int(n_samples[0]), 0, :len(self.probe_ids)] if nv == 1
                           else trace[:int(n_samples[0]), :, :len(self.probe_ids)]).copy(),
                    n_spikes=int(n_spikes[0]), n_events=int(self.n_events[0]) - ev0)

    def v_m(self):
        e_l = np.array([t.E_L for t in self.types])
        return self.U + e_l[self.type_index]


def generate_distance_edges(spec, lo=0, hi=None):
    """CPU restatement of the device-side network generator: the edges into targets [lo, hi) of the specification
    made by bmtk_b200.generator.distance_spec, as (src, trg, weight, delay_steps, port)."""
    from bmtk_b200.generator import GenSpec, as_struct
    L = lib()
    L.orc_generate_distance_edges.restype = C.c_int64
    L.orc_generate_distance_edges.argtypes = [C.c_void_p, C.c_int64] + [C.c_void_p] * 5
    hi = spec['n_neurons'] if hi is None else hi
    s = as_struct(spec, lo, hi, GenSpec)          # orc_gen_spec has the same layout
    n = L.orc_generate_distance_edges(C.byref(s), 0, None, None, None, None, None)
    src, trg = np.empty(n, dtype=np.uint32), np.empty(n, dtype=np.uint32)
    w, d, p = np.empty(n, dtype=np.float32), np.empty(n, dtype=np.uint16), np.empty(n, dtype=np.uint8)
    m = L.orc_generate_distance_edges(C.byref(s), n, _ptr(src), _ptr(trg), _ptr(w), _ptr(d), _ptr(p))
    assert m == n
    return src, trg, w, d, p


class RunArgsF32(C.Structure):
    _fields_ = [
        ('n_neurons', C.c_int64), ('n_virtual', C.c_int64), ('type_index', _p), ('n_types', C.c_int32), ('types', _p),
        ('rowptr', _p), ('target', _p), ('port', _p), ('delay', _p), ('weight', _p),
        ('max_delay', C.c_int32), ('window', C.c_int32), ('theta_any', C.c_int32), ('chunk_steps', C.c_int64),
        ('in_step_ptr', _p), ('in_src', _p), ('poisson_rate_hz', _p), ('poisson_seed', C.c_uint64),
        ('poisson_stream', C.c_uint32),
        ('n_clamp', C.c_int64), ('ce_step', _p), ('ce_target', _p), ('ce_delta', _p),
        ('dt', C.c_double), ('step0', C.c_int64), ('n_steps', C.c_int64),
        ('U', _p), ('asc0', _p), ('asc1', _p), ('y1', _p), ('y2', _p), ('th_spike', _p), ('th_voltage', _p),
        ('i_ext', _p), ('ring', _p), ('refr', _p),
        ('spike_cap', C.c_int64), ('n_spikes', _p), ('spike_step', _p), ('spike_id', _p),
        ('n_probe', C.c_int32), ('probe_ids', _p), ('probe_interval', C.c_int32), ('n_probe_vars', C.c_int32),
        ('probe_vars', C.c_uint32), ('trace', _p), ('n_samples', _p), ('n_events', _p),
    ]


class OracleSimF32:
    """The engine's single-precision arithmetic with deterministic delivery, restated on the CPU (orc_f32_run):
    what the CUDA path must reproduce BIT FOR BIT in deterministic mode. `window` and `chunk_steps` are the
    engine's exchange window and chunk length (they fix which weights are added before they reach a ring cell)."""

    def __init__(self, types, type_index, dt, window, chunk_steps=4096, n_virtual=0, src=None, trg=None, weight=None,
                 delay_steps=None, port=None):
        self.L = lib()
        self.L.orc_f32_run.argtypes = [C.POINTER(RunArgsF32)]
        self.L.orc_f32_run.restype = C.c_int
        self.L.orc_f32_init_state.argtypes = [C.POINTER(RunArgsF32)]
        self.dt, self.N, self.n_virtual = float(dt), int(len(type_index)), int(n_virtual)
        self.window, self.chunk_steps = int(window), int(chunk_steps)
        self.type_index = np.ascontiguousarray(type_index, dtype=np.int32)
        plist = [t if isinstance(t, GlifParams) else make_params(t) for t in types]
        self.types = (GlifParams * len(plist))(*plist)
        self.n_types = len(plist)
        self.theta_any = int(any(p.spike_dependent_threshold or p.adapting_threshold for p in plist))
        n_rows = self.N + self.n_virtual
        if src is None or len(src) == 0:
            src = trg = delay_steps = port = np.zeros(0, dtype=np.int64)
            weight = np.zeros(0, dtype=np.float32)
        delay_steps = np.asarray(delay_steps, dtype=np.int64)
        self.rowptr, order = build_csr(n_rows, src, trg, weight, delay_steps, port)
        self.target = np.ascontiguousarray(np.asarray(trg)[order], dtype=np.int32)
        self.port = np.ascontiguousarray(np.asarray(port)[order], dtype=np.int32)
        self.delay = np.ascontiguousarray(delay_steps[order], dtype=np.int32)
        self.weight = np.ascontiguousarray(np.asarray(weight)[order], dtype=np.float32)
        self.max_delay = int(self.delay.max()) if self.delay.size else 1
        N, S = self.N, self.max_delay + self.window
        f = lambda n: np.zeros(n, dtype=np.float32)
        self.U, self.asc0, self.asc1 = f(N), f(N), f(N)
        self.y1, self.y2 = f(MAX_PORTS * N), f(MAX_PORTS * N)
        self.th_spike, self.th_voltage, self.i_ext = f(N), f(N), f(N)
        self.ring = f(S * MAX_PORTS * N)
        self.refr = np.zeros(N, dtype=np.int32)
        self.step = 0
        self.in_step = np.zeros(0, dtype=np.int64); self.in_src = np.zeros(0, dtype=np.int32)
        self.poisson = None
        self.ce_step = np.zeros(0, dtype=np.int64); self.ce_target = np.zeros(0, dtype=np.int32)
        self.ce_delta = np.zeros(0, dtype=np.float32)
        self.probe_ids = np.zeros(0, dtype=np.int32); self.probe_interval = 1; self.probe_vars = [0]
        self.n_events = np.zeros(1, dtype=np.int64)
        self.L.orc_f32_init_state(C.byref(self._args(0)))

    def set_input_spikes(self, emit_step, virt_index):
        emit_step = np.asarray(emit_step, dtype=np.int64)
        o = np.lexsort((np.asarray(virt_index), emit_step))
        self.in_step = np.ascontiguousarray(emit_step[o])
        self.in_src = np.ascontiguousarray(np.asarray(virt_index)[o], dtype=np.int32)

    def set_poisson(self, rate_hz, seed, stream=0):
        self.poisson = (np.ascontiguousarray(rate_hz, dtype=np.float32), int(seed), int(stream))

    def set_clamp_events(self, step, target, delta):
        step = np.asarray(step, dtype=np.int64)
        o = np.argsort(step, kind='stable')
        self.ce_step = np.ascontiguousarray(step[o])
        self.ce_target = np.ascontiguousarray(np.asarray(target)[o], dtype=np.int32)
        self.ce_delta = np.ascontiguousarray(np.asarray(delta)[o], dtype=np.float32)

    def set_probes(self, ids, interval_steps=1, variables=None):
        self.probe_ids = np.ascontiguousarray(ids, dtype=np.int32)
        self.probe_interval = int(interval_steps)
        self.probe_vars = [int(v) for v in (variables or [0])]

    def _args(self, n_steps):
        a = RunArgsF32()
        a.n_neurons, a.n_virtual = self.N, self.n_virtual
        a.type_index, a.n_types, a.types = _ptr(self.type_index), self.n_types, C.cast(self.types, C.c_void_p)
        a.rowptr, a.target, a.port, a.delay, a.weight = (_ptr(self.rowptr), _ptr(self.target), _ptr(self.port),
                                                         _ptr(self.delay), _ptr(self.weight))
        a.max_delay, a.window, a.theta_any, a.chunk_steps = self.max_delay, self.window, self.theta_any, self.chunk_steps
        a.dt, a.step0, a.n_steps = self.dt, self.step, n_steps
        for k in ('U', 'asc0', 'asc1', 'y1', 'y2', 'th_spike', 'th_voltage', 'i_ext', 'ring', 'refr'):
            setattr(a, k, _ptr(getattr(self, k)))
        return a

    def run(self, n_steps, spike_cap=None):
        n_steps = int(n_steps)
        a = self._args(n_steps)
        end = self.step + n_steps
        self._in_ptr = np.searchsorted(self.in_step, np.arange(end + 1), side='left').astype(np.int64)
        a.in_step_ptr = _ptr(self._in_ptr) if self.in_step.size else None
        a.in_src = _ptr(self.in_src)
        if self.poisson is not None:
            a.poisson_rate_hz, a.poisson_seed, a.poisson_stream = _ptr(self.poisson[0]), self.poisson[1], self.poisson[2]
        a.n_clamp = len(self.ce_step)
        a.ce_step, a.ce_target, a.ce_delta = _ptr(self.ce_step), _ptr(self.ce_target), _ptr(self.ce_delta)
        spike_cap = max(1024, self.N * 64) if spike_cap is None else int(spike_cap)
        n_spikes = np.zeros(1, dtype=np.int64)
        sp_step, sp_id = np.zeros(spike_cap, dtype=np.int64), np.zeros(spike_cap, dtype=np.int32)
        a.spike_cap, a.n_spikes, a.spike_step, a.spike_id = spike_cap, _ptr(n_spikes), _ptr(sp_step), _ptr(sp_id)
        nv = len(self.probe_vars)
        trace = np.zeros((n_steps // max(1, self.probe_interval) + 1, nv, max(1, len(self.probe_ids))), dtype=np.float32)
        n_samples = np.zeros(1, dtype=np.int64)
        a.n_probe, a.probe_ids, a.probe_interval = len(self.probe_ids), _ptr(self.probe_ids), self.probe_interval
        a.n_probe_vars, a.probe_vars = nv, sum(v << (4 * k) for k, v in enumerate(self.probe_vars))
        a.trace, a.n_samples = _ptr(trace), _ptr(n_samples)
        ev0 = int(self.n_events[0])
        a.n_events = _ptr(self.n_events)
        rc = self.L.orc_f32_run(C.byref(a))
        if rc < 0:
            raise MemoryError('oracle allocation failed')
        if rc == 1:
            raise RuntimeError('oracle spike log full (cap %d)' % spike_cap)
        self.step = end
        k = int(n_spikes[0])
        tr = trace[:int(n_samples[0]), :, :len(self.probe_ids)]
        return dict(spike_step=sp_step[:k].copy(), spike_id=sp_id[:k].copy(), trace=(tr[:, 0] if nv == 1 else tr).copy(),
                    n_spikes=k, n_events=int(self.n_events[0]) - ev0)
