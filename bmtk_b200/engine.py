"""Python handle on one engine of the C ABI (one GPU / one rank).

Plays the part PyNEST plays for bmtk.simulator.pointnet: nodes are created per node type, edges
connected one-to-one with weight / delay / receptor arrays, virtual cells replay spike times,
`run` is nest.Simulate, recorders are read back as arrays instead of NEST's .dat files.
"""
import ctypes as C

import numpy as np

from . import _cabi
from ._cabi import GlifParams, check

# NEST's glif_psc defaults for keys a dynamics_params file omits.
GLIF_PSC_DEFAULTS = dict(
    V_m=-78.85, V_th=-51.68, g=9.43, E_L=-78.85, C_m=58.72, t_ref=3.75, V_reset=-78.85,
    asc_init=(0.0, 0.0), asc_decay=(0.003, 0.1), asc_amps=(-9.18, -198.94), asc_r=(1.0, 1.0),
    tau_syn=(2.0,), th_spike_add=0.37, th_spike_decay=0.009, voltage_reset_fraction=0.20,
    voltage_reset_add=18.51, th_voltage_index=0.005, th_voltage_decay=0.09,
    spike_dependent_threshold=False, after_spike_currents=False, adapting_threshold=False, I_e=0.0)

# NEST's iaf_psc_alpha defaults
IAF_PSC_ALPHA_DEFAULTS = dict(V_m=-70.0, E_L=-70.0, C_m=250.0, tau_m=10.0, t_ref=2.0, V_th=-55.0, V_reset=-70.0,
                              tau_syn_ex=2.0, tau_syn_in=2.0, I_e=0.0, V_min=None)


def iaf_psc_alpha_params(d):
    """NEST iaf_psc_alpha parameter dict -> GlifParams with model = iaf_psc_alpha: g = C_m/tau_m,
    receptor ports 0 / 1 carry the excitatory / inhibitory alpha currents."""
    unknown = set(d) - set(IAF_PSC_ALPHA_DEFAULTS)
    if unknown:
        raise ValueError('unknown iaf_psc_alpha parameter(s): %s' % ', '.join(sorted(unknown)))
    q = dict(IAF_PSC_ALPHA_DEFAULTS)
    q.update(d)
    if q['V_min'] is not None and np.isfinite(q['V_min']):
        raise ValueError('iaf_psc_alpha: a finite V_min is not supported')
    p = glif_params(dict(V_m=q['V_m'], E_L=q['E_L'], C_m=q['C_m'], g=q['C_m'] / q['tau_m'], t_ref=q['t_ref'],
                         V_th=q['V_th'], V_reset=q['V_reset'], tau_syn=(q['tau_syn_ex'], q['tau_syn_in']), I_e=q['I_e']))
    p.model = _cabi.MODEL_IAF_PSC_ALPHA
    return p


# NEST's iaf_psc_delta defaults
IAF_PSC_DELTA_DEFAULTS = dict(V_m=-70.0, E_L=-70.0, C_m=250.0, tau_m=10.0, t_ref=2.0, V_th=-55.0, V_reset=-70.0,
                              I_e=0.0, V_min=None, refractory_input=False)


def iaf_psc_delta_params(d):
    """NEST iaf_psc_delta parameter dict -> GlifParams with model = iaf_psc_delta: g = C_m/tau_m, a
    synaptic weight is a jump of V_m in mV, every receptor port adds to the same jump."""
    unknown = set(d) - set(IAF_PSC_DELTA_DEFAULTS)
    if unknown:
        raise ValueError('unknown iaf_psc_delta parameter(s): %s' % ', '.join(sorted(unknown)))
    q = dict(IAF_PSC_DELTA_DEFAULTS)
    q.update(d)
    if q['V_min'] is not None and np.isfinite(q['V_min']):
        raise ValueError('iaf_psc_delta: a finite V_min is not supported')
    if q['refractory_input']:
        raise ValueError('iaf_psc_delta: refractory_input = True is not supported')
    p = glif_params(dict(V_m=q['V_m'], E_L=q['E_L'], C_m=q['C_m'], g=q['C_m'] / q['tau_m'], t_ref=q['t_ref'],
                         V_th=q['V_th'], V_reset=q['V_reset'], tau_syn=(1.0,), I_e=q['I_e']))
    p.model = _cabi.MODEL_IAF_PSC_DELTA
    return p


def glif_params(d):
    """NEST-format glif_psc parameter dict -> GlifParams (unknown keys are rejected). A dict with
    key 'model': 'iaf_psc_alpha' is taken as iaf_psc_alpha parameters."""
    if isinstance(d, GlifParams):
        return d
    if d.get('model') == 'iaf_psc_alpha':
        return iaf_psc_alpha_params({k: v for k, v in d.items() if k != 'model'})
    if d.get('model') == 'iaf_psc_delta':
        return iaf_psc_delta_params({k: v for k, v in d.items() if k != 'model'})
    d = {k: v for k, v in d.items() if k != 'model'}
    unknown = set(d) - set(GLIF_PSC_DEFAULTS)
    if unknown:
        raise ValueError('unknown glif_psc parameter(s): %s' % ', '.join(sorted(unknown)))
    q = dict(GLIF_PSC_DEFAULTS)
    q.update(d)
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
    if not 1 <= len(ts) <= _cabi.MAX_PORTS:
        raise ValueError('tau_syn must have 1..%d entries' % _cabi.MAX_PORTS)
    p.n_ports = len(ts)
    p.tau_syn = (C.c_double * _cabi.MAX_PORTS)(*(ts + [1.0] * (_cabi.MAX_PORTS - len(ts))))
    p.spike_dependent_threshold = int(bool(q['spike_dependent_threshold']))
    p.after_spike_currents = int(bool(q['after_spike_currents']))
    p.adapting_threshold = int(bool(q['adapting_threshold']))
    return p


def _arr(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def time_to_stamp(t_ms, dt):
    """Spike time in ms -> stamp in steps: the first grid point at or after t (spike_generator
    with precise_times, bmtk/simulator/pointnet/pointsimulator.py:69)."""
    t = np.asarray(t_ms, dtype=np.float64)
    return np.ceil(t / dt - 1e-9).astype(np.int64)


class Engine(object):
    def __init__(self, dt, device=0):
        self._lib = _cabi.load()
        self._h = C.c_void_p()
        self.dt = float(dt)
        self.device = int(device)
        check(self._lib.bmtk_engine_create(C.byref(self._h), self.device, self.dt))
        self.n_local = 0
        self.lo = 0
        self.n_probe = 0

    def close(self):
        if getattr(self, '_h', None) is not None and self._h:
            self._lib.bmtk_engine_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- construction
    def set_nodes(self, types, type_index, n_global=None, lo=0):
        ti = _arr(type_index, np.uint16)
        params = (GlifParams * len(types))(*[glif_params(t) for t in types])
        n_local = len(ti)
        n_global = n_local if n_global is None else int(n_global)
        check(self._lib.bmtk_engine_set_nodes(self._h, n_global, int(lo), n_local, _ptr(ti), len(types),
                                              C.cast(params, C.c_void_p)))
        self.n_local, self.lo, self.n_global = n_local, int(lo), n_global

    def set_virtual(self, n_virtual):
        check(self._lib.bmtk_engine_set_virtual(self._h, int(n_virtual)))
        self.n_virtual = int(n_virtual)

    def add_edges(self, src, trg, weight, delay_steps, port):
        src, trg = _arr(src, np.uint32), _arr(trg, np.uint32)
        weight = _arr(weight, np.float32)
        d = np.asarray(delay_steps)
        if d.size and (d.max() > 65535 or d.min() < 0):
            raise ValueError('delay_steps outside 0..65535')
        delay_steps, port = _arr(d, np.uint16), _arr(port, np.uint8)
        n = len(src)
        if not (len(trg) == len(weight) == len(delay_steps) == len(port) == n):
            raise ValueError('edge arrays differ in length')
        check(self._lib.bmtk_engine_add_edges(self._h, n, _ptr(src), _ptr(trg), _ptr(weight), _ptr(delay_steps),
                                              _ptr(port)))

    def set_input_spikes(self, virt_index, stamp_step):
        v, s = _arr(virt_index, np.uint32), _arr(stamp_step, np.uint32)
        if len(v) != len(s):
            raise ValueError('input spike arrays differ in length')
        check(self._lib.bmtk_engine_set_input_spikes(self._h, len(v), _ptr(v), _ptr(s)))

    def set_poisson(self, rate_hz, seed):
        r = _arr(rate_hz, np.float32)
        if len(r) != getattr(self, 'n_virtual', 0):
            raise ValueError('one rate per virtual cell is required')
        check(self._lib.bmtk_engine_set_poisson(self._h, _ptr(r), int(seed)))

    def set_clamp_events(self, step, target, delta_pA):
        s, t, d = _arr(step, np.uint64), _arr(target, np.uint32), _arr(delta_pA, np.float32)
        check(self._lib.bmtk_engine_set_clamp_events(self._h, len(s), _ptr(s), _ptr(t), _ptr(d)))

    def record_spikes(self, enable=True):
        check(self._lib.bmtk_engine_record_spikes(self._h, int(bool(enable))))

    def record_vm(self, ids, interval_steps=1):
        ids = _arr(ids, np.uint32)
        check(self._lib.bmtk_engine_record_vm(self._h, len(ids), _ptr(ids), int(interval_steps)))
        self.n_probe = len(ids)
        self.n_probe_vars = 1

    def record_state(self, ids, interval_steps=1, variables=('V_m',)):
        """Multimeter on `ids` for the named recordables (keys of _cabi.RECORDABLES); fetch_trace then returns
        [samples, variables, ids]."""
        ids = _arr(ids, np.uint32)
        codes = np.array([_cabi.RECORDABLES[v] for v in variables], dtype=np.int32)
        check(self._lib.bmtk_engine_record_state(self._h, len(ids), _ptr(ids), int(interval_steps), len(codes), _ptr(codes)))
        self.n_probe = len(ids)
        self.n_probe_vars = len(codes)

    def set_option(self, key, value):
        check(self._lib.bmtk_engine_set_option(self._h, key.encode(), int(value)))

    def comm_init(self, uid, rank, n_ranks, libnccl=None):
        buf = (C.c_char * 128).from_buffer_copy(bytes(uid)) if uid is not None else None
        check(self._lib.bmtk_engine_comm_init(self._h, buf, int(rank), int(n_ranks),
                                              libnccl.encode() if libnccl else None))

    def local_layout(self):
        """(minimum delay in steps of this rank's edges, neurons of this rank, has clamp changes)."""
        out = np.zeros(4, dtype=np.uint64)
        check(self._lib.bmtk_engine_local_layout(self._h, _ptr(out)))
        return int(out[0]), int(out[1]), bool(out[2])

    def set_global_layout(self, min_delay_steps, max_n_local, any_clamps=False):
        """Network-wide values every rank must pass identically before finalize: the exchange window,
        the spike capacity and the offsets inside the exchange buffers follow from them."""
        a = np.array([int(min_delay_steps), int(max_n_local), int(bool(any_clamps)), 0], dtype=np.uint64)
        check(self._lib.bmtk_engine_set_global_layout(self._h, _ptr(a)))

    def agree_layout(self):
        """Several ranks under torch.distributed: all-reduces the three layout values and sets them."""
        import torch
        import torch.distributed as dist
        d, n, c = self.local_layout()
        dev = torch.device('cuda', self.device) if dist.get_backend() == 'nccl' else torch.device('cpu')
        t = torch.tensor([-min(d, 2 ** 40), n, int(c)], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        self.set_global_layout(int(-t[0].item()), int(t[1].item()), bool(t[2].item()))

    def exchange_layout(self):
        """The 16-word description of this rank's exchange layout (after finalize)."""
        out = np.zeros(16, dtype=np.uint64)
        check(self._lib.bmtk_engine_exchange_layout(self._h, _ptr(out)))
        return out

    def finalize(self):
        check(self._lib.bmtk_engine_finalize(self._h))

    def p2p_handle(self):
        """64-byte handle of this rank's spike-exchange buffer (after finalize, several ranks)."""
        buf = (C.c_char * 64)()
        check(self._lib.bmtk_engine_p2p_handle(self._h, buf))
        return bytes(buf)

    def p2p_connect(self, handles):
        """Maps the exchange buffers of all ranks (list of 64-byte handles in rank order): the stepping
        kernel then exchanges spikes over peer memory instead of NCCL."""
        blob = b''.join(bytes(h) for h in handles)
        buf = (C.c_char * len(blob)).from_buffer_copy(blob)
        check(self._lib.bmtk_engine_p2p_connect(self._h, buf))

    def p2p_buffer(self):
        """Device pointer of this engine's exchange buffer (ranks living in one process)."""
        p = C.c_void_p()
        check(self._lib.bmtk_engine_p2p_buffer(self._h, C.byref(p)))
        return p.value

    def p2p_connect_pointers(self, pointers):
        arr = (C.c_void_p * len(pointers))(*[C.c_void_p(p) for p in pointers])
        check(self._lib.bmtk_engine_p2p_connect_pointers(self._h, arr))

    def connect_peers(self):
        """Exchanges the handles over torch.distributed (any backend) and connects."""
        import torch.distributed as dist
        handles = [None] * dist.get_world_size()
        dist.all_gather_object(handles, self.p2p_handle())
        self.p2p_connect(handles)
        dist.barrier()

    # ---- simulation
    def run(self, n_steps):
        check(self._lib.bmtk_engine_run(self._h, int(n_steps)))

    def fetch_spikes(self):
        """(stamp_step uint32[], id uint32[]) sorted by (stamp, id); drains the store."""
        n = C.c_uint64()
        check(self._lib.bmtk_engine_spike_count(self._h, C.byref(n)))
        st = np.empty(n.value, dtype=np.uint32)
        ids = np.empty(n.value, dtype=np.uint32)
        out = C.c_uint64()
        check(self._lib.bmtk_engine_fetch_spikes(self._h, n.value, _ptr(st), _ptr(ids), C.byref(out)))
        return st[:out.value], ids[:out.value]

    def fetch_trace(self):
        """float32[samples, n_probe] of V_m ([samples, variables, n_probe] after record_state with several
        variables); drains the store."""
        n = C.c_uint64()
        check(self._lib.bmtk_engine_trace_samples(self._h, C.byref(n)))
        nv = getattr(self, 'n_probe_vars', 1)
        tr = np.empty((n.value, nv, self.n_probe), dtype=np.float32)
        out = C.c_uint64()
        check(self._lib.bmtk_engine_fetch_trace(self._h, n.value, _ptr(tr), C.byref(out)))
        return tr[:out.value, 0] if nv == 1 else tr[:out.value]

    def state(self, var):
        """One trial: n_local values. Several trials: n_trials * n_pad1 values, trial-major."""
        t = self.counter('trials')
        out = np.empty(self.n_local if t == 1 else self.counter('n_pad'), dtype=np.float32)
        check(self._lib.bmtk_engine_get_state(self._h, var.encode(), _ptr(out)))
        return out

    def csr_info(self):
        a, b = C.c_uint64(), C.c_uint64()
        c, d, e, f = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        check(self._lib.bmtk_engine_csr_info(self._h, C.byref(a), C.byref(b), C.byref(c), C.byref(d), C.byref(e),
                                             C.byref(f)))
        return dict(n_rows=a.value, n_edges=b.value, target_bits=c.value, max_delay=d.value, min_delay=e.value,
                    ring_slots=f.value)

    def csr(self):
        """(rowptr uint64[n_rows+1], packed uint32[E], weight float32[E])."""
        info = self.csr_info()
        rowptr = np.empty(info['n_rows'] + 1, dtype=np.uint64)
        packed = np.empty(info['n_edges'], dtype=np.uint32)
        weight = np.empty(info['n_edges'], dtype=np.float32)
        check(self._lib.bmtk_engine_get_csr(self._h, _ptr(rowptr), _ptr(packed), _ptr(weight)))
        return rowptr, packed, weight

    def save_state(self, path):
        """Checkpoint: step counter, neuron state and ring buffer."""
        check(self._lib.bmtk_engine_save_state(self._h, str(path).encode()))

    def load_state(self, path):
        """Resume from a checkpoint written for the same network, partition and dt."""
        check(self._lib.bmtk_engine_load_state(self._h, str(path).encode()))

    def p2p_pingpong(self, peer_rank, initiator, rounds=2000):
        """One-way latency (ns) of a tagged 8-byte word between this rank and `peer_rank` over peer memory; both
        ranks call it together, one as initiator."""
        ns = C.c_double()
        check(self._lib.bmtk_engine_p2p_pingpong(self._h, int(peer_rank), int(bool(initiator)), int(rounds), C.byref(ns)))
        return ns.value

    def block_profile(self):
        """uint64[blocks, 4] {producing busy, producing wait, delivering busy, delivering wait} ns per block of the
        pipelined kernel since the last call (option phase_timers); empty when the kernel is not in use."""
        n = C.c_uint64()
        check(self._lib.bmtk_engine_block_profile(self._h, 0, None, C.byref(n)))
        out = np.zeros((n.value * 5 + 40, 4), dtype=np.uint64)
        if n.value:
            check(self._lib.bmtk_engine_block_profile(self._h, n.value * 5 + 40, _ptr(out), C.byref(n)))
        self.update_warp_ns = out[n.value + 40:].reshape(n.value, 16)   # per block and update warp: time to the end of its last step
        self.warp_histograms = out[n.value:n.value + 40].reshape(5, 32)     # bins of 250 ns: update, input, chunk warps at the hand-over; update warps after the step, without / with a spike
        return out[:n.value]

    def mark(self, slot):
        """Records a CUDA event on the engine's stream in slot 0..7."""
        check(self._lib.bmtk_engine_mark(self._h, int(slot)))

    def elapsed_ms(self, from_slot, to_slot):
        """Device time between two marks (waits for the later one)."""
        ms = C.c_double()
        check(self._lib.bmtk_engine_elapsed_ms(self._h, int(from_slot), int(to_slot), C.byref(ms)))
        return ms.value

    def counter(self, name):
        v = C.c_uint64()
        check(self._lib.bmtk_engine_get_counter(self._h, name.encode(), C.byref(v)))
        return v.value


def nccl_unique_id(libnccl=None):
    buf = (C.c_char * 128)()
    check(_cabi.load().bmtk_comm_unique_id(buf, libnccl.encode() if libnccl else None))
    return bytes(buf)


def scatter_reduction_rate(n_cells, n_ops, repeats=5, device=0):
    """Reductions per second the device sustains for one fp32 `red` per op into random cells of a
    buffer of n_cells floats (the ceiling of atomic spike delivery)."""
    ms = C.c_double()
    check(_cabi.load().bmtk_probe_scatter_reductions(int(device), int(n_cells), int(n_ops), int(repeats), C.byref(ms)))
    return n_ops / (ms.value * 1e-3)
