"""`nest` stand-in for the verification shim (test infrastructure).

Implements the PyNEST names bmtk.simulator.pointnet calls, with NEST 3 conventions (the reference
switches on nest.__version__, bmtk/simulator/pointnet/nest_utils.py:36-54): Create returns a
NodeCollection, recorders write ascii `<label>-<id>-<rank>.dat` files with `#` comment lines and a
`sender<TAB>time_ms[<TAB>variable]` header (read back by modules/record_spikes.py:76-82 and
modules/multimeter_reporter.py:53-56).

Every call is recorded in `calls` (tests compare them with what bmtk_b200.pointnet derives from the
same files). Simulate() turns the recorded network into one engine of the bmtk_b200.engine.Engine
API made by `_engine_factory(dt)`, runs it, and writes the recorder files.
"""
import os

import numpy as np

__version__ = 'nest-3.3'
NEURON_MODELS = ('glif_psc', 'iaf_psc_alpha', 'iaf_psc_delta')
_engine_factory = None


def version():
    return __version__


class NodeCollection(object):
    def __init__(self, ids):
        self._ids = [int(i) for i in ids]

    def tolist(self):
        return list(self._ids)

    def __iter__(self):
        return iter(NodeCollection([i]) for i in self._ids)

    def __len__(self):
        return len(self._ids)

    def __getitem__(self, k):
        r = self._ids[k]
        return NodeCollection(r if isinstance(r, list) else [r])

    def __add__(self, other):
        return NodeCollection(self._ids + _ids_of(other))

    def get(self, key=None):
        vals = [_K.nodes[i]['params'].get(key) if key else dict(_K.nodes[i]['params']) for i in self._ids]
        return vals[0] if len(vals) == 1 else vals

    def set(self, params=None, **kw):
        SetStatus(self, dict(params or {}, **kw))


class _BadDelay(Exception):
    def __init__(self, msg):
        super(_BadDelay, self).__init__(msg)
        self.errorname = 'BadDelay'
        self.errormessage = msg


class _Errors(object):
    BadDelay = _BadDelay


class kernel(object):
    NESTErrors = _Errors


class _Kernel(object):
    def __init__(self):
        self.reset()

    def reset(self):
        self.status = {'resolution': 0.1, 'overwrite_files': False, 'print_time': False, 'local_num_threads': 1,
                       'min_delay': 0.1, 'max_delay': 0.1, 'biological_time': 0.0}
        self.nodes = {}          # nest id -> dict(model, params)
        self.next_id = 1
        self.connections = []    # dict(pre, post, weight, delay, receptor, model)
        self.recorder_links = [] # (recorder id, [neuron ids])
        self.clamp_links = []    # (generator id, [neuron ids], delay)
        self.calls = []
        self.engine = None
        self.time = 0.0


_K = _Kernel()
calls = _K.calls


def _ids_of(x):
    if isinstance(x, NodeCollection):
        return x.tolist()
    if np.isscalar(x):
        return [int(x)]
    return [int(i) for i in (x.tolist() if hasattr(x, 'tolist') else x)]


def ResetKernel():
    global calls
    _K.reset()
    calls = _K.calls


def SetKernelStatus(d):
    _K.status.update(d)
    _K.status['min_delay'] = _K.status['max_delay'] = _K.status['resolution']


def GetKernelStatus(key=None):
    return dict(_K.status) if key is None else _K.status[key]


def set_verbosity(level):
    pass


def Rank():
    return 0


def NumProcesses():
    return 1


def SyncProcesses():
    pass


def Create(model, n=1, params=None):
    params = dict(params or {})
    ids = list(range(_K.next_id, _K.next_id + int(n)))
    _K.next_id += int(n)
    for i in ids:
        _K.nodes[i] = dict(model=model, params=dict(params))
    _K.calls.append(('Create', model, int(n), params, ids[0]))
    return NodeCollection(ids)


def CopyModel(existing, new, params=None):
    raise NotImplementedError('CopyModel (weight recorder) is outside the point-neuron path covered here')


def SetStatus(obj, params, val=None):
    if val is not None:
        params = {params: val}
    for i in _ids_of(obj):
        _K.nodes[i]['params'].update({k: (np.array(v, dtype=np.float64) if k == 'spike_times' else v) for k, v in params.items()})
    _K.calls.append(('SetStatus', _ids_of(obj), dict(params)))


def GetStatus(obj, key=None):
    out = [_K.nodes[i]['params'].get(key) if key else dict(_K.nodes[i]['params']) for i in _ids_of(obj)]
    return out


def Connect(pre, post, conn_spec=None, syn_spec=None):
    pre, post = _ids_of(pre), _ids_of(post)
    syn = dict(syn_spec or {})
    res = _K.status['resolution']
    pre_models = {_K.nodes[i]['model'] for i in pre}
    post_models = {_K.nodes[i]['model'] for i in post}
    _K.calls.append(('Connect', np.array(pre), np.array(post), conn_spec, {k: (np.array(v) if not np.isscalar(v) else v) for k, v in syn.items()}))
    if post_models <= {'spike_recorder', 'spike_detector'}:
        for r in post:
            _K.recorder_links.append((r, list(pre)))
        return
    if pre_models <= {'multimeter'}:
        for r in pre:
            _K.recorder_links.append((r, list(post)))
        return
    if pre_models <= {'step_current_generator'}:
        d = float(syn.get('delay', res))
        if d < res * (1 - 1e-9):
            raise _BadDelay('Delay must be greater than or equal to resolution')
        for g in pre:
            _K.clamp_links.append((g, list(post), d))
        return
    rule = conn_spec if isinstance(conn_spec, str) else (conn_spec or {}).get('rule', 'all_to_all')
    if rule != 'one_to_one':
        raise NotImplementedError('Connect rule %r between cells' % (rule,))
    if len(pre) != len(post):
        raise ValueError('one_to_one needs equally many sources and targets')
    n = len(pre)
    w = np.broadcast_to(np.asarray(syn.get('weight', 1.0), dtype=np.float64), (n,))
    d = np.broadcast_to(np.asarray(syn.get('delay', 1.0), dtype=np.float64), (n,))
    if n and np.any(d < res * (1 - 1e-9)):
        raise _BadDelay('Delay must be greater than or equal to resolution')
    rec = np.broadcast_to(np.asarray(syn.get('receptor_type', 0), dtype=np.int64), (n,))
    _K.connections.append(dict(pre=np.array(pre, dtype=np.int64), post=np.array(post, dtype=np.int64), weight=w.copy(),
                               delay=d.copy(), receptor=rec.copy(), model=syn.get('synapse_model', syn.get('model', 'static_synapse'))))
    if n:
        _K.status['min_delay'] = float(min(_K.status['min_delay'] if _K.connections[:-1] else d.min(), d.min()))
        _K.status['max_delay'] = float(max(_K.status['max_delay'], d.max()))


def network():
    """What the recorded calls describe, in engine terms (neurons numbered in creation order)."""
    res = _K.status['resolution']
    neurons = sorted(i for i, nd in _K.nodes.items() if nd['model'] in NEURON_MODELS)
    virtual = sorted(i for i, nd in _K.nodes.items() if nd['model'] == 'spike_generator')
    eng_of = {i: k for k, i in enumerate(neurons)}
    virt_of = {i: k for k, i in enumerate(virtual)}
    types, type_of, type_index = [], {}, []
    for i in neurons:
        nd = _K.nodes[i]
        p = {k: (np.asarray(v).tolist() if isinstance(v, (np.ndarray, list, tuple)) else v) for k, v in nd['params'].items()}
        if nd['model'] != 'glif_psc':
            p['model'] = nd['model']
        key = repr(sorted(p.items()))
        if key not in type_of:
            type_of[key] = len(types)
            types.append(p)
        type_index.append(type_of[key])
    model_of_type = [t.get('model', 'glif_psc') for t in types]
    src, trg, w, d, port = [], [], [], [], []
    for c in _K.connections:
        s = np.array([eng_of[i] if i in eng_of else len(neurons) + virt_of[i] for i in c['pre']], dtype=np.int64)
        t = np.array([eng_of[i] for i in c['post']], dtype=np.int64)
        tm = np.array([model_of_type[type_index[k]] for k in t]) if len(t) else np.zeros(0, dtype='U1')
        prt = np.where(c['receptor'] > 0, c['receptor'] - 1, 0)
        prt = np.where(tm == 'iaf_psc_alpha', (c['weight'] < 0).astype(np.int64), prt)   # the sign picks the PSC of iaf_psc_alpha
        prt = np.where(tm == 'iaf_psc_delta', 0, prt)
        src.append(s); trg.append(t); w.append(c['weight']); d.append(c['delay']); port.append(prt)
    cat = lambda xs, dt: np.concatenate(xs).astype(dt) if xs else np.zeros(0, dtype=dt)
    in_virt, in_time = [], []
    for i in virtual:
        st = _K.nodes[i]['params'].get('spike_times')
        if st is not None and len(st):
            in_virt.append(np.full(len(st), virt_of[i], dtype=np.int64))
            in_time.append(np.asarray(st, dtype=np.float64))
    return dict(dt=res, neurons=neurons, virtual=virtual, types=types, type_index=np.array(type_index, dtype=np.uint16),
                src=cat(src, np.int64), trg=cat(trg, np.int64), weight=cat(w, np.float64), delay_ms=cat(d, np.float64),
                port=cat(port, np.uint8), in_virt=cat(in_virt, np.int64), in_time_ms=cat(in_time, np.float64))


def _build_engine():
    from bmtk_b200.engine import time_to_stamp
    net = network()
    dt = net['dt']
    eng = _engine_factory(dt)
    eng.set_nodes(net['types'], net['type_index'], n_global=len(net['neurons']), lo=0)
    eng.set_virtual(len(net['virtual']))
    eng.add_edges(net['src'], net['trg'], net['weight'], np.round(net['delay_ms'] / dt).astype(np.int64), net['port'])
    if len(net['in_virt']):
        eng.set_input_spikes(net['in_virt'], time_to_stamp(net['in_time_ms'], dt))
    eng_of = {i: k for k, i in enumerate(net['neurons'])}
    steps, targets, deltas = [], [], []
    for g, posts, delay in _K.clamp_links:
        p = _K.nodes[g]['params']
        prev = 0.0
        for t, v in sorted(zip(p.get('amplitude_times', []), p.get('amplitude_values', []))):
            # the generator's current reaches the cell one connection delay (= dt) after the listed time
            s = int(round(t / dt)) + int(round(delay / dt))
            ids = np.array([eng_of[i] for i in posts], dtype=np.uint32)
            steps.append(np.full(len(ids), s, dtype=np.uint64)); targets.append(ids)
            deltas.append(np.full(len(ids), v - prev, dtype=np.float32))
            prev = v
    if steps:
        eng.set_clamp_events(np.concatenate(steps), np.concatenate(targets), np.concatenate(deltas))
    eng.record_spikes(any(_K.nodes[r]['model'] in ('spike_recorder', 'spike_detector') for r, _ in _K.recorder_links))
    probes, interval, variables = [], None, []
    for r, ids in _K.recorder_links:
        nd = _K.nodes[r]
        if nd['model'] != 'multimeter':
            continue
        rf = nd['params'].get('record_from')
        variables.extend(v for v in ([rf] if isinstance(rf, str) else list(rf)) if v not in variables)
        k = int(round(float(nd['params'].get('interval', dt)) / dt))
        interval = k if interval is None else int(np.gcd(interval, k))
        probes.extend(eng_of[i] for i in ids)
    _K.probe_ids = np.array(sorted(set(probes)), dtype=np.uint32)
    _K.probe_interval = interval or 1
    _K.probe_vars = variables
    if len(_K.probe_ids):
        eng.record_state(_K.probe_ids, _K.probe_interval, variables)
    eng.finalize()
    _K.engine, _K.net = eng, net


def Simulate(ms):
    if _K.engine is None:
        _build_engine()
    dt = _K.status['resolution']
    n_steps = int(round(ms / dt))
    _K.engine.run(n_steps)
    _K.time += n_steps * dt
    _K.status['biological_time'] = _K.time
    _write_recorders()


def _write_recorders():
    """NEST-3 ascii recording backend: `<label>-<node id>-<rank>.dat`."""
    eng, net, dt = _K.engine, _K.net, _K.status['resolution']
    nest_of = np.array(net['neurons'], dtype=np.int64)
    header = '# NEST version: 3.3.0\n# RecordingBackendASCII version: 2\n'
    st = ids = None
    trace = None
    for r in sorted({r for r, _ in _K.recorder_links}):
        nd = _K.nodes[r]
        label = nd['params'].get('label') or nd['model']
        path = '%s-%d-0.dat' % (label, r)
        watched = sorted({i for rr, lst in _K.recorder_links if rr == r for i in lst})
        mode = 'a' if os.path.exists(path) and getattr(_K, 'files_started', set()) & {path} else 'w'
        if nd['model'] in ('spike_recorder', 'spike_detector'):
            if st is None:
                st, ids = eng.fetch_spikes()
            sender = nest_of[ids.astype(np.int64)]
            keep = np.isin(sender, np.array(watched, dtype=np.int64))
            with open(path, mode) as f:
                if mode == 'w':
                    f.write(header + 'sender\ttime_ms\n')
                for s, t in zip(sender[keep].tolist(), (st[keep].astype(np.float64) * dt).tolist()):
                    f.write('%d\t%.3f\n' % (s, t))
        elif nd['model'] == 'multimeter':
            if trace is None:
                trace = eng.fetch_trace()            # [samples at multiples of probe_interval, (variables,) probes]
                if trace.ndim == 2:
                    trace = trace[:, None, :]
            rf = nd['params']['record_from']
            rf = [rf] if isinstance(rf, str) else list(rf)
            vcols = [_K.probe_vars.index(v) for v in rf]
            k = int(round(float(nd['params'].get('interval', dt)) / dt)) // _K.probe_interval
            t0, t1 = float(nd['params'].get('start', 0.0)), float(nd['params'].get('stop', np.inf))
            cols = np.searchsorted(_K.probe_ids, np.array([net['neurons'].index(i) for i in watched]))
            n_done = getattr(_K, 'samples_written', {}).get(r, 0)
            with open(path, mode) as f:
                if mode == 'w':
                    f.write(header + 'sender\ttime_ms\t' + '\t'.join(rf) + '\n')
                for j in range(k - 1, trace.shape[0], k):
                    t = (n_done + j + 1) * _K.probe_interval * dt
                    if t <= t0 + 1e-9 or t > t1 + 1e-9:
                        continue
                    for i, c in zip(watched, cols):
                        f.write('%d\t%.3f\t%s\n' % (i, t, '\t'.join(repr(float(trace[j, v, c])) for v in vcols)))
            _K.__dict__.setdefault('samples_written', {})[r] = n_done + trace.shape[0]
        _K.__dict__.setdefault('files_started', set()).add(path)
