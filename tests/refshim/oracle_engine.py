"""An engine with the API of bmtk_b200.engine.Engine that computes with the fp64 CPU oracle (test
infrastructure). The verification shim drives it from the fake `nest` module, and the adapter test lets
bmtk_b200.pointnet drive the same class, so that the two adapters can be compared file for file in a
container without a GPU. It is never used by the product."""
import numpy as np

from oracle import glif_oracle as O


class OracleEngine(object):
    def __init__(self, dt, device=0):
        self.dt = float(dt)
        self._edges = []
        self._inputs = None
        self._clamps = None
        self._probes = (np.zeros(0, dtype=np.uint32), 1)
        self._record = False
        self._spikes = [np.zeros(0, dtype=np.uint32), np.zeros(0, dtype=np.uint32)]
        self._trace = []
        self.n_virtual = 0
        self.sim = None
        self.options = {}

    def set_nodes(self, types, type_index, n_global=None, lo=0):
        assert lo == 0 and (n_global is None or n_global == len(type_index))
        self.types, self.type_index = list(types), np.asarray(type_index, dtype=np.uint16)
        self.n_local = len(self.type_index)

    def set_virtual(self, n):
        self.n_virtual = int(n)

    def add_edges(self, src, trg, weight, delay_steps, port):
        d = np.asarray(delay_steps)
        if d.size and d.min() < 1:
            from bmtk_b200._cabi import BadDelay, E_DELAY
            raise BadDelay(E_DELAY, 'delay shorter than the resolution dt = %g ms' % self.dt)
        self._edges.append((np.asarray(src, dtype=np.int64), np.asarray(trg, dtype=np.int64),
                            np.asarray(weight, dtype=np.float32), d.astype(np.int64), np.asarray(port, dtype=np.int64)))

    def set_input_spikes(self, virt, stamps):
        self._inputs = (np.asarray(virt, dtype=np.int64), np.asarray(stamps, dtype=np.int64))

    def set_poisson(self, rates, seed):
        raise NotImplementedError

    def set_clamp_events(self, step, target, delta):
        self._clamps = (np.asarray(step), np.asarray(target), np.asarray(delta, dtype=np.float32))

    def record_spikes(self, enable=True):
        self._record = bool(enable)

    def record_vm(self, ids, interval_steps=1):
        self._probes = (np.asarray(ids, dtype=np.uint32), int(interval_steps))
        self.n_probe = len(ids)

    def record_state(self, ids, interval_steps=1, variables=('V_m',)):
        from bmtk_b200._cabi import RECORDABLES
        self._probes = (np.asarray(ids, dtype=np.uint32), int(interval_steps))
        self._vars = [RECORDABLES[v] for v in variables]
        self.n_probe = len(ids)

    def set_option(self, key, value):
        self.options[key] = value

    def finalize(self):
        cat = lambda k, dt: np.concatenate([e[k] for e in self._edges]).astype(dt) if self._edges else np.zeros(0, dtype=dt)
        self.sim = O.OracleSim(self.types, self.type_index, self.dt, n_virtual=self.n_virtual, src=cat(0, np.int64),
                               trg=cat(1, np.int64), weight=cat(2, np.float32).astype(np.float64),
                               delay_steps=cat(3, np.int64), port=cat(4, np.int64))
        if self._inputs is not None:
            self.sim.set_input_spikes(self._inputs[1] - 1, self._inputs[0])
        if self._clamps is not None:
            self.sim.set_clamp_events(self._clamps[0], self._clamps[1], self._clamps[2].astype(np.float64))
        if len(self._probes[0]):
            self.sim.set_probes(self._probes[0], self._probes[1], getattr(self, '_vars', [0]))

    def connect_peers(self):
        pass

    def run(self, n_steps):
        r = self.sim.run(int(n_steps))
        if self._record:
            self._spikes[0] = np.concatenate([self._spikes[0], r['spike_step'].astype(np.uint32)])
            self._spikes[1] = np.concatenate([self._spikes[1], r['spike_id'].astype(np.uint32)])
        if len(self._probes[0]):
            self._trace.append(r['trace'].astype(np.float32))

    def fetch_spikes(self):
        st, ids = self._spikes
        self._spikes = [np.zeros(0, dtype=np.uint32), np.zeros(0, dtype=np.uint32)]
        return st, ids

    def fetch_trace(self):
        nv = len(getattr(self, '_vars', [0]))
        empty = np.zeros((0, len(self._probes[0])) if nv == 1 else (0, nv, len(self._probes[0])), dtype=np.float32)
        tr = np.concatenate(self._trace) if self._trace else empty
        self._trace = []
        return tr

    def counter(self, name):
        return {'events': int(self.sim.n_events[0]), 'steps': self.sim.step}.get(name, 0)

    def close(self):
        pass
