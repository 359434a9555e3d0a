"""Seeded synthetic point-neuron networks with the shapes of the benchmark configurations.

No dataset is involved: the reference publishes no benchmark network for this path, so the
workloads are generated here (numpy Generator(PCG64), fixed seeds) in the style of
examples/point_450glifs (GLIF-3 `glif_psc` cells, alpha-PSC ports 1..4 chosen by the
excitatory/inhibitory class of source and target, virtual Poisson cells as input).

  c0  450 neurons / 5 types, Erdos-Renyi p = 0.1, 100 virtual cells       (CPU-runnable case)
  c1  10 000 unconnected neurons, one current step each (0..300 pA)
  c2  50 000 E/I neurons, fixed in-degree 1000
  c3  230 924 neurons / 17 types on a disk, Gaussian distance rule, ~70 M edges
  c4  the c2 network as 64 independent trials over one CSR (per-trial Poisson streams)

Every generator works target block by target block with its own child seed, so a rank that
owns neurons [lo, hi) generates exactly its own edges and all ranks agree on the network.
"""
import numpy as np

TAU_SYN = (5.5, 8.5, 2.8, 5.8)
BLOCK = 8192  # targets per generation block (the unit of seeding)


class Network(object):
    """Plain description of one workload, in engine units (steps, 0-based ports, pA)."""

    def __init__(self, name, dt, n_steps):
        self.name = name
        self.dt = float(dt)
        self.n_steps = int(n_steps)
        self.types = []                 # NEST-format glif_psc dicts
        self.type_names = []
        self.type_is_inh = np.zeros(0, dtype=bool)
        self.type_index = np.zeros(0, dtype=np.uint16)   # [n_neurons], neurons sorted by type
        self.n_virtual = 0
        self.lo, self.hi = 0, 0         # target block these edges cover
        self.src = np.zeros(0, dtype=np.uint32)          # global source id; >= n_neurons is virtual
        self.trg = np.zeros(0, dtype=np.uint32)
        self.weight = np.zeros(0, dtype=np.float32)
        self.delay_steps = np.zeros(0, dtype=np.uint16)
        self.port = np.zeros(0, dtype=np.uint8)
        self.in_virt = np.zeros(0, dtype=np.uint32)      # replayed virtual spikes (index, stamp step)
        self.in_stamp = np.zeros(0, dtype=np.uint32)
        self.poisson_rate_hz = None                      # on-line Poisson instead of replay
        self.poisson_seed = 0
        self.clamp_step = np.zeros(0, dtype=np.uint64)
        self.clamp_target = np.zeros(0, dtype=np.uint32)
        self.clamp_delta = np.zeros(0, dtype=np.float32)
        self.probe_ids = np.zeros(0, dtype=np.uint32)
        self.meta = {}

    @property
    def n_neurons(self):
        return int(len(self.type_index))

    @property
    def n_edges(self):
        return int(len(self.src))


def _glif3_type(rng, inhibitory):
    """One glif_lif_asc_psc parameter set in the ranges of the benchmark configuration
    (C_m 50-150 pF, g 3-10 nS, E_L -70 mV, V_th -50..-40 mV, asc_decay 0.003/0.1 per ms)."""
    return dict(
        V_m=-70.0, E_L=-70.0, V_reset=-70.0,
        V_th=float(rng.uniform(-50.0, -40.0)),
        g=float(rng.uniform(3.0, 10.0)),
        C_m=float(rng.uniform(50.0, 150.0)),
        t_ref=float(np.round(rng.uniform(1.4, 3.2), 1)),
        asc_init=(0.0, 0.0), asc_decay=(0.003, 0.1),
        asc_amps=(float(rng.uniform(-40.0, -5.0)), float(rng.uniform(-300.0, -50.0))),
        asc_r=(1.0, 1.0), tau_syn=TAU_SYN,
        spike_dependent_threshold=False, after_spike_currents=True, adapting_threshold=False)


def _port_of(src_inh, trg_inh):
    """0-based receptor port by class pair, as examples/point_450glifs' synaptic models do
    (e2e 1, i2e 2, e2i 3, i2i 4 in NEST numbering)."""
    return (np.where(src_inh, 1, 0) + np.where(trg_inh, 2, 0)).astype(np.uint8)


def _poisson_trains(rng, rates_hz, t_stop_ms, dt):
    """Homogeneous Poisson trains by exponential inter-spike intervals, the construction of
    PoissonSpikeGenerator (bmtk/utils/reports/spike_trains/spike_trains.py:166-206).
    Returns (virtual index, stamp step) with stamps = ceil(t/dt) >= 1."""
    idx, stamps = [], []
    for v, r in enumerate(np.asarray(rates_hz, dtype=np.float64)):
        if r <= 0:
            continue
        n_exp = int(r * t_stop_ms * 1e-3 * 1.5 + 20)
        t = np.cumsum(rng.exponential(1000.0 / r, size=n_exp))
        while t[-1] < t_stop_ms:
            t = np.concatenate([t, t[-1] + np.cumsum(rng.exponential(1000.0 / r, size=n_exp))])
        t = t[t < t_stop_ms]
        s = np.maximum(np.ceil(t / dt - 1e-9), 1).astype(np.uint32)
        idx.append(np.full(len(s), v, dtype=np.uint32))
        stamps.append(s)
    if not idx:
        return np.zeros(0, dtype=np.uint32), np.zeros(0, dtype=np.uint32)
    return np.concatenate(idx), np.concatenate(stamps)


def _block_rngs(seed, n_blocks):
    return [np.random.default_rng(s) for s in np.random.SeedSequence(seed).spawn(n_blocks)]


def _finish_edges(net, parts):
    if parts:
        net.src = np.concatenate([p[0] for p in parts]).astype(np.uint32)
        net.trg = np.concatenate([p[1] for p in parts]).astype(np.uint32)
        net.weight = np.concatenate([p[2] for p in parts]).astype(np.float32)
        net.delay_steps = np.concatenate([p[3] for p in parts]).astype(np.uint16)
        net.port = np.concatenate([p[4] for p in parts]).astype(np.uint8)


def _sizes(n, fractions):
    s = np.floor(np.asarray(fractions) * n).astype(np.int64)
    s[0] += n - s.sum()
    return s


def _virtual_edges(rng, n_neurons, n_virtual, out_degree, weight, delay_steps, lo, hi, port=0):
    """Each virtual cell projects to `out_degree` random neurons; keeps targets in [lo, hi)."""
    trg = rng.integers(0, n_neurons, size=(n_virtual, out_degree), dtype=np.int64).ravel()
    src = np.repeat(np.arange(n_virtual, dtype=np.int64) + n_neurons, out_degree)
    w = np.broadcast_to(np.asarray(weight, dtype=np.float32), (n_virtual, out_degree)).ravel() \
        if np.ndim(weight) == 2 else np.full(len(trg), weight, dtype=np.float32)
    keep = (trg >= lo) & (trg < hi)
    n = int(keep.sum())
    return (src[keep], trg[keep], w[keep], np.full(n, delay_steps, dtype=np.uint16), np.full(n, port, dtype=np.uint8))


# ---------------------------------------------------------------------------------------------
def c0(seed=1234, t_stop_ms=3000.0, dt=0.1, input_weight=5.0, input_gain=14.0, poisson_online=False):
    """450 GLIF-3 neurons in 5 types (3 excitatory x 120, 2 inhibitory x 45), directed
    Erdos-Renyi p = 0.1 without self loops, weights lognormal(ln 2, 0.5) pA with inhibitory
    sources negated, delays uniform 1-2 ms on the dt grid, 100 Poisson virtual cells at 15 Hz
    projecting to 40 random targets each.

    The configuration's 5 pA input weight alone leaves every neuron more than 15 mV below
    threshold (mean drive ~10 pA against g*(V_th-E_L) of 60-300 pA), i.e. a silent network with
    nothing to propagate. `input_gain` multiplies it (default 14 -> 70 pA peak PSC) so that the
    network fires; pass input_gain=1 for the literal configuration.
    """
    rng = np.random.default_rng(seed)
    net = Network('c0', dt, round(t_stop_ms / dt))
    sizes = [120, 120, 120, 45, 45]
    inh = np.array([False, False, False, True, True])
    net.types = [_glif3_type(rng, i) for i in inh]
    net.type_names = ['e0', 'e1', 'e2', 'i0', 'i1']
    net.type_is_inh = inh
    net.type_index = np.repeat(np.arange(5), sizes).astype(np.uint16)
    n = net.n_neurons
    net.lo, net.hi = 0, n
    adj = rng.random((n, n)) < 0.1
    np.fill_diagonal(adj, False)
    src, trg = np.nonzero(adj)
    w = rng.lognormal(np.log(2.0), 0.5, size=len(src)).astype(np.float32)
    src_inh = inh[net.type_index[src]]
    w = np.where(src_inh, -w, w).astype(np.float32)
    d = np.round(rng.uniform(1.0, 2.0, size=len(src)) / dt).astype(np.uint16)
    port = _port_of(src_inh, inh[net.type_index[trg]])
    n_virtual = 100
    net.n_virtual = n_virtual
    ve = _virtual_edges(rng, n, n_virtual, 40, input_weight * input_gain, round(1.0 / dt), 0, n)
    _finish_edges(net, [(src, trg, w, d, port), ve])
    rates = np.full(n_virtual, 15.0)
    if poisson_online:
        net.poisson_rate_hz = rates.astype(np.float32)
        net.poisson_seed = 4321
    else:
        net.in_virt, net.in_stamp = _poisson_trains(np.random.default_rng(4321), rates, t_stop_ms, dt)
    net.probe_ids = np.array([0, 130, 250, 370, 420], dtype=np.uint32)
    net.meta = dict(input_gain=input_gain)
    return net


def c1(n=10000, t_stop_ms=1500.0, dt=0.05, seed=1235):
    """Current-clamp sweep: n unconnected GLIF-3 neurons cycling through 5 types, neuron i gets a
    step of 300*i/(n-1) pA from 100 ms to 1100 ms (IClamp semantics: the change listed at time T
    is effective from step round(T/dt)+1)."""
    rng = np.random.default_rng(seed)
    net = Network('c1', dt, round(t_stop_ms / dt))
    net.types = [_glif3_type(rng, False) for _ in range(5)]
    net.type_names = ['t%d' % i for i in range(5)]
    net.type_is_inh = np.zeros(5, dtype=bool)
    # neurons sorted by type; amplitude grid is assigned through a fixed permutation so that every
    # type sees the whole amplitude range
    net.type_index = np.sort(np.arange(n) % 5).astype(np.uint16)
    net.lo, net.hi = 0, n
    amp = (300.0 * rng.permutation(n) / max(n - 1, 1)).astype(np.float32)
    on, off = round(100.0 / dt) + 1, round(1100.0 / dt) + 1
    ids = np.arange(n, dtype=np.uint32)
    net.clamp_step = np.concatenate([np.full(n, on), np.full(n, off)]).astype(np.uint64)
    net.clamp_target = np.concatenate([ids, ids])
    net.clamp_delta = np.concatenate([amp, -amp]).astype(np.float32)
    net.probe_ids = np.linspace(0, n - 1, 16).astype(np.uint32)
    net.meta = dict(amp=amp)
    return net


def c2(n=50000, in_degree=1000, t_stop_ms=1000.0, dt=0.1, seed=1236, n_virtual=2000, lo=0, hi=None,
       input_weight=120.0, poisson_online=True, w_scale=1.0):
    """E/I network: 80 % excitatory / 20 % inhibitory in 4 types each, every neuron receives
    exactly `in_degree` synapses from uniformly drawn sources (no self loops, multapses allowed),
    weights lognormal(ln 1.5, 0.6) pA with inhibitory sources scaled by -4, delays uniform
    0.8-3.0 ms on the dt grid, ports uniform over the 4 receptors; `n_virtual` Poisson cells at
    10 Hz with out-degree 200 (scaled with n). The configuration leaves the input weight open: 120 pA
    puts the full-size network at about 6 Hz per neuron."""
    hi = n if hi is None else hi
    rng = np.random.default_rng(seed)
    net = Network('c2', dt, round(t_stop_ms / dt))
    inh = np.array([False] * 4 + [True] * 4)
    net.types = [_glif3_type(rng, i) for i in inh]
    net.type_names = ['e%d' % i for i in range(4)] + ['i%d' % i for i in range(4)]
    net.type_is_inh = inh
    sizes = _sizes(n, [0.2] * 4 + [0.05] * 4)
    net.type_index = np.repeat(np.arange(8), sizes).astype(np.uint16)
    net.lo, net.hi = lo, hi
    n_blocks = (n + BLOCK - 1) // BLOCK
    rngs = _block_rngs(seed + 1, n_blocks)
    parts = []
    for b in range(n_blocks):
        b0, b1 = b * BLOCK, min((b + 1) * BLOCK, n)
        if b1 <= lo or b0 >= hi:
            continue
        r = rngs[b]
        t = np.repeat(np.arange(b0, b1, dtype=np.int64), in_degree)
        s = r.integers(0, n - 1, size=len(t), dtype=np.int64)
        s += s >= t  # skip the target itself
        w = r.lognormal(np.log(1.5), 0.6, size=len(t)).astype(np.float32) * np.float32(w_scale)
        w = np.where(inh[net.type_index[s]], np.float32(-4.0) * w, w).astype(np.float32)
        d = np.round(r.uniform(0.8, 3.0, size=len(t)) / dt).astype(np.uint16)
        p = r.integers(0, 4, size=len(t), dtype=np.uint8)
        keep = (t >= lo) & (t < hi)
        parts.append((s[keep], t[keep], w[keep], d[keep], p[keep]))
    net.n_virtual = n_virtual
    out_deg = max(1, min(200, n // 4))
    ve = _virtual_edges(np.random.default_rng(seed + 2), n, n_virtual, out_deg, input_weight, round(1.0 / dt), lo, hi)
    parts.append(ve)
    _finish_edges(net, parts)
    rates = np.full(n_virtual, 10.0)
    if poisson_online:
        net.poisson_rate_hz = rates.astype(np.float32)
        net.poisson_seed = 4323
    else:
        net.in_virt, net.in_stamp = _poisson_trains(np.random.default_rng(4323), rates, t_stop_ms, dt)
    net.probe_ids = np.linspace(lo, hi - 1, 16).astype(np.uint32)
    return net


def c4(n=50000, in_degree=1000, t_stop_ms=500.0, dt=0.1, trials=64, **kw):
    """Trial sweep: the c2 network simulated as `trials` independent trials that share one CSR, each
    with its own Philox stream for the Poisson cells (engine option "trials"); 500 ms."""
    net = c2(n=n, in_degree=in_degree, t_stop_ms=t_stop_ms, dt=dt, poisson_online=True, **kw)
    net.name = 'c4'
    net.meta = dict(trials=int(trials))
    return net


def c3(n=230924, mean_in_degree=330.0, t_stop_ms=1000.0, dt=0.25, seed=1237, n_virtual=17400, lo=0, hi=None,
       radius_um=845.0, input_weight=45.0, poisson_online=True, w_scale=1.0, virt_out_degree=200):
    """V1-scale network: n GLIF-3 neurons in 17 types (13 excitatory, 4 inhibitory; 85 % / 15 %)
    placed uniformly on a disk; P(i -> j) proportional to exp(-d^2 / 2 sigma^2) with sigma drawn in
    100-200 um per (source class, target type); weights lognormal per (source type, target type)
    with inhibitory sources negative; delays uniform 0.5-4.0 ms on the dt grid; 4 receptor ports
    by class pair; `n_virtual` Poisson cells at rates uniform 2-20 Hz with ~200 targets each.

    Sampling: for every target a Poisson number of candidate synapses is drawn; each candidate
    picks a source class, a Gaussian displacement with that pair's sigma, and then a uniformly
    random neuron of that class inside the 20 um grid cell the displaced point falls in; a cell
    holding c neurons keeps the candidate with probability c / c_max, which makes every neuron's
    chance proportional to the kernel at its cell. Candidates landing outside the disk are
    dropped, which thins in-degree near the rim exactly as a distance rule does; mean_in_degree
    = 330 candidates gives ~303 synapses per neuron, ~70 M in all.
    """
    hi = n if hi is None else hi
    rng = np.random.default_rng(seed)
    net = Network('c3', dt, round(t_stop_ms / dt))
    n_types = 17
    inh = np.array([False] * 13 + [True] * 4)
    net.types = [_glif3_type(rng, i) for i in inh]
    net.type_names = ['e%d' % i for i in range(13)] + ['i%d' % i for i in range(4)]
    net.type_is_inh = inh
    frac = np.concatenate([rng.dirichlet(np.full(13, 8.0)) * 0.85, rng.dirichlet(np.full(4, 8.0)) * 0.15])
    sizes = _sizes(n, frac)
    net.type_index = np.repeat(np.arange(n_types), sizes).astype(np.uint16)
    net.lo, net.hi = lo, hi
    # positions: uniform on the disk, independent of type
    rad = radius_um * np.sqrt(rng.random(n))
    ang = rng.uniform(0, 2 * np.pi, n)
    x, y = rad * np.cos(ang), rad * np.sin(ang)
    sigma = rng.uniform(100.0, 200.0, size=(2, n_types))       # (source class, target type)
    w_mu = np.log(rng.uniform(0.8, 2.5, size=(n_types, n_types)))  # (source type, target type)
    w_sigma = 0.5
    is_inh = inh[net.type_index]
    # 20 um grid per source class: neurons of the class sorted by cell
    cell = 20.0
    g = int(np.ceil(2 * radius_um / cell)) + 1
    grids = []
    for c in (False, True):
        ids = np.nonzero(is_inh == c)[0]
        cx = ((x[ids] + radius_um) / cell).astype(np.int64)
        cy = ((y[ids] + radius_um) / cell).astype(np.int64)
        key = cx * g + cy
        order = np.argsort(key, kind='stable')
        cnt = np.bincount(key, minlength=g * g)
        start = np.concatenate([[0], np.cumsum(cnt)[:-1]])
        grids.append((ids[order], start, cnt, float(cnt.max())))
    n_class = np.array([np.sum(~is_inh), np.sum(is_inh)], dtype=np.float64)
    # expected fraction of candidates that survive the density correction, per class
    acc = np.array([n_class[c] / (np.count_nonzero(grids[c][2]) * grids[c][3]) for c in (0, 1)])
    n_blocks = (n + BLOCK - 1) // BLOCK
    rngs = _block_rngs(seed + 1, n_blocks)

    def make_block(b):
        b0, b1 = b * BLOCK, min((b + 1) * BLOCK, n)
        r = rngs[b]
        tb0, tb1 = max(b0, lo), min(b1, hi)
        # candidates are drawn for the whole block (the stream does not depend on the partition)
        tt_blk = net.type_index[b0:b1]
        pe = n_class[0] * sigma[0, tt_blk] ** 2
        pi = n_class[1] * sigma[1, tt_blk] ** 2
        # oversample so that mean_in_degree survives the density correction on average
        lam = mean_in_degree * (pe / acc[0] + pi / acc[1]) / (pe + pi)
        k = r.poisson(lam)
        t = np.repeat(np.arange(b0, b1, dtype=np.int64), k)
        tt = net.type_index[t]
        qe = np.repeat(pe / acc[0], k)
        qi = np.repeat(pi / acc[1], k)
        sc = (r.random(len(t)) * (qe + qi) >= qe).astype(np.int64)
        sg = sigma[sc, tt]
        px = x[t] + r.normal(size=len(t)) * sg
        py = y[t] + r.normal(size=len(t)) * sg
        u = r.random(len(t))
        u2 = r.random(len(t))
        wz = r.normal(size=len(t))
        dd = r.uniform(0.5, 4.0, size=len(t))
        ok = px * px + py * py < radius_um * radius_um
        ok &= (t >= tb0) & (t < tb1)
        t, sc, px, py, u, u2, wz, dd = t[ok], sc[ok], px[ok], py[ok], u[ok], u2[ok], wz[ok], dd[ok]
        key = ((px + radius_um) / cell).astype(np.int64) * g + ((py + radius_um) / cell).astype(np.int64)
        s = np.zeros(len(t), dtype=np.int64)
        good = np.zeros(len(t), dtype=bool)
        for c in (0, 1):
            m = np.nonzero(sc == c)[0]
            ids, start, cnt, cmax = grids[c]
            kc = key[m]
            cn = cnt[kc]
            # density correction: a cell with cn neurons keeps a candidate with probability cn/cmax,
            # so every neuron is hit in proportion to the kernel at its cell, not to 1/local density
            has = u2[m] * cmax < cn
            pick = start[kc] + np.minimum((u[m] * cn).astype(np.int64), np.maximum(cn - 1, 0))
            s[m] = np.where(has, ids[np.minimum(pick, len(ids) - 1)], 0)
            good[m] = has
        good &= s != t
        t, s, wz, dd = t[good], s[good], wz[good], dd[good]
        st, tt = net.type_index[s], net.type_index[t]
        w = np.exp(w_mu[st, tt] + w_sigma * wz).astype(np.float32) * np.float32(w_scale)
        w = np.where(inh[st], np.float32(-4.0) * w, w).astype(np.float32)
        d = np.maximum(np.round(dd / dt), 1).astype(np.uint16)
        p = _port_of(inh[st], inh[tt])
        return (s.astype(np.uint32), t.astype(np.uint32), w, d, p)

    todo = [b for b in range(n_blocks) if not (min((b + 1) * BLOCK, n) <= lo or b * BLOCK >= hi)]
    import concurrent.futures
    import os
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(16, os.cpu_count() or 1))) as ex:
        parts = list(ex.map(make_block, todo))
    net.n_virtual = n_virtual
    vr = np.random.default_rng(seed + 2)
    ve = _virtual_edges(vr, n, n_virtual, virt_out_degree, input_weight, max(1, round(1.0 / dt)), lo, hi)
    parts.append(ve)
    _finish_edges(net, parts)
    rates = np.random.default_rng(seed + 3).uniform(2.0, 20.0, size=n_virtual)
    if poisson_online:
        net.poisson_rate_hz = rates.astype(np.float32)
        net.poisson_seed = 4324
    else:
        net.in_virt, net.in_stamp = _poisson_trains(np.random.default_rng(4324), rates, t_stop_ms, dt)
    net.probe_ids = np.linspace(lo, hi - 1, 16).astype(np.uint32)
    net.meta = dict(x=x, y=y)
    return net


def build_engine(net, device=0, deterministic=False, record_spikes=True, record_vm=True, options=None,
                 rank=0, n_ranks=1, nccl_uid=None, libnccl=None, p2p=False):
    """Creates and finalizes an Engine for `net` (whose edges must cover [net.lo, net.hi))."""
    from .engine import Engine
    e = Engine(net.dt, device=device)
    e.set_nodes(net.types, net.type_index[net.lo:net.hi], n_global=net.n_neurons, lo=net.lo)
    e.set_virtual(net.n_virtual)
    e.add_edges(net.src, net.trg, net.weight, net.delay_steps, net.port)
    if net.poisson_rate_hz is not None:
        e.set_poisson(net.poisson_rate_hz, net.poisson_seed)
    elif len(net.in_virt):
        e.set_input_spikes(net.in_virt, net.in_stamp)
    if len(net.clamp_step):
        m = (net.clamp_target >= net.lo) & (net.clamp_target < net.hi)
        e.set_clamp_events(net.clamp_step[m], net.clamp_target[m], net.clamp_delta[m])
    e.record_spikes(record_spikes)
    if record_vm and len(net.probe_ids):
        ids = net.probe_ids[(net.probe_ids >= net.lo) & (net.probe_ids < net.hi)]
        e.record_vm(ids, 1)
    e.set_option('deterministic', int(deterministic))
    for k, v in (options or {}).items():
        e.set_option(k, v)
    if n_ranks > 1:
        e.comm_init(nccl_uid, rank, n_ranks, libnccl)
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() == n_ranks:
            e.agree_layout()    # window, spike capacity and buffer offsets must be the same on every rank
    e.finalize()
    if n_ranks > 1 and p2p and not deterministic:
        e.connect_peers()       # spike exchange over peer memory inside the persistent kernel
    return e
