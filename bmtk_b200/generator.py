"""Synthetic distance-dependent network, sampled on the GPU.

Stands in for bmtk.builder on the point-neuron path (the reference builds its example networks on the
host by evaluating a Python connection rule per node pair, examples/point_450glifs/build_network.py):
`distance_spec` lays out nodes, type-pair parameters, the spatial grids and the two quantile tables with
numpy; `generate_edges` hands them to bmtk_generate_distance_edges, which draws every target's incoming
synapses with counter-based random numbers on the device (bmtk_b200/csrc/generate.cu). The edge list is a
pure function of the specification: any partition of the targets over calls, ranks or devices yields
the same edges. `c3_device` assembles the V1-scale workload this way (same node types, positions and
parameter ranges as workloads.c3, whose edges are drawn by numpy on the host)."""
import ctypes as C

import numpy as np

from . import _cabi
from . import workloads as W
from ._cabi import check

N_QUANTILES = 4096


class GenSpec(C.Structure):
    """bmtk_gen_spec (include/bmtk_b200.h)."""
    _fields_ = [
        ('n_neurons', C.c_uint32), ('n_types', C.c_uint32), ('lo', C.c_uint32), ('hi', C.c_uint32),
        ('type_index', C.c_void_p), ('type_is_inh', C.c_void_p), ('x', C.c_void_p), ('y', C.c_void_p),
        ('sigma', C.c_void_p), ('w_base', C.c_void_p), ('q_exc', C.c_void_p), ('q_inh', C.c_void_p),
        ('lam', C.c_void_p), ('gauss_table', C.c_void_p), ('lognorm_table', C.c_void_p),
        ('cell_start', C.c_void_p * 2), ('cell_count', C.c_void_p * 2), ('cell_ids', C.c_void_p * 2),
        ('class_size', C.c_uint32 * 2), ('cell_max', C.c_float * 2), ('grid', C.c_uint32),
        ('radius', C.c_float), ('inv_cell', C.c_float), ('inh_scale', C.c_float), ('delay_min_ms', C.c_float),
        ('delay_max_ms', C.c_float), ('dt', C.c_float), ('seed', C.c_uint64),
    ]


def quantile_tables(w_sigma):
    """Standard normal quantiles at (i + 0.5) / 4096 and the lognormal factors exp(w_sigma z), float32."""
    from scipy.special import ndtri
    z = ndtri((np.arange(N_QUANTILES) + 0.5) / N_QUANTILES)
    return z.astype(np.float32), np.exp(w_sigma * z).astype(np.float32)


def distance_spec(type_index, type_is_inh, x, y, sigma, w_mu, radius_um, mean_in_degree, dt, seed, cell_um=20.0,
                  w_sigma=0.5, inh_scale=4.0, delay_ms=(0.5, 4.0)):
    """Arrays of a generator specification (dict; `as_struct` turns it into the C structure)."""
    type_index = np.ascontiguousarray(type_index, dtype=np.uint16)
    inh = np.ascontiguousarray(type_is_inh, dtype=np.uint8)
    n, nt = len(type_index), len(inh)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.ascontiguousarray(y, dtype=np.float32)
    is_inh = inh[type_index].astype(bool)
    grid = int(np.ceil(2 * radius_um / cell_um)) + 1
    inv_cell = np.float32(1.0 / cell_um)
    R = np.float32(radius_um)
    spec = dict(n_neurons=n, n_types=nt, type_index=type_index, type_is_inh=inh, x=x, y=y,
                sigma=np.ascontiguousarray(sigma, dtype=np.float32), w_base=np.exp(np.asarray(w_mu)).astype(np.float32),
                grid=grid, radius=float(R), inv_cell=float(inv_cell), inh_scale=float(inh_scale),
                delay_min_ms=float(delay_ms[0]), delay_max_ms=float(delay_ms[1]), dt=float(dt), seed=int(seed))
    n_class = np.zeros(2)
    acc = np.zeros(2)
    for c in (0, 1):
        ids = np.nonzero(is_inh == bool(c))[0]
        # the cell of a neuron, with the arithmetic the generator applies to a displaced point
        cx = np.floor((x[ids] + R) * inv_cell).astype(np.int64)
        cy = np.floor((y[ids] + R) * inv_cell).astype(np.int64)
        key = cx * grid + cy
        order = np.argsort(key, kind='stable')
        cnt = np.bincount(key, minlength=grid * grid)
        start = np.concatenate([[0], np.cumsum(cnt)[:-1]])
        spec['cell_ids%d' % c] = ids[order].astype(np.uint32)
        spec['cell_start%d' % c] = start.astype(np.uint32)
        spec['cell_count%d' % c] = cnt.astype(np.uint32)
        spec['cell_max%d' % c] = float(cnt.max()) if len(ids) else 1.0
        n_class[c] = len(ids)
        acc[c] = n_class[c] / max(1.0, np.count_nonzero(cnt) * spec['cell_max%d' % c])
    sg = np.asarray(sigma, dtype=np.float64)
    pe = n_class[0] * sg[0] ** 2 / max(acc[0], 1e-30)
    pi = n_class[1] * sg[1] ** 2 / max(acc[1], 1e-30) if n_class[1] else np.zeros(nt)
    spec['q_exc'] = pe.astype(np.float32)
    spec['q_inh'] = pi.astype(np.float32)
    # candidates per target so that mean_in_degree of them survive the density correction on average
    spec['lam'] = (mean_in_degree * (pe + pi) / (n_class[0] * sg[0] ** 2 + n_class[1] * sg[1] ** 2)).astype(np.float32)
    spec['gauss_table'], spec['lognorm_table'] = quantile_tables(w_sigma)
    return spec


def as_struct(spec, lo, hi, cls=GenSpec):
    s = cls()
    s.n_neurons, s.n_types, s.lo, s.hi = spec['n_neurons'], spec['n_types'], int(lo), int(hi)
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    for k in ('type_index', 'type_is_inh', 'x', 'y', 'sigma', 'w_base', 'q_exc', 'q_inh', 'lam', 'gauss_table', 'lognorm_table'):
        setattr(s, k, ptr(spec[k]))
    for c in (0, 1):
        s.cell_start[c] = ptr(spec['cell_start%d' % c])
        s.cell_count[c] = ptr(spec['cell_count%d' % c])
        s.cell_ids[c] = ptr(spec['cell_ids%d' % c])
        s.class_size[c] = len(spec['cell_ids%d' % c])
        s.cell_max[c] = spec['cell_max%d' % c]
    for k in ('grid', 'radius', 'inv_cell', 'inh_scale', 'delay_min_ms', 'delay_max_ms', 'dt', 'seed'):
        setattr(s, k, spec[k])
    return s


def generate_edges(spec, lo=0, hi=None, device=0):
    """(src, trg, weight, delay_steps, port) of the edges into targets [lo, hi), drawn on the device."""
    hi = spec['n_neurons'] if hi is None else hi
    lib = _cabi.load()
    s = as_struct(spec, lo, hi)
    n = C.c_uint64()
    check(lib.bmtk_generate_distance_edges(C.byref(s), int(device), 0, None, None, None, None, None, C.byref(n)))
    m = int(n.value)
    src, trg = np.empty(m, dtype=np.uint32), np.empty(m, dtype=np.uint32)
    w, d, p = np.empty(m, dtype=np.float32), np.empty(m, dtype=np.uint16), np.empty(m, dtype=np.uint8)
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    check(lib.bmtk_generate_distance_edges(C.byref(s), int(device), m, ptr(src), ptr(trg), ptr(w), ptr(d), ptr(p), C.byref(n)))
    return src, trg, w, d, p


def c3_device(n=230924, mean_in_degree=346.0, t_stop_ms=1000.0, dt=0.25, seed=1237, n_virtual=17400, lo=0, hi=None,
              radius_um=845.0, input_weight=45.0, virt_out_degree=200, device=0):
    """The V1-scale workload with its recurrent edges sampled on the GPU: node types, positions, sigma and weight
    tables are drawn exactly as workloads.c3 draws them (same numpy stream), the ~70 M synapses by the device
    generator; virtual-cell edges and Poisson rates as in workloads.c3."""
    hi = n if hi is None else hi
    rng = np.random.default_rng(seed)
    net = W.Network('c3_device', dt, round(t_stop_ms / dt))
    n_types = 17
    inh = np.array([False] * 13 + [True] * 4)
    net.types = [W._glif3_type(rng, i) for i in inh]
    net.type_names = ['e%d' % i for i in range(13)] + ['i%d' % i for i in range(4)]
    net.type_is_inh = inh
    frac = np.concatenate([rng.dirichlet(np.full(13, 8.0)) * 0.85, rng.dirichlet(np.full(4, 8.0)) * 0.15])
    net.type_index = np.repeat(np.arange(n_types), W._sizes(n, frac)).astype(np.uint16)
    net.lo, net.hi = lo, hi
    rad = radius_um * np.sqrt(rng.random(n))
    ang = rng.uniform(0, 2 * np.pi, n)
    x, y = rad * np.cos(ang), rad * np.sin(ang)
    sigma = rng.uniform(100.0, 200.0, size=(2, n_types))
    w_mu = np.log(rng.uniform(0.8, 2.5, size=(n_types, n_types)))
    spec = distance_spec(net.type_index, inh, x, y, sigma, w_mu, radius_um, mean_in_degree, dt, seed + 1)
    parts = [generate_edges(spec, lo, hi, device)]
    net.n_virtual = n_virtual
    parts.append(W._virtual_edges(np.random.default_rng(seed + 2), n, n_virtual, virt_out_degree, input_weight,
                                  max(1, round(1.0 / dt)), lo, hi))
    W._finish_edges(net, parts)
    net.poisson_rate_hz = np.random.default_rng(seed + 3).uniform(2.0, 20.0, size=n_virtual).astype(np.float32)
    net.poisson_seed = 4324
    net.probe_ids = np.linspace(lo, hi - 1, 16).astype(np.uint32)
    net.meta = dict(x=x, y=y, spec=spec)
    return net
