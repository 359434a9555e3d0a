"""PointNetwork: SONATA populations -> the arrays the engine is built from.

Mirrors bmtk.simulator.pointnet.PointNetwork (bmtk/simulator/pointnet/pointnetwork.py:70-248 over
bmtk/simulator/core/simulator_network.py:207-267): from_config loads node / edge populations and
components, build_nodes groups nodes into one batch per node type (engine ids in creation order,
like NEST ids but 0-based), build_recurrent_edges expands every edge type to
(source, target, weight = nsyns * syn_weight | weight_function, delay, receptor port), and
add_spike_trains attaches virtual cells and their edges. Nothing touches the GPU here: the
PointSimulator hands the collected arrays to the engine.
"""
import json
import os
from collections import namedtuple

import numpy as np

from . import sonata
from .glif_utils import convert_aibs2nest
from .io_tools import io
from .pyfunction_cache import py_modules

PopulationID = namedtuple('PopulationID', 'population node_id')

_GLIF_MODES = {
    'glif_lif_psc': (False, False, False), 'glif_lif_r_psc': (True, False, False),
    'glif_lif_asc_psc': (False, True, False), 'glif_lif_r_asc_psc': (True, True, False),
    'glif_lif_r_asc_a_psc': (True, True, True),
}


class BadDelay(Exception):
    """A synaptic delay is shorter than the simulation resolution (NEST's BadDelay,
    bmtk/simulator/pointnet/pointnetwork.py:234-243)."""


class GidPool(object):
    """(population, node_id) <-> engine id (bmtk/simulator/pointnet/gids.py:24-107). Engine ids are
    0-based and contiguous in creation order; look-ups are vectorised."""

    def __init__(self):
        self._pops = {}          # name -> (sorted node_ids, engine ids in that order)
        self._engine_pop = []    # per engine id: population index
        self._engine_node = []   # per engine id: node id
        self._pop_names = []

    @property
    def gids(self):
        return list(range(len(self)))

    @property
    def populations(self):
        return list(self._pop_names)

    def add_nestids(self, name, node_ids, nest_ids):
        node_ids = np.asarray(node_ids, dtype=np.int64)
        nest_ids = np.asarray(nest_ids, dtype=np.int64)
        if name not in self._pop_names:
            self._pop_names.append(name)
        pi = self._pop_names.index(name)
        if len(nest_ids) and nest_ids[0] != len(self._engine_node):
            raise Exception('engine ids must be added in creation order')
        self._engine_pop.extend([pi] * len(nest_ids))
        self._engine_node.extend(node_ids.tolist())
        if name in self._pops:
            old_n, old_g = self._pops[name]
            node_ids = np.concatenate([old_n, node_ids])
            nest_ids = np.concatenate([old_g, nest_ids])
        o = np.argsort(node_ids, kind='stable')
        self._pops[name] = (node_ids[o], nest_ids[o])

    add_gids = add_nestids

    def get_nestids(self, name, node_ids):
        nids, gids = self._pops[name]
        q = np.asarray(node_ids, dtype=np.int64)
        pos = np.searchsorted(nids, q)
        pos = np.minimum(pos, max(len(nids) - 1, 0))
        if len(nids) == 0 or np.any(nids[pos] != q):
            raise KeyError('node_id(s) not in population {}'.format(name))
        return gids[pos]

    get_gids = get_nestids

    def get_gid(self, name, node_id):
        return int(self.get_nestids(name, [node_id])[0])

    def get_pool_id(self, gid):
        return PopulationID(self._pop_names[self._engine_pop[gid]], self._engine_node[gid])

    def get_node_ids(self, nest_ids, with_populations=True):
        g = np.asarray(nest_ids, dtype=np.int64)
        node = np.asarray(self._engine_node, dtype=np.int64)[g]
        if not with_populations:
            return node
        names = np.asarray(self._pop_names, dtype=object)[np.asarray(self._engine_pop, dtype=np.int64)[g]]
        return node, names

    def __len__(self):
        return len(self._engine_node)


class NodeSet(object):
    """A selection of nodes (bmtk/simulator/core/node_sets.py:4-53): a list is taken as engine ids,
    a dict filters populations by equality on node / node-type columns."""

    def __init__(self, filter_params, network):
        self._network = network
        self._preselected = None
        self._filter = {}
        if isinstance(filter_params, (list, tuple, np.ndarray)):
            self._preselected = [int(g) for g in filter_params]
            self._populations = []
        elif isinstance(filter_params, dict):
            f = dict(filter_params)
            pops = None
            for k in ('population', 'populations'):
                if k in f:
                    v = f.pop(k)
                    pops = [network.get_node_population(p) for p in (v if isinstance(v, (list, tuple)) else [v])]
            self._filter = f
            self._populations = pops if pops is not None else network.get_node_populations()
        else:
            io.log_exception('Unknown node set params type {}'.format(type(filter_params)))

    def populations(self):
        return self._populations

    def population_names(self):
        return [p.name for p in self._populations]

    def node_ids_by_population(self):
        return [(p, p.filter(**self._filter)) for p in self._populations]

    @property
    def node_ids(self):
        out = []
        for _p, ids in self.node_ids_by_population():
            out.extend(ids.tolist())
        return out

    def gids(self):
        if self._preselected is not None:
            return list(self._preselected)
        out = []
        pool = self._network.gid_pool
        for p, ids in self.node_ids_by_population():
            if p.name in pool.populations and len(ids):
                out.extend(pool.get_nestids(p.name, ids).tolist())
        return out


def balanced_bounds(load, parts):
    """Bounds b[0..parts] of contiguous blocks of len(load) items whose load sums are as equal as contiguous cuts
    allow: cut k lies where the running sum first reaches k/parts of the total (items without load count 1 so that
    unconnected neurons still spread). Every block gets at least one item when there are enough."""
    w = np.maximum(np.asarray(load, dtype=np.int64), 1)
    c = np.concatenate([[0], np.cumsum(w)])
    n = len(w)
    b = np.searchsorted(c, c[-1] * np.arange(parts + 1) / float(parts), side='left').astype(np.int64)
    b[0], b[-1] = 0, n
    for k in range(1, parts):               # strictly increasing while items are left
        b[k] = min(max(b[k], b[k - 1] + (1 if n >= parts else 0)), n)
    return b


class PointNetwork(object):
    def __init__(self, **properties):
        self._components = {}
        self._node_populations = {}
        self._edge_populations = []
        self._node_sets = {}
        self._gid_pool = GidPool()
        self._io = io
        self._dt = None
        # build products
        self.types = []               # one NEST glif_psc dict per node-type batch
        self.type_labels = []         # (population, node_type_id)
        self.type_index = np.zeros(0, dtype=np.uint16)
        self.target_block = None      # (lo, hi) engine ids whose incoming edges this rank expands; None = all
        self.block_bounds = None
        self.edge_batches = []        # dict(src, trg, weight, delay, port) in engine ids, recurrent
        self.virtual_index = {}       # population -> (sorted node_ids, virtual index)
        self.n_virtual = 0
        self.virtual_edge_batches = []
        self.input_spikes = []        # (virtual index array, time ms array)
        self._nodes_built = False
        self._edges_built = False

    # ---- configuration
    @property
    def io(self):
        return self._io

    @property
    def dt(self):
        return self._dt

    @dt.setter
    def dt(self, v):
        self._dt = float(v)

    @property
    def gid_pool(self):
        return self._gid_pool

    gid_map = gid_pool

    @property
    def _nestid2gid(self):
        return self._gid_pool

    def add_component(self, name, path):
        self._components[name] = path

    def get_component(self, name):
        if name not in self._components:
            self.io.log_exception('No network component set with name {}'.format(name))
        return self._components[name]

    def has_component(self, name):
        return name in self._components

    @classmethod
    def from_config(cls, conf, **properties):
        """bmtk/simulator/core/simulator_network.py:207-267."""
        network = cls(**properties)
        if isinstance(conf, str):
            from .config import Config
            conf = Config.from_json(conf)
        for name, value in conf.get('components', {}).items():
            network.add_component(name, value)
        nets = conf.get('networks', {})
        for nodes_cfg in nets.get('nodes', []):
            for pop in sonata.load_nodes(nodes_cfg['nodes_file'], nodes_cfg['node_types_file'],
                                         nodes_cfg.get('population')):
                network.add_nodes(pop)
        for edges_cfg in nets.get('edges', []):
            if not edges_cfg.get('enabled', True):
                continue
            for pop in sonata.load_edges(edges_cfg['edges_file'], edges_cfg['edge_types_file'],
                                         edges_cfg.get('population')):
                network.add_edges(pop)
        for name, ns in conf.get('node_sets', {}).items():
            network.add_node_set(name, ns)
        return network

    # ---- populations
    def add_nodes(self, node_population):
        name = node_population.name
        if name in self._node_populations:
            self.io.log_exception('There are multiple node populations with name {}.'.format(name))
        self._preprocess_node_types(node_population)
        self._node_populations[name] = node_population

    def _load_json(self, component, fname):
        path = fname if os.path.isabs(fname) else os.path.join(self.get_component(component), fname)
        with open(path, 'r') as f:
            return json.load(f)

    def _preprocess_node_types(self, pop):
        """dynamics_params file -> dict; Allen-format GLIF files -> NEST parameters
        (core/sonata_reader/node_adaptor.py:102-165, pointnet/sonata_adaptors.py:154-167)."""
        for t in np.unique(pop.node_type_ids):
            row = pop.types_table[t]
            if row.get('model_type') == 'virtual':
                continue
            dp = row.get('dynamics_params')
            if isinstance(dp, str):
                dp = self._load_json('point_neuron_models_dir', dp)
            elif dp is None:
                dp = {}
            mt = row.get('model_template')
            if isinstance(mt, str) and mt.startswith('nest:glif') and dp.get('type') == 'GLIF':
                mt, dp = convert_aibs2nest(mt, dp)
            row['model_template'] = mt
            row['dynamics_params'] = dp

    def add_edges(self, edge_population):
        for t in np.unique(edge_population.edge_type_ids):
            row = edge_population.types_table[t]
            dp = row.get('dynamics_params')
            if isinstance(dp, str):
                row['dynamics_params'] = self._load_json('synaptic_models_dir', dp)
            elif dp is None:
                row['dynamics_params'] = {}
            mt = row.get('model_template')
            if isinstance(mt, str) and mt.startswith('nest:'):
                row['model_template'] = mt[5:]
        self._edge_populations.append(edge_population)

    @property
    def node_populations(self):
        return list(self._node_populations.values())

    def get_node_populations(self):
        return self.node_populations

    def get_node_population(self, name):
        return self._node_populations[name]

    def add_node_set(self, name, node_set):
        self._node_sets[name] = node_set

    def get_node_set(self, node_set):
        """A name of a population / of a node_sets entry / 'all', a filter dict, or a list of ids
        (core/simulator_network.py:101-131)."""
        if isinstance(node_set, str):
            if node_set in self._node_sets:
                return self.get_node_set(self._node_sets[node_set])
            if node_set in self._node_populations:
                return NodeSet({'population': node_set}, self)
            if node_set == 'all':
                return NodeSet({}, self)
            self.io.log_exception('Unknown node set {}'.format(node_set))
        return NodeSet(node_set, self)

    def find_edges(self, source_nodes=None, target_nodes=None):
        out = self._edge_populations
        if source_nodes is not None:
            out = [e for e in out if e.source_population == source_nodes]
        if target_nodes is not None:
            out = [e for e in out if e.target_population == target_nodes]
        return out

    # ---- building
    def build(self):
        self.build_nodes()
        self.build_recurrent_edges()

    def _node_type_params(self, pop, type_id):
        row = pop.types_table[type_id]
        mt = row.get('model_template') or ''
        model = mt.split(':', 1)[1] if ':' in mt else mt
        dp = dict(row.get('dynamics_params') or {})
        if model in _GLIF_MODES:
            r, a, v = _GLIF_MODES[model]
            dp.setdefault('spike_dependent_threshold', r)
            dp.setdefault('after_spike_currents', a)
            dp.setdefault('adapting_threshold', v)
        elif model in ('iaf_psc_alpha', 'iaf_psc_delta'):
            dp['model'] = model
        elif model != 'glif_psc':
            self.io.log_exception('node type {} of population {}: model_template "{}" is not supported by this '
                                  'engine (supported: nest:glif_psc, the nest:glif_lif*_psc variants and '
                                  'nest:iaf_psc_alpha, nest:iaf_psc_delta)'.format(type_id, pop.name, mt))
        dp.pop('type', None)
        return {k: (np.asarray(v).tolist() if isinstance(v, np.ndarray) else v) for k, v in dp.items()}

    def build_nodes(self):
        """One batch per node type in order of first appearance (sonata_adaptors.py:132-152); engine
        ids follow creation order (pointnetwork.py:144-159)."""
        if self._nodes_built:
            return
        type_index = []
        for pop in self.node_populations:
            if pop.is_mixed:
                self.io.log_exception('population {} mixes virtual and non-virtual nodes; not supported '
                                      '(the reference cannot run it either)'.format(pop.name))
            if pop.is_virtual:
                continue
            if pop.has_dynamics_params:
                self.io.log_exception('population {}: per-node dynamics_params in the nodes file are not supported'
                                      .format(pop.name))
            _, first = np.unique(pop.node_type_ids, return_index=True)
            for t in pop.node_type_ids[np.sort(first)]:
                ids = pop.node_ids[pop.node_type_ids == t]
                n0 = len(self._gid_pool)
                self.types.append(self._node_type_params(pop, t))
                self.type_labels.append((pop.name, int(t)))
                type_index.append(np.full(len(ids), len(self.types) - 1, dtype=np.uint16))
                self._gid_pool.add_nestids(pop.name, ids, np.arange(n0, n0 + len(ids)))
        self.type_index = np.concatenate(type_index) if type_index else np.zeros(0, dtype=np.uint16)
        self._nodes_built = True

    # ---- several ranks: contiguous blocks of engine ids, balanced by in-degree
    def partition(self, rank, world):
        """Cuts the engine ids into `world` contiguous blocks whose in-degree sums (recurrent and virtual
        edges) are as equal as contiguous cuts allow, and makes this network expand only the edges that end
        in block `rank`: a rank then never holds the other ranks' weight, delay and port arrays. Returns the
        block bounds (world + 1 engine ids). Call before build_recurrent_edges / add_spike_trains."""
        if not self._nodes_built:
            self.build_nodes()
        n = len(self._gid_pool)
        indeg = np.zeros(n, dtype=np.int64)
        for epop in self._edge_populations:
            tp = epop.target_population
            if tp not in self._node_populations or self._node_populations[tp].is_virtual:
                continue
            indeg += np.bincount(self._gid_pool.get_nestids(tp, epop.target_node_ids), minlength=n)
        self.block_bounds = balanced_bounds(indeg, world)
        self.target_block = (int(self.block_bounds[rank]), int(self.block_bounds[rank + 1]))
        return self.block_bounds

    def _expand_edges(self, epop, src_lookup, trg_pop_name):
        """Per edge type: weight, delay, port (sonata_adaptors.py:268-357). Yields dict batches with
        sources already mapped by `src_lookup` and targets mapped to engine ids."""
        nsyns_col, w_col, d_col = epop.column('nsyns'), epop.column('syn_weight'), epop.column('delay')
        local = None
        if self.target_block is not None:
            # with several ranks only the edges that end in this rank's block are expanded
            trg_all = self._gid_pool.get_nestids(trg_pop_name, epop.target_node_ids)
            local = (trg_all >= self.target_block[0]) & (trg_all < self.target_block[1])
        # batches in ascending edge_type_id, the order of the reference's groupby('etid') (sonata_adaptors.py:298)
        for t in np.unique(epop.edge_type_ids):
            row = epop.types_table[t]
            m = np.nonzero(epop.edge_type_ids == t if local is None else (epop.edge_type_ids == t) & local)[0]
            n = len(m)
            model = row.get('model_template')
            if model not in (None, 'static_synapse'):
                self.io.log_exception('edge type {} of {}: synapse model "{}" is not supported (static_synapse only)'
                                      .format(t, epop.name, model))
            dyn = row.get('dynamics_params') or {}
            port = int(dyn.get('receptor_type', 1) or 1) - 1
            if port < 0 or port > 3:
                self.io.log_exception('edge type {}: receptor_type {} outside 1..4'.format(t, dyn.get('receptor_type')))
            if d_col is not None:
                delay = d_col[m].astype(np.float64)
            elif row.get('delay') is not None:
                delay = np.full(n, float(row['delay']))
            elif 'delay' in dyn:
                delay = np.full(n, float(dyn['delay']))
            else:
                delay = np.full(n, 1.0)          # NEST's static_synapse default
            wf = row.get('weight_function')
            if wf is not None:
                if not py_modules.has_synaptic_weight(wf):
                    self.io.log_exception('Unable to calculate synaptic weight for "{}" edges, missing "weight_function" '
                                          'attribute value {} function.'.format(epop.name, wf))
                import pandas as pd
                edges_df = pd.DataFrame({'edge_type_id': epop.edge_type_ids[m], 'source_node_id': epop.source_node_ids[m],
                                         'target_node_id': epop.target_node_ids[m]})
                for c, col in (('nsyns', nsyns_col), ('syn_weight', w_col), ('delay', d_col)):
                    if col is not None:
                        edges_df[c] = col[m]
                for c, v in row.items():
                    if c not in edges_df.columns and c not in ('dynamics_params',):
                        edges_df[c] = v
                src_df = self._node_populations[epop.source_population].to_dataframe().loc[epop.source_node_ids[m]]
                trg_df = self._node_populations[epop.target_population].to_dataframe().loc[epop.target_node_ids[m]]
                weight = np.asarray(py_modules.synaptic_weight(wf)(edges_df, src_df, trg_df), dtype=np.float64)
            else:
                nsyns = nsyns_col[m] if nsyns_col is not None else (row.get('nsyns') if row.get('nsyns') is not None else 1)
                if w_col is not None:
                    sw = w_col[m]
                elif row.get('syn_weight') is not None:
                    sw = row['syn_weight']
                else:
                    raise Exception('Could not find syn_weight value')
                weight = np.asarray(nsyns * np.asarray(sw, dtype=np.float64), dtype=np.float64)
                if weight.ndim == 0:
                    weight = np.full(n, float(weight))
            if self._dt is not None and n and np.any(delay < self._dt * (1 - 1e-9)):
                msg = 'BadDelay: delay {} ms of edge type {} in {} is shorter than the resolution dt = {} ms'.format(
                    float(delay.min()), t, epop.name, self._dt)
                self.io.log_error(msg)
                raise BadDelay(msg)
            trg = self._gid_pool.get_nestids(trg_pop_name, epop.target_node_ids[m])
            ports = np.full(n, port, dtype=np.uint8)
            # iaf_psc_alpha targets have no receptor ports: the sign of the weight picks the
            # excitatory (port 0) or inhibitory (port 1) alpha current
            iaf = self._type_is_iaf()[self.type_index[trg]] if n else np.zeros(0, dtype=bool)
            if np.any(iaf):
                ports = np.where(iaf, (weight < 0).astype(np.uint8), ports).astype(np.uint8)
            # iaf_psc_delta targets have one receptor: weights of either sign are jumps of V_m
            delta = self._type_is_delta()[self.type_index[trg]] if n else np.zeros(0, dtype=bool)
            if np.any(delta):
                ports = np.where(delta, 0, ports).astype(np.uint8)
            yield dict(src=src_lookup(epop.source_node_ids[m]), trg=trg, weight=weight, delay=delay, port=ports,
                       edge_type_id=int(t), population=epop.name)

    def _type_is_delta(self):
        return np.array([t.get('model') == 'iaf_psc_delta' for t in self.types], dtype=bool)

    def _type_is_iaf(self):
        return np.array([t.get('model') == 'iaf_psc_alpha' for t in self.types], dtype=bool)

    def build_recurrent_edges(self):
        """pointnetwork.py:161-173: every edge population between non-virtual populations."""
        if self._edges_built:
            return
        if not self._nodes_built:
            self.build_nodes()
        if self.io.mpi_size > 1 and self.target_block is None:
            self.partition(self.io.mpi_rank, self.io.mpi_size)
        for epop in self._edge_populations:
            sp, tp = epop.source_population, epop.target_population
            if sp not in self._node_populations or tp not in self._node_populations:
                self.io.log_exception('edges {}: unknown node population {} or {}'.format(epop.name, sp, tp))
            if self._node_populations[sp].is_virtual:
                continue
            if self._node_populations[tp].is_virtual:
                self.io.log_exception('edges {}: virtual cells cannot be targets'.format(epop.name))
            look = (lambda ids, _sp=sp: self._gid_pool.get_nestids(_sp, ids))
            self.edge_batches.extend(self._expand_edges(epop, look, tp))
        self._edges_built = True

    def add_spike_trains(self, spike_trains, node_set, sg_params=None):
        """Virtual cells of `node_set` replay `spike_trains`; their edges are connected
        (pointnetwork.py:187-227). Spike times <= 0 are refused (pointnetwork.py:58-59)."""
        if not self._nodes_built:
            self.build_nodes()
        ns = node_set if isinstance(node_set, NodeSet) else self.get_node_set(node_set)
        for pop in ns.populations():
            if not pop.is_virtual or pop.name in self.virtual_index:
                continue
            ids = np.sort(pop.node_ids)
            vidx = np.arange(self.n_virtual, self.n_virtual + len(ids), dtype=np.int64)
            self.virtual_index[pop.name] = (ids, vidx)
            self.n_virtual += len(ids)
            v_all, t_all = [], []
            fast = hasattr(spike_trains, 'to_dataframe') and pop.name in getattr(spike_trains, 'populations', [])
            if fast:
                df = spike_trains.to_dataframe(populations=pop.name, with_population_col=False)
                t = df['timestamps'].values.astype(np.float64)
                nid = df['node_ids'].values.astype(np.int64)
                keep = np.isin(nid, ids)
                t, nid = t[keep], nid[keep]
                if np.any(t <= 0.0):
                    self.io.log_exception('spike train of population {} contains negative/zero time, unable to run '
                                          'virtual cell'.format(pop.name))
                v_all.append(vidx[np.searchsorted(ids, nid)])
                t_all.append(t)
            else:
                for nid, v in zip(ids, vidx):
                    try:
                        st = spike_trains.get_times(node_id=int(nid), population=pop.name)
                    except TypeError:
                        st = spike_trains.get_times(node_id=int(nid))
                    if st is None or len(st) == 0:
                        continue
                    st = np.sort(np.asarray(st, dtype=np.float64))
                    if np.any(st <= 0.0):
                        self.io.log_exception('spike train {} contains negative/zero time, unable to run virtual '
                                              'cell'.format(st))
                    v_all.append(np.full(len(st), v, dtype=np.int64))
                    t_all.append(st)
            if v_all:
                self.input_spikes.append((np.concatenate(v_all), np.concatenate(t_all)))
            for epop in self.find_edges(source_nodes=pop.name):
                tp = epop.target_population
                if self._node_populations[tp].is_virtual:
                    continue

                def look(q, _ids=ids, _vidx=vidx):
                    pos = np.searchsorted(_ids, q)
                    return -1 - _vidx[pos]          # virtual sources are marked negative: -(index+1)
                self.virtual_edge_batches.extend(self._expand_edges(epop, look, tp))

    # ---- what the simulator hands to the engine
    def edge_arrays(self):
        """All edges as engine arrays: (src, trg, weight f32, delay ms f64, port u8); virtual source v
        becomes n_neurons + v."""
        n = len(self._gid_pool)
        parts = self.edge_batches + self.virtual_edge_batches
        if not parts:
            z = np.zeros(0)
            return z.astype(np.uint32), z.astype(np.uint32), z.astype(np.float32), z, z.astype(np.uint8)
        src = np.concatenate([np.asarray(b['src'], dtype=np.int64) for b in parts])
        src = np.where(src < 0, n + (-1 - src), src)
        trg = np.concatenate([b['trg'] for b in parts])
        w = np.concatenate([b['weight'] for b in parts]).astype(np.float32)
        d = np.concatenate([b['delay'] for b in parts])
        p = np.concatenate([b['port'] for b in parts])
        return src.astype(np.uint32), trg.astype(np.uint32), w, d, p
