"""SONATA nodes / edges files as arrays.

The reference walks these files through per-row Node/Edge objects
(bmtk/utils/sonata/{file,file_root,population,group,types_table}.py); the engine wants whole
columns, so populations are loaded here as numpy arrays with the same semantics:
  * types CSV: space separated, index column node_type_id / edge_type_id, NONE/NULL -> None
    (bmtk/utils/sonata/types_table.py:31-35,170-220, utils.py:61-67);
  * nodes.h5: /nodes/<pop>/{node_id, node_type_id, node_group_id, node_group_index} and
    /nodes/<pop>/<group>/<columns> (population.py:161-179, group.py:38-65);
  * edges.h5: /edges/<pop>/{source_node_id[@node_population], target_node_id[@node_population],
    edge_type_id, edge_group_id, edge_group_index} and /edges/<pop>/<group>/<columns>
    (population.py:349-378,416-455). edge_group_index is honoured (the reference pairs whole
    group datasets with population order, which is the same thing for builder-written files).
"""
import numpy as np
import pandas as pd

from .. import h5io


def _clean(v):
    if v is None:
        return None
    if isinstance(v, float) and np.isnan(v):
        return None
    if isinstance(v, (np.integer,)):
        return int(v)
    if isinstance(v, (np.floating,)):
        return float(v)
    if isinstance(v, (np.bool_,)):
        return bool(v)
    return v


class TypesTable(object):
    """type id -> dict of the CSV columns (NaN/NONE -> None)."""

    def __init__(self, index_col):
        self.index_col = index_col
        self.columns = []
        self._rows = {}

    def add_csv(self, path):
        df = pd.read_csv(path, sep=' ', na_values=['NONE', 'NULL', 'None'], keep_default_na=True)
        if self.index_col not in df.columns:
            raise Exception('{} has no column {}'.format(path, self.index_col))
        for c in df.columns:
            if c not in self.columns and c != self.index_col:
                self.columns.append(c)
        for _, row in df.iterrows():
            tid = int(row[self.index_col])
            if tid in self._rows:
                raise Exception('{}: duplicate {} {}'.format(path, self.index_col, tid))
            self._rows[tid] = {c: _clean(row[c]) for c in df.columns}
        return self

    def __getitem__(self, type_id):
        return self._rows[int(type_id)]

    def __contains__(self, type_id):
        return int(type_id) in self._rows

    @property
    def type_ids(self):
        return list(self._rows.keys())

    def column(self, name, type_ids, default=None):
        return [self._rows[int(t)].get(name, default) for t in type_ids]


class _Population(object):
    def __init__(self, name, types_table):
        self.name = name
        self.types_table = types_table
        self.groups = {}           # group id -> {column: array}

    def _read_groups(self, grp, group_ids):
        for gid in np.unique(group_ids):
            g = grp[str(int(gid))]
            cols = {}
            for k in g.keys():
                node = g[k]
                if hasattr(node, 'keys'):
                    continue      # dynamics_params sub-group: per-node parameters are not supported
                cols[k] = node[()]
            self.groups[int(gid)] = cols
        self.has_dynamics_params = any('dynamics_params' in grp[str(int(g))].keys() for g in np.unique(group_ids))


class NodePopulation(_Population):
    def __init__(self, name, h5grp, types_table):
        super().__init__(name, types_table)
        self.node_ids = h5grp['node_id'][()].astype(np.int64)
        self.node_type_ids = h5grp['node_type_id'][()].astype(np.int64)
        n = len(self.node_ids)
        self.group_ids = h5grp['node_group_id'][()].astype(np.int64) if 'node_group_id' in h5grp else np.zeros(n, np.int64)
        self.group_index = h5grp['node_group_index'][()].astype(np.int64) if 'node_group_index' in h5grp \
            else np.arange(n, dtype=np.int64)
        self._read_groups(h5grp, self.group_ids)
        missing = set(np.unique(self.node_type_ids).tolist()) - set(types_table.type_ids)
        if missing:
            raise Exception('node population {}: node_type_id(s) {} missing from the node types table'.format(
                name, sorted(missing)))
        self._df = None

    def __len__(self):
        return len(self.node_ids)

    @property
    def type_ids(self):
        return self.node_type_ids

    def type_column(self, name, default=None):
        """Per-node value of a node-types column."""
        lut = {t: self.types_table[t].get(name, default) for t in np.unique(self.node_type_ids)}
        return np.array([lut[t] for t in self.node_type_ids], dtype=object)

    @property
    def is_virtual(self):
        mt = [self.types_table[t].get('model_type') for t in np.unique(self.node_type_ids)]
        return all(m == 'virtual' for m in mt)

    @property
    def is_mixed(self):
        mt = [self.types_table[t].get('model_type') == 'virtual' for t in np.unique(self.node_type_ids)]
        return any(mt) and not all(mt)

    def to_dataframe(self):
        """One row per node (index node_id): group columns, then node-type columns."""
        if self._df is None:
            df = pd.DataFrame({'node_id': self.node_ids, 'node_type_id': self.node_type_ids})
            cols = sorted({c for g in self.groups.values() for c in g})
            for c in cols:
                vals = np.empty(len(self), dtype=object)
                vals[:] = None
                for gid, g in self.groups.items():
                    if c in g:
                        m = self.group_ids == gid
                        vals[m] = np.asarray(g[c])[self.group_index[m]]
                try:
                    df[c] = pd.to_numeric(pd.Series(vals), errors='raise')
                except (ValueError, TypeError):
                    df[c] = vals
            for c in self.types_table.columns:
                if c not in df.columns:
                    df[c] = self.type_column(c)
            self._df = df.set_index('node_id', drop=False)
        return self._df

    def filter(self, **query):
        """node_ids matching equality (or membership, for lists) on node / node-type columns
        (bmtk/utils/sonata/group.py:245-312)."""
        df = self.to_dataframe()
        mask = np.ones(len(df), dtype=bool)
        for k, v in query.items():
            if k in ('node_ids',):
                k = 'node_id'
            if k not in df.columns:
                return np.zeros(0, dtype=np.int64)
            col = df[k].values
            mask &= np.isin(col, list(v)) if isinstance(v, (list, tuple, np.ndarray)) else (col == v)
        return df['node_id'].values[mask].astype(np.int64)


class EdgePopulation(_Population):
    def __init__(self, name, h5grp, types_table):
        super().__init__(name, types_table)
        s, t = h5grp['source_node_id'], h5grp['target_node_id']
        self.source_node_ids = s[()].astype(np.int64)
        self.target_node_ids = t[()].astype(np.int64)
        self.source_population = _as_str(s.attrs.get('node_population') if 'node_population' in s.attrs else None)
        self.target_population = _as_str(t.attrs.get('node_population') if 'node_population' in t.attrs else None)
        self.edge_type_ids = h5grp['edge_type_id'][()].astype(np.int64)
        n = len(self.edge_type_ids)
        self.group_ids = h5grp['edge_group_id'][()].astype(np.int64) if 'edge_group_id' in h5grp else np.zeros(n, np.int64)
        self.group_index = h5grp['edge_group_index'][()].astype(np.int64) if 'edge_group_index' in h5grp \
            else np.arange(n, dtype=np.int64)
        self._read_groups(h5grp, self.group_ids)
        missing = set(np.unique(self.edge_type_ids).tolist()) - set(types_table.type_ids)
        if missing:
            raise Exception('edge population {}: edge_type_id(s) {} missing from the edge types table'.format(
                name, sorted(missing)))

    def __len__(self):
        return len(self.edge_type_ids)

    @property
    def type_ids(self):
        return self.edge_type_ids

    def column(self, name):
        """Per-edge values of a group column, or None when no group has it."""
        if not any(name in g for g in self.groups.values()):
            return None
        out = None
        for gid, g in self.groups.items():
            m = self.group_ids == gid
            if name in g:
                vals = np.asarray(g[name])[self.group_index[m]]
                if out is None:
                    out = np.full(len(self), np.nan, dtype=np.float64) if vals.dtype.kind in 'iuf' \
                        else np.empty(len(self), dtype=object)
                out[m] = vals
        return out


def _as_str(v):
    if v is None:
        return None
    if isinstance(v, bytes):
        return v.decode()
    if isinstance(v, np.ndarray):
        return _as_str(v.ravel()[0])
    return str(v)


def load_nodes(nodes_file, node_types_file, population=None):
    """-> list of NodePopulation (bmtk/simulator/core/sonata_reader/network_reader.py:120-127)."""
    table = TypesTable('node_type_id').add_csv(node_types_file)
    with h5io.File(nodes_file, 'r') as h:
        root = h['nodes']
        names = [population] if population else list(root.keys())
        return [NodePopulation(n, root[n], table) for n in names]


def load_edges(edges_file, edge_types_file, population=None):
    table = TypesTable('edge_type_id').add_csv(edge_types_file)
    with h5io.File(edges_file, 'r') as h:
        root = h['edges']
        names = [population] if population else list(root.keys())
        return [EdgePopulation(n, root[n], table) for n in names]
