"""Registries for user functions: synaptic_weight, synapse_model, cell_model, model_processing.

Same decorators and add_* helpers as the reference (bmtk/simulator/core/pyfunction_cache.py:171-324);
weight functions are called once per edge type with (edges_df, source_nodes_df, target_nodes_df)
and return one weight per edge (bmtk/simulator/pointnet/sonata_adaptors.py:319-335).
"""
from functools import wraps


class _Cache(object):
    def __init__(self):
        self.clear()

    def clear(self):
        self.synaptic_weights = {}
        self.synapse_models = {}
        self.cell_models = {}
        self.cell_processors = {}

    def add(self, table, name, func, overwrite=True):
        t = getattr(self, table)
        if overwrite or name not in t:
            t[name] = func

    def has_synaptic_weight(self, name):
        return name in self.synaptic_weights

    def synaptic_weight(self, name):
        return self.synaptic_weights[name]

    def has_synapse_model(self, name):
        return name in self.synapse_models

    def synapse_model(self, name):
        return self.synapse_models[name]

    def has_cell_model(self, directive, model_type):
        return (directive, model_type) in self.cell_models

    def cell_model(self, directive, model_type):
        return self.cell_models[(directive, model_type)]


py_modules = _Cache()


def _decorator(table, key_fn):
    def outer(*wargs, **wkwargs):
        if len(wargs) == 1 and callable(wargs[0]) and not wkwargs:
            func = wargs[0]
            py_modules.add(table, key_fn(func.__name__, {}), func)

            @wraps(func)
            def plain(*a, **k):
                return func(*a, **k)
            return plain

        def deco(func):
            py_modules.add(table, key_fn(wkwargs.get('name', func.__name__), wkwargs), func)

            @wraps(func)
            def wrapped(*a, **k):
                return func(*a, **k)
            return wrapped
        return deco
    return outer


synaptic_weight = _decorator('synaptic_weights', lambda n, kw: n)
synapse_model = _decorator('synapse_models', lambda n, kw: n)
model_processing = _decorator('cell_processors', lambda n, kw: n)
cell_model = _decorator('cell_models', lambda n, kw: (kw.get('directive'), kw.get('model_type')))


def add_weight_function(func, name=None, overwrite=True):
    py_modules.add('synaptic_weights', name or func.__name__, func, overwrite)


def add_synapse_model(func, name=None, overwrite=True):
    py_modules.add('synapse_models', name or func.__name__, func, overwrite)


def add_cell_model(func, directive, model_type, overwrite=True):
    py_modules.add('cell_models', (directive, model_type), func, overwrite)


def add_cell_processor(func, name=None, overwrite=True):
    py_modules.add('cell_processors', name or func.__name__, func, overwrite)


def load_py_modules(cell_models=None, syn_models=None, syn_weights=None):
    for mod, adder in ((cell_models, None), (syn_models, add_synapse_model), (syn_weights, add_weight_function)):
        if mod is None or adder is None:
            continue
        for name in dir(mod):
            f = getattr(mod, name)
            if callable(f) and not name.startswith('_') and getattr(f, '__module__', None) == mod.__name__:
                adder(f, name, overwrite=False)


# Default weight functions (bmtk/simulator/pointnet/default_setters/synaptic_weights.py:6-12):
# weight = syn_weight * nsyns
def default_weight_fnc(edge_props, source_nodes, target_nodes):
    import numpy as np
    nsyns = edge_props['nsyns'].values if 'nsyns' in edge_props else 1
    return np.asarray(edge_props['syn_weight'].values * nsyns, dtype=float)


add_weight_function(default_weight_fnc, 'default_weight_fnc', overwrite=False)
