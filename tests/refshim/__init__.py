"""Verification shim (test infrastructure): runs the UNMODIFIED reference adapter,
bmtk.simulator.pointnet of the reference tree, against this repository's engine contract.

BMTK PointNet touches NEST through a dozen PyNEST names and HDF5 through h5py. `install()` registers
two stand-in modules in sys.modules before the reference package is imported:

  nest  (tests/refshim/nest.py)  records Create / Connect / SetStatus calls, and on Simulate() builds an
        engine from them, runs it and writes the recorders' output as NEST-3 ascii files;
  h5py  (tests/refshim/h5py.py)  the bmtk_b200.h5io reader / writer under h5py's names.

The reference's own get_batches / GidPool / add_spike_trains / SpikesMod / MultimeterMod / IClampMod
code then runs as it is, so node batches, id bookkeeping, edge expansion (weights, delays, receptor
ports), virtual-cell spike times, clamp tables and the output files can be compared with what
bmtk_b200.pointnet produces from the same SONATA files, with no restatement of the adapter in between.
"""
import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def install(reference_root, engine_factory):
    """Puts the stand-ins and the reference tree on the import path; returns the fake `nest` module.
    `engine_factory(dt)` makes the engine Simulate() drives (the Engine API of bmtk_b200.engine)."""
    for name in [m for m in sys.modules if m == 'bmtk' or m.startswith('bmtk.')]:
        del sys.modules[name]
    _pandas_compat()
    import bmtk_b200.h5io  # noqa: F401  (decides on a real h5py before the stand-in becomes importable)
    if HERE not in sys.path:
        sys.path.insert(0, HERE)
    for name in ('nest', 'h5py'):
        sys.modules.pop(name, None)
    nest = importlib.import_module('nest')
    importlib.import_module('h5py')
    assert os.path.dirname(os.path.abspath(nest.__file__)) == HERE
    nest._engine_factory = engine_factory
    if reference_root not in sys.path:
        sys.path.insert(0, reference_root)
    return nest


def _pandas_compat():
    """The reference (bmtk 1.0.8) was written for pandas 1.x; two settings let it run unmodified under the
    pandas 3 of this image: string columns stay numpy object arrays (group.py:203 hands the column dtype to
    numpy), and DataFrame.append (removed in pandas 2; population.py:243-245) is provided through concat."""
    import pandas as pd
    try:
        pd.set_option('future.infer_string', False)
    except Exception:
        pass
    if not hasattr(pd.DataFrame, 'append'):
        def _append(self, other, ignore_index=False, **kw):
            return pd.concat([self, other], ignore_index=ignore_index)
        pd.DataFrame.append = _append


def uninstall(reference_root):
    for name in [m for m in sys.modules if m == 'bmtk' or m.startswith('bmtk.') or m in ('nest', 'h5py')]:
        del sys.modules[name]
    for p in (HERE, reference_root):
        while p in sys.path:
            sys.path.remove(p)
