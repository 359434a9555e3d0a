"""`h5py` stand-in for the verification shim: bmtk_b200.h5io under h5py's names (the subset the
reference's SONATA readers and report writers use)."""
import numpy as np

from bmtk_b200 import h5io

__version__ = '3.0.0-h5io'
version = type('version', (), {'version': __version__, 'hdf5_version': '1.10-subset'})

Group = (h5io.RGroup, h5io.WGroup)
Dataset = (h5io.RDataset, h5io.WDataset)


class _FileMeta(type):
    def __instancecheck__(cls, obj):
        return isinstance(obj, (h5io.RFile, h5io.WFile))


class File(metaclass=_FileMeta):
    """h5py.File(path, mode): returns the h5io file object; isinstance(x, h5py.File) works on it."""

    def __new__(cls, path, mode='r', **kw):
        return h5io.File(path, mode, **kw)


def special_dtype(vlen=None, **kw):
    return np.dtype(object) if vlen is not None else np.dtype(object)


def string_dtype(encoding='utf-8', length=None):
    return np.dtype(object) if length is None else np.dtype('S%d' % length)


def check_dtype(**kw):
    return None
