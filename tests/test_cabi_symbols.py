"""The C-ABI library loads and exports every function include/bmtk_b200.h declares. No compute
is attempted without a GPU; without one, creating an engine must fail loudly."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, 'include', 'bmtk_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(bmtk_[a-z0-9_]+)\s*\(', text)))


def test_header_and_binding_agree():
    from bmtk_b200 import _cabi
    assert declared_functions() == _cabi.exported_symbols()


def test_library_exports_every_declared_symbol(cabi):
    for name in declared_functions():
        assert hasattr(cabi, name), name
    assert b'sm_100a' in cabi.bmtk_version()


def test_struct_layout_matches_header(cabi):
    from bmtk_b200 import _cabi
    # 7 + 4*2 + 4 + 6 doubles, 4 int32, I_e double, model + reserved int32
    assert C.sizeof(_cabi.GlifParams) == (7 + 8 + 4 + 6) * 8 + 4 * 4 + 8 + 8


def test_argument_errors_do_not_need_a_gpu(cabi):
    from bmtk_b200 import _cabi
    h = C.c_void_p()
    assert cabi.bmtk_engine_create(C.byref(h), 0, -1.0) == _cabi.E_INVALID
    assert b'dt' in cabi.bmtk_last_error()
    assert cabi.bmtk_engine_run(None, 10) == _cabi.E_INVALID


def test_engine_fails_loudly_without_a_device(cabi):
    import torch
    if torch.cuda.is_available():
        pytest.skip('a CUDA device is present')
    from bmtk_b200.engine import Engine
    from bmtk_b200._cabi import EngineError
    with pytest.raises(EngineError) as ei:
        Engine(0.1)
    assert 'no CPU path' in str(ei.value)
