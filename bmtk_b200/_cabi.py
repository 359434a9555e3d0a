"""ctypes binding of the C ABI declared in include/bmtk_b200.h.

This is the stub a maintainer of bmtk.simulator.pointnet would add in place of `import nest`:
every function below stands for the PyNEST calls named beside its declaration in the header.
The shared object is bmtk_b200/lib/libbmtk_b200.so, built in-tree by `python -m bmtk_b200.build`.
There is no CPU implementation behind it: loading fails loudly when the library is missing, and
creating an engine fails loudly when no CUDA device is present.
"""
import ctypes as C
import os

MAX_PORTS = 4
MODEL_GLIF_PSC, MODEL_IAF_PSC_ALPHA, MODEL_IAF_PSC_DELTA = 0, 1, 2
LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'lib', 'libbmtk_b200.so')

# recorder variables (BMTK_VAR_*), by the names NEST's glif_psc gives its recordables
RECORDABLES = {'V_m': 0, 'I_syn': 1, 'ASCurrents_sum': 2, 'threshold': 3, 'threshold_spike': 4, 'threshold_voltage': 5, 'I': 6}

OK, E_INVALID, E_CUDA, E_OVERFLOW, E_UNSUPPORTED, E_COMM, E_DELAY = 0, -1, -2, -3, -4, -5, -6


class GlifParams(C.Structure):
    """bmtk_glif_params: NEST glif_psc parameters under their NEST names (fp64)."""
    _fields_ = [
        ('V_m', C.c_double), ('V_th', C.c_double), ('g', C.c_double), ('E_L', C.c_double),
        ('C_m', C.c_double), ('t_ref', C.c_double), ('V_reset', C.c_double),
        ('asc_init', C.c_double * 2), ('asc_decay', C.c_double * 2), ('asc_amps', C.c_double * 2),
        ('asc_r', C.c_double * 2), ('tau_syn', C.c_double * MAX_PORTS),
        ('th_spike_add', C.c_double), ('th_spike_decay', C.c_double),
        ('voltage_reset_fraction', C.c_double), ('voltage_reset_add', C.c_double),
        ('th_voltage_index', C.c_double), ('th_voltage_decay', C.c_double),
        ('n_ports', C.c_int32), ('spike_dependent_threshold', C.c_int32),
        ('after_spike_currents', C.c_int32), ('adapting_threshold', C.c_int32),
        ('I_e', C.c_double), ('model', C.c_int32), ('reserved', C.c_int32),
    ]


class EngineError(RuntimeError):
    def __init__(self, code, message):
        super().__init__('bmtk_b200 error %d: %s' % (code, message))
        self.code = code


class BadDelay(EngineError):
    """A synaptic delay is shorter than the resolution (NEST raises BadDelay for the same input,
    bmtk/simulator/pointnet/pointnetwork.py:234-243)."""


_P = C.c_void_p
_SIGNATURES = {
    'bmtk_last_error': (C.c_char_p, []),
    'bmtk_version': (C.c_char_p, []),
    'bmtk_engine_create': (C.c_int, [C.POINTER(_P), C.c_int, C.c_double]),
    'bmtk_engine_destroy': (C.c_int, [_P]),
    'bmtk_engine_set_nodes': (C.c_int, [_P, C.c_uint64, C.c_uint64, C.c_uint64, _P, C.c_int32, _P]),
    'bmtk_engine_set_virtual': (C.c_int, [_P, C.c_uint64]),
    'bmtk_engine_add_edges': (C.c_int, [_P, C.c_uint64, _P, _P, _P, _P, _P]),
    'bmtk_engine_set_input_spikes': (C.c_int, [_P, C.c_uint64, _P, _P]),
    'bmtk_engine_set_poisson': (C.c_int, [_P, _P, C.c_uint64]),
    'bmtk_engine_set_clamp_events': (C.c_int, [_P, C.c_uint64, _P, _P, _P]),
    'bmtk_engine_record_spikes': (C.c_int, [_P, C.c_int]),
    'bmtk_engine_record_vm': (C.c_int, [_P, C.c_uint64, _P, C.c_uint32]),
    'bmtk_engine_record_state': (C.c_int, [_P, C.c_uint64, _P, C.c_uint32, C.c_int32, _P]),
    'bmtk_engine_set_option': (C.c_int, [_P, C.c_char_p, C.c_int64]),
    'bmtk_comm_unique_id': (C.c_int, [_P, C.c_char_p]),
    'bmtk_engine_comm_init': (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_char_p]),
    'bmtk_engine_finalize': (C.c_int, [_P]),
    'bmtk_engine_local_layout': (C.c_int, [_P, _P]),
    'bmtk_engine_set_global_layout': (C.c_int, [_P, _P]),
    'bmtk_engine_exchange_layout': (C.c_int, [_P, _P]),
    'bmtk_exchange_layout_compare': (C.c_int, [_P, _P, C.c_int]),
    'bmtk_engine_p2p_handle': (C.c_int, [_P, _P]),
    'bmtk_engine_p2p_connect': (C.c_int, [_P, _P]),
    'bmtk_engine_p2p_buffer': (C.c_int, [_P, C.POINTER(_P)]),
    'bmtk_engine_p2p_connect_pointers': (C.c_int, [_P, C.POINTER(_P)]),
    'bmtk_engine_run': (C.c_int, [_P, C.c_uint64]),
    'bmtk_engine_spike_count': (C.c_int, [_P, C.POINTER(C.c_uint64)]),
    'bmtk_engine_fetch_spikes': (C.c_int, [_P, C.c_uint64, _P, _P, C.POINTER(C.c_uint64)]),
    'bmtk_engine_trace_samples': (C.c_int, [_P, C.POINTER(C.c_uint64)]),
    'bmtk_engine_fetch_trace': (C.c_int, [_P, C.c_uint64, _P, C.POINTER(C.c_uint64)]),
    'bmtk_engine_get_state': (C.c_int, [_P, C.c_char_p, _P]),
    'bmtk_engine_csr_info': (C.c_int, [_P] + [C.POINTER(C.c_uint64)] * 2 + [C.POINTER(C.c_uint32)] * 4),
    'bmtk_engine_get_csr': (C.c_int, [_P, _P, _P, _P]),
    'bmtk_engine_get_counter': (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_uint64)]),
    'bmtk_propagate_spikes': (C.c_int, [_P, _P, C.c_uint32, C.c_uint32, _P, _P, _P, C.c_uint32, C.c_uint32, C.c_int, _P]),
    'bmtk_propagate_spikes_noalloc': (C.c_int, [_P, _P, C.c_uint32, C.c_uint32, _P, _P, _P, C.c_uint32, C.c_uint32, _P]),
    'bmtk_probe_scatter_reductions': (C.c_int, [C.c_int, C.c_uint64, C.c_uint64, C.c_int, C.POINTER(C.c_double)]),
    'bmtk_generate_distance_edges': (C.c_int, [_P, C.c_int, C.c_uint64, _P, _P, _P, _P, _P, C.POINTER(C.c_uint64)]),
    'bmtk_engine_save_state': (C.c_int, [_P, C.c_char_p]),
    'bmtk_engine_load_state': (C.c_int, [_P, C.c_char_p]),
    'bmtk_engine_p2p_pingpong': (C.c_int, [_P, C.c_int, C.c_int, C.c_uint32, C.POINTER(C.c_double)]),
    'bmtk_engine_block_profile': (C.c_int, [_P, C.c_uint64, _P, C.POINTER(C.c_uint64)]),
    'bmtk_engine_mark': (C.c_int, [_P, C.c_int]),
    'bmtk_engine_elapsed_ms': (C.c_int, [_P, C.c_int, C.c_int, C.POINTER(C.c_double)]),
}

_lib = None


def exported_symbols():
    """Names include/bmtk_b200.h declares (used by the symbol-table test)."""
    return sorted(_SIGNATURES)


def load():
    """dlopen the engine library and set every prototype. Raises when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError('%s is missing: run `python -m bmtk_b200.build` (needs nvcc). '
                              'bmtk_b200 has no CPU fallback.' % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(code):
    if code != OK:
        msg = load().bmtk_last_error().decode('utf-8', 'replace')
        raise (BadDelay if code == E_DELAY else EngineError)(code, msg)
