"""Allen Cell Types GLIF parameter files -> NEST `glif_psc` parameters.

Same mapping as the reference's converter for NEST >= 2.20
(bmtk/simulator/pointnet/glif_utils.py:259-418), written as one table-driven function: SI units
to mV / pF / nS / ms / pA, V_th = coeffs.th_inf*th_inf + El_reference, g = coeffs.G / R_input,
t_ref = spike_cut_length*dt, asc_decay = 1/asc_tau, fixed tau_syn = [5.5, 8.5, 2.8, 5.8] ms and the
three mode flags per model name. Applied when a node type's dynamics_params carry
"type": "GLIF" (bmtk/simulator/pointnet/sonata_adaptors.py:154-167).
"""
import numpy as np

TAU_SYN = (5.5, 8.5, 2.8, 5.8)

# model_template -> (spike_dependent_threshold, after_spike_currents, adapting_threshold)
_MODES = {
    'nest:glif_lif_psc': (False, False, False),
    'nest:glif_lif_r_psc': (True, False, False),
    'nest:glif_lif_asc_psc': (False, True, False),
    'nest:glif_lif_r_asc_psc': (True, True, False),
    'nest:glif_lif_r_asc_a_psc': (True, True, True),
}


def convert_aibs2nest(model_template, dynamics_params):
    """-> (model_template, params). Templates other than the five *_psc GLIF names pass through."""
    if model_template not in _MODES:
        return model_template, dynamics_params
    r_mode, asc_mode, a_mode = _MODES[model_template]
    c = dynamics_params
    k = c['coeffs']
    e_ref = c['El_reference'] * 1.0e03
    p = {
        'V_m': c['El'] * 1.0e03 + e_ref,
        'V_th': k['th_inf'] * c['th_inf'] * 1.0e03 + e_ref,
        'g': k['G'] / c['R_input'] * 1.0e09,
        'E_L': c['El'] * 1.0e03 + e_ref,
        'C_m': k['C'] * c['C'] * 1.0e12,
        't_ref': c['spike_cut_length'] * c['dt'] * 1.0e03,
    }
    if r_mode:
        th = c['threshold_dynamics_method']['params']
        rs = c['voltage_reset_method']['params']
        p['th_spike_add'] = th['a_spike'] * 1.0e03
        p['th_spike_decay'] = th['b_spike'] * 1.0e-03
        p['voltage_reset_fraction'] = rs['a']
        p['voltage_reset_add'] = rs['b'] * 1.0e03
        if a_mode:
            p['th_voltage_index'] = th['a_voltage'] * k['a'] * 1.0e-03
            p['th_voltage_decay'] = th['b_voltage'] * k['b'] * 1.0e-03
    else:
        p['V_reset'] = e_ref
    if asc_mode:
        p['asc_init'] = np.array(c['init_AScurrents']) * 1.0e12
        p['asc_decay'] = 1.0 / np.array(c['asc_tau_array']) * 1.0e-03
        p['asc_amps'] = np.array(c['asc_amp_array']) * np.array(k['asc_amp_array']) * 1.0e12
        if r_mode:
            p['asc_r'] = (1.0, 1.0)
    p['tau_syn'] = np.array(TAU_SYN)
    p['spike_dependent_threshold'] = r_mode
    p['after_spike_currents'] = asc_mode
    p['adapting_threshold'] = a_mode
    return 'nest:glif_psc', p
