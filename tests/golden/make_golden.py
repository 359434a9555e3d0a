"""Generates tests/golden/glif_known_answers.json from the reference tree.

Run in a container that has the reference checked out (not needed at test time):
    python tests/golden/make_golden.py /path/to/reference

For each of the five *_psc GLIF variants of the reference's only numerical known-answer test
(bmtk/tests/simulator/pointnet/test_glif_utils.py:16-44) it stores
  - the Allen-format input file content (glif_models/637930677_*.json),
  - the NEST-format parameters produced by the reference's own converter
    (bmtk/simulator/pointnet/glif_utils.py:259-418, loaded by file path with a stub `nest`
    module that only reports version 'nest-3.3'),
  - the stimulus of the test (spike times/weights, receptor, resolution, duration) and the
    expected spike times with their tolerance, parsed from the test file's text.
"""
import importlib.util
import json
import os
import re
import sys
import types

import numpy as np


def load_reference_converter(ref):
    nest = types.ModuleType('nest')
    nest.__version__ = 'nest-3.3'
    sys.modules['nest'] = nest
    pkg = types.ModuleType('refpointnet')
    pkg.__path__ = [os.path.join(ref, 'bmtk/simulator/pointnet')]
    sys.modules['refpointnet'] = pkg
    mods = {}
    for name in ('nest_utils', 'glif_utils'):
        spec = importlib.util.spec_from_file_location(
            'refpointnet.' + name, os.path.join(pkg.__path__[0], name + '.py'))
        m = importlib.util.module_from_spec(spec)
        sys.modules['refpointnet.' + name] = m
        spec.loader.exec_module(m)
        mods[name] = m
    return mods['glif_utils'].convert_aibs2nest


def jsonable(v):
    if isinstance(v, np.ndarray):
        return [float(x) for x in v]
    if isinstance(v, (tuple, list)):
        return [jsonable(x) for x in v]
    if isinstance(v, (np.floating,)):
        return float(v)
    if isinstance(v, (np.bool_,)):
        return bool(v)
    return v


def main(ref):
    convert = load_reference_converter(ref)
    tdir = os.path.join(ref, 'bmtk/tests/simulator/pointnet')
    text = open(os.path.join(tdir, 'test_glif_utils.py')).read()
    block = text[text.index('@pytest.mark.parametrize'):text.index('def test_converter_psc')]
    cases = re.findall(r"\('([^']+)',\s*'([^']+)',\s*\[([^\]]*)\]\)", block)
    assert len(cases) == 5, cases
    res = float(re.search(r'"resolution":\s*([0-9.]+)', text).group(1))
    times = [float(x) for x in re.search(r"'spike_times':\s*\[([^\]]*)\]", text).group(1).split(',')]
    weight = float(re.search(r"'spike_weights':\s*\[([0-9.]+)\]", text).group(1))
    receptor = int(re.search(r'"receptor_type":\s*(\d+)', text).group(1))
    tstop = float(re.search(r'nest\.Simulate\(([0-9.]+)\)', text).group(1))
    atol = float(re.search(r'atol=([0-9.]+)', text).group(1))
    out = {
        'source': 'bmtk/tests/simulator/pointnet/test_glif_utils.py:16-44',
        'resolution_ms': res, 'tstop_ms': tstop, 'atol_ms': atol,
        'stimulus': {'spike_times_ms': times, 'spike_weight_pA': weight, 'receptor_type': receptor,
                     'delay_ms': 1.0, 'delay_note': 'static_synapse default delay (no delay in syn_spec)'},
        'cases': [],
    }
    for model, path, expected in cases:
        aibs = json.load(open(os.path.join(tdir, path)))
        nest_model, params = convert(model, aibs)
        out['cases'].append({
            'model_template': model, 'fixture': path, 'aibs_params': aibs,
            'nest_model': nest_model,
            'nest_params': {k: jsonable(v) for k, v in params.items()},
            'expected_spike_times_ms': [float(x) for x in expected.split(',') if x.strip()],
        })
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'glif_known_answers.json')
    with open(dst, 'w') as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print('wrote', dst)


if __name__ == '__main__':
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get('BMTK_REFERENCE', '/root/reference'))
