"""The "inputs" and "reports" sections of a configuration as lists of settings objects.

Same parsing rules as bmtk/simulator/utils/simulation_inputs.py:44-129 and
simulation_reports.py:30-355: `module` (and `input_type` for inputs) are required, `enabled: false`
drops an entry, membrane reports get default cells / file_name / tmp_dir, and a spikes report is
always appended from the "output" section (spikes_file, spikes_file_csv, spikes_sort_order,
compression 'gzip', tmp_dir = output_dir, cache_to_disk).
"""


class SimInput(object):
    def __init__(self, name, input_type, module, params):
        self.name, self.input_type, self.module = name, input_type, module
        self.params = {k: v for k, v in params.items() if k not in ('module', 'input_type', 'enabled')}
        self.enabled = params.get('enabled', True)

    @property
    def node_set(self):
        return self.params.get('node_set', None)


def inputs_from_config(cfg):
    out = []
    for name, params in cfg.get('inputs', {}).items():
        if 'module' not in params:
            raise Exception('inputs setting {} does not specify the "module".'.format(name))
        if 'input_type' not in params:
            raise Exception('inputs setting {} does not specify the "input_type".'.format(name))
        si = SimInput(name, params['input_type'], params['module'], params)
        if si.enabled:
            out.append(si)
    return out


class SimReport(object):
    def __init__(self, name, module, params):
        self.report_name, self.module = name, module
        self.params = {k: v for k, v in params.items() if k not in ('module', 'enabled')}
        self.enabled = params.get('enabled', True)

    @property
    def node_set(self):
        return self.params.get('cells', 'all')


_MEMBRANE = ('membrane_report', 'multimeter_report', 'multimeter')


def reports_from_config(cfg):
    output = cfg.get('output', {})
    out_dir = output.get('output_dir', '.')
    out, has_spikes = [], False
    for name, params in cfg.get('reports', {}).items():
        if not params.get('enabled', True):
            continue
        if 'module' not in params:
            raise Exception('report {} does not specify the module.'.format(name))
        module = params['module']
        if module == 'spikes_report':
            has_spikes = True
            continue                      # the reference's SpikesReport.build returns None here too
        r = SimReport(name, module, params)
        if module in _MEMBRANE:
            p = r.params
            p.setdefault('cells', 'biophysical')
            p.setdefault('tmp_dir', out_dir)
            if 'file_name' not in p:
                p['file_name'] = name if name.endswith(('.h5', '.hdf', '.hdf5')) else '{}.h5'.format(name)
            for k in ('sections', 'buffer', 'transform'):
                p.pop(k, None)
        out.append(r)
    if not has_spikes:
        params = {
            'spikes_file': output.get('spikes_file'), 'compression': output.get('compression', 'gzip'),
            'spikes_file_csv': output.get('spikes_file_csv'), 'spikes_file_nwb': output.get('spikes_file_nwb'),
            'spikes_sort_order': output.get('spikes_sort_order'), 'tmp_dir': output.get('output_dir', out_dir),
            'cache_to_disk': output.get('cache_to_disk', True),
        }
        out.append(SimReport('spikes_report', 'spikes_report', params))
    return out
