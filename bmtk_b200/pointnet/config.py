"""SONATA simulation configuration: JSON with a manifest of path variables.

Semantics follow the reference parser (bmtk/utils/sonata/config/sonata_config.py:258-444) and its
simulator wrapper (bmtk/simulator/core/simulation_config.py:30-99, pointnet/config.py:31-48):
  * "$VAR" and "${VAR}" are replaced from the manifest, which may itself chain variables;
    built-ins ${configdir} ${configfname} ${workingdir} ${date} ${time} ${datetime}; keyword
    arguments given to from_json/from_dict override the manifest; a value that consists of
    nothing but one variable keeps the variable's type (int, bool, list ...).
  * "network" / "simulation" entries naming other JSON files are parsed and merged in.
  * in "output", log_file and spikes_file* are prefixed with output_dir unless absolute or
    already below it; "node_sets_file" is loaded into "node_sets".
  * attribute views (run, inputs, reports, networks, output, components, node_sets, output_dir,
    log_file, dt, tstop, ...) and build_env() = logging + (wipe and) create output_dir + copy of
    the resolved config.
"""
import datetime
import json
import os
import re

from .io_tools import io as _io

_VAR = re.compile(r'\$\{?[\w]+\}?')


class ConfigParser(object):
    def __init__(self, **usr_vars):
        self.usr_vars = usr_vars

    def parse(self, cfg):
        if isinstance(cfg, str):
            with open(cfg, 'r') as f:
                conf = json.load(f)
            conf['config_path'] = os.path.abspath(cfg)
            conf['config_dir'] = os.path.dirname(conf['config_path'])
        elif isinstance(cfg, dict):
            conf = dict(cfg)
        else:
            raise Exception('{} is not a file or file path.'.format(cfg))
        if 'config_path' not in conf:
            conf['config_path'] = os.path.join(os.getcwd(), 'sonata_config.json')
            conf['config_dir'] = os.path.dirname(conf['config_path'])
        manifest = self._manifest(conf)
        conf['manifest'] = manifest
        for k in list(conf.keys()):
            if k != 'manifest':
                conf[k] = self._insert(conf[k], manifest)
        for child in ('network', 'simulation'):
            if isinstance(conf.get(child), str):
                p = conf[child]
                p = p if p.startswith('/') else os.path.join(conf['config_dir'], p)
                sub = self.parse(p)
                del sub['config_path']
                conf.update(sub)
        self._post(conf)
        return conf

    @staticmethod
    def _builtins(conf):
        now = datetime.datetime.now()
        out = {'workingdir': os.getcwd()}
        if 'config_path' in conf:
            out['configdir'] = os.path.dirname(conf['config_path'])
            out['configfname'] = conf['config_path']
        out['time'] = now.strftime('%H-%M-%S')
        out['date'] = now.strftime('%Y-%m-%d')
        out['datetime'] = now.strftime('%Y-%m-%d_%H-%M-%S')
        return out

    def _manifest(self, conf):
        resolved = self._builtins(conf)
        if 'manifest' not in conf:
            return resolved
        todo = {(k[1:] if k.startswith('$') else k): v for k, v in conf['manifest'].items()}
        while todo:
            done = []
            for k, v in todo.items():
                val = self._substitute(v, resolved)
                if not isinstance(val, str) or '$' not in val:
                    resolved[k] = val
                    done.append(k)
            if not done:
                raise Exception('Unable to resolve manifest variables: {}'.format(set(todo)))
            for k in done:
                del todo[k]
        return resolved

    def _insert(self, obj, manifest):
        if isinstance(obj, str):
            return self._substitute(obj, manifest)
        if isinstance(obj, list):
            return [self._insert(x, manifest) for x in obj]
        if isinstance(obj, dict):
            return {k: (v if k == 'manifest' else self._insert(v, manifest)) for k, v in obj.items()}
        return obj

    def _substitute(self, s, manifest):
        if not isinstance(s, str):
            return s
        out = s
        for m in _VAR.finditer(s):
            tok = m.group()
            key = tok[2:-1] if tok.startswith('${') and tok.endswith('}') else tok[1:]
            if key in self.usr_vars:
                val = self.usr_vars[key]
            elif key in manifest:
                val = manifest[key]
            else:
                continue
            if isinstance(val, str) or len(s) > len(tok):
                out = out.replace(tok, str(val))
            else:
                return val       # the whole value is one non-string variable: keep its type
        return out

    @staticmethod
    def _post(conf):
        out = conf.get('output')
        if isinstance(out, dict) and 'output_dir' in out:
            od = out['output_dir']
            for k, p in list(out.items()):
                if (k == 'log_file' or k.startswith('spikes_file')) and isinstance(p, str):
                    if not (os.path.isabs(p) or p.startswith(od)):
                        out[k] = os.path.join(od, p)
        if 'node_sets' not in conf and 'node_sets_file' in conf:
            with open(conf['node_sets_file'], 'r') as f:
                conf['node_sets'] = json.load(f)


class Config(dict):
    """Parsed configuration: a dict with the attribute views the simulator reads."""

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.env_built = False
        self._io = _io
        self._set_props()

    # ---- factories (pointnet/config.py:41-48, sonata_config.py:148-172)
    @classmethod
    def from_json(cls, config_file, validator=None, validate=False, **opts):
        return cls(ConfigParser(**opts).parse(config_file))

    @classmethod
    def from_dict(cls, config_dict, validator=None, validate=False, **opts):
        return cls(ConfigParser(**opts).parse(config_dict))

    @classmethod
    def load(cls, config_file, validator=None, **opts):
        if isinstance(config_file, dict):
            return cls.from_dict(config_file, validator, **opts)
        if isinstance(config_file, str):
            if config_file.endswith(('yml', 'yaml')):
                raise NotImplementedError('yaml configurations are not supported')
            return cls.from_json(config_file, validator, **opts)
        raise Exception('Unable to open {}'.format(config_file))

    def validate(self):
        return True      # the reference has no schema for PointNet either (pointnet/config.py:30)

    @property
    def io(self):
        return self._io

    def _set_props(self):
        g = self.get
        self.run = g('run', {})
        self.conditions = g('conditions', {})
        self.components = g('components', {})
        self.output = g('output', {})
        self.inputs = g('inputs', {})
        self.reports = g('reports', {})
        self.networks = g('networks', {})
        self.engine = g('engine', {})      # knobs of this engine; the reference ignores the section
        self.output_dir = self.output.get('output_dir', '.')
        self.log_file = self.output.get('log_file', None)
        self.overwrite_output = self.output.get('overwrite_output_dir', False)
        self.nodes = self.networks.get('nodes', [])
        self.edges = self.networks.get('edges', [])
        self.gap_juncs = self.networks.get('gap_juncs', [])
        self.with_networks = 'networks' in self and len(self.nodes) > 0
        self.dt = self.run.get('dt', 0.1)
        self.tstart = self.run.get('tstart', 0.0)
        self.tstop = self.run.get('tstop', None)
        self.node_sets = g('node_sets', {})

    def copy_to_output(self):
        path = os.path.join(self.output_dir, os.path.basename(self['config_path']))
        out = {k: v for k, v in self.items() if k != 'manifest'}
        with open(path, 'w') as f:
            json.dump(out, f, indent=2)

    def build_env(self, force=False):
        """Logging, output directory (wiped when overwrite_output_dir), copy of the resolved config
        (bmtk/simulator/core/simulation_config.py:76-99)."""
        if self.env_built and not force:
            return
        o = self.output
        if 'log_format' in o:
            self.io.set_log_format(o['log_format'])
        if 'log_level' in o:
            self.io.set_log_level(o['log_level'])
        if 'log_to_console' in o:
            self.io.log_to_console = o['log_to_console']
        self.io.setup_output_dir(self.output_dir, self.log_file, self.overwrite_output)
        if self.io.mpi_rank == 0:
            self.copy_to_output()
        self.env_built = True


def from_json(config_file, validate=False, **opts):
    return Config.from_json(config_file, validate=validate, **opts)


def from_dict(config_dict, validate=False, **opts):
    return Config.from_dict(config_dict, validate=validate, **opts)
