"""Drop-in counterpart of bmtk.simulator.pointnet (bmtk/simulator/pointnet/__init__.py:23-27):

    from bmtk_b200 import pointnet
    configure = pointnet.Config.from_json('config.json'); configure.build_env()
    network = pointnet.PointNetwork.from_config(configure)
    sim = pointnet.PointSimulator.from_config(configure, network)
    sim.run()
"""
from .config import Config
from .pointnetwork import BadDelay, GidPool, NodeSet, PointNetwork
from .pointsimulator import PointSimulator
from .pyfunction_cache import (add_cell_model, add_cell_processor, add_synapse_model, add_weight_function,
                               cell_model, model_processing, synapse_model, synaptic_weight)
from .spike_trains import PoissonSpikeGenerator, SpikeTrains
from . import io_tools, modules
