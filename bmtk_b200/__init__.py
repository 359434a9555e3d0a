"""bmtk_b200: a B200-native engine for the point-neuron path of the Brain Modeling Toolkit.

`bmtk_b200.pointnet` mirrors bmtk.simulator.pointnet (Config, PointNetwork, PointSimulator);
`bmtk_b200.engine.Engine` is the handle on the C ABI (include/bmtk_b200.h) that the CUDA kernels
sit behind. There is no CPU execution path.
"""
__version__ = '0.1.0'
