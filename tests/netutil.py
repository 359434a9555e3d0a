"""Test helpers: the oracle side of a workloads.Network (tests only)."""
import numpy as np

from oracle import glif_oracle as O


def oracle_from_network(net, n_threads=1, f32_weights=True):
    """OracleSim over the same nodes, edges, inputs and clamps as `net` (full network)."""
    assert net.lo == 0 and net.hi == net.n_neurons, 'oracle needs the whole network'
    w = net.weight.astype(np.float32).astype(np.float64) if f32_weights else net.weight.astype(np.float64)
    sim = O.OracleSim(net.types, net.type_index, net.dt, n_virtual=net.n_virtual, src=net.src, trg=net.trg,
                      weight=w, delay_steps=net.delay_steps, port=net.port, n_threads=n_threads)
    if net.poisson_rate_hz is not None:
        steps, srcs = O.poisson_spikes(net.poisson_rate_hz, net.dt, net.poisson_seed, 0, net.n_steps)
        sim.set_input_spikes(steps, srcs)
    elif len(net.in_virt):
        sim.set_input_spikes(net.in_stamp.astype(np.int64) - 1, net.in_virt)
    if len(net.clamp_step):
        # device deltas are fp32; give the oracle the same numbers
        sim.set_clamp_events(net.clamp_step, net.clamp_target, net.clamp_delta.astype(np.float64))
    if len(net.probe_ids):
        sim.set_probes(net.probe_ids, 1)
    return sim


def rates_by_type(net, spike_ids, t_ms):
    """Mean firing rate (Hz) per node type: spikes / neurons / seconds
    (the definition of bmtk/analyzer/spike_trains.py:302-349)."""
    cnt = np.bincount(net.type_index[np.asarray(spike_ids, dtype=np.int64)], minlength=len(net.types))
    n = np.bincount(net.type_index, minlength=len(net.types))
    return cnt / np.maximum(n, 1) / (t_ms * 1e-3)


def oracle_f32_from_network(net, window, chunk_steps=4096):
    """OracleSimF32 (the engine's fp32 arithmetic, deterministic delivery, restated on the CPU) over `net`."""
    assert net.lo == 0 and net.hi == net.n_neurons
    sim = O.OracleSimF32(net.types, net.type_index, net.dt, window, chunk_steps, n_virtual=net.n_virtual, src=net.src,
                         trg=net.trg, weight=net.weight.astype(np.float32), delay_steps=net.delay_steps, port=net.port)
    if net.poisson_rate_hz is not None:
        sim.set_poisson(net.poisson_rate_hz, net.poisson_seed)
    elif len(net.in_virt):
        sim.set_input_spikes(net.in_stamp.astype(np.int64) - 1, net.in_virt)
    if len(net.clamp_step):
        sim.set_clamp_events(net.clamp_step, net.clamp_target, net.clamp_delta)
    if len(net.probe_ids):
        sim.set_probes(net.probe_ids, 1)
    return sim
