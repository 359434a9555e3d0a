"""bmtk_propagate_spikes: stateless spike delivery over caller-owned device memory, against a
numpy statement of the same sums (fp64) and against itself (deterministic = bitwise stable)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def make_case(oracle, seed, n_rows=500, n_targets=300, n_edges=40000, ring_slots=12, max_delay=9):
    rng = np.random.default_rng(seed)
    src = rng.integers(0, n_rows, n_edges)
    trg = rng.integers(0, n_targets, n_edges)
    d = rng.integers(1, max_delay + 1, n_edges)
    port = rng.integers(0, 4, n_edges)
    w = rng.normal(size=n_edges).astype(np.float32)
    rowptr, order = oracle.build_csr(n_rows, src, trg, w, d, port)
    n_pad = (n_targets + 3) // 4 * 4
    tb = max(1, int(np.ceil(np.log2(n_pad))))
    packed = (d[order].astype(np.uint32) << (tb + 2)) | (port[order].astype(np.uint32) << tb) | trg[order].astype(np.uint32)
    entries = np.empty((n_edges, 2), dtype=np.uint32)
    entries[:, 0] = packed
    entries[:, 1] = w[order].view(np.uint32)
    return dict(rowptr=rowptr.astype(np.uint64), entries=entries, tb=tb, n_pad=n_pad, ring_slots=ring_slots,
                trg=trg[order], d=d[order], port=port[order], w=w[order], n_rows=n_rows)


def reference_ring(case, ring, spike_src, spike_step):
    """fp64 statement: ring[(step + delay) % S][port][target] += weight for every row entry."""
    S, n_pad = case['ring_slots'], case['n_pad']
    out = ring.astype(np.float64).reshape(S, 4, n_pad)
    for s, n in zip(spike_src, spike_step):
        b, e = int(case['rowptr'][s]), int(case['rowptr'][s + 1])
        np.add.at(out, ((n + case['d'][b:e]) % S, case['port'][b:e], case['trg'][b:e]), case['w'][b:e].astype(np.float64))
    return out.reshape(-1)


def call(cabi, name, case, t, spike_src, spike_step, ring, *extra):
    import torch
    src = torch.from_numpy(spike_src.astype(np.int32)).cuda()
    stp = torch.from_numpy(spike_step.astype(np.int32)).cuda()
    fn = getattr(cabi, name)
    rc = fn(C.c_void_p(t['rowptr'].data_ptr()), C.c_void_p(t['entries'].data_ptr()), case['tb'], len(spike_src),
            C.c_void_p(src.data_ptr()), C.c_void_p(stp.data_ptr()), C.c_void_p(ring.data_ptr()), case['ring_slots'],
            case['n_pad'], *extra)
    torch.cuda.synchronize()
    return rc


def to_device(case):
    import torch
    return dict(rowptr=torch.from_numpy(case['rowptr'].view(np.int64)).cuda(),
                entries=torch.from_numpy(case['entries'].view(np.int32)).cuda())


@pytest.mark.parametrize('deterministic', [1, 0])
def test_stateless_delivery_matches_numpy(cabi, oracle, deterministic):
    import torch
    case = make_case(oracle, 1)
    t = to_device(case)
    rng = np.random.default_rng(2)
    ring = torch.zeros(case['ring_slots'] * 4 * case['n_pad'], dtype=torch.float32, device='cuda')
    expect = np.zeros(ring.numel())
    for k in range(2):
        src = rng.integers(0, case['n_rows'], 700)
        step = rng.integers(1000, 1010, 700)
        assert call(cabi, 'bmtk_propagate_spikes', case, t, src, step, ring, deterministic, None) == 0
        expect = reference_ring(case, expect, src, step)
        got = ring.cpu().numpy().astype(np.float64)
        assert np.allclose(got, expect, rtol=1e-4, atol=1e-3)


def test_stateless_deterministic_is_bitwise_stable(cabi, oracle):
    import torch
    case = make_case(oracle, 3)
    t = to_device(case)
    rng = np.random.default_rng(4)
    src = rng.integers(0, case['n_rows'], 2000)
    step = rng.integers(0, 6, 2000)
    outs = []
    for perm in (np.arange(2000), rng.permutation(2000)):     # the order of the spike list must not matter
        ring = torch.zeros(case['ring_slots'] * 4 * case['n_pad'], dtype=torch.float32, device='cuda')
        assert call(cabi, 'bmtk_propagate_spikes', case, t, src[perm], step[perm], ring, 1, None) == 0
        outs.append(ring.cpu().numpy())
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))


def test_stateless_argument_errors(cabi):
    from bmtk_b200 import _cabi
    assert cabi.bmtk_propagate_spikes(None, None, 4, 0, None, None, None, 4, 16, 1, None) == _cabi.E_INVALID
