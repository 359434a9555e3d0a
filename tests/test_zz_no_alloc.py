"""bmtk_propagate_spikes_noalloc: the delivery entry point for callers that cannot allocate.

A plugin inside another application's memory pool, or a process whose network already fills the
GPU, cannot afford a cudaMalloc per delivery. This test calls the allocation-free entry point
through the C ABI and requires its ring buffer to equal, bit for bit, what the allocating entry
point (bmtk_propagate_spikes, deterministic) produces from the same inputs - both sum in the same
fixed order - on two calls in a row that accumulate into the same ring, and checks that inputs
beyond the built-in scratch are refused with a clear message and leave the ring untouched.
Collected last so that a failure here cannot hide the other tests of a run that stops early.
"""
import numpy as np
import pytest

from test_gpu_propagate_stateless import call, make_case, reference_ring, to_device

pytestmark = pytest.mark.gpu


def test_noalloc_equals_allocating_entry_point_twice_in_a_row(cabi, oracle):
    import torch
    case = make_case(oracle, 11)
    t = to_device(case)
    rng = np.random.default_rng(12)
    n_cells = case['ring_slots'] * 4 * case['n_pad']
    ring_ref = torch.zeros(n_cells, dtype=torch.float32, device='cuda')
    ring_new = torch.zeros(n_cells, dtype=torch.float32, device='cuda')
    expect = np.zeros(n_cells)
    for k in range(2):
        src = rng.integers(0, case['n_rows'], 900 + 300 * k)
        step = rng.integers(50, 58, len(src))
        assert call(cabi, 'bmtk_propagate_spikes', case, t, src, step, ring_ref, 1, None) == 0
        assert call(cabi, 'bmtk_propagate_spikes_noalloc', case, t, src, step, ring_new, None) == 0, \
            cabi.bmtk_last_error()
        a, b = ring_ref.cpu().numpy(), ring_new.cpu().numpy()
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), 'call %d differs' % k
        expect = reference_ring(case, expect, src, step)
        assert np.allclose(b.astype(np.float64), expect, rtol=1e-4, atol=1e-3)
    assert np.abs(ring_new.cpu().numpy()).sum() > 0


def test_noalloc_refuses_what_does_not_fit(cabi, oracle):
    import torch
    from bmtk_b200 import _cabi
    case = make_case(oracle, 13, n_rows=50, n_targets=64, n_edges=50 * 8000)   # rows of ~8000 entries
    t = to_device(case)
    ring = torch.zeros(case['ring_slots'] * 4 * case['n_pad'], dtype=torch.float32, device='cuda')
    # too many spikes for the built-in scratch
    src = np.zeros(5000, dtype=np.int64)
    rc = call(cabi, 'bmtk_propagate_spikes_noalloc', case, t, src, src, ring, None)
    assert rc == _cabi.E_INVALID and b'at most 4096' in cabi.bmtk_last_error()
    # few spikes, but their rows hold more events than fit: refused before the ring is touched
    src = np.arange(50, dtype=np.int64)
    rc = call(cabi, 'bmtk_propagate_spikes_noalloc', case, t, src, np.zeros(50, dtype=np.int64), ring, None)
    assert rc == _cabi.E_OVERFLOW and b'at most 262144' in cabi.bmtk_last_error()
    assert float(ring.abs().sum()) == 0.0
    # and the entry point still works afterwards
    src = np.arange(20, dtype=np.int64)
    assert call(cabi, 'bmtk_propagate_spikes_noalloc', case, t, src, np.zeros(20, dtype=np.int64), ring, None) == 0
    exp = reference_ring(case, np.zeros(ring.numel()), src, np.zeros(20, dtype=np.int64))
    assert np.allclose(ring.cpu().numpy().astype(np.float64), exp, rtol=1e-4, atol=1e-3)


def test_noalloc_event_total_cannot_wrap(cabi):
    """4096 listings of one row of 1 048 640 entries add up to 2^32 + 262 144 events: formed in 32 bits
    that total would read 262 144 and pass the capacity check. It must be refused, in both deterministic
    entry points, with the ring untouched."""
    import torch
    from bmtk_b200 import _cabi
    n_row = 1048640
    n_pad, tb, S = 64, 6, 4
    entries = np.empty((n_row, 2), dtype=np.uint32)
    entries[:, 0] = (1 << (tb + 2)) | (np.arange(n_row, dtype=np.uint32) % 60)     # delay 1, port 0
    entries[:, 1] = np.float32(1.0).view(np.uint32)
    case = dict(rowptr=np.array([0, n_row], dtype=np.uint64), entries=entries, tb=tb, n_pad=n_pad, ring_slots=S)
    t = to_device(case)
    ring = torch.zeros(S * 4 * n_pad, dtype=torch.float32, device='cuda')
    src = np.zeros(4096, dtype=np.int64)
    assert (4096 * n_row) % (1 << 32) == 262144
    rc = call(cabi, 'bmtk_propagate_spikes_noalloc', case, t, src, src, ring, None)
    assert rc == _cabi.E_OVERFLOW, cabi.bmtk_last_error()
    assert float(ring.abs().sum()) == 0.0
    rc = call(cabi, 'bmtk_propagate_spikes', case, t, src, src, ring, 1, None)
    assert rc == _cabi.E_OVERFLOW, cabi.bmtk_last_error()
    assert float(ring.abs().sum()) == 0.0
