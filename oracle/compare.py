"""Comparison of two recorded spike lists under the tolerances the path is graded on (test
infrastructure, like the rest of oracle/): spike times within one step over an initial span,
first step at which the (stamp, id)-sorted lists differ, firing rate per node type as
bmtk/analyzer/spike_trains.py:302-349 defines it (spikes / neurons / seconds).
"""
import numpy as np


def first_divergence(st_a, id_a, st_b, id_b):
    """First stamp at which two (stamp, id)-sorted lists differ; None if they are identical."""
    st_a, st_b = np.asarray(st_a, dtype=np.int64), np.asarray(st_b, dtype=np.int64)
    id_a, id_b = np.asarray(id_a, dtype=np.int64), np.asarray(id_b, dtype=np.int64)
    n = min(len(st_a), len(st_b))
    neq = np.nonzero((st_a[:n] != st_b[:n]) | (id_a[:n] != id_b[:n]))[0]
    if len(neq):
        return int(min(st_a[neq[0]], st_b[neq[0]]))
    if len(st_a) == len(st_b):
        return None
    return int((st_a if len(st_a) > n else st_b)[n])


def within_one_step(st_a, id_a, st_b, id_b, upto_step, n_ids):
    """Spike trains of every neuron compared over stamps <= upto_step, in both directions.

    Spikes stamped upto_step or upto_step + 1 in one list may pair with a partner just outside the
    span in the other; the span of list b is therefore widened by one step when a neuron's counts
    differ by exactly that boundary spike.
    Returns dict(n_a, n_b, neurons_with_other_count, spikes_beyond_one_step, ok).
    """
    st_a, st_b = np.asarray(st_a, dtype=np.int64), np.asarray(st_b, dtype=np.int64)
    id_a, id_b = np.asarray(id_a, dtype=np.int64), np.asarray(id_b, dtype=np.int64)

    def pick(st, ids, upto):
        m = st <= upto
        o = np.lexsort((st[m], ids[m]))
        return st[m][o], ids[m][o]
    sa, ia = pick(st_a, id_a, upto_step)
    sb, ib = pick(st_b, id_b, upto_step)
    ca, cb = np.bincount(ia, minlength=n_ids), np.bincount(ib, minlength=n_ids)
    differ = np.nonzero(ca != cb)[0]
    if len(differ):
        # a spike stamped upto_step whose partner is stamped upto_step + 1 is not a difference
        sb1, ib1 = pick(st_b, id_b, upto_step + 1)
        sa1, ia1 = pick(st_a, id_a, upto_step + 1)
        cb1, ca1 = np.bincount(ib1, minlength=n_ids), np.bincount(ia1, minlength=n_ids)
        last_a = np.zeros(n_ids, dtype=np.int64)
        last_b = np.zeros(n_ids, dtype=np.int64)
        last_a[ia] = sa          # sorted by (id, stamp): the last write per id is its latest stamp
        last_b[ib] = sb
        d = differ
        edge = d[((ca[d] == cb[d] + 1) & (cb1[d] == ca[d]) & (last_a[d] == upto_step)) |
                 ((cb[d] == ca[d] + 1) & (ca1[d] == cb[d]) & (last_b[d] == upto_step))]
        differ = np.setdiff1d(differ, edge)
    same = ca == cb
    keep_a, keep_b = same[ia], same[ib]
    da = np.abs(sa[keep_a] - sb[keep_b])
    beyond = int(np.count_nonzero(da > 1))
    return dict(n_a=int(len(sa)), n_b=int(len(sb)), neurons_with_other_count=int(len(differ)),
                spikes_beyond_one_step=beyond, ok=bool(len(differ) == 0 and beyond == 0))


def rates_by_type(type_index, n_types, spike_ids, t_ms):
    """Mean firing rate (Hz) of every node type: spikes / neurons / seconds."""
    type_index = np.asarray(type_index)
    cnt = np.bincount(type_index[np.asarray(spike_ids, dtype=np.int64)], minlength=n_types)
    n = np.bincount(type_index, minlength=n_types)
    return cnt / np.maximum(n, 1) / (t_ms * 1e-3), cnt, n


def rate_agreement(type_index, n_types, ids_a, ids_b, t_ms, rel=0.02, sigmas=3.0):
    """Per-type rates of two runs. Once two runs of a recurrent network have parted (one spike a step
    earlier is enough), they are two realisations of the same process and a type's spike counts
    differ by counting noise: for counts c_a, c_b of (near-)Poisson trains the difference has standard
    deviation sqrt(c_a + c_b). The allowance is rel x rate plus `sigmas` of that, in Hz.
    Returns dict(max_rel_err, worst_type, ok, rates_a, rates_b, allowance)."""
    ra, ca, n = rates_by_type(type_index, n_types, ids_a, t_ms)
    rb, cb, _ = rates_by_type(type_index, n_types, ids_b, t_ms)
    noise = sigmas * np.sqrt(ca + cb) / np.maximum(n, 1) / (t_ms * 1e-3)
    allow = rel * rb + noise
    err = np.abs(ra - rb)
    relerr = err / np.maximum(rb, 1e-12)
    worst = int(np.argmax(relerr))
    return dict(max_rel_err=float(relerr[worst]), worst_type=worst, ok=bool(np.all(err <= allow)),
                within_rel_only=bool(np.all(err <= rel * rb)), rates_a=ra, rates_b=rb, allowance=allow)
