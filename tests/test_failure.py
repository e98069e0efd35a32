"""Failure detection without any GPU fault: every failure is produced on the host, among CPU/gloo ranks.

* a rank raises between steps -> its peers learn of it from the heartbeat store before their next launch;
* a rank silently stops beating -> peers time it out;
* a rank never joins a collective -> the short process-group timeout ends the peers' collective with an error;
* an asynchronous gradient reduction that nobody collected -> ``synchronize`` raises.
"""
import os
import time

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_dist


def _peer_exception():
    from cubework_b200.utils.health import Heartbeat, PeerFailure
    hb = Heartbeat()
    dist.barrier()
    x = torch.ones(4)
    dist.all_reduce(x)          # step 0 works on every rank
    hb.beat(0)
    dist.barrier()
    if dist.get_rank() == 1:
        try:
            raise ValueError("loss is NaN")
        except ValueError as e:
            hb.fail(e)          # between steps, nothing in flight
        return
    time.sleep(0.5)
    with pytest.raises(PeerFailure) as info:
        hb.check_peers(timeout_s=30)
    assert info.value.rank == 1 and "loss is NaN" in info.value.reason
    # no collective is launched towards the dead rank: the test returns instead of hanging


def _peer_silent():
    from cubework_b200.utils.health import Heartbeat, PeerFailure
    hb = Heartbeat()
    dist.barrier()
    if dist.get_rank() == 1:
        time.sleep(3.0)         # stops beating (but stays alive so the store survives)
        return
    deadline = time.time() + 20
    while True:
        hb.beat(1)
        try:
            hb.check_peers(timeout_s=1.0)
        except PeerFailure as e:
            assert e.rank == 1 and "silent" in e.reason
            break
        assert time.time() < deadline, "silent peer was never detected"
        time.sleep(0.2)


def _collective_timeout():
    import datetime
    g = dist.new_group([0, 1], backend="gloo", timeout=datetime.timedelta(seconds=2))
    x = torch.ones(4)
    if dist.get_rank() == 1:
        time.sleep(6)           # never joins the collective
        return
    t0 = time.time()
    with pytest.raises(RuntimeError):
        dist.all_reduce(x, group=g)
    assert time.time() - t0 < 30


def _uncollected_async_grad():
    from cubework_b200.parallel import common
    p = torch.nn.Parameter(torch.zeros(3))

    class NeverDone:

        def wait(self):
            raise RuntimeError("reduction lost")

    common.push_async_grad(NeverDone(), torch.zeros(3), id(p))
    with pytest.raises(RuntimeError):
        common.synchronize([p])
    common._bucket.pending.clear()


def test_peer_exception_is_seen_before_next_launch():
    run_dist(_peer_exception, 2, tp="1d", tp_size=2)


def test_silent_peer_times_out():
    run_dist(_peer_silent, 2, tp="1d", tp_size=2)


def test_missing_rank_ends_collective_with_error():
    run_dist(_collective_timeout, 2)


def test_uncollected_async_gradient_raises():
    _uncollected_async_grad()
