"""Host-side failure detection between steps.

The reference has none: a dead rank simply hangs the next NCCL call (no timeout is passed to
``init_process_group``, cubework/initialize.py:33-35).  Here every rank publishes a heartbeat (step counter
+ wall time, or a failure record) in the job's key-value store after each step and, before launching the next
one, checks its peers: a peer that reported an exception, or whose heartbeat is older than ``timeout_s``, raises
:class:`PeerFailure` on the host, so no kernel that would wait for that peer is launched.  Device-side waits are
time-bounded as a second line of defence (``cubework_b200.ops.ext.check_status``).
"""
import time
import traceback

import torch.distributed as dist


class PeerFailure(RuntimeError):

    def __init__(self, rank, reason):
        super().__init__(f"rank {rank}: {reason}")
        self.rank, self.reason = rank, reason


class Heartbeat:

    def __init__(self, store=None, rank=None, world_size=None, prefix="cubework_b200/hb"):
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.prefix = prefix
        self.beat(-1)

    def _key(self, rank):
        return f"{self.prefix}/{rank}"

    def beat(self, step):
        self.store.set(self._key(self.rank), f"ok|{step}|{time.time():.3f}")

    def fail(self, exc):
        """Tell the peers this rank is going away (call from an ``except`` block, between steps)."""
        msg = "".join(traceback.format_exception_only(type(exc), exc)).strip().replace("|", "/")
        self.store.set(self._key(self.rank), f"failed|{msg}|{time.time():.3f}")

    def leave(self):
        self.store.set(self._key(self.rank), f"left||{time.time():.3f}")

    def check_peers(self, timeout_s=30.0, min_step=None):
        """Raises PeerFailure if a peer failed, left, or has been silent for ``timeout_s`` seconds."""
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                state, info, stamp = self.store.get(self._key(r)).decode().split("|")
            except Exception as e:  # noqa: BLE001
                raise PeerFailure(r, f"no heartbeat record ({type(e).__name__})")
            if state == "failed":
                raise PeerFailure(r, f"reported an exception: {info}")
            if state == "left":
                raise PeerFailure(r, "left the job")
            if now - float(stamp) > timeout_s:
                raise PeerFailure(r, f"silent for {now - float(stamp):.1f} s (last step {info})")
            if min_step is not None and int(info) < min_step:
                raise PeerFailure(r, f"is behind: step {info} < {min_step}")
