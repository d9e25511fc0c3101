"""Host-side liveness check for the sharded paths (KV heads or sequences spread over the GPUs of one box).

The sharded kernels never wait for a peer without a bound: the fused gather's consumer gives up after its time
limit and raises a status bit (ingot_gather_wait). This module is the host half of the same policy. Before a rank
launches step s it publishes "I am about to run step s" in the job's key-value store and checks that every peer has
published the same within a time limit; a peer that has left (crashed, been preempted, stopped calling) is found on
the host, BEFORE any kernel that would wait for its data is launched, and the step raises PeerLost instead.
A rank only ever leaves between steps, with none of its kernels in flight.

The reference is single-device and has nothing like this; its only failure handling is the exception that
propagates to main() (src/main.cpp:458-461).
"""
import time


class PeerLost(RuntimeError):
    """A peer did not announce the step in time; .missing lists the ranks."""

    def __init__(self, step, missing):
        super().__init__(f"step {step}: no sign of rank(s) {missing} within the time limit")
        self.step, self.missing = step, missing


class PeerMonitor:
    """store: a torch.distributed Store (TCPStore / FileStore / the default group's store); any object with
    set(key, value) and a non-blocking check([keys]) -> bool works."""

    def __init__(self, store, rank, world, prefix="ingot/step", poll_s=0.005):
        self.store, self.rank, self.world, self.prefix, self.poll_s = store, rank, world, prefix, poll_s

    def _key(self, rank, step):
        return f"{self.prefix}/{step}/{rank}"

    def announce(self, step):
        self.store.set(self._key(self.rank, step), b"1")

    def missing(self, step):
        return [r for r in range(self.world) if r != self.rank and not self.store.check([self._key(r, step)])]

    def begin_step(self, step, timeout_s=5.0):
        """Announces `step` and returns once every peer has; raises PeerLost after timeout_s."""
        self.announce(step)
        deadline = time.monotonic() + timeout_s
        while True:
            gone = self.missing(step)
            if not gone:
                return
            if time.monotonic() > deadline:
                raise PeerLost(step, gone)
            time.sleep(self.poll_s)
