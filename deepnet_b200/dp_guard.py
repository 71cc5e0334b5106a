"""Host-side failure detection for the data-parallel ranks.

The reference has no multi-GPU layer and no failure handling beyond Python exceptions
(cudamat/cudamat.py:101-123).  With one NCCL all-reduce per update, a rank that is gone
(crashed, raised, never started) would leave the others waiting inside a collective that can
never complete.  The guard keeps that from happening: every rank publishes the number of the
update it is about to enqueue in a small file of a shared directory and, before it launches,
waits a bounded time until every other rank has published the same number.  A rank that leaves
says so (`leave()`, also called when `guarded()` sees an exception).  A missing or departed peer
is detected on the host, BEFORE the next launch: the survivors tear the communicator down
(`dp_abort`, nothing of theirs is in flight between updates) and raise `RankLost`.
"""
import os
import time


class RankLost(RuntimeError):
    pass


class RankGuard(object):
    def __init__(self, directory, world, rank, timeout=30.0, poll=0.005, on_abort=None):
        """directory: shared by the ranks of one launch (one node: any local path).  on_abort: called
        once before RankLost is raised (the engines pass `cm.dp_abort`)."""
        self.dir, self.world, self.rank = directory, world, rank
        self.timeout, self.poll, self.on_abort = timeout, poll, on_abort
        os.makedirs(directory, exist_ok=True)
        self._next = 0                                 # updates this rank has taken part in so far
        self._write("start")

    def _path(self, rank):
        return os.path.join(self.dir, "rank%d" % rank)

    def _write(self, text):
        tmp = self._path(self.rank) + ".tmp"
        with open(tmp, "w") as f:
            f.write(text)
        os.replace(tmp, self._path(self.rank))        # readers see the old or the new text, never half of one

    def _read(self, rank):
        try:
            with open(self._path(rank)) as f:
                return f.read()
        except OSError:
            return None

    def _lost(self, why):
        if self.on_abort is not None:
            try:
                self.on_abort()
            finally:
                self.on_abort = None
        self._write("left %d" % self._next)
        raise RankLost(why)

    def before_step(self, step):
        """Call between updates, before enqueueing update `step`.  Returns once every rank is about
        to enqueue the same update; raises RankLost if one has left or does not show up in time."""
        self._write("step %d" % step)
        deadline = time.time() + self.timeout
        waiting = [r for r in range(self.world) if r != self.rank]
        while waiting:
            for r in list(waiting):
                text = self._read(r)
                if text is not None and text.startswith("left "):
                    # "left n": the peer took part in updates 0 .. n-1 (their collectives are enqueued) and no further
                    if int(text[5:]) <= step:
                        self._lost("rank %d left before update %d" % (r, step))
                    waiting.remove(r)
                elif text is not None and text.startswith("step ") and int(text[5:]) >= step:
                    waiting.remove(r)
            if waiting:
                if time.time() > deadline:
                    self._lost("rank(s) %s did not reach update %d within %.1f s" % (waiting, step, self.timeout))
                time.sleep(self.poll)
        self._next = step + 1

    def leave(self):
        """This rank stops taking part (call between updates, with nothing of its own in flight)."""
        self._write("left %d" % self._next)

    def guarded(self, fn, *args, **kw):
        """Runs fn; if it raises, the peers are told before the exception travels on."""
        try:
            return fn(*args, **kw)
        except BaseException:
            self.leave()
            raise
