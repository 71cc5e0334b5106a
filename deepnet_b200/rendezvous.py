"""Bring-up of the data-parallel ranks of one node without any framework.

The reference has no multi-GPU layer; a launcher (torchrun or any other) only has to start one
process per GPU with RANK / LOCAL_RANK / WORLD_SIZE in the environment.  Rank 0 creates the NCCL
id and publishes it in a file that the other ranks poll; after `dp_init` every other exchange
(barrier, gathering one number per rank) is an all-reduce of a few floats on the library stream.
"""
import os
import tempfile
import time

import numpy as np


def _id_path():
    # one launch = one parent process (the launcher) and one master port: a name no earlier or
    # concurrent launch shares
    tag = "%s_%s_%s" % (os.environ.get("MASTER_PORT", "0"), os.environ.get("TORCHELASTIC_RUN_ID", "none"), os.getppid())
    return os.path.join(tempfile.gettempdir(), "b200mat_nccl_id_" + tag)


class Group(object):
    """The ranks of one launch.  world == 1 needs no NCCL and no files."""

    def __init__(self, cm, world, rank, timeout=120.0, path=None):
        self.cm, self.world, self.rank = cm, world, rank
        self._slots = None
        self._path = path or _id_path()
        if world == 1:
            return
        path = self._path
        if rank == 0:
            uid = cm.dp_unique_id()
            with open(path + ".tmp", "wb") as f:
                f.write(uid)
            os.rename(path + ".tmp", path)           # appears whole or not at all
        else:
            deadline = time.time() + timeout
            while not os.path.exists(path):
                if time.time() > deadline:
                    raise RuntimeError("rank %d: rank 0 published no NCCL id within %.0f s" % (rank, timeout))
                time.sleep(0.02)
            with open(path, "rb") as f:
                uid = f.read()
        cm.dp_init(uid, world, rank)
        self._slots = cm.empty((1, max(world, 4)))
        self.gather(0.0)                             # first collective: every rank has read the file
        if rank == 0:
            try:
                os.remove(path)
            except OSError:
                pass

    def gather(self, x):
        """One float per rank -> list of all ranks' values on every rank (blocks)."""
        if self.world == 1:
            return [float(x)]
        v = np.zeros((1, self._slots.shape[1]), np.float32)
        v[0, self.rank] = x
        self._slots.overwrite(v)
        self.cm.dp_allreduce(self._slots)
        return [float(t) for t in np.array(self._slots.asarray())[0, :self.world]]

    def exchange(self, tag, payload, timeout=120.0):
        """Every rank contributes some bytes; returns all ranks' contributions in rank order."""
        if self.world == 1:
            return [payload]
        base = "%s_%s_" % (self._path, tag)
        with open(base + "%d.tmp" % self.rank, "wb") as f:
            f.write(payload)
        os.rename(base + "%d.tmp" % self.rank, base + str(self.rank))
        out = []
        deadline = time.time() + timeout
        for r in range(self.world):
            while not os.path.exists(base + str(r)):
                if time.time() > deadline:
                    raise RuntimeError("rank %d: rank %d published no %s within %.0f s" % (self.rank, r, tag, timeout))
                time.sleep(0.01)
            with open(base + str(r), "rb") as f:
                out.append(f.read())
        self.gather(0.0)                             # everyone has read everything
        try:
            os.remove(base + str(self.rank))
        except OSError:
            pass
        return out

    def barrier(self):
        self.cm.cuda_sync_threads()
        self.gather(0.0)

    def max(self, x):
        return max(self.gather(x))

    def close(self):
        if self.world > 1:
            self.cm.dp_destroy()
