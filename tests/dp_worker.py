"""One rank of the two-GPU data-parallel test: trains its shard of the global minibatch
with the fused engine and writes its final weights and hidden draw.  Launched by
tests/test_gpu_dp.py as a child process (one per GPU); not collected by pytest."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, tmp = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    scale = float(sys.argv[4]) if len(sys.argv) > 4 else 0.5
    from deepnet_b200 import b200mat as cm
    from deepnet_b200 import configs
    from deepnet_b200.fused_rbm import FusedRBM
    cm.cuda_set_device(rank)
    cm.cublas_init()
    from deepnet_b200.rendezvous import Group
    group = Group(cm, world, rank, timeout=60, path=os.path.join(tmp, "nccl_id"))
    cfg = configs.build(0, cases=400, dims_scale=scale)
    gb = cfg["batchsize"]                       # global minibatch, split evenly over the ranks
    b = gb // world
    V, H = cfg["layers"][0]["numdims"], cfg["layers"][1]["numdims"]
    eng = FusedRBM(cm, V, H, b, cfg["edges"][0]["weight"], cfg["hyperparams"],
                   edge_hyperparams=cfg["edges"][0].get("hyperparams"), binary_data=True, seed=cfg["seed"], world_size=world,
                   rank=rank, group=group)
    data = cm.CUDAMatrix(cfg["data"])
    if len(sys.argv) > 5 and sys.argv[5] == "absent":
        # Failure detection: rank 1 is alive but never enqueues its update (it left between updates, no
        # kernel of its in flight).  Rank 0's update waits for rank 1's statistics with a short limit,
        # gives up by itself and leaves a status word; its context stays usable.
        status, usable = 0, True
        if rank == 1:
            group.barrier()                     # (the host barrier that opens rank 0's first update)
        else:
            cm.set_wait_limit(20000)            # peer waits: sixteen times that, a fraction of a second
            eng.TrainOneBatch(0, data.slice(0, b))
            status = cm.read_status()           # blocks until the kernels have returned by themselves
            cm.set_wait_limit(0)
            a = np.random.default_rng(0).standard_normal((64, 64)).astype(np.float32)
            usable = bool(np.allclose(np.array(cm.dot(cm.CUDAMatrix(a), cm.CUDAMatrix(a)).asarray()), a @ a, atol=1e-3))
        np.savez(os.path.join(tmp, "rank%d.npz" % rank), status=status, usable=usable, peer=int(eng.dp_peer))
        eng.close(group)
        cm.dp_destroy()
        return
    for step in range(3):
        s = step * gb + rank * b
        eng.TrainOneBatch(step, data.slice(s, s + b))
    cm.dp_wait(20000)        # bounded: a peer that never joined would end here with an error, not a hang
    cm.dp_check()
    np.savez(os.path.join(tmp, "rank%d.npz" % rank), W=np.array(eng.W.asarray()), hs=np.array(eng.h_samp.asarray()),
             loss=eng.read_loss(), status=cm.read_status(), peer=int(eng.dp_peer), peer_mode=cm.dp_peer_mode())
    eng.close(group)         # nobody unmaps a peer's memory while another rank may still write to it
    cm.dp_destroy()          # leaves only after its last collective has completed


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        # do not leave the peer waiting in a collective this rank will never join
        try:
            from deepnet_b200 import b200mat
            b200mat._lib.dp_abort()
        finally:
            raise
