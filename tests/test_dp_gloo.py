"""Host-side data-parallel logic on CPU, world size 2 over gloo: each rank runs the CD step
of its minibatch shard on the oracle with its global column offset, the packed sufficient
statistics are summed across ranks (gloo stands in for the NCCL all-reduce), and the result
must equal the single-process run on the whole minibatch: identical Bernoulli bits,
statistics and updated weights within fp32 summation-order tolerance."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cd1_stats(em, W, bv, bh, data, seed, col0):
    """One CD-1 pass of a binary RBM issued as the reference calls (deepnet/dbm.py:118-238)."""
    em.EigenMatrix.init_random(seed, col0=col0)
    V, H = W.shape
    B = data.shape[1]
    w, v0 = em.CUDAMatrix(W), em.CUDAMatrix(data)
    h = em.empty((H, B))
    em.dot(w.T, v0, target=h)
    h.add_col_vec(em.CUDAMatrix(bh))
    em.sigmoid(h)
    suff_w = em.dot(v0, h.T)
    suff_v, suff_h = v0.sum(axis=1), h.sum(axis=1)
    hs = h.sample_bernoulli(target=em.empty((H, B)))
    v = em.empty((V, B))
    em.dot(w, hs, target=v)
    v.add_col_vec(em.CUDAMatrix(bv))
    em.sigmoid(v)
    em.dot(w.T, v, target=h)
    h.add_col_vec(em.CUDAMatrix(bh))
    em.sigmoid(h)
    hs2 = h.sample_bernoulli(target=em.empty((H, B)))
    suff_w.add_dot(v, h.T, mult=-1.0)
    suff_v.add_sums(v, axis=1, mult=-1.0)
    suff_h.add_sums(h, axis=1, mult=-1.0)
    pack = np.concatenate([suff_w.asarray().ravel(order="F"), suff_v.asarray().ravel(), suff_h.asarray().ravel()])
    return pack.astype(np.float32), hs.asarray().copy(), hs2.asarray().copy()


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from oracle import eigenmat_oracle as em
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(123)                      # same on every rank
    V, H, B = 48, 32, 16
    W = (rng.standard_normal((V, H)) * 0.1).astype(np.float32)
    bv = (rng.standard_normal((V, 1)) * 0.1).astype(np.float32)
    bh = (rng.standard_normal((H, 1)) * 0.1).astype(np.float32)
    data = (rng.random((V, B * world)) < 0.3).astype(np.float32)
    shard = np.asfortranarray(data[:, rank * B:(rank + 1) * B])
    pack, hs, hs2 = _cd1_stats(em, W, bv, bh, shard, seed=77, col0=rank * B)
    t = torch.from_numpy(pack.copy())
    dist.all_reduce(t)                                     # the one exchange of the update
    # every rank applies the identical update with 1 / (B * world)
    n = V * H
    w, d = em.CUDAMatrix(W), em.CUDAMatrix(np.zeros_like(W))
    w.momentum_update(d, em.CUDAMatrix(np.zeros_like(W)), em.CUDAMatrix(t.numpy()[:n].reshape(V, H, order="F")),
                      1.0 / (B * world), 0.5, 0.1, l2=2e-4)
    gathered = [None] * world
    dist.all_gather_object(gathered, (hs, hs2, w.asarray().copy()))
    if rank == 0:
        full_pack, full_hs, full_hs2 = _cd1_stats(em, W, bv, bh, np.asfortranarray(data), seed=77, col0=0)
        q.put((t.numpy().copy(), full_pack, gathered, full_hs, full_hs2))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shards_reproduce_the_single_process_update():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    summed, full_pack, gathered, full_hs, full_hs2 = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # Bernoulli bits of the shards are the columns of the full-batch draw (stream is GPU-count independent)
    assert np.array_equal(np.concatenate([g[0] for g in gathered], axis=1), full_hs)
    assert np.array_equal(np.concatenate([g[1] for g in gathered], axis=1), full_hs2)
    np.testing.assert_allclose(summed, full_pack, rtol=1e-5, atol=1e-5)
    # replicas end bit-identical
    assert np.array_equal(gathered[0][2], gathered[1][2])


def test_packed_statistics_views_cover_the_buffer():
    # layout of the one all-reduced buffer: [V*H weight statistics | V | H]
    V, H = 12, 8
    total = V * H + V + H
    offs = [(0, V * H), (V * H, V * H + V), (V * H + V, total)]
    assert offs[0][1] == offs[1][0] and offs[1][1] == offs[2][0] and offs[2][1] == total
