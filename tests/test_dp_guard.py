"""Failure detection among data-parallel ranks, on the host: a rank that leaves between updates,
one that raises, and one that never starts are noticed by the others before their next launch
(bounded wait), the communicator is torn down once, and RankLost is raised.  CPU processes only:
no GPU is faulted, hung or even touched."""
import multiprocessing as mp
import os
import time

import pytest

from deepnet_b200.dp_guard import RankGuard, RankLost


def _rank(directory, world, rank, script, q):
    aborts = []
    guard = RankGuard(directory, world, rank, timeout=2.0, on_abort=lambda: aborts.append(1))
    done, outcome = 0, "finished"
    try:
        for step in range(6):
            if script == "leaves" and step == 2:
                guard.leave()                       # between updates, nothing in flight
                outcome = "left"
                break
            if script == "raises" and step == 3:
                guard.guarded(lambda: 1 / 0)
            guard.before_step(step)
            done += 1                               # here the update (and its all-reduce) would be enqueued
    except RankLost as e:
        outcome = "lost: %s" % e
    except ZeroDivisionError:
        outcome = "raised"
    q.put((rank, done, outcome, len(aborts)))


def _run(tmp_path, scripts, absent=()):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = len(scripts)
    procs = [ctx.Process(target=_rank, args=(str(tmp_path), world, r, scripts[r], q)) for r in range(world) if r not in absent]
    t0 = time.time()
    for p in procs:
        p.start()
    out = dict()
    for _ in procs:
        r, done, outcome, aborts = q.get(timeout=60)
        out[r] = (done, outcome, aborts)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    return out, time.time() - t0


def test_all_ranks_present_run_to_the_end(tmp_path):
    out, _ = _run(tmp_path, ["ok", "ok", "ok"])
    assert all(v == (6, "finished", 0) for v in out.values())


def test_a_rank_that_leaves_between_updates_is_noticed_before_the_next_launch(tmp_path):
    out, dt = _run(tmp_path, ["ok", "ok", "leaves"])
    assert out[2] == (2, "left", 0)
    for r in (0, 1):
        done, outcome, aborts = out[r]
        assert done == 2 and outcome.startswith("lost: rank") and aborts == 1      # stopped at the same update, one teardown
    assert dt < 30


def test_a_rank_that_raises_tells_its_peers(tmp_path):
    out, _ = _run(tmp_path, ["raises", "ok"])
    assert out[0][1] == "raised" and out[0][0] == 3
    assert out[1][0] == 3 and "left before update 3" in out[1][1] and out[1][2] == 1


def test_a_rank_that_never_starts_times_out(tmp_path):
    out, dt = _run(tmp_path, ["ok", "ok"], absent=(1,))
    done, outcome, aborts = out[0]
    assert done == 0 and "did not reach update 0" in outcome and aborts == 1
    assert 1.5 < dt < 30                              # the bounded wait, not forever
