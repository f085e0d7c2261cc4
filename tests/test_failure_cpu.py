"""Failure detection with host-injected failures among CPU ranks (gloo): a rank that raises, a rank that exits between
steps, a rank that never joins, a silent rank (heartbeat timeout).  No GPU is involved."""
import multiprocessing as mp
import os
import time

import pytest
import torch
import torch.distributed as dist

from dart_pytorch_b200.parallel.health import Heartbeat, PeerFailure, wait_collective, wait_for_peers


def _worker(rank, world, port, scenario, q):
    try:
        store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=__import__("datetime").timedelta(seconds=60))
        if scenario == "never_joins" and rank == world - 1:
            time.sleep(12.0)                      # holds the store connection but never starts the job
            q.put((rank, "idle"))
            return
        # limits with room for a loaded test machine: a healthy rank must never look late
        hb = Heartbeat(store, rank, world, timeout=4.0, background_interval=0.2)
        if scenario == "never_joins":
            try:
                wait_for_peers(hb, deadline_s=6.0)
                q.put((rank, "joined"))
            except PeerFailure as e:
                q.put((rank, f"detected:{e.rank}"))
            return
        wait_for_peers(hb, deadline_s=30.0)
        dist.init_process_group("gloo", store=store, rank=rank, world_size=world,
                                timeout=__import__("datetime").timedelta(seconds=10))
        x = torch.ones(4)
        for step in range(6):
            if scenario == "silent" and rank == 1 and step == 2:
                time.sleep(9.0)                   # alive (background beats continue) but stuck between steps
                q.put((rank, "stalled"))
                time.sleep(0.5)
                return
            try:
                with hb.guard():
                    if scenario == "raises" and rank == 1 and step == 2:
                        raise ValueError("injected failure")
                    if scenario == "exits" and rank == 1 and step == 2:
                        hb.report_failure("leaving between steps")
                        q.put((rank, "left"))
                        return
                    wait_collective(dist.all_reduce(x, async_op=True), hb)     # the step's collective
                # the culprit reaches its failure point while the others are still between steps
                time.sleep(0.0 if (rank == 1 and step == 1) or step == 0 else 0.4)
            except PeerFailure as e:
                q.put((rank, f"detected:{e.rank}:{step}"))
                return
            except RuntimeError:
                # the other documented path: the collective itself ends with an error; the store says who it was
                time.sleep(0.2)
                bad = hb.failed_peers()
                q.put((rank, f"detected:{min(bad) if bad else -1}:{step}"))
                return
            except ValueError:
                q.put((rank, "raised"))
                return
        q.put((rank, "finished"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"error:{type(e).__name__}:{e}"))


def _run(scenario, world=3):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() + hash(scenario)) % 200
    procs = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    deadline = time.time() + 120
    while len(out) < world and time.time() < deadline:
        try:
            r, msg = q.get(timeout=1.0)
            out[r] = msg
        except Exception:
            pass
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.terminate()
    return out


@pytest.mark.parametrize("scenario,culprit_msg", [("raises", "raised"), ("exits", "left"), ("silent", "stalled")])
def test_peers_learn_of_a_failed_rank_before_their_next_collective(scenario, culprit_msg):
    out = _run(scenario)
    assert out.get(1) == culprit_msg, out
    for r in (0, 2):
        assert out.get(r, "").startswith("detected:1:"), out
        assert int(out[r].split(":")[2]) >= 2          # steps 0 and 1 completed normally


def test_rank_that_never_joins_is_reported():
    out = _run("never_joins")
    assert out.get(2) == "idle", out
    assert out.get(0) == "detected:2" and out.get(1) == "detected:2", out


def test_heartbeat_local_semantics():
    store = dist.HashStore()
    a, b = Heartbeat(store, 0, 2, timeout=0.2), Heartbeat(store, 1, 2, timeout=0.2)
    a.check()
    b.check()
    with pytest.raises(ZeroDivisionError):
        with a.guard():
            1 / 0
    with pytest.raises(PeerFailure) as ei:
        b.check()
    assert ei.value.rank == 0 and "ZeroDivisionError" in ei.value.reason
    c = Heartbeat(dist.HashStore(), 0, 2, timeout=0.2)
    c.check()                                             # peer 1 not seen yet: grace period
    time.sleep(0.3)
    with pytest.raises(PeerFailure) as ei:
        c.check()
    assert "never joined" in ei.value.reason
    # progress: a live peer that stays behind is flagged only by check_progress
    st = dist.HashStore()
    e, f = Heartbeat(st, 0, 2, timeout=0.2), Heartbeat(st, 1, 2, timeout=0.2)
    e.enter_step()
    e.check_progress()
    time.sleep(0.3)
    f.beat()
    e.check()
    with pytest.raises(PeerFailure) as ei:
        e.check_progress()
    assert "stuck at step 0" in ei.value.reason
