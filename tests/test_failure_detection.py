"""Failure detection, exercised on the host only (no GPU is faulted or hung): heartbeat watchdog,
a rank that stops stepping, a rank that raises, a short process-group timeout, an incomplete
checkpoint."""
import os
import time

import pytest
import torch
import torch.distributed as dist

from distributed_helpers import run_distributed


class FakeStore(dict):
    def set(self, k, v):
        self[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self[k]


def test_watchdog_flags_a_rank_that_stopped_beating():
    from picotron_b200.runtime.watchdog import StepWatchdog
    store = FakeStore()
    a = StepWatchdog(store, rank=0, world_size=1, timeout_s=0.2)          # no thread for world 1
    a.world_size = 3
    t0 = 1000.0                                   # the reader's own (monotonic) clock
    store.set("pico_hb/1", "5")                   # rank 1 keeps up
    store.set("pico_hb/2", "2")                   # rank 2 is behind
    a.beat(5)
    assert a.check_once(t0) == []                 # first sighting: nobody is stale yet
    store.set("pico_hb/1", "6")
    assert a.check_once(t0 + 10) == [2]           # rank 2 has not moved for longer than the timeout
    store.set("pico_hb/2", "6")                   # it recovers
    assert a.check_once(t0 + 10.1) == []
    a._my_step = 1                                # peers that are ahead of us are never failures
    assert a.check_once(t0 + 30) == []


def test_watchdog_flags_a_job_stuck_inside_one_step():
    """One rank hangs inside a step and the others block in its collectives: every heartbeat carries
    the same step number. A rank whose own last beat is as old as its peers' flags them all."""
    from picotron_b200.runtime.watchdog import StepWatchdog
    store = FakeStore()
    a = StepWatchdog(store, rank=0, world_size=1, timeout_s=0.2)
    a.world_size = 3
    store.set("pico_hb/1", "7")
    store.set("pico_hb/2", "7")
    a.beat(7)
    t0 = 2000.0
    a._my_beat_at = t0
    assert a.check_once(t0) == []
    assert a.check_once(t0 + 0.1) == []           # everyone in step 7, but not for long yet
    assert a.check_once(t0 + 10) == [1, 2]        # nobody, this rank included, has moved since
    a.beat(8)                                     # this rank did make progress: peers in step 7 are behind
    a._my_beat_at = t0 + 10
    assert a.check_once(t0 + 10.05) == [1, 2]


def _stalled_rank_worker(rank, world):
    """Rank 1 stops stepping; rank 0's watchdog thread notices within the timeout."""
    from picotron_b200.runtime.watchdog import StepWatchdog
    store = dist.distributed_c10d._get_default_store()
    failures = []
    wd = StepWatchdog(store, rank, world, timeout_s=0.5, poll_s=0.1, on_failure=failures.append)
    for step in range(1, 4):
        wd.beat(step)
        time.sleep(0.05)
    if rank == 0:
        for step in range(4, 30):
            wd.beat(step)
            time.sleep(0.1)
            if failures:
                break
        assert failures and failures[0] == [1], failures
    else:
        time.sleep(2.5)       # alive but not making progress
    wd.stop()


def test_watchdog_detects_stalled_rank_over_the_store():
    run_distributed(_stalled_rank_worker, 2)


def _raising_rank_worker(rank, world):
    if rank == 1:
        raise RuntimeError("injected failure on rank 1")
    time.sleep(0.2)


def test_a_raising_rank_fails_the_job():
    with pytest.raises(AssertionError, match="injected failure"):
        run_distributed(_raising_rank_worker, 2, timeout=60)


def _timeout_worker(rank, world):
    """A collective that one rank never joins ends with an error after a short group timeout."""
    import datetime
    g = dist.new_group(ranks=list(range(world)), timeout=datetime.timedelta(seconds=2))
    t = torch.ones(1)
    if rank == 0:
        with pytest.raises(Exception):
            dist.all_reduce(t, group=g)       # rank 1 never calls it
    else:
        time.sleep(4)


def test_collective_times_out_when_a_rank_never_joins():
    try:
        run_distributed(_timeout_worker, 2, timeout=60)
    except AssertionError as e:          # gloo may tear the pair down on the peer as well
        assert "rank 1" in str(e) or "Connection" in str(e) or "exit codes" in str(e)


def test_incomplete_checkpoint_is_refused(tmp_path):
    import json
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.checkpoint import CheckpointManager
    pgm.process_group_manager = None
    model = torch.nn.Linear(4, 4)
    ck = CheckpointManager()
    out = str(tmp_path / "1")
    ck.save_checkpoint(model, None, 1, 10, out)
    assert ck.load_checkpoint(model, None, out) == (1, 10)
    man = json.load(open(os.path.join(out, "manifest.json")))
    man["files"].append("weights_tp_rank_world_size=1_2_pp_rank_world_size=0_1.pth")
    json.dump(man, open(os.path.join(out, "manifest.json"), "w"))
    with pytest.raises(FileNotFoundError, match="incomplete"):
        ck.load_checkpoint(model, None, out)


def test_flag_protocol_double_buffer_model():
    """Pure-Python model of the two-copy buffer rule used by the fused collectives: an op may start
    writing copy n%2 on a peer only after every rank finished the op n-1 that precedes it; with that
    rule no write of op n+2 can overlap a read of op n."""
    import itertools
    world, ops_count = 3, 6
    # progress[r] = number of ops rank r has completed; op n on rank r needs every rank to have
    # *started* op n (their data), modelled as progress >= n
    for order in itertools.islice(itertools.permutations(range(world)), 6):
        progress = [0] * world
        reading = {}
        for _ in range(ops_count * world * 4):
            for r in order:
                n = progress[r]
                if n >= ops_count:
                    continue
                # rank r can complete op n once all ranks have reached op n
                if min(progress) >= n:
                    # writing copy n%2 of peers: nobody may still be reading op n-2 from it
                    for peer in range(world):
                        assert reading.get((peer, n % 2), n) >= n - 1 or progress[peer] > n - 2
                    reading[(r, n % 2)] = n
                    progress[r] = n + 1
        assert progress == [ops_count] * world
