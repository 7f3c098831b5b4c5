"""Failure detection of the N-partitioned path, made to fail on the HOST only: CPU ranks over gloo where one
rank leaves between steps or never joins, and a fake communicator that reports an asynchronous error.
No GPU is involved and nothing is made to hang: every wait here has a deadline of a second or two."""
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tilebench_b200 import comm, npart


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir, scenario):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    hb = comm.Heartbeat(store, rank, world, prefix=f"hb/{scenario}")
    log = []
    try:
        local = torch.full((2, 3), float(rank))
        for step in range(4):
            if scenario == "leaves" and rank == 1 and step == 2:
                hb.leave("planned exit after step 1")          # between steps: nothing of this rank is in flight
                log.append("left")
                break
            if scenario == "silent" and rank == 1 and step == 2:
                log.append("went silent")
                time.sleep(3.0)                                 # outlives the others' deadline, then exits
                break
            try:
                hb.begin_step(step, timeout_s=1.0)
            except comm.PeerLost as e:
                log.append(f"step {step}: lost {e.ranks}: {e.reason[e.ranks[0]]}")
                break                                           # no collective is launched with a lost peer
            full = npart.all_gather_columns(local + step)
            assert full.shape == (2, 3 * world) and float(full[0, -1]) == world - 1 + step
            log.append(f"step {step}: ok")
    finally:
        with open(os.path.join(out_dir, f"log_{rank}.txt"), "w") as f:
            f.write("\n".join(log))
        # no destroy_process_group barrier: a rank that lost its peer must be able to finish on its own


@pytest.mark.parametrize("scenario", ["leaves", "silent"])
def test_rank_that_leaves_or_goes_silent_is_seen_before_the_next_collective(tmp_path, scenario):
    world = 3
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path), scenario), nprocs=world, join=True)
    logs = {r: (tmp_path / f"log_{r}.txt").read_text().splitlines() for r in range(world)}
    for r in (0, 2):
        assert logs[r][:2] == ["step 0: ok", "step 1: ok"]
        assert len(logs[r]) == 3 and logs[r][2].startswith("step 2: lost [1]")
        assert ("planned exit" if scenario == "leaves" else "silent for 1 s") in logs[r][2]
    assert logs[1][:2] == ["step 0: ok", "step 1: ok"]


def test_rank_that_never_joins_is_reported_as_never_seen():
    store = dist.HashStore()
    hb = comm.Heartbeat(store, 0, 2)
    t0 = time.monotonic()
    with pytest.raises(comm.PeerLost) as e:
        hb.begin_step(0, timeout_s=0.3)
    assert e.value.ranks == [1] and "never" in e.value.reason[1] and time.monotonic() - t0 < 2.0
    # once the peer shows up the same call passes
    comm.Heartbeat(store, 1, 2).beat(0)
    hb.begin_step(0, timeout_s=0.3)


class FakeCommunicator:
    """Stands in for an NCCL communicator: healthy until `fail_after` polls, then reports an async error."""

    def __init__(self, fail_after):
        self.fail_after, self.polls, self.aborts = fail_after, 0, 0

    def get_async_error(self):
        self.polls += 1
        return None if self.polls <= self.fail_after else "ncclRemoteError"

    def abort(self):
        self.aborts += 1


def test_watchdog_reports_async_error_and_aborts_once():
    fake = FakeCommunicator(fail_after=3)
    wd = comm.CommWatchdog(fake.get_async_error, fake.abort, period_s=0.01).start()
    wd.check()                                       # healthy so far
    deadline = time.monotonic() + 2.0
    while wd.error is None and time.monotonic() < deadline:
        time.sleep(0.01)
    with pytest.raises(comm.CommError, match="ncclRemoteError"):
        wd.check()
    assert wd.aborted and fake.aborts == 1
    time.sleep(0.05)
    assert fake.aborts == 1 and fake.polls == 4      # the poller stopped after the first error
    wd.stop()


def test_watchdog_source_exception_and_guarded_steps():
    def broken():
        raise OSError("driver call failed")
    wd = comm.CommWatchdog(broken, None, period_s=0.01).start()
    time.sleep(0.1)
    with pytest.raises(comm.CommError, match="driver call failed"):
        wd.check()
    wd.stop()
    # guarded_steps: watchdog first, then heartbeat, then the step is handed out
    store = dist.HashStore()
    hb0, hb1 = comm.Heartbeat(store, 0, 2), comm.Heartbeat(store, 1, 2)
    hb1.beat(1)
    healthy = comm.CommWatchdog(lambda: None, None, period_s=0.01).start()
    assert list(comm.guarded_steps(hb0, range(2), healthy, timeout_s=0.3)) == [0, 1]
    hb1.leave("done")
    with pytest.raises(comm.PeerLost):
        list(comm.guarded_steps(hb0, [2], healthy, timeout_s=0.3))
    healthy.stop()
