"""Child process of the rank-failure test: gloo ranks on the CPU; one rank fails on the host between steps."""

import datetime
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from mfq_b200.parallel.health import RankFailure, RankHealth, reform_group  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    victim, fail_step = int(os.environ["VICTIM"]), int(os.environ["FAIL_STEP"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["STORE_PORT"]), world, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=30), wait_for_workers=True)
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=20))
    health = RankHealth(dist.PrefixStore("hb", store), rank, world, timeout=5.0)
    group, my_rank, my_world = dist.group.WORLD, rank, world
    sums, detected = [], None
    for step in range(6):
        try:
            if rank == victim and step == fail_step:
                raise RuntimeError("injected host-side failure")  # the fault: an exception in this rank's step
            # ranks agree on the host that everyone is still there BEFORE launching the step's collective
            dist.barrier(group=group) if detected is None and step < fail_step else None
            health.check()
        except RankFailure as f:
            detected = sorted(f.failed)
            group, my_rank, my_world = reform_group(health.survivors(), backend="gloo")
            health = RankHealth(dist.PrefixStore(f"hb{step}", store), my_rank, my_world, timeout=5.0)
        except RuntimeError as exc:
            health.report_failure(str(exc))
            print("HEALTH_RESULT " + json.dumps({"rank": rank, "left_at": step}), flush=True)
            return  # leaves between steps: nothing of this rank is in flight
        t = torch.tensor([float(my_rank + 1)])
        if step == fail_step and detected is None:
            # the victim reports before the others check; give its store write a moment (host-side only)
            import time
            deadline = time.time() + 10
            while time.time() < deadline and not health.failed():
                time.sleep(0.05)
            try:
                health.check()
            except RankFailure as f:
                detected = sorted(f.failed)
                group, my_rank, my_world = reform_group(health.survivors(), backend="gloo")
                health = RankHealth(dist.PrefixStore(f"hb{step}", store), my_rank, my_world, timeout=5.0)
                t = torch.tensor([float(my_rank + 1)])
        dist.all_reduce(t, group=group)
        sums.append(float(t))
        health.beat()
    print("HEALTH_RESULT " + json.dumps({"rank": rank, "detected": detected, "world_after": my_world, "sums": sums}), flush=True)


if __name__ == "__main__":
    main()
