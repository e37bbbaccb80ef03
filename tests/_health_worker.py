"""Worker of the failure-detection tests: gloo ranks on CPU that lose a peer in a scripted way."""
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    scenario, port = sys.argv[1], int(sys.argv[2])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    from tensorrt_edge_llm_b200.parallel.comm import TorchComm
    from tensorrt_edge_llm_b200.parallel.health import GuardedComm, HealthMonitor, RankLostError
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=4))
    mon = HealthMonitor(dist.PrefixStore("health", store), rank, world, interval_s=0.1, timeout_s=1.0).start()
    comm = GuardedComm(TorchComm(), mon)
    t0 = time.monotonic()
    try:
        for step in range(6):
            if rank == 1 and step == 2:
                if scenario == "leave":
                    mon.leave()                     # orderly, between steps
                    os._exit(0)
                if scenario == "vanish":
                    os._exit(0)                     # no goodbye: heartbeats just stop
                if scenario == "raise":
                    try:
                        raise ValueError("bad weights on this rank")
                    except ValueError as e:
                        mon.report_failure(str(e))
                        os._exit(3)
            if scenario == "vanish" and step == 2:
                time.sleep(1.6)                     # the step's host work; the dead peer goes stale meanwhile
            x = torch.full((4,), float(rank + 1))
            y = comm.all_reduce(x)
            assert float(y[0]) == sum(range(1, world + 1))
            time.sleep(0.15)
        print(f"rank {rank}: finished all steps", flush=True)
        os._exit(0 if scenario == "healthy" else 5)
    except RankLostError as e:
        print(f"rank {rank}: lost rank {e.rank} ({e.reason}) after {time.monotonic() - t0:.1f} s at step {step}", flush=True)
        os._exit(42)


if __name__ == "__main__":
    main()
