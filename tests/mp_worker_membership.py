"""Worker of the membership test (CPU, gloo-free: only a TCPStore): rank 2 leaves cleanly after step 3,
rank 1 disappears without a word after step 5; ranks 0 and the others must notice on the host, before
the step in which the peer would be missing, and carry on with the survivors."""
import os
import sys
import time
from datetime import timedelta

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torch.distributed import TCPStore  # noqa: E402

from parameter_server_b200.parallel.membership import Membership, RankLost  # noqa: E402


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=30), wait_for_workers=True)
    m = Membership(store, rank, world, timeout_s=1.0)
    events = []
    for step in range(1, 9):
        if rank == 2 and step == 4:
            m.leave()                      # clean departure between steps
            print("rank 2 left", flush=True)
            time.sleep(3.0)                # keep the process (and its store connection) around
            return
        if rank == 1 and step == 6:
            print("rank 1 vanishes", flush=True)
            time.sleep(6.0)                # silent: no heartbeat, no announcement
            os._exit(0)
        try:
            m.step(step)
        except RankLost as e:
            events.append((step, e.ranks, e.left))
            # the survivors agree on the new membership and go on (a real job would restore / re-shard here)
        time.sleep(0.01)                   # the "kernel" of this step
    print(f"rank {rank} events {events} survivors {m.survivors()}", flush=True)
    if rank == 0:
        time.sleep(1.0)                    # the store's master outlives its clients


if __name__ == "__main__":
    main()
