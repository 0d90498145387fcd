"""Every rank of a multi-GPU launch checks the kernel library when it loads it: concurrent builders must take turns."""

import multiprocessing as mp
import time


def _worker(log_path: str, idx: int) -> None:
    from nestor_b200.csrc import build as B

    def fake(verbose, force, checked):          # stands in for the compile + link; records when it ran
        with open(log_path, "a") as f:
            f.write(f"enter {idx}\n")
        time.sleep(0.15)
        with open(log_path, "a") as f:
            f.write(f"leave {idx}\n")
        return B.LIB

    B._build_locked = fake
    B.build()


def test_concurrent_builders_are_serialised(tmp_path):
    log = tmp_path / "order.log"
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(str(log), i)) for i in range(4)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    lines = log.read_text().split("\n")[:-1]
    assert len(lines) == 8
    for a, b in zip(lines[0::2], lines[1::2]):      # never two builders inside at once
        assert a.startswith("enter") and b.startswith("leave") and a.split()[1] == b.split()[1]
