"""Worker of the host-side failure test (gloo, CPU): rank 1 raises before the gradient exchange, rank 0 must
get an error from its all-reduce within the process group's timeout. No GPU is involved."""
import sys
import time
from datetime import timedelta
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main(out_dir: str) -> None:
    dist.init_process_group("gloo", timeout=timedelta(seconds=10))
    rank = dist.get_rank()
    dist.barrier()
    if rank == 1:
        raise SystemExit(3)                       # this rank never reaches the exchange
    buf = torch.ones(1 << 16)
    t0 = time.perf_counter()
    try:
        dist.all_reduce(buf, async_op=True).wait()
        outcome = "completed"
    except Exception as e:  # noqa: BLE001 - the class is what the test looks at
        outcome = type(e).__name__
    (Path(out_dir) / "survivor.txt").write_text(f"{outcome}|{time.perf_counter() - t0:.2f}|")


if __name__ == "__main__":
    main(sys.argv[1])
