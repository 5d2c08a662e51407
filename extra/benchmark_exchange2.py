"""Exchange at one fixed size across every partner offset.

    torchrun --nproc-per-node 8 extra/benchmark_exchange2.py

Rank r swaps 2^26 fp16 elements with rank (r + offset) mod world for offset =
1..world-1 paired so that partners name each other (r <-> r XOR offset), which
on NVSwitch should cost the same for every offset; the reference's
extra/benchmark_exchange2.py sweeps `gpu_offset` the same way to expose uneven
NIC/GPU paths between nodes.
"""
import json

import torch

from _bench_common import NVLINK_GBS
from penny_b200.utils import bench_device, initialize_distributed, shutdown


def main():
    rank, world, comm = initialize_distributed(heap_bytes=2 << 30)
    n = 1 << 26
    x = torch.randn(n, device="cuda").half()
    for offset in range(1, world):
        peer = rank ^ offset
        if peer >= world:
            continue
        want = None
        buf = x.clone()
        comm.exchange(buf, peer)
        comm.check()
        t = bench_device(lambda: comm.exchange(buf, peer), 5, 20)["median_us"]
        gbs = n * 2 / t / 1e3
        if rank == 0:
            print(json.dumps({"op": "exchange", "offset": offset, "bytes": n * 2, "t_us": round(t, 1),
                              "gbs": round(gbs, 1), "frac_nvlink": round(gbs / NVLINK_GBS, 3)}), flush=True)
    shutdown()


if __name__ == "__main__":
    main()
