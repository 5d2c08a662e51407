"""`from penny.utils import initialize_distributed, bench_kineto` – the reference's import path."""
from penny_b200.utils import (bench_device, bench_kineto, bus_bandwidth_gbs, flush_l2,  # noqa: F401
                              global_communicator, initialize_distributed, shutdown)
