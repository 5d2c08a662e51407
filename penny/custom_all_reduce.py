"""`from penny.custom_all_reduce import CustomAllreduce` – the reference's import path."""
from penny_b200.parallel.custom_all_reduce import (CustomAllreduce, _can_p2p, custom_ar,  # noqa: F401
                                                  is_weak_contiguous, nnodes)
