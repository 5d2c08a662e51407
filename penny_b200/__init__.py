"""penny_b200: Blackwell-native collectives with the capabilities of Penny.

    penny_b200.parallel   communicators (symmetric heap, NVLS), CustomAllreduce,
                          the gloo CPU backend, the tuner, schedule math
    penny_b200.ops        all_reduce / all_gather / reduce_scatter / exchange /
                          all_to_all and the fused ops
    penny_b200.models     Llama-3-8B-shaped TP decode and sequence-parallel prefill,
                          Mixtral-shaped EP layer
    penny_b200.utils      initialize_distributed, device-side benchmarking
    penny_b200.config     PennyConfig: every PENNY_* environment knob in one object

`import penny` and `import penny_cpp` keep the reference's import paths.
"""
__version__ = "0.1.0"

from .config import PennyConfig  # noqa: E402,F401
