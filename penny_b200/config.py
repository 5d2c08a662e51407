"""One place for every knob: environment variables `PENNY_*` (plus the two the
reference already reads, `NNODES` and `VLLM_CUSTOM_ALLREDUCE_ALGO`) with keyword
overrides on top.

    cfg = PennyConfig.from_env(timeout_ms=2000)     # env first, then overrides
    comm = Communicator.create(group, config=cfg)
    print(cfg.describe())

The reference scatters its configuration over import-time `os.getenv("NNODES")`
(penny/custom_all_reduce.py:13, penny/utils.py:43, required there, optional
here), a C++ `getenv("VLLM_CUSTOM_ALLREDUCE_ALGO")` (csrc/custom_all_reduce.cuh:803-818)
and per-call arguments; there is no configuration object.

Variables that native code reads on its own (when a kernel family is first
used) are exported back to the environment by `apply_env()`, so a value given
as a keyword reaches them too.
"""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass
from typing import Optional

_TRUE = ("1", "true", "yes", "on")


def _env_bool(name: str, default: bool) -> bool:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return v.strip().lower() in _TRUE


def _env_int(name: str, default: int) -> int:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return int(v, 0)


@dataclass
class PennyConfig:
    # --- communicator
    heap_bytes: int = 1 << 30             # PENNY_HEAP_BYTES: symmetric heap per GPU
    timeout_ms: int = 10000               # PENNY_TIMEOUT_MS: bound of every device-side wait
    disable_nvls: bool = False            # PENNY_DISABLE_NVLS=1: never bind the NVSwitch multicast object
    heap_mode: str = "auto"               # PENNY_HEAP_MODE: auto | vmm | ipc
    nnodes: int = 1                       # NNODES: virtual nodes (shapes double ring / tree / node-aware ring)
    # --- algorithm choice
    algo: Optional[str] = None            # PENNY_ALGO: force one all-reduce algorithm
    vllm_algo: Optional[str] = None       # VLLM_CUSTOM_ALLREDUCE_ALGO: 1stage | oneshot | 2stage | twoshot
    tuner_cache: Optional[str] = None     # PENNY_TUNER_CACHE: JSON table of measured best algorithms
    custom_ar_blocks: int = 0             # PENNY_CUSTOM_AR_BLOCKS: block cap of the drop-in CustomAllreduce (0 = default)
    # --- GEMM kernels
    gemm_pair: bool = True                # PENNY_GEMM_PAIR=0: single-CTA tiles only (no cta_group::2)
    gemm_split_tail: bool = False         # PENNY_GEMM_SPLIT_TAIL=1: split the ragged last wave along K
    # --- debugging
    debug_poison: bool = False            # PENNY_DEBUG_POISON=1: fill scratch with NaN patterns between calls

    @classmethod
    def from_env(cls, **overrides) -> "PennyConfig":
        cfg = cls(
            heap_bytes=_env_int("PENNY_HEAP_BYTES", cls.heap_bytes),
            timeout_ms=_env_int("PENNY_TIMEOUT_MS", cls.timeout_ms),
            disable_nvls=_env_bool("PENNY_DISABLE_NVLS", cls.disable_nvls),
            heap_mode=os.environ.get("PENNY_HEAP_MODE", cls.heap_mode) or cls.heap_mode,
            nnodes=_env_int("NNODES", cls.nnodes),
            algo=os.environ.get("PENNY_ALGO") or None,
            vllm_algo=os.environ.get("VLLM_CUSTOM_ALLREDUCE_ALGO") or None,
            tuner_cache=os.environ.get("PENNY_TUNER_CACHE") or None,
            custom_ar_blocks=_env_int("PENNY_CUSTOM_AR_BLOCKS", cls.custom_ar_blocks),
            gemm_pair=_env_bool("PENNY_GEMM_PAIR", cls.gemm_pair),
            gemm_split_tail=_env_bool("PENNY_GEMM_SPLIT_TAIL", cls.gemm_split_tail),
            debug_poison=_env_bool("PENNY_DEBUG_POISON", cls.debug_poison),
        )
        unknown = set(overrides) - {f.name for f in dataclasses.fields(cls)}
        if unknown:
            raise TypeError(f"unknown PennyConfig field(s): {sorted(unknown)}")
        cfg = dataclasses.replace(cfg, **{k: v for k, v in overrides.items() if v is not None})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.heap_mode not in ("auto", "vmm", "ipc"):
            raise ValueError(f"PENNY_HEAP_MODE must be auto, vmm or ipc, not {self.heap_mode!r}")
        if self.heap_bytes < (16 << 20):
            raise ValueError("the symmetric heap must be at least 16 MiB")
        if self.timeout_ms < 0 or self.nnodes < 1 or self.custom_ar_blocks < 0:
            raise ValueError("timeout_ms >= 0, nnodes >= 1 and custom_ar_blocks >= 0 are required")
        if self.vllm_algo is not None and self.vllm_algo.lower() not in ("1stage", "oneshot", "2stage", "twoshot"):
            raise ValueError(f"VLLM_CUSTOM_ALLREDUCE_ALGO: unknown value {self.vllm_algo!r}")

    def apply_env(self) -> None:
        """Exports the fields that native code or other modules read from the environment."""
        os.environ["PENNY_HEAP_BYTES"] = str(int(self.heap_bytes))
        os.environ["PENNY_TIMEOUT_MS"] = str(int(self.timeout_ms))
        os.environ["PENNY_DISABLE_NVLS"] = "1" if self.disable_nvls else "0"
        if self.heap_mode != "auto":
            os.environ["PENNY_HEAP_MODE"] = self.heap_mode
        os.environ["NNODES"] = str(int(self.nnodes))
        os.environ["PENNY_GEMM_PAIR"] = "1" if self.gemm_pair else "0"
        os.environ["PENNY_GEMM_SPLIT_TAIL"] = "1" if self.gemm_split_tail else "0"
        for name, val in (("PENNY_ALGO", self.algo), ("VLLM_CUSTOM_ALLREDUCE_ALGO", self.vllm_algo),
                          ("PENNY_TUNER_CACHE", self.tuner_cache)):
            if val:
                os.environ[name] = str(val)
        if self.custom_ar_blocks:
            os.environ["PENNY_CUSTOM_AR_BLOCKS"] = str(int(self.custom_ar_blocks))

    def describe(self) -> str:
        return ", ".join(f"{f.name}={getattr(self, f.name)!r}" for f in dataclasses.fields(self))
