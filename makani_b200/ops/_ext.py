"""Loader for the in-tree sm_100a extension (`makani_b200/csrc/_C.so`).

The extension is built by `python -m makani_b200.csrc.build` (or `__graft_entry__.build()`); it is never
JIT-compiled at import time.  `require()` raises with build instructions when a CUDA tensor reaches an op
and the extension cannot be loaded, so that a GPU run can never silently fall back to eager PyTorch.
"""

from __future__ import annotations

import importlib.util
import os
import threading

_LOCK = threading.Lock()
_MOD = None
_ERR = None

SO_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "_C.so")


def _load():
    global _MOD, _ERR
    with _LOCK:
        if _MOD is not None or _ERR is not None:
            return
        try:
            import torch  # noqa: F401  (libtorch must be loaded before the extension)

            if not os.path.exists(SO_PATH):
                raise FileNotFoundError(f"{SO_PATH} not built")
            spec = importlib.util.spec_from_file_location("makani_b200.csrc._C", SO_PATH)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.set_gelu_tanh(1 if _GELU_TANH else 0)
            _MOD = mod
        except Exception as e:  # pragma: no cover - depends on the machine
            _ERR = e


# MAKANI_B200_NATIVE=0 (or `set_native(False)`) routes every op through its plain PyTorch formulation: the
# op-for-op restatement of the reference's execution (cuDNN/cuBLAS/cuFFT/ATen/NCCL) used as the same-box comparison arm.
_NATIVE = os.environ.get("MAKANI_B200_NATIVE", "1") != "0"
_GELU_TANH = os.environ.get("MAKANI_B200_GELU", "erf") == "tanh"


def set_native(flag: bool) -> None:
    global _NATIVE
    _NATIVE = bool(flag)


def native() -> bool:
    return _NATIVE


def available() -> bool:
    _load()
    return _MOD is not None


# number of kernels of this extension launched by the current process (each binding call launches exactly one)
LAUNCHES = 0
_NON_KERNEL = {"read_error_flag", "clear_error_flag", "lp_scratch_floats", "adam_entry_bytes", "peer_alloc", "peer_open",
               "peer_close", "peer_free", "tensor_from_ptr", "set_gelu_tanh"}


class _Counting:
    """Thin proxy over the extension module that counts kernel launches."""

    def __init__(self, mod):
        self._mod = mod
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._mod, name)
            if name in _NON_KERNEL:
                fn = raw
            else:
                def fn(*args, __raw=raw, **kwargs):
                    global LAUNCHES
                    LAUNCHES += 1
                    return __raw(*args, **kwargs)
            self._cache[name] = fn
        return fn


_PROXY = None


def require():
    global _PROXY
    _load()
    if _MOD is None:
        raise RuntimeError(
            "makani_b200: the sm_100a extension is not available "
            f"({_ERR!r}). Build it with `python -m makani_b200.csrc.build`."
        )
    if _PROXY is None:
        _PROXY = _Counting(_MOD)
    return _PROXY


_SM_COUNT = {}


def sm_count(device=None) -> int:
    """Number of SMs of `device` (148 on B200); used to size split-k factors and grids."""
    import torch

    if not torch.cuda.is_available():
        return 148
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def set_gelu_approximation(kind: str) -> None:
    """"none" (default): GELU is the exact erf form everywhere, as torch.nn.GELU(); "tanh": the tanh approximation
    (hardware tanh.approx in the kernels, `approximate="tanh"` in the torch fallbacks)."""
    global _GELU_TANH
    assert kind in ("none", "tanh")
    _GELU_TANH = kind == "tanh"
    if _MOD is not None or available():
        _MOD.set_gelu_tanh(1 if _GELU_TANH else 0)


def gelu_approximation() -> str:
    return "tanh" if _GELU_TANH else "none"


def launch_count() -> int:
    return LAUNCHES


def add_launches(n: int) -> None:
    """Account for kernels of this extension that a CUDA-graph replay launched (counted once at capture time)."""
    global LAUNCHES
    LAUNCHES += int(n)


# Codes written to the per-device error word by kernels whose bounded waits (2 s) ran out.
ERROR_CODES = {
    1: "GEMM producer: shared-memory stage never freed (empty barrier)",
    2: "GEMM MMA issuer: accumulator buffer never drained (TMEM-empty barrier)",
    3: "GEMM MMA issuer: operands never arrived (full barrier / TMA load)",
    4: "GEMM epilogue: accumulator never completed (TMEM-full barrier)",
    5: "GEMM producer: epilogue-operand buffer never freed",
    6: "GEMM epilogue: epilogue operand never arrived",
    16: "peer all-reduce: a rank did not reach the barrier",
    32: "GEMM: peers did not deliver / release the first handshake buffer",
    33: "GEMM: peers did not deliver / release the second handshake buffer",
    40: "publish kernel: peers still read the previous contents",
    44: "segment-sum kernel: a peer's segment did not arrive",
    56: "instance-norm statistics: peers still read the previous sums",
    57: "instance-norm apply: a peer's sums did not arrive",
}


def describe_error(code: int) -> str:
    return ERROR_CODES.get(int(code), "unknown code")


def check_device_errors(device=None) -> None:
    """Raise if a kernel recorded an expired bounded wait on `device` (synchronises)."""
    import torch

    if _MOD is None or not torch.cuda.is_available():
        return
    dev = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    code = _MOD.read_error_flag(int(dev))
    if code != 0:
        _MOD.clear_error_flag(int(dev))
        raise RuntimeError(f"makani_b200: a device-side bounded wait expired (code {code}: {describe_error(code)})")
