"""A fixed split of the GPU's SMs between two streams (CUDA green contexts).

``SmSplit(device, decode_pct)`` asks the driver for two SM partitions and a stream in each.  The engine's prefill
lane runs on the stream of the ``100 - decode_pct`` percent partition, so prompt chunks can never occupy the SMs that
decode steps need; decode itself stays on the process's ordinary stream and may use every SM that is idle.  The split
belongs to the process and disappears with it.

Reference parity: pegainfer-qwen3/src/green_ctx.rs (``--decode-sm-pct``), pegainfer-gemma4/src/green_ctx.rs.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native


class SmSplit:
    def __init__(self, device, decode_pct: int):
        if not 10 <= decode_pct <= 90:
            raise ValueError("--decode-sm-pct must be between 10 and 90")
        self.device = torch.device(device)
        lib = _native.load()
        if not lib.pg_green_available():
            raise RuntimeError("this driver offers no green contexts: --decode-sm-pct is not available")
        total = torch.cuda.get_device_properties(self.device).multi_processor_count
        want = max(8, min(total - 8, round(total * decode_pct / 100)))
        h = ctypes.c_void_p()
        _native.check(lib.pg_green_split(ctypes.c_int(self.device.index or 0), ctypes.c_int(want), ctypes.byref(h)))
        self._handle, self._lib = h, lib
        sa, sb, na, nb = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int(), ctypes.c_int()
        _native.check(lib.pg_green_info(h, ctypes.byref(sa), ctypes.byref(sb), ctypes.byref(na), ctypes.byref(nb)))
        self.decode_sms, self.prefill_sms = na.value, nb.value
        self.decode_stream = torch.cuda.ExternalStream(sa.value, device=self.device)
        self.prefill_stream = torch.cuda.ExternalStream(sb.value, device=self.device)

    def close(self) -> None:
        if self._handle is not None:
            torch.cuda.synchronize(self.device)
            self._lib.pg_green_destroy(self._handle)
            self._handle = None
