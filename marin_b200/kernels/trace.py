"""Which kernels were running when a launch failed: the host side of the ``-DMB_TRACE`` build.

With ``MARIN_B200_DEFINES=MB_TRACE`` in the environment every kernel's first block leaves a mark (library, source line
of the kernel's entry) in a small buffer of pinned host memory before it waits for the kernels ahead of it.  Host
memory outlives a fault of the CUDA context, so after ``unspecified launch failure`` the last marks still say which
kernels had started: with programmatic dependent launch up to three neighbours are on the device at once, and the one
that faulted is among them.  Usage::

    from marin_b200.kernels import trace
    marks = trace.Marks()          # before the work
    ...                            # run; call marks.arm() again after new libraries were loaded
    print(marks.last(12))          # after the failure: [(library, line), ...], oldest first

A measuring aid: the engine never uses this build (marks cost a system-wide atomic per kernel).
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

import torch

from . import build

#: library ids as the sources define them (MB_LIB_ID next to MB_LIB)
LIBRARIES = {1: "elementwise.cu", 2: "gemm_tc.cu", 3: "attention_fast.cu", 4: "attention_tc.cu", 5: "sampling.cu",
             6: "gemm_simple.cu", 7: "attention_simple.cu"}
SLOTS = 1023


class Marks:
    def __init__(self):
        self.buffer = torch.zeros(1 + SLOTS, dtype=torch.int32).pin_memory()
        self.arm()

    def arm(self) -> int:
        """Hands the buffer to every library loaded so far that was built with MB_TRACE; returns how many took it."""
        took = 0
        for lib in list(build._loaded.values()):
            if hasattr(lib, "mb_set_trace") and lib.mb_set_trace(ctypes.c_void_p(self.buffer.data_ptr())) == 0:
                took += 1
        return took

    def count(self) -> int:
        return int(self.buffer[0])

    def last(self, n: int = 12) -> List[Tuple[str, int]]:
        values = self.buffer.numpy()
        total = int(values[0])
        marks = [int(values[1 + i % SLOTS]) for i in range(max(0, total - min(n, SLOTS)), total)]
        return [(LIBRARIES.get(m >> 20, str(m >> 20)), m & 0xFFFFF) for m in marks]
