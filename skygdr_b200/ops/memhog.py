"""Best-effort HBM task (skygdr_b200/csrc/kernels/memhog.cu)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .._ext import load
from .flow import CreditPage, new_status, read_status

OPS = {"read": 0, "write": 1, "rw": 2, "copy": 3, "axpy": 4}
BYTES_PER_VEC = {0: 16, 1: 16, 2: 32, 3: 32, 4: 48}


class Memhog:
    """A working set of ``gb`` GiB (two halves unless read-only) and a persistent kernel over it.

    Reference: src/gpu_be_memhog_task.cu (flags :142-201) and
    llm_problem_analysis/decode_hbm_stress.cu (axpy over half/half of the working set)."""

    def __init__(self, device, gb: float = 16.0, op: str = "rw", ctas: Optional[int] = None, threads: int = 256,
                 chunk_bytes: int = 1 << 20, page: Optional[CreditPage] = None):
        self._C = load()
        self.device = torch.device(device)
        self.op = OPS[op]
        total = int(gb * (1 << 30))
        half = total if op == "read" else total // 2
        half -= half % 16
        self.a = torch.zeros(half // 4, dtype=torch.float32, device=self.device)
        self.b = torch.zeros(half // 4 if op != "read" else 0, dtype=torch.float32, device=self.device)
        self.sink = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.status = new_status(self.device)
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.ctas = ctas or sms * 4
        self.threads, self.chunk_bytes, self.page = threads, chunk_bytes, page
        self.consumed = 0

    def bytes_per_pass(self) -> int:
        return (self.a.numel() * 4 // 16) * BYTES_PER_VEC[self.op]

    def launch(self, iters: int = 1, seconds: float = 0.0, duty_on_ms: float = 0.0, duty_off_ms: float = 0.0,
               alpha: float = 0.5, max_wait_ms: float = 2.0) -> None:
        self._C.reset_status(self.status)
        self._C.memhog(self.a, self.b, self.op, iters, int(seconds * 1e9), int(duty_on_ms * 1e6), int(duty_off_ms * 1e6),
                       self.chunk_bytes, self.ctas, self.threads, self.page.dev_ptr if self.page else 0, self.consumed,
                       int(max_wait_ms * 1e6), alpha, self.sink, self.status)

    def result(self) -> Dict[str, float]:
        torch.cuda.synchronize(self.device)
        st = read_status(self.status)
        self.consumed += st["bytes_done"]
        dt = (st["t_end_ns"] - st["t_start_ns"]) * 1e-9
        st["seconds"] = dt
        st["gib_s"] = st["bytes_done"] / dt / (1 << 30) if dt > 0 else 0.0
        st["gb_s"] = st["bytes_done"] / dt / 1e9 if dt > 0 else 0.0
        return st
