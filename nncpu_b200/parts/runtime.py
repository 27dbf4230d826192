"""What parts need from their surroundings: the device, the run's element
type, a device status word for kernels with bounded waits, and the choice
between the tensor-core and the CUDA-core matrix product.
"""
from __future__ import annotations

import torch

from .. import perf
from ..errors import ExtensionError
from ..kernels import ops


class Runtime:
    def __init__(self, device, dtype: torch.dtype):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ExtensionError(f"models run on a CUDA device, not on {self.device}: there is no CPU path")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ExtensionError(f"run element type {dtype} is not supported (bfloat16 or float32)")
        self.dtype = dtype
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._workspace = None
        self._status_host = None
        self._status_posted = []
        self._status_turn = 0

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    @property
    def workspace(self) -> ops.GemmWorkspace:
        """Made when the first tensor-core product needs it (a float32 run never does)."""
        if self._workspace is None:
            self._workspace = ops.GemmWorkspace(self.device)
        return self._workspace

    def tensor_cores_take(self, x_dtype, w, k: int) -> bool:
        return x_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ops.linear_tc_supported(1, w.shape[0], k)

    def linear(self, x, w, bias, out, accumulate: bool = False, epilogue: str = "plain") -> None:
        """out (+)= x . w^T + bias.  bfloat16 inputs whose sizes keep TMA's
        alignment rule go to the tensor cores; everything else, and every
        float32 product, runs in true 32-bit on CUDA cores."""
        if self.tensor_cores_take(x.dtype, w, x.shape[1]):
            if x.shape[0] <= ops.SKINNY_MAX_TOKENS:
                ops.linear_skinny(x, w, bias, out, accumulate, epilogue)
            else:
                ops.linear_tc(x, w, bias, out, self.workspace, accumulate, epilogue)
        else:
            assert epilogue == "plain", "the fused epilogue exists on the tensor-core path only"
            ops.linear_simt(x, w, bias, out, accumulate)

    def phase(self, slot: str, weight=None, n_tokens: int = 0, nbytes: float = 0, flops: float = 0):
        """A profiler scope for the launches of one phase (free when the profiler is off).  With ``weight`` the
        phase is a product of ``n_tokens`` rows with that matrix: it streams the matrix once and does two
        operations per element and row."""
        if not perf.enabled():
            return perf._NULL
        if weight is not None:
            nbytes += weight.numel() * weight.element_size()
            flops += 2.0 * n_tokens * weight.numel()
        return perf.scope(slot, nbytes, flops)

    def post_status(self) -> None:
        """Starts a copy of the status word to pinned host memory, in stream order.  A caller that then waits
        for later work of the same stream (an event, a copy) can ``check_status()`` without waiting again."""
        if self._workspace is None:
            return
        if self._status_host is None:
            self._status_host = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(8)]
            self._status_events = [torch.cuda.Event() for _ in range(8)]
            self._status_posted = []
        i = self._status_turn = (self._status_turn + 1) % len(self._status_host)
        self._status_posted = [j for j in self._status_posted if j != i]
        self._status_host[i].copy_(self._workspace.status, non_blocking=True)
        self._status_events[i].record()
        self._status_posted.append(i)

    def check_status(self) -> None:
        """Raises if a kernel's bounded wait ran out.  Reads the copies that ``post_status`` started and that
        have arrived; when none was posted it reads the word itself, which waits for the stream."""
        if self._workspace is None:
            return
        code = 0
        if self._status_posted:
            waiting = []
            for i in self._status_posted:
                if self._status_events[i].query():
                    code = code or int(self._status_host[i][0])
                else:
                    waiting.append(i)
            self._status_posted = waiting
        else:
            code = int(self._workspace.status.item())
        if code:
            torch.cuda.synchronize(self.device)
            self._workspace.status.zero_()
            self._status_posted = []
            raise ExtensionError(f"a kernel gave up waiting (status {code}); the step's results are not valid")
