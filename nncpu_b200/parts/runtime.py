"""What parts need from their surroundings: the device, the run's element
type, a device status word for kernels with bounded waits, and the choice
between the tensor-core and the CUDA-core matrix product.
"""
from __future__ import annotations

import torch

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
        self._workspace = None

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

    def check_status(self) -> None:
        """Call after a synchronisation: raises if a kernel's bounded wait ran out."""
        if self._workspace is None:
            return
        code = int(self._workspace.status.item())
        if code:
            self._workspace.status.zero_()
            raise ExtensionError(f"a kernel gave up waiting (status {code}); the step's results are not valid")
