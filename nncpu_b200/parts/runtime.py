"""What parts need from their surroundings: the device, the run's element
type, a device status word for kernels with bounded waits, and the choice
between the tensor-core and the CUDA-core matrix product.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import List, Optional

import torch

from .. import perf
from ..errors import ExtensionError
from ..kernels import ops
from .base import DeferredNorm


class Arena:
    """The memory of one step's intermediate tensors: one device buffer that ``Runtime.empty`` carves pieces
    from, front to back, so that a step asks the allocator for nothing
    (the reference sizes its forward scratch once: crates/nncpu/src/model/kv.rs:45-47,295-332).

    * ``begin()`` starts a step: everything handed out before is void.
    * ``mark()`` / ``release(mark)`` give back what a part of the step no longer needs (a block's
      temporaries when the block is done), so the buffer holds the widest moment of a step, not its sum.
      What must live until the step ends although it is made inside such a part (a table that later layers
      read) is taken with ``keep=True``, from the buffer's other end.
    * ``measure()``: pieces are shape-only (``meta``) tensors and only the sizes are added up; a forward pass
      run this way launches nothing and tells how large the buffer must be.
    * A request that does not fit is served by the allocator once, and the next ``begin()`` makes the buffer
      large enough for it; an arena that a CUDA graph has captured is ``frozen`` instead and refuses, because its
      addresses are part of the graph."""
    ALIGN = 256

    def __init__(self, device):
        self.device = torch.device(device)
        self.buf: Optional[torch.Tensor] = None
        self.typed = {}                 # the buffer seen as each element type that was asked for
        self.capacity = 0
        self.offset = 0                 # bytes in use from the front (given back by release)
        self.top = 0                    # bytes in use from the back (kept until the step ends)
        self.peak = 0
        self.overflow: List[torch.Tensor] = []
        self.measuring = False
        self.frozen = False

    def reserve(self, nbytes: int) -> None:
        nbytes = (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN    # pieces from the back are aligned too
        if nbytes > self.capacity:
            if self.frozen:
                raise ExtensionError("a captured step's arena cannot grow")
            self.buf = None             # the old buffer goes back before the new one is asked for
            self.typed = {}
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            self.capacity = nbytes

    def begin(self) -> None:
        self.overflow.clear()
        if self.peak > self.capacity and not self.measuring:
            self.reserve(self.peak)
        self.offset = self.top = 0

    def mark(self) -> int:
        return self.offset

    def release(self, mark: int) -> None:
        self.offset = mark

    def alloc(self, shape, dtype: torch.dtype, keep: bool = False) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        size = dtype.itemsize
        nbytes = n * size
        if keep:
            self.top += (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
            start = self.capacity - self.top
        else:
            start = (self.offset + self.ALIGN - 1) // self.ALIGN * self.ALIGN
            self.offset = start + nbytes
        self.peak = max(self.peak, self.offset + self.top)
        if self.measuring:
            return torch.empty(shape, dtype=dtype, device="meta")
        if self.offset + self.top <= self.capacity:
            whole = self.typed.get(dtype)
            if whole is None:
                whole = self.typed[dtype] = self.buf[:self.capacity // size * size].view(dtype)
            return whole[start // size:start // size + n].view(shape)
        if self.frozen:
            raise ExtensionError(f"a captured step asked for {nbytes} bytes beyond its arena of {self.capacity}")
        t = torch.empty(shape, dtype=dtype, device=self.device)
        self.overflow.append(t)
        return t


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
        self.arena: Optional[Arena] = None      # set by the engine around a step; without one, the allocator serves
        self._norm_bins = None          # accumulators of the norms that ride on products, during such a step
        self._norm_rows = [None, None]
        self._norm_turn = 0
        self._status_host = None
        self._status_posted = []
        self._status_turn = 0

    def empty(self, *shape, dtype=None, keep: bool = False) -> torch.Tensor:
        """An uninitialised tensor for this step: a piece of the step's arena, void when the next step begins, or
        when the part that asked for it is done (``scope``) unless it is to ``keep``."""
        if self.arena is not None:
            return self.arena.alloc(shape, dtype or self.dtype, keep)
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    @contextmanager
    def using(self, arena: Optional[Arena]):
        """Steps inside take their tensors from ``arena``."""
        before, self.arena = self.arena, arena
        try:
            yield arena
        finally:
            self.arena = before

    @contextmanager
    def scope(self):
        """What is taken from the arena inside is given back at the end: for a part's temporaries."""
        arena = self.arena
        mark = arena.mark() if arena is not None else 0
        try:
            yield
        finally:
            if arena is not None and self.arena is arena:
                arena.release(mark)

    @property
    def workspace(self) -> ops.GemmWorkspace:
        """Made when the first tensor-core product needs it (a float32 run never does)."""
        if self._workspace is None:
            self._workspace = ops.GemmWorkspace(self.device)
        return self._workspace

    def tensor_cores_take(self, x_dtype, w, k: int) -> bool:
        return x_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ops.linear_tc_supported(1, w.shape[0], k)

    def linear(self, x, w, bias, out, accumulate: bool = False, epilogue: str = "plain", then_norm=None) -> None:
        """out (+)= x . w^T + bias.  bfloat16 inputs whose sizes keep TMA's
        alignment rule go to the tensor cores; everything else, and every
        float32 product, runs in true 32-bit on CUDA cores.

        ``x`` may be a ``DeferredNorm`` (a norm's unfinished output): the few-token product and the product of
        whole prompts finish it, any other path makes the ordinary tensor first.  ``then_norm`` (a ``NormRequest``):
        this product is the last write into ``out`` before that norm reads it; the same two products fulfil it."""
        deferred = x if isinstance(x, DeferredNorm) else None
        takes = self.tensor_cores_take(x.dtype, w, x.shape[1])
        few = takes and x.shape[0] <= ops.SKINNY_MAX_TOKENS
        # which norms this product can carry: the one before it (bit 0), the one after it (bit 1)
        roles = 3 if few else (ops.linear_tc_norm_roles(x.shape[0], w.shape[0], x.shape[1]) if takes else 0)
        fuses = bool(roles & 2)
        if deferred is not None:
            if roles & 1:
                x, norm_in = deferred.x_gamma, (deferred.bins, deferred.request.eps)
            else:
                x, norm_in = deferred.finish(), None
        else:
            norm_in = None
        if takes:
            norm_out = None
            if (fuses and then_norm is not None and self._norm_bins is not None and epilogue == "plain"
                    and out.dtype == torch.float32 and out.shape[1] == then_norm.size == w.shape[0] and out.is_contiguous()
                    and self._norm_bins.shape[1] == (ops.SKINNY_MAX_TOKENS if few else out.shape[0])):
                # two sets of accumulators (and of rows times gamma) take turns: this product adds into one (zero
                # since it was last cleared) and clears the other, whose consumer has run by now
                turn = self._norm_turn
                self._norm_turn = 1 - turn
                if self._norm_rows[turn] is None:
                    self._norm_rows[turn] = self.empty(*out.shape, keep=True)
                made = DeferredNorm(self._norm_rows[turn], self._norm_bins[turn], then_norm)
                norm_out = (made.x_gamma, then_norm.gamma, made.bins, self._norm_bins[1 - turn])
            if few:
                ops.linear_skinny(x, w, bias, out, accumulate, epilogue,
                                  norm_out and (norm_out[0], norm_out[1], norm_out[2].view(-1), norm_out[3].view(-1)),
                                  norm_in and (norm_in[0].view(-1), norm_in[1]))
            else:
                ops.linear_tc(x, w, bias, out, self.workspace, accumulate, epilogue, norm_out=norm_out, norm_in=norm_in)
            if norm_out is not None:
                then_norm.result = made
        else:
            assert epilogue == "plain", "the fused epilogue exists on the tensor-core path only"
            ops.linear_simt(x, w, bias, out, accumulate)

    def fuses_norms(self, n_tokens: int, n_out: int) -> bool:
        """Whether the bfloat16 products of a step of ``n_tokens`` rows (``n_out`` output features) may carry the norms
        around them: the few-token product always, the tensor-core product on pairs of SMs, and from 17 to 64
        tokens the kernels that ``ops.linear_tc_norm_roles`` names (each product is asked when its turn comes; one
        that cannot leaves the norm to its own kernel)."""
        return (n_tokens <= ops.SKINNY_MAX_TOKENS or ops.linear_tc_fuses_norms(n_tokens, n_out)
                or n_tokens <= ops.CLUSTER_MAX_TOKENS)

    def begin_norm_fusion(self, n_tokens: int) -> None:
        """Once per step whose products may carry norms: two sets of exact accumulators, one row each per token (16
        rows for a step of few tokens), start at zero (one fill), whatever an earlier step or another captured graph
        left in them; the rows times gamma that go with them are taken when the first product needs them."""
        rows = ops.SKINNY_MAX_TOKENS if n_tokens <= ops.SKINNY_MAX_TOKENS else n_tokens
        self._norm_bins = self.empty(2, rows, ops.NORM_ROW_WORDS, dtype=torch.int64, keep=True)
        self._norm_bins.zero_()
        self._norm_rows = [None, None]
        self._norm_turn = 0

    def end_norm_fusion(self) -> None:
        """The step is over: its accumulators belong to the step's arena."""
        self._norm_bins = None
        self._norm_rows = [None, None]

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
