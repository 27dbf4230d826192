"""A model: the parts its spec names, their weights, and the forward pass of
one step over a schedule of layers.

The forward pass follows the reference's order
(crates/nncpu/src/model/forward.rs:848-965): embedding rows, the schedule's
blocks over a float32 residual stream, and, only for the rows whose logits
are wanted, the final norm and the vocabulary projection
(crates/nncpu/src/model/forward.rs:974-985,1017-1030).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache import KVRequest, StateRequest
from ..config import ModelSpec, load_config
from ..errors import BadFormat, InvalidArgument, translating_oom
from ..kernels import ops
from ..parts import Runtime, build
from ..weights import ParamSpec, load_tensors, random_tensors_on_device

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise InvalidArgument(f"dtype {dtype!r} is not supported (bfloat16 or float32)") from None


def _gib(params: List[ParamSpec], dtype: torch.dtype) -> float:
    esize = 2 if dtype == torch.bfloat16 else 4
    n = 0
    for p in params:
        c = 1
        for d in p.shape:
            c *= d
        n += c
    return n * esize / 2 ** 30


def _shares(spec: ModelSpec) -> List[bool]:
    """Per layer: whether its runs read another entry's keys and values."""
    share: List[Optional[bool]] = [None] * len(spec.layers)
    for i, e in enumerate(spec.schedule):
        if not 0 <= e.layer < len(spec.layers):
            raise BadFormat(f"schedule entry {i} names layer {e.layer}, but there are {len(spec.layers)} layers")
        s = e.cache_of is not None
        if share[e.layer] is not None and share[e.layer] != s:
            raise BadFormat(f"layer {e.layer} runs both with a cache of its own and on another entry's cache")
        share[e.layer] = s
    return [bool(s) for s in share]


def build_blocks(spec: ModelSpec) -> list:
    shares = _shares(spec)
    return [build("block", b, **({"reads_other_cache": True} if shares[i] else {}))
            for i, b in enumerate(spec.layers)]


def parameter_list(spec: ModelSpec) -> List[ParamSpec]:
    """Every tensor the model of ``spec`` reads from its file."""
    e, o = spec.embedding, spec.output
    params = [ParamSpec(f"{e.name}.weight", (e.vocab_size, e.hidden_size))]
    for block in build_blocks(spec):
        params += block.params()
    params += build("norm", o.norm).params()
    if not o.tied:
        params.append(ParamSpec(f"{o.name}.weight", (o.vocab_size, o.hidden_size)))
    return params


class Model:
    """Built by ``Model.load``; run through an ``Engine``."""

    def __init__(self, config, tensors: Dict[str, torch.Tensor], rt: Runtime):
        self.config = config
        self.spec = spec = config.model_spec()
        self.rt = rt
        self.blocks = build_blocks(spec)
        self.final_norm = build("norm", spec.output.norm)
        # `tensors` is consumed: parts take what they fuse out of it, so that no second copy stays alive
        self.embed_table = tensors[f"{spec.embedding.name}.weight"]
        self.lm_head = self.embed_table if spec.output.tied else tensors[f"{spec.output.name}.weight"]
        for block in self.blocks:
            block.bind(tensors, rt)
        self.final_norm.bind(tensors, rt)
        self.schedule = list(spec.schedule)
        self._cache_plan = self._plan_cache()

    @classmethod
    def load(cls, folder, dtype="bfloat16", device="cuda:0", progress=None) -> "Model":
        """Reads ``folder/config.json``, picks the architecture's configuration
        class from the registry, checks the folder's safetensors file (or the
        files of its index) against what the parts ask for, and moves the
        weights to ``device``."""
        config = load_config(folder)
        dt = resolve_dtype(dtype)
        rt = Runtime(device, dt)
        params = parameter_list(config.model_spec())
        with translating_oom(f"the weights of {folder} ({_gib(params, dt):.2f} GiB in {dtype})"):
            tensors = load_tensors(folder, params, dt, rt.device, progress)
            return cls(config, tensors, rt)

    @classmethod
    def random(cls, config, seed: int, dtype="bfloat16", device="cuda:0") -> "Model":
        """A model of ``config`` with random weights made on the device (no
        files).  ``write_model_folder`` is the mode that writes a folder."""
        dt = resolve_dtype(dtype)
        rt = Runtime(device, dt)
        params = parameter_list(config.model_spec())
        with translating_oom(f"random weights ({_gib(params, dt):.2f} GiB in {dtype})"):
            return cls(config, random_tensors_on_device(params, seed, dt, rt.device), rt)

    # -- storage the schedule asks for ------------------------------------------

    def cache_requests(self) -> Tuple[List[Tuple[Optional[KVRequest], Optional[StateRequest]]], List[Optional[int]]]:
        return self._cache_plan

    def _plan_cache(self):
        """What the cache must hold: one (keys/values, state) request per cache user, and for each user the
        user whose keys and values it reads instead of its own.  A schedule entry has as many users as its
        block asks for (``Block.cache_requests()``: one per mixer, none for a block without one); an entry that
        reads another entry's cache pairs its users with that entry's, in order."""
        requests, cache_of = [], []
        self._users = []   # per schedule entry: (first user, number of users)
        for i, e in enumerate(self.schedule):
            asked = self.blocks[e.layer].cache_requests()
            if e.cache_of is not None and self._users[e.cache_of][1] != len(asked):
                raise BadFormat(f"schedule entry {i} reads the cache of entry {e.cache_of}, whose block keeps "
                                f"{self._users[e.cache_of][1]} caches where this one needs {len(asked)}")
            self._users.append((len(requests), len(asked)))
            for k, (kv, state) in enumerate(asked):
                requests.append((None if e.cache_of is not None else kv, state))
                cache_of.append(None if e.cache_of is None else self._users[e.cache_of][0] + k)
        return requests, cache_of

    # -- numbers for reports ------------------------------------------------------

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a decode step reads: every scheduled block once
        and the output matrix; the embedding table is gathered, not streamed."""
        head = self.lm_head.numel() * self.lm_head.element_size()
        return sum(self.blocks[e.layer].weight_bytes() for e in self.schedule) + head

    def info(self) -> dict:
        """What the model is, in the reference's terms (crates/nncpu/src/lib.rs:150-190): sizes, counts and the
        bytes its weights hold on the device.  Head counts are those of the first mixer that has heads."""
        n_params = sum(int(torch.tensor(p.shape).prod()) for p in parameter_list(self.spec) if p.required)
        heads = next((b.mixer for b in self.spec.layers if hasattr(b.mixer, "n_heads")), None)
        weights = self.weight_bytes_per_step() + (0 if self.spec.output.tied else
                                                  self.embed_table.numel() * self.embed_table.element_size())
        return {"architecture": self.spec.architecture, "dtype": str(self.rt.dtype).replace("torch.", ""),
                "layers": len(self.spec.layers), "schedule": len(self.schedule),
                "hidden_size": self.spec.hidden_size, "vocab_size": self.spec.vocab_size,
                "n_heads": getattr(heads, "n_heads", None), "n_kv_heads": getattr(heads, "n_kv_heads", None),
                "head_dim": getattr(heads, "head_dim", None),
                "parameters": n_params, "weight_bytes": weights, "max_positions": self.spec.max_positions}

    # -- one step -------------------------------------------------------------------

    def forward(self, ctx, cache) -> Optional[torch.Tensor]:
        """Runs the step's tokens through the schedule and returns float32
        logits [n_wanted, vocab] (None when no row is wanted)."""
        rt, spec = self.rt, self.spec
        residual = rt.empty(ctx.n_tokens, spec.hidden_size, dtype=torch.float32)
        with rt.phase("embed"):
            ops.embed(self.embed_table, ctx.tok_ids, residual, spec.embedding.scale)
        ctx.next_norm = ctx.after_block = None
        fusing = rt.dtype == torch.bfloat16 and rt.fuses_norms(ctx.n_tokens, spec.hidden_size)
        if fusing:
            rt.begin_norm_fusion(ctx.n_tokens)      # norms may ride on the products around them
        for i, (e, (first, count)) in enumerate(zip(self.schedule, self._users)):
            if i + 1 < len(self.schedule):
                # the block that follows may ask this one to leave its first norm's input (a few tokens only)
                ctx.after_block = self.blocks[self.schedule[i + 1].layer].entry_norm_request(ctx, residual)
            self.blocks[e.layer].forward(ctx, residual, [ctx.entry_cache(cache, u) for u in range(first, first + count)])
        ctx.next_norm = ctx.after_block = None
        if fusing:
            rt.end_norm_fusion()
        if ctx.n_wanted == 0:
            return None
        x = self.final_norm.forward(ctx, residual, rows=ctx.logit_rows)
        logits = rt.empty(ctx.n_wanted, spec.vocab_size, dtype=torch.float32)
        with rt.phase("lm_head", self.lm_head, ctx.n_wanted):
            rt.linear(x, self.lm_head, None, logits)
        return logits
