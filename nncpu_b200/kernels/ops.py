"""Python faces of the CUDA kernels: one function per kernel, taking torch
tensors on the GPU and launching on torch's current stream.

Nothing here computes: every function checks what only Python can see
(devices, element types, contiguity), then calls the C entry point, which
checks sizes and either launches or refuses with a message.
"""
from __future__ import annotations

import ctypes
import functools
from typing import Optional

import torch

from ..errors import ExtensionError, InvalidArgument
from . import library

_DT = {torch.float32: 0, torch.bfloat16: 1}
_vp = ctypes.c_void_p


def _code(t: Optional[torch.Tensor]) -> int:
    if t is None:
        return 0
    try:
        return _DT[t.dtype]
    except KeyError:
        raise InvalidArgument(f"kernels take float32 or bfloat16 tensors, not {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    # asked several times per launch (a prompt step of a few tokens is bound by the host): the usual case first
    if t is None:
        return None             # a null pointer
    if t.is_cuda and t.is_contiguous():
        return _vp(t.data_ptr())
    if t.is_meta and _dry:
        return None             # a pass over shapes alone: nothing is launched, so nothing is pointed at
    if not t.is_cuda:
        raise ExtensionError("the kernels run on the GPU: a tensor on the CPU was passed, and there is no CPU path")
    raise InvalidArgument("kernels take contiguous tensors")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream of the current device as a raw handle (the short way when torch offers it: this is
    asked once per kernel launch)."""
    if _raw_stream is not None:
        return _vp(_raw_stream(torch._C._cuda_getDevice()))
    return _vp(torch.cuda.current_stream().cuda_stream)


_launches = 0
_dry = False


class shapes_only:
    """Inside, every function of this module checks its arguments and launches nothing: a forward pass over
    shape-only (``meta``) tensors, which the engine runs once to learn how much memory a step needs."""

    def __enter__(self):
        global _dry
        self.before, _dry = _dry, True

    def __exit__(self, *exc):
        global _dry
        _dry = self.before
        return False



def launch_count() -> int:
    """Kernels of this library launched so far in this process, graph replays included."""
    return _launches


def add_launches(n: int) -> None:
    """A CUDA graph that holds ``n`` of this library's kernels was replayed."""
    global _launches
    _launches += n


_last_fn = ""      # the entry point that launched last (a hint for launches that can overlap with their like)


_entry_points = {}     # (library, function) -> (the function, its library): found once


def _call(libname: str, fn: str, *args) -> None:
    global _launches, _last_fn
    found = _entry_points.get((libname, fn))
    if found is None:
        lib = library.load(libname)
        found = _entry_points[libname, fn] = (getattr(lib, fn), lib)
    if _dry:
        return
    _last_fn = ""
    if found[0](*args) != 0:
        raise ExtensionError(found[1].last_error().decode())
    _launches += 1
    _last_fn = fn


def launch_overlap(on: bool) -> None:
    """Whether kernels that can do so are launched to start while the kernel before them ends: a few-token
    product after another one (it asks for its first weights before it waits for that one's results), the
    tensor-core products (their set-up; up to 64 tokens also their first weight tiles), prefill attention (its
    set-up) and the norms between them.
    On by default; off, every kernel waits for the one before it to be over, and the results are the same bits."""
    for name in ("linear_skinny", "gemm_sm100", "generic", "attention_tc"):
        getattr(library.load(name), f"nncpu_launch_overlap_{name}")(ctypes.c_int(1 if on else 0))


_i = int      # a C int: ctypes passes a Python int as one (sizes, counts, flags, type codes; booleans become 0 or 1)


def _f(v) -> ctypes.c_float:
    return ctypes.c_float(float(v))


def embed(table, ids, out, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale; out is float32 [n, hidden]; ids int32."""
    n, hidden = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and ids.numel() >= n
    _call("generic", "nncpu_embed", _ptr(table), _i(_code(table)), _ptr(ids), _ptr(out), _i(n), _i(hidden),
          _i(table.shape[0]), _f(scale), _stream())


def rmsnorm(x, gamma, eps: float, out, rows=None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * gamma over the last axis."""
    dim = x.shape[-1]
    n_rows = out.numel() // dim
    assert gamma is None or gamma.numel() == dim
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= n_rows)
    _call("generic", "nncpu_rmsnorm", _ptr(x), _i(_code(x)), _ptr(gamma), _i(_code(gamma)), _ptr(out),
          _i(_code(out)), _ptr(rows), _i(n_rows), _i(dim), _f(eps), _stream())


def linear_simt(x, w, bias, out, accumulate: bool = False) -> None:
    """out (+)= x . w^T + bias on CUDA cores in 32-bit; any sizes and element types."""
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    _call("generic", "nncpu_linear_simt", _ptr(x), _i(_code(x)), _ptr(w), _i(_code(w)), _ptr(bias),
          _i(_code(bias)), _ptr(out), _i(_code(out)), _i(m), _i(n), _i(k), _i(k), _i(n), _i(accumulate), _stream())


def linear_tc_supported(m: int, n: int, k: int) -> bool:
    return m > 0 and k % 8 == 0


class GemmWorkspace:
    """Device memory the tensor-core kernels need besides their operands:
    scratch for the partial tiles of products that deal their k-blocks out
    evenly, and the status word that a kernel sets when a bounded wait ran
    out.  Launches that share a workspace must not overlap on the GPU (one
    stream)."""

    def __init__(self, device):
        lib = library.load("gemm_sm100")
        lib.nncpu_linear_tc_scratch_floats.restype = ctypes.c_long
        self.scratch = torch.empty(lib.nncpu_linear_tc_scratch_floats(), dtype=torch.float32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)


# Which kernel a tensor-core product runs with, where a measurement or a test wants another than its sizes would get.
PLANS = {"auto": 0, "even_from_17": 1, "never_even": 2, "no_pairs": 4, "narrow_units": 8}

EPILOGUES = {"plain": 0, "swiglu": 1}


@functools.lru_cache(maxsize=4096)
def linear_tc_fuses_norms(m: int, n: int) -> bool:
    """Whether the tensor-core product of ``m`` tokens with ``n`` output features can carry the norms around it
    (``linear_tc``'s ``norm_out`` and ``norm_in``): the products of whole prompts."""
    return bool(library.load("gemm_sm100").nncpu_linear_tc_fuses_norms(m, n))


@functools.lru_cache(maxsize=4096)
def linear_tc_norm_roles(m: int, n: int, k: int) -> int:
    """Which norms the tensor-core product of ``m`` tokens, ``n`` output features and width ``k`` can carry: bit 0 the
    norm before it (``norm_in``), bit 1 the norm after it (``norm_out``).  Whole prompts both; 17 to 64 tokens the
    norm before, and the norm after where a cluster shares every output tile."""
    return int(library.load("gemm_sm100").nncpu_linear_tc_norm_roles(m, n, k))


def linear_tc(x, w, bias, out, workspace: GemmWorkspace, accumulate: bool = False, epilogue: str = "plain",
              plan: str = "auto", norm_out=None, norm_in=None) -> None:
    """out (+)= x . w^T + bias on the tensor cores; x and w bfloat16.  With
    ``epilogue="swiglu"`` the rows of w hold gate and up rows interleaved in
    blocks of 8 and out [m, n/2] receives silu(gate) * up.  ``plan``: "auto",
    or for measurements and tests "even_from_17" (17 to 64 tokens deal their
    k-blocks out evenly like 65 to 256), "never_even", "no_pairs".

    Where ``linear_tc_norm_roles(m, n, k)`` says so, the product can carry the RMS norms around it as
    ``linear_skinny`` does: ``norm_out = (xg, gamma, bins, bins_clear)`` and ``norm_in = (bins, eps)`` with accumulators of
    ``NORM_ROW_WORDS`` 64-bit words per row (int64 [m, NORM_ROW_WORDS])."""
    m, k = x.shape
    n = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert w.shape[1] == k and out.shape == (m, n // 2 if epilogue == "swiglu" else n)
    xg = gamma = bins_out = bins_clear = bins_in = None
    eps = 0.0
    if norm_out is not None:
        xg, gamma, bins_out, bins_clear = norm_out
        assert xg.dtype == torch.bfloat16 and xg.shape == (m, n) and xg.is_contiguous() and gamma.numel() == n
        assert bins_out.dtype == torch.int64 and bins_out.shape == (m, NORM_ROW_WORDS) and bins_out.is_contiguous()
        assert bins_clear is None or (bins_clear.dtype == torch.int64 and bins_clear.shape == (m, NORM_ROW_WORDS))
    if norm_in is not None:
        bins_in, eps = norm_in
        assert bins_in.dtype == torch.int64 and bins_in.shape == (m, NORM_ROW_WORDS) and bins_in.is_contiguous()
    _call("gemm_sm100", "nncpu_linear_tc", _ptr(x), _ptr(w), _ptr(bias), _i(_code(bias)), _ptr(out),
          _i(_code(out)), _i(m), _i(n), _i(k), _i(x.stride(0)), _i(out.shape[1]), _i(accumulate), _i(EPILOGUES[epilogue]),
          _i(PLANS[plan]), _ptr(xg), _ptr(gamma), _i(_code(gamma)), _ptr(bins_out), _ptr(bins_clear), _ptr(bins_in),
          _f(eps), _ptr(workspace.scratch), _ptr(workspace.status), _stream())


def linear_tc_wait_probe(x, w, out, workspace: GemmWorkspace, limit_ms: int = 5) -> None:
    """The library's check of its own failure path: one tile of x [128, K] . w [256, K]^T whose copies are
    expected to bring more bytes than they do, with every wait limited to ``limit_ms``.  The kernel gives up in
    order, frees what it holds and sets the workspace's status word; ``out`` is not written."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.float32
    assert x.shape[0] == 128 and w.shape[0] == 256 and x.shape[1] == w.shape[1] and out.shape == (128, 256)
    _call("gemm_sm100", "nncpu_linear_tc_wait_probe", _ptr(x), _ptr(w), _ptr(out), _i(x.shape[1]), _i(limit_ms),
          _ptr(workspace.status), _stream())


def linear_tc_qkv_supported(x, n_heads: int, n_kv: int, head_dim: int) -> bool:
    """Whether the q/k/v projection of these tokens can run with its epilogue fused."""
    lib = library.load("gemm_sm100")
    return x.dtype == torch.bfloat16 and bool(
        lib.nncpu_linear_tc_qkv_supported(x.shape[0], x.shape[1], x.stride(0), n_heads, n_kv, head_dim))


def linear_tc_qkv(x, w_qkv, q_gamma, k_gamma, eps, cos_sin, tok_seq, tok_pos, block_table, k_pages, v_pages, q_out,
                  workspace: GemmWorkspace, n_heads: int, n_kv: int, head_dim: int, norm_in=None) -> None:
    """x . w_qkv^T with the per-head norm, the rotation and the stores fused into the product's epilogue:
    queries to ``q_out``, keys and values to the tokens' rows of the cache pages.  bfloat16 throughout,
    32-bit accumulators, norm and rotation.  ``cos_sin`` is the rotation table laid out by pair:
    float32 [head_dim / 2, tokens, 2].  ``norm_in = (bins, eps)``: ``x`` holds the rows of the norm before the
    projection times gamma, and the rows' scales are applied to the accumulators (as in ``linear_tc``)."""
    m, k = x.shape
    bins_in, norm_eps = norm_in if norm_in is not None else (None, 0.0)
    assert bins_in is None or (bins_in.dtype == torch.int64 and bins_in.shape == (m, NORM_ROW_WORDS))
    assert w_qkv.shape == ((n_heads + 2 * n_kv) * head_dim, k) and q_out.shape == (m, n_heads * head_dim)
    assert x.dtype == w_qkv.dtype == q_out.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16
    assert q_out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert k_pages.shape[1:] == (n_kv, 64, head_dim) and v_pages.shape == k_pages.shape
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (head_dim // 2, m, 2))
    assert q_gamma is None or k_gamma is None or q_gamma.dtype == k_gamma.dtype
    g = q_gamma if q_gamma is not None else k_gamma
    _call("gemm_sm100", "nncpu_linear_tc_qkv", _ptr(x), _ptr(w_qkv), _i(m), _i(k), _i(x.stride(0)), _ptr(q_out),
          _ptr(k_pages), _ptr(v_pages), _ptr(q_gamma), _ptr(k_gamma), _i(_code(g)), _f(eps), _ptr(cos_sin),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(block_table), _i(block_table.shape[1]), _i(n_heads), _i(n_kv),
          _i(head_dim), _ptr(bins_in), _f(norm_eps), _ptr(workspace.status), _stream())


SKINNY_MAX_TOKENS = 16
CLUSTER_MAX_TOKENS = 64    # up to here a tensor-core product's weights are the 128-row operand of one tile row


def linear_skinny(x, w, bias, out, accumulate: bool = False, epilogue: str = "plain", norm_out=None,
                  norm_in=None) -> None:
    """The same product for at most 16 tokens: a stream over the weights that
    uses every SM, with no scratch memory.

    The product can carry the RMS norms around it.  ``norm_out = (xg, gamma, bins, bins_clear)``: besides ``out``
    it leaves ``xg`` (bfloat16 [m, n]) = out * gamma and adds the sums of squares of out's rows into ``bins`` (int64
    [NORM_WORDS], zero before the call: exact accumulators that do not depend on the order of additions);
    ``bins_clear`` (or None) is another such block, which is set to zero.  ``norm_in = (bins, eps)``: ``x`` holds
    such rows times gamma, and the result is multiplied by 1 / sqrt(sum / k + eps) per row before bias and
    activation."""
    m, k = x.shape
    n = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert w.shape[1] == k and out.shape == (m, n // 2 if epilogue == "swiglu" else n)
    xg = gamma = bins_out = bins_clear = bins_in = None
    eps = 0.0
    if norm_out is not None:
        xg, gamma, bins_out, bins_clear = norm_out
        assert xg.dtype == torch.bfloat16 and xg.shape == (m, n) and gamma.numel() == n
        assert bins_out.dtype == torch.int64 and bins_out.numel() == NORM_WORDS
        assert bins_clear is None or (bins_clear.dtype == torch.int64 and bins_clear.numel() == NORM_WORDS)
    if norm_in is not None:
        assert norm_out is None, "a product is a norm's producer or its consumer"
        bins_in, eps = norm_in
        assert bins_in.dtype == torch.int64 and bins_in.numel() == NORM_WORDS
    # a product that follows another one may start while that one ends (see launch_overlap)
    after_skinny = _last_fn == "nncpu_linear_skinny"
    _call("linear_skinny", "nncpu_linear_skinny", _ptr(x), _ptr(w), _ptr(bias), _i(_code(bias)), _ptr(out),
          _i(_code(out)), _i(m), _i(n), _i(k), _i(k), _i(out.shape[1]), _i(accumulate), _i(EPILOGUES[epilogue]),
          _ptr(xg), _ptr(gamma), _i(_code(gamma)), _ptr(bins_out), _ptr(bins_clear), _ptr(bins_in), _f(eps),
          _i(after_skinny), _stream())


def linear_skinny_force_warps(warps: int) -> None:
    """For measurements and tests: the few-token product runs as blocks of 8 or of 4 warps whatever the sizes;
    0: chosen by the sizes (4 warps where 16-row blocks number more than two per SM and at most four)."""
    library.load("linear_skinny").nncpu_linear_skinny_force_warps(ctypes.c_int(int(warps)))


NORM_ROW_WORDS = 16  # 64-bit words of one row's accumulator: 8 bins, a word that says "not finite", spare
NORM_WORDS = 256    # the accumulators of one norm of a few-token step: 16 rows


def rope_table(positions, inv_freq, out, position_scale: float = 1.0, by_pair: bool = False) -> None:
    """out[t, i] = (cos, sin)(positions[t] * position_scale * inv_freq[i]); out float32 [n, half, 2], or with
    ``by_pair`` [half, n, 2] holding the same values as out[i, t]."""
    if by_pair:
        half, n, two = out.shape
    else:
        n, half, two = out.shape
    assert two == 2 and out.dtype == torch.float32 and inv_freq.dtype == torch.float32
    assert inv_freq.numel() == half and positions.dtype == torch.int32 and positions.numel() >= n
    _call("generic", "nncpu_rope_table", _ptr(positions), _ptr(inv_freq), _ptr(out), _i(n), _i(half),
          _f(position_scale), _i(by_pair), _stream())


def qk_norm_rope_append(qkv, q_gamma, k_gamma, eps, cos_sin, tok_seq, tok_pos, block_table, k_pages, v_pages,
                        q_out, n_heads: int, n_kv: int, head_dim: int) -> None:
    """Per-head norm and rotation of q and k, and the append of k and v to
    their pages.  ``n_kv`` 0: qkv holds q only and nothing is appended."""
    n = q_out.shape[0]
    rot_half = 0 if cos_sin is None else cos_sin.shape[1]
    assert qkv.shape == (n, (n_heads + 2 * n_kv) * head_dim) and q_out.shape == (n, n_heads * head_dim)
    assert q_gamma is None or k_gamma is None or q_gamma.dtype == k_gamma.dtype
    g = q_gamma if q_gamma is not None else k_gamma
    bt_stride = block_table.shape[1] if block_table is not None else 0
    _call("generic", "nncpu_qk_norm_rope_append", _ptr(qkv), _i(_code(qkv)), _ptr(q_gamma), _ptr(k_gamma),
          _i(_code(g)), _f(eps), _ptr(cos_sin), _i(rot_half), _ptr(tok_seq), _ptr(tok_pos), _ptr(block_table),
          _i(bt_stride), _ptr(k_pages), _ptr(v_pages), _i(_code(k_pages)), _ptr(q_out), _i(_code(q_out)), _i(n),
          _i(n_heads), _i(n_kv), _i(head_dim), _stream())


def attention(q, k_pages, v_pages, block_table, tok_seq, tok_pos, out, n_heads: int, n_kv: int, head_dim: int,
              scale: float, window: int = 0) -> None:
    """Causal attention of each token over its sequence's pages."""
    n = q.shape[0]
    assert q.shape == (n, n_heads * head_dim) and out.shape == q.shape
    assert k_pages.dtype == v_pages.dtype and block_table.dtype == torch.int32
    _call("generic", "nncpu_attention", _ptr(q), _i(_code(q)), _ptr(k_pages), _ptr(v_pages), _i(_code(k_pages)),
          _ptr(block_table), _i(block_table.shape[1]), _ptr(tok_seq), _ptr(tok_pos), _ptr(out), _i(_code(out)),
          _i(n), _i(n_heads), _i(n_kv), _i(head_dim), _f(scale), _i(window), _stream())


def attention_mma_supported(n_heads: int, n_kv: int, head_dim: int, *tensors) -> bool:
    """The tensor-core attention kernels take bfloat16 q, cache and output with
    head size 64 or 128 and at most 16 query heads per key/value head."""
    return (head_dim in (64, 128) and n_kv > 0 and n_heads % n_kv == 0 and n_heads // n_kv <= 16
            and all(t.dtype == torch.bfloat16 for t in tensors))


# How decode attention cuts a sequence's keys into splits: the kernel's launch bounds let two of its blocks run on
# an SM at once, and a split shorter than this many keys costs more in merging than it gains.
DECODE_BLOCKS_PER_SM = 2
DECODE_MIN_KEYS_PER_SPLIT = 256
DECODE_CLUSTER_MAX_SPLITS = 8      # up to here the splits merge inside a thread-block cluster, without scratch


def attention_decode_splits(n_tokens: int, n_kv: int, longest: int, sm_count: int) -> int:
    """As many splits as keep every block of the grid running at once (never a second wave), each with at
    least ``DECODE_MIN_KEYS_PER_SPLIT`` keys of the longest sequence.  Up to twice what a cluster merges is cut
    back to what it merges: one launch instead of two costs less than the finer cut gains (one sequence of 3 072
    keys: 8 splits in a cluster 9.1 us, 12 through scratch and a merge kernel 9.3 us before the kernel boundary)."""
    pairs = max(1, n_tokens * n_kv)
    n = max(1, min(DECODE_BLOCKS_PER_SM * sm_count // pairs, longest // DECODE_MIN_KEYS_PER_SPLIT))
    return DECODE_CLUSTER_MAX_SPLITS if DECODE_CLUSTER_MAX_SPLITS < n <= 2 * DECODE_CLUSTER_MAX_SPLITS else n


def attention_decode_scratch_floats(n_tok: int, n_heads: int, n_kv: int, head_dim: int, n_splits: int) -> int:
    return 0 if n_splits <= 1 else n_tok * n_kv * n_splits * (n_heads // n_kv) * (head_dim + 2)


def attention_decode_mma(q, k_pages, v_pages, block_table, tok_seq, tok_pos, out, scratch, n_heads: int, n_kv: int,
                         head_dim: int, scale: float, window: int, n_splits: int) -> None:
    """One token per sequence; each token's keys are cut into ``n_splits``
    splits that run in parallel.  With ``scratch`` (float32,
    ``attention_decode_scratch_floats`` elements) a second kernel merges them;
    with ``scratch`` None and at most 8 splits they form a thread-block
    cluster and merge through distributed shared memory."""
    n = q.shape[0]
    assert q.shape == (n, n_heads * head_dim) and out.shape == q.shape
    assert scratch is None or scratch.dtype == torch.float32
    _call("attention_mma", "nncpu_attention_decode_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
          _i(block_table.shape[1]), _ptr(tok_seq), _ptr(tok_pos), _ptr(out), _ptr(scratch),
          ctypes.c_long(0 if scratch is None else scratch.numel()), _i(n), _i(n_heads), _i(n_kv), _i(head_dim),
          _f(scale), _i(window), _i(n_splits), _stream())


def attention_decode_mma_from_qkv(qkv, q_gamma, k_gamma, eps, cos_sin, k_pages, v_pages, append: bool, block_table,
                                  tok_seq, tok_pos, out, scratch, n_heads: int, n_kv: int, head_dim: int, scale: float,
                                  window: int, n_splits: int) -> None:
    """Decode attention that starts from the float32 projections ``qkv`` [n, per_tok * head_dim] (q heads, then with
    ``append`` the k and v heads): every block makes its queries itself (per-head norm, rotation by ``cos_sin``
    [n, head_dim / 2, 2]), and with ``append`` the token's key and value are made, written to the cache and used.
    One launch in place of ``qk_norm_rope_append`` and ``attention_decode_mma``, with the same arithmetic."""
    n = out.shape[0]
    per_tok = n_heads + 2 * n_kv if append else n_heads
    assert qkv.dtype == torch.float32 and qkv.shape == (n, per_tok * head_dim) and qkv.is_contiguous()
    assert out.shape == (n, n_heads * head_dim) and out.dtype == torch.bfloat16
    assert k_pages.dtype == v_pages.dtype == torch.bfloat16 and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (n, head_dim // 2, 2))
    assert q_gamma is None or k_gamma is None or q_gamma.dtype == k_gamma.dtype
    assert scratch is None or scratch.dtype == torch.float32
    g = q_gamma if q_gamma is not None else k_gamma
    _call("attention_mma", "nncpu_attention_decode_mma_from_qkv", _ptr(qkv), _ptr(q_gamma), _ptr(k_gamma), _i(_code(g)),
          _f(eps), _ptr(cos_sin), _ptr(k_pages), _ptr(v_pages), _i(append), _ptr(block_table), _i(block_table.shape[1]),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(out), _ptr(scratch), ctypes.c_long(0 if scratch is None else scratch.numel()),
          _i(n), _i(n_heads), _i(n_kv), _i(head_dim), _f(scale), _i(window), _i(n_splits), _stream())


def attention_prefill_mma(q, k_pages, v_pages, block_table, cu_seqlens, tok_pos, out, n_seqs: int, n_heads: int,
                          n_kv: int, head_dim: int, scale: float, window: int) -> None:
    """Any number of new tokens per sequence, at consecutive positions."""
    n = q.shape[0]
    assert q.shape == (n, n_heads * head_dim) and out.shape == q.shape and cu_seqlens.numel() >= n_seqs + 1
    _call("attention_mma", "nncpu_attention_prefill_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
          _i(block_table.shape[1]), _ptr(cu_seqlens), _ptr(tok_pos), _ptr(out), _i(n), _i(n_seqs), _i(n_heads),
          _i(n_kv), _i(head_dim), _f(scale), _i(window), _stream())


def attention_prefill_tc_supported(n_heads: int, n_kv: int, head_dim: int, *tensors) -> bool:
    """Whether the tcgen05 prefill kernel takes these sizes (and these tensors: all bfloat16)."""
    lib = library.load("attention_tc")
    return bool(lib.nncpu_attention_prefill_tc_supported(n_heads, n_kv, head_dim)) and \
        all(t.dtype == torch.bfloat16 for t in tensors)


def attention_prefill_tc(q, k_pages, v_pages, block_table, cu_seqlens, tok_pos, out, status, n_seqs: int,
                         n_heads: int, n_kv: int, head_dim: int, scale: float, window: int) -> None:
    """Prefill attention on the tcgen05 tensor cores: any number of new tokens per sequence, at consecutive
    positions; ``status`` is an int32 word on the device that receives a code if a bounded wait runs out."""
    n = q.shape[0]
    assert q.shape == (n, n_heads * head_dim) and out.shape == q.shape and cu_seqlens.numel() >= n_seqs + 1
    assert q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert k_pages.shape[1:] == (n_kv, 64, head_dim) and v_pages.shape == k_pages.shape
    assert status.dtype == torch.int32
    _call("attention_tc", "nncpu_attention_prefill_tc", _ptr(q), _ptr(k_pages), _ptr(v_pages), _i(k_pages.shape[0]),
          _ptr(block_table), _i(block_table.shape[1]), _ptr(cu_seqlens), _ptr(tok_pos), _ptr(out), _i(n), _i(n_seqs),
          _i(n_heads), _i(n_kv), _i(head_dim), _f(scale), _i(window), _ptr(status), _stream())


def swiglu(gate_up, out) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    n, inter = out.shape
    assert gate_up.shape == (n, 2 * inter)
    _call("generic", "nncpu_swiglu", _ptr(gate_up), _i(_code(gate_up)), _ptr(out), _i(_code(out)), _i(n),
          _i(inter), _stream())


def gather_rows(x, rows, out) -> None:
    n, dim = out.shape
    assert x.dtype == torch.float32 and out.dtype == torch.float32 and rows.dtype == torch.int32
    _call("generic", "nncpu_gather_rows", _ptr(x), _ptr(rows), _ptr(out), _i(n), _i(dim), _stream())


def argmax(logits, out) -> None:
    """out[r] = the first largest of logits[r]; logits float32 [n, vocab], out int32 [n]."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() >= n
    lib = library.load("generic")
    lib.nncpu_argmax_scratch_bytes.restype = ctypes.c_long
    need = lib.nncpu_argmax_scratch_bytes(_i(n), _i(vocab))      # long rows are searched in chunks
    scratch = torch.empty(need, dtype=torch.uint8, device=logits.device) if need else None
    _call("generic", "nncpu_argmax", _ptr(logits), _ptr(out), _i(n), _i(vocab), _ptr(scratch), ctypes.c_long(need),
          _stream())


def topk(logits, vals, ids) -> None:
    """The k = vals.shape[1] best entries of every row by (logit descending, id
    ascending), NaN as -inf, in no particular order: vals float32 [n, k], ids int32 [n, k]."""
    n, vocab = logits.shape
    k = vals.shape[1]
    assert logits.dtype == torch.float32 and vals.dtype == torch.float32 and ids.dtype == torch.int32
    assert vals.shape == (n, k) and ids.shape == (n, k)
    _call("generic", "nncpu_topk", _ptr(logits), _ptr(vals), _ptr(ids), _i(n), _i(vocab), _i(k), _stream())


def sample_chain(logits, u, out, top_k: int, temperature: float, top_p: float, min_p: float) -> None:
    """The whole chain on the device for 0 < top_k <= 1024: out[r] = the token drawn from row r with the
    uniform u[r] (float64 in [0, 1)) after top-k, top-p, min-p and temperature, in rank order."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and u.dtype == torch.float64 and out.dtype == torch.int32
    assert u.numel() >= n and out.numel() >= n
    lib = library.load("generic")
    lib.nncpu_sample_chain_scratch_bytes.restype = ctypes.c_long
    need = lib.nncpu_sample_chain_scratch_bytes(_i(n), _i(vocab))   # long rows: candidates found by the whole GPU
    scratch = torch.empty(need, dtype=torch.uint8, device=logits.device) if need else None
    _call("generic", "nncpu_sample_chain", _ptr(logits), _ptr(u), _ptr(out), _i(n), _i(vocab), _i(top_k),
          _f(temperature), _f(top_p), _f(min_p), _ptr(scratch), ctypes.c_long(need), _stream())


def row_exp_sum(logits, out) -> None:
    """out[r] (float64) = sum over the row of exp(logit - the row's largest logit), NaN as -inf."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.float64 and out.shape == (n,)
    _call("generic", "nncpu_row_exp_sum", _ptr(logits), _ptr(out), _i(n), _i(vocab), _stream())


def sample_temperature(logits, uniforms, out, temperature: float) -> None:
    """One draw per row at ``temperature`` over the whole vocabulary in id
    order; uniforms float64 [n] in [0, 1)."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and uniforms.dtype == torch.float64 and out.dtype == torch.int32
    lib = library.load("generic")
    lib.nncpu_sample_temperature_scratch_bytes.restype = ctypes.c_long
    need = lib.nncpu_sample_temperature_scratch_bytes(_i(n), _i(vocab))   # long rows are summed in chunks
    scratch = torch.empty(need, dtype=torch.uint8, device=logits.device) if need else None
    _call("generic", "nncpu_sample_temperature", _ptr(logits), _ptr(uniforms), _ptr(out), _i(n), _i(vocab),
          _f(temperature), _ptr(scratch), ctypes.c_long(need), _stream())
