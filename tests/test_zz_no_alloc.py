"""The decode-attention entry point that allocates nothing, called through its
exported C symbol the way a foreign caller would, against the regular entry
point that takes scratch from its caller.

Such a caller (a process whose GPU memory is all spoken for, a binding that
only holds raw pointers, a loop that must not enter the driver's allocator)
passes inputs and output and nothing else; the scratch is the library's own
fixed device array.  Two calls in a row with different sizes show that what one
call leaves in that array does not disturb the next.  This file sorts last, so
a run that stops at the first failure has already run every other test; it
passes alone in a fresh process too, where its first call is the one that looks
the array's address up.
"""
import ctypes
import math

import pytest
import torch

from gpu_util import DEV, check, scatter_pages

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def call_static(lib, q, kp, vp, table, tok_seq, tok_pos, out, nh, nkv, hd, window, n_splits):
    fn = lib.nncpu_attention_decode_mma_static
    fn.restype = ctypes.c_int
    return fn(_ptr(q), _ptr(kp), _ptr(vp), _ptr(table), ctypes.c_int(table.shape[1]), _ptr(tok_seq), _ptr(tok_pos),
              _ptr(out), ctypes.c_int(q.shape[0]), ctypes.c_int(nh), ctypes.c_int(nkv), ctypes.c_int(hd),
              ctypes.c_float(1.0 / math.sqrt(hd)), ctypes.c_int(window), ctypes.c_int(n_splits),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_entry_point_without_allocation_matches_the_regular_one_twice_in_a_row():
    from nncpu_b200.kernels import library, ops
    lib = library.load("attention_mma")
    lib.nncpu_attention_decode_mma_static_max_floats.restype = ctypes.c_long
    assert lib.nncpu_attention_decode_mma_static_max_floats() == 1 << 20
    cases = [  # (heads, kv heads, head size, window, splits, sequence lengths)
        (8, 2, 128, 0, 6, [700, 33, 64, 1]),
        (4, 4, 64, 50, 3, [129, 300]),
    ]
    for nh, nkv, hd, window, n_splits, seqs in cases:
        kp, vp, table, _, _ = scatter_pages(24, nkv, hd, seqs, torch.bfloat16, seed=nh)
        n = len(seqs)
        tok_seq = torch.arange(n, dtype=torch.int32, device=DEV)
        tok_pos = torch.tensor([s - 1 for s in seqs], dtype=torch.int32, device=DEV)
        q = torch.randn(n, nh * hd, generator=torch.Generator().manual_seed(hd)).bfloat16().to(DEV)
        floats = ops.attention_decode_scratch_floats(n, nh, nkv, hd, n_splits)
        want = torch.empty_like(q)
        ops.attention_decode_mma(q, kp, vp, table, tok_seq, tok_pos, want, torch.empty(floats, device=DEV), nh, nkv, hd,
                                 1.0 / math.sqrt(hd), window, n_splits)
        got = torch.full_like(q, 9.0)
        before = torch.cuda.memory_allocated()
        rc = call_static(lib, q, kp, vp, table, tok_seq, tok_pos, got, nh, nkv, hd, window, n_splits)
        assert rc == 0, lib.last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        check(got, want, 1.5e-2, f"static scratch, {nh} heads of {hd}")
        assert torch.equal(got, want)      # the same kernel on the same inputs


def test_stale_scratch_padding_rows_one_split_and_many_splits():
    """What the built-in array holds from an earlier call never shows: a large call first, then a batch with a
    padding row (zeros expected), a call with a single split (which needs no scratch at all) and one with more
    splits than a cluster merges; each against the plain 32-bit attention kernel, not only its sibling entry."""
    from nncpu_b200.kernels import library, ops
    lib = library.load("attention_mma")
    nh, nkv, hd = 8, 2, 128
    seqs = [900, 700, 1100, 64]
    kp, vp, table, _, _ = scatter_pages(64, nkv, hd, seqs, torch.bfloat16, seed=5)
    n = len(seqs)
    q = torch.randn(n, nh * hd, generator=torch.Generator().manual_seed(1)).bfloat16().to(DEV)
    pos = torch.tensor([s - 1 for s in seqs], dtype=torch.int32, device=DEV)
    for tok_seq, n_splits in (([0, 1, 2, 3], 16), ([0, -1, 2, 3], 3), ([0, 1, -1, 3], 1), ([0, 1, 2, 3], 12)):
        seq = torch.tensor(tok_seq, dtype=torch.int32, device=DEV)
        got = torch.full_like(q, 9.0)
        rc = call_static(lib, q, kp, vp, table, seq, pos, got, nh, nkv, hd, 0, n_splits)
        assert rc == 0, lib.last_error().decode()
        want = torch.zeros(n, nh * hd, device=DEV)
        live = [i for i, s in enumerate(tok_seq) if s >= 0]
        idx = torch.tensor(live, device=DEV)
        part = torch.empty(len(live), nh * hd, device=DEV)
        ops.attention(q[idx].float().contiguous(), kp.float(), vp.float(), table, seq[idx].contiguous(),
                      pos[idx].contiguous(), part, nh, nkv, hd, 1.0 / math.sqrt(hd), 0)
        want[idx] = part
        check(got, want, 1.5e-2, f"{n_splits} splits, rows {tok_seq}")
        for i, s in enumerate(tok_seq):
            if s < 0:
                assert float(got[i].float().abs().max()) == 0.0     # a padding row is zeros whatever the array held


def test_entry_point_without_allocation_refuses_what_does_not_fit():
    from nncpu_b200.kernels import library
    lib = library.load("attention_mma")
    kp, vp, table, _, _ = scatter_pages(2, 8, 128, [10], torch.bfloat16)
    n = 64
    z = torch.zeros(n, dtype=torch.int32, device=DEV)
    q = torch.zeros(n, 32 * 128, dtype=torch.bfloat16, device=DEV)
    out = torch.full_like(q, 3.0)
    # 64 tokens x 8 key/value heads x 16 splits x 4 heads x 130 floats = 4.26 M floats > 1 Mi floats
    rc = call_static(lib, q, kp, vp, table.expand(n, -1).contiguous(), z, z, out, 32, 8, 128, 0, 16)
    assert rc != 0
    msg = lib.last_error().decode()
    assert "built-in buffer holds 1048576" in msg and "4259840" in msg
    torch.cuda.synchronize()
    assert float(out.float().min()) == 3.0      # nothing was launched
    rc = call_static(lib, q[:1], kp, vp, table, z[:1], z[:1], out[:1], 32, 8, 96, 0, 2)
    assert rc != 0 and "head size 64 or 128" in lib.last_error().decode()
