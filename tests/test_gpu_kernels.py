"""Each CUDA kernel alone against a plain float32/float64 reference of the same
operation, at sizes other than the models' (odd widths, tails, many pages)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from gpu_util import DEV, check, rel_err, scatter_pages
from nncpu_b200.cache import PAGE
from nncpu_b200.errors import ExtensionError

pytestmark = pytest.mark.gpu
DT = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from nncpu_b200.kernels import ops
    return ops


def test_embed(ops):
    table = torch.randn(37, 50, device=DEV)
    ids = torch.tensor([3, 36, -1, 0, 3], dtype=torch.int32, device=DEV)
    for t in (table, table.bfloat16()):
        out = torch.empty(5, 50, device=DEV)
        ops.embed(t, ids, out, 2.0)
        want = t.float()[ids.clamp_min(0).long()] * 2.0
        want[2] = 0
        assert torch.equal(out, want)


@pytest.mark.parametrize("dim", [1, 7, 80, 129, 1024, 1028, 4096, 5120, 8192])
@pytest.mark.parametrize("dt", DT)
def test_rmsnorm(ops, dim, dt):
    g = torch.Generator().manual_seed(dim)
    x = (torch.randn(9, dim, generator=g) * 3).to(DEV)
    gamma = (1 + 0.1 * torch.randn(dim, generator=g)).to(dt).to(DEV)
    want = P.rmsnorm(x.cpu().numpy(), gamma.float().cpu().numpy(), 1e-5)
    out = torch.empty(9, dim, dtype=dt, device=DEV)
    ops.rmsnorm(x, gamma, 1e-5, out)
    check(out, want, 1e-5 if dt == torch.float32 else 8e-3, "rmsnorm")
    rows = torch.tensor([8, -1, 0, 8], dtype=torch.int32, device=DEV)
    out = torch.empty(4, dim, dtype=torch.float32, device=DEV)
    ops.rmsnorm(x, gamma, 1e-5, out, rows)
    w = np.stack([want[8], np.zeros(dim, np.float32), want[0], want[8]])
    check(out, w, 1e-5, "rmsnorm of gathered rows")


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 307, 81), (17, 64, 409), (70, 130, 33), (300, 31, 200)])
def test_linear_simt(ops, m, n, k):
    g = torch.Generator().manual_seed(m * n + k)
    x, w, b = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g) * 0.1, torch.randn(n, generator=g)
    want = (x.double() @ w.double().T + b.double()).float()
    out = torch.empty(m, n, device=DEV)
    ops.linear_simt(x.to(DEV), w.to(DEV), b.to(DEV), out)
    check(out, want, 2e-6, "linear")
    acc = torch.ones(m, n, device=DEV)
    ops.linear_simt(x.to(DEV), w.to(DEV), None, acc, accumulate=True)
    check(acc, want - b + 1, 2e-6, "linear accumulate")
    # mixed element types: bfloat16 activations, float32 weights, bfloat16 out
    xb = x.bfloat16()
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.linear_simt(xb.to(DEV), w.to(DEV), b.bfloat16().to(DEV), out)
    check(out, xb.float() @ w.T + b.bfloat16().float(), 1e-2, "linear mixed")


def test_linear_simt_row_does_not_depend_on_the_batch(ops):
    x, w = torch.randn(70, 200, device=DEV), torch.randn(90, 200, device=DEV)
    whole = torch.empty(70, 90, device=DEV)
    ops.linear_simt(x, w, None, whole)
    for rows in (slice(0, 1), slice(13, 14), slice(20, 37)):
        part = torch.empty(rows.stop - rows.start, 90, device=DEV)
        ops.linear_simt(x[rows].contiguous(), w, None, part)
        assert torch.equal(part, whole[rows])


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (3, 307, 80), (16, 1000, 512), (17, 130, 72), (64, 2048, 1024),
                                   (65, 100, 200), (128, 128, 128), (129, 384, 96), (256, 300, 264),
                                   (257, 512, 128), (700, 307, 80), (1000, 1111, 1096), (512, 512, 64),
                                   (513, 777, 4096), (2048, 6144, 512), (900, 520, 72)])
def test_linear_tensor_core(ops, m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.1).bfloat16().to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    status = ops.GemmWorkspace(DEV)
    want = (x.double() @ w.double().T).float()
    out = torch.full((m, n), 9.0, device=DEV)
    ops.linear_tc(x, w, b, out, status)
    check(out, want + b, 1e-5, "tensor-core linear, float32 out")
    outb = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(x, w, b.bfloat16(), outb, status)
    check(outb, want + b.bfloat16().float(), 8e-3, "tensor-core linear, bfloat16 out")
    acc = torch.full((m, n), 0.5, device=DEV)
    ops.linear_tc(x, w, None, acc, status, accumulate=True)
    check(acc, want + 0.5, 1e-5, "tensor-core linear, accumulate")
    accb = torch.full((m, n), 0.5, dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(x, w, None, accb, status, accumulate=True)
    check(accb, want + 0.5, 8e-3, "tensor-core linear, accumulate in bfloat16")
    assert int(status.status.item()) == 0


@pytest.mark.parametrize("m,inter,k", [(1, 8, 64), (7, 136, 80), (64, 12288, 512), (100, 1000, 264), (300, 320, 128),
                                       (1000, 2048, 1024)])
def test_linear_tensor_core_with_gated_epilogue(ops, m, inter, k):
    g = torch.Generator().manual_seed(m + inter)
    x = torch.randn(m, k, generator=g).bfloat16()
    gate = (torch.randn(inter, k, generator=g) * 0.1).bfloat16()
    up = (torch.randn(inter, k, generator=g) * 0.1).bfloat16()
    w = torch.stack([gate.view(-1, 8, k), up.view(-1, 8, k)], dim=1).reshape(-1, k).contiguous()
    want = P.swiglu((x.double() @ gate.double().T).float().numpy(), (x.double() @ up.double().T).float().numpy())
    ws = ops.GemmWorkspace(DEV)
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 8e-3)):
        out = torch.full((m, inter), 9.0, dtype=dt, device=DEV)
        ops.linear_tc(x.to(DEV), w.to(DEV), None, out, ws, epilogue="swiglu")
        check(out, want, tol, "gated epilogue")
    assert int(ws.status.item()) == 0


@pytest.mark.parametrize("plan", ["even_from_17", "narrow_units"])
@pytest.mark.parametrize("m,n,k", [(20, 1000, 1096), (40, 25600, 512), (70, 640, 4096), (100, 25000, 264),
                                   (130, 4096, 1024), (256, 19000, 520), (200, 128, 8192), (128, 300, 2048),
                                   (65, 12288, 4096), (100, 25600, 264), (200, 19008, 520)])
def test_linear_tensor_core_with_work_cut_evenly(ops, m, n, k, plan):
    """17 to 256 tokens with the k-blocks of all tiles dealt out evenly to the blocks: fewer tiles than SMs
    (every tile in parts), more tiles than SMs (whole tiles and parts), one tile, every epilogue; twice, and
    the runs agree bit for bit.  From 65 tokens on a unit holds 256 weight rows (two tiles that share the tokens'
    k-block; the last may be short of rows or lack its second tile), with "narrow_units" 128 as below that."""
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.1).bfloat16().to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    ws = ops.GemmWorkspace(DEV)
    want = (x.double() @ w.double().T).float()
    out = torch.full((m, n), 9.0, device=DEV)
    ops.linear_tc(x, w, b, out, ws, plan=plan)
    check(out, want + b, 1e-5, "float32 out with bias")
    again = torch.full((m, n), 9.0, device=DEV)
    ops.linear_tc(x, w, b, again, ws, plan=plan)
    assert torch.equal(out, again)
    acc = torch.full((m, n), 0.5, dtype=torch.bfloat16, device=DEV)
    ops.linear_tc(x, w, None, acc, ws, accumulate=True, plan=plan)
    check(acc, want + 0.5, 8e-3, "accumulate in bfloat16")
    if n % 16 == 0:
        gated = torch.full((m, n // 2), 9.0, device=DEV)
        ops.linear_tc(x, w, None, gated, ws, epilogue="swiglu", plan=plan)
        y = want.cpu().numpy().reshape(m, -1, 2, 8)
        check(gated, P.swiglu(y[:, :, 0].reshape(m, -1), y[:, :, 1].reshape(m, -1)), 1e-5, "gated epilogue")
    assert int(ws.status.item()) == 0


def test_linear_tensor_core_is_repeatable_and_row_independent(ops):
    # K is cut into slices for few tokens: the slices are added in slice order, so runs agree bit for bit
    x = torch.randn(8, 4096).bfloat16().to(DEV)
    w = (torch.randn(512, 4096) * 0.05).bfloat16().to(DEV)
    ws = ops.GemmWorkspace(DEV)
    outs = []
    for _ in range(5):
        out = torch.empty(8, 512, device=DEV)
        ops.linear_tc(x, w, None, out, ws)
        outs.append(out)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    one = torch.empty(1, 512, device=DEV)
    ops.linear_tc(x[3:4].contiguous(), w, None, one, ws)
    assert torch.equal(one[0], outs[0][3])


@pytest.mark.parametrize("m,n,k", [(1, 16, 32), (1, 307, 80), (3, 6144, 4096), (8, 100, 264), (9, 64, 4096),
                                   (16, 1000, 1096), (5, 24, 8)])
def test_linear_for_few_tokens(ops, m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.1).bfloat16().to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    want = (x.double() @ w.double().T).float()
    out = torch.full((m, n), 9.0, device=DEV)
    ops.linear_skinny(x, w, b, out)
    check(out, want + b, 1e-5, "few tokens, float32 out")
    outb = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.linear_skinny(x, w, b.bfloat16(), outb)
    check(outb, want + b.bfloat16().float(), 8e-3, "few tokens, bfloat16 out")
    acc = torch.full((m, n), 0.5, device=DEV)
    ops.linear_skinny(x, w, None, acc, accumulate=True)
    check(acc, want + 0.5, 1e-5, "few tokens, accumulate")
    again = torch.full((m, n), 0.5, device=DEV)
    ops.linear_skinny(x, w, None, again, accumulate=True)
    assert torch.equal(acc, again)                            # the same bits every time
    if m > 1:                                                 # a row does not depend on its neighbours
        one = torch.empty(1, n, device=DEV)
        ops.linear_skinny(x[m - 1:].contiguous(), w, b, one)
        assert torch.equal(one[0], out[m - 1])


@pytest.mark.parametrize("m,inter,k", [(1, 8, 64), (7, 136, 80), (8, 12288, 512), (13, 1000, 264), (16, 320, 4096)])
def test_linear_for_few_tokens_with_gated_epilogue(ops, m, inter, k):
    g = torch.Generator().manual_seed(m + inter)
    x = torch.randn(m, k, generator=g).bfloat16()
    gate = (torch.randn(inter, k, generator=g) * 0.1).bfloat16()
    up = (torch.randn(inter, k, generator=g) * 0.1).bfloat16()
    w = torch.stack([gate.view(-1, 8, k), up.view(-1, 8, k)], dim=1).reshape(-1, k).contiguous()
    want = P.swiglu((x.double() @ gate.double().T).float().numpy(), (x.double() @ up.double().T).float().numpy())
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 8e-3)):
        out = torch.full((m, inter), 9.0, dtype=dt, device=DEV)
        ops.linear_skinny(x.to(DEV), w.to(DEV), None, out, epilogue="swiglu")
        check(out, want, tol, "few tokens, gated epilogue")


@pytest.mark.parametrize("m,hidden,inter", [(1, 64, 48), (5, 200, 136), (8, 4096, 512), (13, 1000, 264), (16, 320, 4096),
                                            (3, 5120, 64), (16, 8192, 32)])
def test_few_token_products_carry_the_norm_between_them(ops, m, hidden, inter):
    """residual += act . w_down^T, then rmsnorm(residual) . w_next^T: the first product leaves residual * gamma and
    its blocks' sums of squares, the second one finishes the norm in its epilogue.  Against the plain norm and
    products, for the plain and the gated epilogue, with a width that is no multiple of 16."""
    g = torch.Generator().manual_seed(m + hidden + inter)
    act = torch.randn(m, inter, generator=g).bfloat16().to(DEV)
    w_down = (torch.randn(hidden, inter, generator=g) * 0.1).bfloat16().to(DEV)
    residual0 = torch.randn(m, hidden, generator=g).to(DEV)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().to(DEV)
    eps = 1e-5
    residual = residual0.clone()
    xg = torch.full((m, hidden), 9.0, dtype=torch.bfloat16, device=DEV)
    bins = torch.zeros(ops.NORM_WORDS, dtype=torch.int64, device=DEV)
    stale = torch.full((ops.NORM_WORDS,), 77, dtype=torch.int64, device=DEV)
    ops.linear_skinny(act, w_down, None, residual, accumulate=True, norm_out=(xg, gamma, bins, stale))
    plain = residual0.clone()
    ops.linear_skinny(act, w_down, None, plain, accumulate=True)
    assert torch.equal(residual, plain)                                   # the product itself is untouched
    assert int(stale.abs().max()) == 0                                    # the other norm's accumulators are cleared
    check(xg, residual * gamma.float(), 8e-3, "residual * gamma")
    # the accumulators hold the sums of the blocks' float sums exactly: bin b counts units of 2^(32 b - 150)
    words = bins.view(16, 16).cpu().numpy().astype(object)
    total = np.array([float(sum(int(words[t][b]) * 2.0 ** (32 * b - 150) for b in range(8))) for t in range(m)])
    want_ss = (residual.double() ** 2).sum(-1).cpu().numpy()
    assert np.abs(total - want_ss).max() <= 1e-6 * want_ss.max() and int(bins.view(16, 16)[:, 8].sum()) == 0
    again_bins = torch.zeros_like(bins)                                   # the same bits whatever the blocks' order
    ops.linear_skinny(act, w_down, None, residual0.clone(), accumulate=True, norm_out=(torch.empty_like(xg), gamma, again_bins, None))
    assert torch.equal(again_bins, bins)
    normed = P.rmsnorm(residual.cpu().numpy(), gamma.float().cpu().numpy(), eps)
    n_out = 16 * ((inter + 15) // 16)
    w_next = (torch.randn(n_out, hidden, generator=g) * 0.1).bfloat16().to(DEV)
    bias = torch.randn(n_out, generator=g).to(DEV)
    out = torch.full((m, n_out), 9.0, device=DEV)
    ops.linear_skinny(xg, w_next, bias, out, norm_in=(bins, eps))
    want = P.linear(normed, w_next.float().cpu().numpy(), bias.cpu().numpy())
    check(out, want, 8e-3, "consumer, plain epilogue")                    # x * gamma was rounded to bfloat16 on the way
    gated = torch.full((m, n_out // 2), 9.0, device=DEV)
    ops.linear_skinny(xg, w_next, None, gated, epilogue="swiglu", norm_in=(bins, eps))
    y = P.linear(normed, w_next.float().cpu().numpy()).reshape(m, -1, 2, 8)
    check(gated, P.swiglu(y[:, :, 0].reshape(m, -1), y[:, :, 1].reshape(m, -1)), 8e-3, "consumer, gated epilogue")
    # a row that is not finite has no finite scale: NaN comes out, as from the norm itself
    bad = residual0.clone()
    bad[0, 3] = float("inf")
    bins.zero_()
    ops.linear_skinny(act, w_down, None, bad, accumulate=True, norm_out=(xg, gamma, bins, None))
    ops.linear_skinny(xg, w_next, None, out, norm_in=(bins, eps))
    assert torch.isnan(out[0]).all() and (m == 1 or torch.isfinite(out[1:]).all())


def test_linear_for_few_tokens_refuses(ops):
    x = torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ExtensionError, match="at most 16 tokens"):
        ops.linear_skinny(x, w, None, torch.empty(17, 8, device=DEV))


def test_linear_tensor_core_refuses_unaligned(ops):
    x = torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    assert not ops.linear_tc_supported(4, 8, 20)
    with pytest.raises(ExtensionError, match="multiples of 8"):
        ops.linear_tc(x, w, None, torch.empty(4, 8, device=DEV), ops.GemmWorkspace(DEV))


def test_rope_table(ops):
    pos = torch.tensor([0, 1, 5, 1000, 40959], dtype=torch.int32, device=DEV)
    for theta, half in ((1e4, 8), (1e6, 64), (5e5, 24)):
        inv = torch.pow(torch.tensor(theta, dtype=torch.float64),
                        -2.0 * torch.arange(half, dtype=torch.float64) / (2 * half)).float()
        out = torch.empty(5, half, 2, device=DEV)
        ops.rope_table(pos, inv.to(DEV), out)
        ang = (pos.cpu().float()[:, None] * inv[None, :]).double()
        assert (out[..., 0].cpu() - torch.cos(ang).float()).abs().max() < 2e-6
        assert (out[..., 1].cpu() - torch.sin(ang).float()).abs().max() < 2e-6


@pytest.mark.parametrize("m,n,k", [(3, 307, 4104), (8, 64, 8192), (13, 5120, 2560), (16, 1000, 136)])
def test_few_token_product_in_blocks_of_four_warps(ops, m, n, k):
    """Grids of a little more than two 16-row blocks per SM run as blocks of 4 warps (every thread finishes two
    output elements): forced here at other sizes too, every epilogue, with and without the norms riding on it, and
    bit for bit what blocks of 8 warps give wherever a warp's share of K is the same."""
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16().to(DEV)
    b = torch.randn(n, generator=g).to(DEV)
    want = (x.double() @ w.double().T).float()
    try:
        ops.linear_skinny_force_warps(4)
        out = torch.full((m, n), 9.0, device=DEV)
        ops.linear_skinny(x, w, b, out)
        check(out, want + b, 1e-5, "float32 out with bias")
        again = torch.full((m, n), 9.0, device=DEV)
        ops.linear_skinny(x, w, b, again)
        assert torch.equal(out, again)
        acc = torch.full((m, n), 0.5, dtype=torch.bfloat16, device=DEV)
        ops.linear_skinny(x, w, None, acc, accumulate=True)
        check(acc, want + 0.5, 8e-3, "accumulate in bfloat16")
        if n % 16 == 0:
            gated = torch.full((m, n // 2), 9.0, device=DEV)
            ops.linear_skinny(x, w, None, gated, epilogue="swiglu")
            y = want.cpu().numpy().reshape(m, -1, 2, 8)
            check(gated, P.swiglu(y[:, :, 0].reshape(m, -1), y[:, :, 1].reshape(m, -1)), 1e-5, "gated")
            gamma = (1 + 0.1 * torch.randn(n, generator=g)).bfloat16().to(DEV)
            residual = torch.full((m, n), 0.25, device=DEV)
            xg = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
            bins = torch.zeros(ops.NORM_WORDS, dtype=torch.int64, device=DEV)
            stale = torch.full((ops.NORM_WORDS,), 5, dtype=torch.int64, device=DEV)
            ops.linear_skinny(x, w, None, residual, accumulate=True, norm_out=(xg, gamma, bins, stale))
            check(residual, want + 0.25, 1e-5, "producer")
            assert int(stale.abs().max()) == 0
            check(xg, residual * gamma.float(), 8e-3, "residual * gamma")
            w2 = (torch.randn(64, n, generator=g) * 0.05).bfloat16().to(DEV)
            out2 = torch.empty(m, 64, device=DEV)
            ops.linear_skinny(xg, w2, None, out2, norm_in=(bins, 1e-6))
            normed = P.rmsnorm(residual.cpu().numpy(), gamma.float().cpu().numpy(), 1e-6)
            check(out2, P.linear(normed, w2.float().cpu().numpy()), 8e-3, "consumer")
            ops.linear_skinny_force_warps(8)
            wide = torch.zeros_like(bins)
            ops.linear_skinny(x, w, None, torch.full((m, n), 0.25, device=DEV), accumulate=True,
                              norm_out=(torch.empty_like(xg), gamma, wide, None))
            ss = lambda t: np.array([sum(int(v) * 2.0 ** (32 * i - 150) for i, v in enumerate(row[:8]))
                                     for row in t.view(16, 16).cpu().numpy().astype(object)])
            assert np.abs(ss(bins) - ss(wide)).max() <= 1e-4 * max(ss(wide).max(), 1e-30)
    finally:
        ops.linear_skinny_force_warps(0)


@pytest.mark.parametrize("m,hidden,inter", [(512, 512, 1024), (700, 1040, 528)])
def test_products_of_prompts_carry_the_norm_between_them(ops, m, hidden, inter):
    """The same on the tensor cores for 512 tokens and more: the product that adds into the residual stream leaves
    residual * gamma and one exact accumulator of the sum of squares per row; the product that follows (plain or
    gated epilogue) multiplies its accumulators by the rows' scales.  A token count and widths that are no multiples
    of the 256 x 256 tiles."""
    g = torch.Generator().manual_seed(m + hidden)
    act = torch.randn(m, inter, generator=g).bfloat16().to(DEV)
    w_down = (torch.randn(hidden, inter, generator=g) * 0.1).bfloat16().to(DEV)
    residual0 = torch.randn(m, hidden, generator=g).to(DEV)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().to(DEV)
    eps = 1e-5
    ws = ops.GemmWorkspace(DEV)
    assert ops.linear_tc_fuses_norms(m, hidden) and not ops.linear_tc_fuses_norms(511, hidden)
    residual = residual0.clone()
    xg = torch.full((m, hidden), 9.0, dtype=torch.bfloat16, device=DEV)
    bins = torch.zeros(m, ops.NORM_ROW_WORDS, dtype=torch.int64, device=DEV)
    stale = torch.full((m, ops.NORM_ROW_WORDS), 77, dtype=torch.int64, device=DEV)
    ops.linear_tc(act, w_down, None, residual, ws, accumulate=True, norm_out=(xg, gamma, bins, stale))
    plain = residual0.clone()
    ops.linear_tc(act, w_down, None, plain, ws, accumulate=True)
    assert torch.equal(residual, plain)                                   # the product itself is untouched
    assert int(stale.abs().max()) == 0                                    # the other norm's accumulators are cleared
    check(xg, residual * gamma.float(), 8e-3, "residual * gamma")
    words = bins.cpu().numpy().astype(object)
    total = np.array([float(sum(int(words[t][b]) * 2.0 ** (32 * b - 150) for b in range(8))) for t in range(m)])
    want_ss = (residual.double() ** 2).sum(-1).cpu().numpy()
    assert np.abs(total - want_ss).max() <= 1e-6 * want_ss.max() and int(bins[:, 8].sum()) == 0
    again = torch.zeros_like(bins)                                        # the same bits whatever the blocks' order
    ops.linear_tc(act, w_down, None, residual0.clone(), ws, accumulate=True, norm_out=(torch.empty_like(xg), gamma, again, None))
    assert torch.equal(again, bins)
    normed = P.rmsnorm(residual.cpu().numpy(), gamma.float().cpu().numpy(), eps)
    n_out = 16 * ((inter + 15) // 16)
    w_next = (torch.randn(n_out, hidden, generator=g) * 0.1).bfloat16().to(DEV)
    bias = torch.randn(n_out, generator=g).to(DEV)
    out = torch.full((m, n_out), 9.0, device=DEV)
    ops.linear_tc(xg, w_next, bias, out, ws, norm_in=(bins, eps))
    want = P.linear(normed, w_next.float().cpu().numpy(), bias.cpu().numpy())
    check(out, want, 8e-3, "consumer, plain epilogue")
    gated = torch.full((m, n_out // 2), 9.0, device=DEV)
    ops.linear_tc(xg, w_next, None, gated, ws, epilogue="swiglu", norm_in=(bins, eps))
    y = P.linear(normed, w_next.float().cpu().numpy()).reshape(m, -1, 2, 8)
    check(gated, P.swiglu(y[:, :, 0].reshape(m, -1), y[:, :, 1].reshape(m, -1)), 8e-3, "consumer, gated epilogue")
    with pytest.raises(ExtensionError):                                   # sizes whose kernel cannot carry a norm say so
        ops.linear_tc(xg[:100].contiguous(), w_next, None, torch.empty(100, n_out, device=DEV), ws, norm_in=(bins[:100].contiguous(), eps))
    assert int(ws.status.item()) == 0


@pytest.mark.parametrize("m", [17, 40, 64])
def test_products_of_17_to_64_tokens_carry_the_norm_between_them(ops, m):
    """With the weights as the 128-row operand a token is a column: the cluster kernel that adds into the residual
    stream leaves residual * gamma and adds each warp's part of a token's sum of squares into the token's
    accumulator; the cluster kernel and the kernel of whole tiles per block multiply their columns by the tokens'
    scales (plain and gated epilogue)."""
    g = torch.Generator().manual_seed(m)
    hidden, inter, wide = 1024, 2816, 19200
    act = torch.randn(m, inter, generator=g).bfloat16().to(DEV)
    w_down = (torch.randn(hidden, inter, generator=g) * 0.1).bfloat16().to(DEV)
    residual0 = torch.randn(m, hidden, generator=g).to(DEV)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().to(DEV)
    eps = 1e-5
    ws = ops.GemmWorkspace(DEV)
    assert ops.linear_tc_norm_roles(m, hidden, inter) == 3 and ops.linear_tc_norm_roles(m, wide, hidden) == 1
    assert ops.linear_tc_norm_roles(100, hidden, inter) == 0
    residual = residual0.clone()
    xg = torch.full((m, hidden), 9.0, dtype=torch.bfloat16, device=DEV)
    bins = torch.zeros(m, ops.NORM_ROW_WORDS, dtype=torch.int64, device=DEV)
    stale = torch.full((m, ops.NORM_ROW_WORDS), 77, dtype=torch.int64, device=DEV)
    ops.linear_tc(act, w_down, None, residual, ws, accumulate=True, norm_out=(xg, gamma, bins, stale))
    plain = residual0.clone()
    ops.linear_tc(act, w_down, None, plain, ws, accumulate=True)
    assert torch.equal(residual, plain) and int(stale.abs().max()) == 0
    check(xg, residual * gamma.float(), 8e-3, "residual * gamma")
    words = bins.cpu().numpy().astype(object)
    total = np.array([float(sum(int(words[t][b]) * 2.0 ** (32 * b - 150) for b in range(8))) for t in range(m)])
    want_ss = (residual.double() ** 2).sum(-1).cpu().numpy()
    assert np.abs(total - want_ss).max() <= 1e-6 * want_ss.max() and int(bins[:, 8].sum()) == 0
    again = torch.zeros_like(bins)
    ops.linear_tc(act, w_down, None, residual0.clone(), ws, accumulate=True, norm_out=(torch.empty_like(xg), gamma, again, None))
    assert torch.equal(again, bins)
    normed = P.rmsnorm(residual.cpu().numpy(), gamma.float().cpu().numpy(), eps)
    for n_out in (inter, wide):     # a cluster per tile; whole tiles per block
        w_next = (torch.randn(n_out, hidden, generator=g) * 0.1).bfloat16().to(DEV)
        bias = torch.randn(n_out, generator=g).to(DEV)
        out = torch.full((m, n_out), 9.0, device=DEV)
        ops.linear_tc(xg, w_next, bias, out, ws, norm_in=(bins, eps))
        want = P.linear(normed, w_next.float().cpu().numpy(), bias.cpu().numpy())
        check(out, want, 8e-3, f"consumer, plain epilogue, {n_out} features")
        gated = torch.full((m, n_out // 2), 9.0, device=DEV)
        ops.linear_tc(xg, w_next, None, gated, ws, epilogue="swiglu", norm_in=(bins, eps))
        y = P.linear(normed, w_next.float().cpu().numpy()).reshape(m, -1, 2, 8)
        check(gated, P.swiglu(y[:, :, 0].reshape(m, -1), y[:, :, 1].reshape(m, -1)), 8e-3, f"consumer, gated, {n_out}")
    assert int(ws.status.item()) == 0


@pytest.mark.parametrize("m", [3, 13])
def test_products_that_start_under_their_predecessor_give_the_same_bits(ops, m):
    """A chain of few-token products, each reading what the one before wrote (with a norm carried between two of
    them): launched so that each may start while its predecessor ends, and launched one after the other, in a
    plain stream and in a captured graph, it leaves the same bits.  The chain is long and its matrices differ in
    size, so that blocks of three kernels are in flight at once."""
    g = torch.Generator().manual_seed(m)
    hidden, inter = 1024, 2816
    w_up = [(torch.randn(2 * inter, hidden, generator=g) * 0.05).bfloat16().to(DEV) for _ in range(4)]
    w_down = [(torch.randn(hidden, inter, generator=g) * 0.05).bfloat16().to(DEV) for _ in range(4)]
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().to(DEV)
    x0 = torch.randn(m, hidden, generator=g).to(DEV)

    def chain():
        residual = x0.clone()
        xg = (x0 * gamma.float()).bfloat16()
        bins = torch.zeros(2, ops.NORM_WORDS, dtype=torch.int64, device=DEV)
        ss = (x0.double() ** 2).sum(-1)
        act = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
        first = torch.empty(m, 2 * inter, dtype=torch.bfloat16, device=DEV)
        ops.linear_skinny(xg, w_up[0], None, first)                       # nothing of this kind before it
        for layer in range(4):
            if layer == 0:
                ops.linear_skinny(xg, w_up[0], None, act, epilogue="swiglu")
            else:
                ops.linear_skinny(xg, w_up[layer], None, act, epilogue="swiglu", norm_in=(bins[layer % 2], 1e-6))
            ops.linear_skinny(act, w_down[layer], None, residual, accumulate=True,
                              norm_out=(xg, gamma, bins[(layer + 1) % 2], bins[layer % 2]))
        return residual, xg.clone(), bins.clone()

    try:
        ops.launch_overlap(False)
        want = chain()
        ops.launch_overlap(True)
        for _ in range(3):
            got = chain()
            assert all(torch.equal(a, b) for a, b in zip(got, want))
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = chain()
        for _ in range(3):
            graph.replay()
            torch.cuda.synchronize()
            assert all(torch.equal(a, b) for a, b in zip(captured, want))
    finally:
        ops.launch_overlap(True)
    assert bool(torch.isfinite(want[0]).all())


@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (5, 1, 48, 48), (3, 3, 80, 32), (8, 2, 128, 128)])
@pytest.mark.parametrize("dt", DT)
def test_qk_norm_rope_append(ops, nh, nkv, hd, rot, dt):
    g = torch.Generator().manual_seed(nh * hd)
    lens, new = [70, 3], [5, 3]       # sequence 0 already holds 65 tokens, sequence 1 starts
    n = sum(new)
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, generator=g)
    qg, kg = (1 + 0.1 * torch.randn(hd, generator=g) for _ in range(2))
    tok_seq = torch.tensor([0] * 5 + [1] * 3, dtype=torch.int32)
    tok_pos = torch.tensor(list(range(65, 70)) + [0, 1, 2], dtype=torch.int32)
    table = torch.tensor([[4, 1], [2, -1]], dtype=torch.int32)
    theta = 1e4
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)
    cs = torch.empty(n, rot // 2, 2, device=DEV)
    ops.rope_table(tok_pos.to(DEV), inv.float().to(DEV), cs)
    kp = torch.full((6, nkv, PAGE, hd), 7.0, dtype=dt, device=DEV)
    vp = torch.full((6, nkv, PAGE, hd), 7.0, dtype=dt, device=DEV)
    q_out = torch.empty(n, nh * hd, dtype=dt, device=DEV)
    ops.qk_norm_rope_append(qkv.to(dt).to(DEV), qg.to(DEV), kg.to(DEV), 1e-6, cs, tok_seq.to(DEV), tok_pos.to(DEV),
                            table.to(DEV), kp, vp, q_out, nh, nkv, hd)
    x = qkv.to(dt).float().numpy()
    q = x[:, :nh * hd].reshape(n, nh, hd)
    k = x[:, nh * hd:(nh + nkv) * hd].reshape(n, nkv, hd)
    v = x[:, (nh + nkv) * hd:].reshape(n, nkv, hd)
    q = P.rope_neox(P.rmsnorm(q, qg.numpy(), 1e-6), tok_pos.numpy(), theta, rot)
    k = P.rope_neox(P.rmsnorm(k, kg.numpy(), 1e-6), tok_pos.numpy(), theta, rot)
    tol = 1e-5 if dt == torch.float32 else 8e-3
    check(q_out.view(n, nh, hd), q, tol, "q")
    for t in range(n):
        page = int(table[tok_seq[t], tok_pos[t] // PAGE])
        check(kp[page, :, tok_pos[t] % PAGE], k[t], tol, f"k of token {t}")
        check(vp[page, :, tok_pos[t] % PAGE], v[t], tol, f"v of token {t}")
    # nothing else was written
    written = torch.zeros(6, PAGE, dtype=torch.bool)
    for t in range(n):
        written[int(table[tok_seq[t], tok_pos[t] // PAGE]), tok_pos[t] % PAGE] = True
    untouched = ~written[:, None, :, None].expand(6, nkv, PAGE, hd)
    assert bool((kp.float().cpu()[untouched] == 7.0).all()) and bool((vp.float().cpu()[untouched] == 7.0).all())


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 128), (4, 2, 64), (3, 1, 128)])
def test_qk_norm_rope_append_float32_in_bfloat16_out(ops, nh, nkv, hd):
    """The combination a bfloat16 run uses: float32 projections in, bfloat16 q and cache out."""
    g = torch.Generator().manual_seed(hd + nh)
    new = [70, 3, 1]
    starts = [65, 0, 200]
    n = sum(new)
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, generator=g)
    qg, kg = (1 + 0.1 * torch.randn(hd, generator=g) for _ in range(2))
    tok_seq = torch.tensor([b for b, k in enumerate(new) for _ in range(k)], dtype=torch.int32)
    tok_pos = torch.tensor([s + i for s, k in zip(starts, new) for i in range(k)], dtype=torch.int32)
    table = torch.tensor([[4, 1, 7, -1], [2, -1, -1, -1], [0, 3, 5, 6]], dtype=torch.int32)
    theta = 1e6
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    cs = torch.empty(n, hd // 2, 2, device=DEV)
    ops.rope_table(tok_pos.to(DEV), inv.float().to(DEV), cs)
    kp = torch.full((8, nkv, PAGE, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    vp = torch.full((8, nkv, PAGE, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
    ops.qk_norm_rope_append(qkv.to(DEV), qg.bfloat16().to(DEV), kg.bfloat16().to(DEV), 1e-6, cs, tok_seq.to(DEV),
                            tok_pos.to(DEV), table.to(DEV), kp, vp, q_out, nh, nkv, hd)
    x = qkv.numpy()
    q = x[:, :nh * hd].reshape(n, nh, hd)
    k = x[:, nh * hd:(nh + nkv) * hd].reshape(n, nkv, hd)
    v = x[:, (nh + nkv) * hd:].reshape(n, nkv, hd)
    q = P.rope_neox(P.rmsnorm(q, qg.bfloat16().float().numpy(), 1e-6), tok_pos.numpy(), theta, hd)
    k = P.rope_neox(P.rmsnorm(k, kg.bfloat16().float().numpy(), 1e-6), tok_pos.numpy(), theta, hd)
    check(q_out.view(n, nh, hd), q, 8e-3, "q")
    written = torch.zeros(8, PAGE, dtype=torch.bool)
    for t in range(n):
        page = int(table[tok_seq[t], tok_pos[t] // PAGE])
        check(kp[page, :, tok_pos[t] % PAGE], k[t], 8e-3, f"k of token {t}")
        check(vp[page, :, tok_pos[t] % PAGE], v[t], 8e-3, f"v of token {t}")
        written[page, tok_pos[t] % PAGE] = True
    untouched = ~written[:, None, :, None].expand(8, nkv, PAGE, hd)
    assert bool((kp.float().cpu()[untouched] == 7.0).all()) and bool((vp.float().cpu()[untouched] == 7.0).all())


@pytest.mark.parametrize("nh,nkv,k,with_norm,with_rope", [(4, 2, 256, True, True), (2, 2, 136, False, True),
                                                          (6, 4, 64, True, False)])
def test_linear_qkv_fused_epilogue(ops, nh, nkv, k, with_norm, with_rope):
    """The q/k/v projection of prompts with norm, rotation and cache append in its epilogue: three sequences
    (one continuing at position 130, one with a padded row in the middle), a token count that does not fill
    the last 256-row tile."""
    hd = 128
    g = torch.Generator().manual_seed(nh + k)
    new, starts = [300, 257, 43], [130, 0, 64]
    n = sum(new)
    x = (torch.randn(n, k, generator=g) * 0.5).bfloat16()
    w = (torch.randn((nh + 2 * nkv) * hd, k, generator=g) / math.sqrt(k)).bfloat16()
    qg, kg = ((1 + 0.1 * torch.randn(hd, generator=g)).bfloat16() for _ in range(2))
    tok_seq = torch.tensor([b for b, c in enumerate(new) for _ in range(c)], dtype=torch.int32)
    tok_pos = torch.tensor([s0 + i for s0, c in zip(starts, new) for i in range(c)], dtype=torch.int32)
    pad = 310
    tok_seq[pad] = -1                                                     # a padded row: q is written, the cache is not
    n_pages = 16
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((3, 8), -1, dtype=torch.int32)
    it = iter(perm)
    for b, (s0, c) in enumerate(zip(starts, new)):
        for pg in range((s0 + c + PAGE - 1) // PAGE):
            table[b, pg] = next(it)
    theta = 1e6
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    cs = None
    if with_rope:
        cs = torch.empty(hd // 2, n, 2, device=DEV)
        ops.rope_table(tok_pos.to(DEV), inv.float().to(DEV), cs, by_pair=True)
        by_token = torch.empty(n, hd // 2, 2, device=DEV)
        ops.rope_table(tok_pos.to(DEV), inv.float().to(DEV), by_token)
        assert torch.equal(cs.transpose(0, 1), by_token)
    kp = torch.full((n_pages, nkv, PAGE, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    vp = torch.full((n_pages, nkv, PAGE, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.full((n, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
    xd = x.to(DEV)
    assert ops.linear_tc_qkv_supported(xd, nh, nkv, hd) and not ops.linear_tc_qkv_supported(xd[:100], nh, nkv, hd)
    assert not ops.linear_tc_qkv_supported(xd, nh, nkv, 64) and not ops.linear_tc_qkv_supported(xd, 3, nkv, hd)
    ws = ops.GemmWorkspace(DEV)
    ops.linear_tc_qkv(xd, w.to(DEV), qg.to(DEV) if with_norm else None, kg.to(DEV) if with_norm else None, 1e-6, cs,
                      tok_seq.to(DEV), tok_pos.to(DEV), table.to(DEV), kp, vp, q_out, ws, nh, nkv, hd)
    assert int(ws.status.item()) == 0
    y = P.linear(x.float().numpy(), w.float().numpy())
    q = y[:, :nh * hd].reshape(n, nh, hd)
    kk = y[:, nh * hd:(nh + nkv) * hd].reshape(n, nkv, hd)
    v = y[:, (nh + nkv) * hd:].reshape(n, nkv, hd)
    if with_norm:
        q, kk = P.rmsnorm(q, qg.float().numpy(), 1e-6), P.rmsnorm(kk, kg.float().numpy(), 1e-6)
    if with_rope:
        q, kk = P.rope_neox(q, tok_pos.numpy(), theta, hd), P.rope_neox(kk, tok_pos.numpy(), theta, hd)
    check(q_out.view(n, nh, hd), q, 8e-3, "q")
    written = torch.zeros(n_pages, PAGE, dtype=torch.bool)
    for t in list(range(0, n, 7)) + [299, 300, 556, 557, n - 1]:
        if t == pad:
            continue
        page = int(table[tok_seq[t], tok_pos[t] // PAGE])
        check(kp[page, :, tok_pos[t] % PAGE], kk[t], 8e-3, f"k of token {t}")
        check(vp[page, :, tok_pos[t] % PAGE], v[t], 8e-3, f"v of token {t}")
    for t in range(n):
        if t != pad:
            written[int(table[tok_seq[t], tok_pos[t] // PAGE]), tok_pos[t] % PAGE] = True
    untouched = ~written[:, None, :, None].expand(n_pages, nkv, PAGE, hd)
    assert bool((kp.float().cpu()[untouched] == 7.0).all()) and bool((vp.float().cpu()[untouched] == 7.0).all())
    assert bool((kp.float().cpu()[~untouched] != 7.0).any())


def test_qk_norm_rope_append_padding_and_no_norm(ops):
    n, nh, nkv, hd = 3, 2, 1, 16
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, device=DEV)
    tok_seq = torch.tensor([0, -1, 0], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([0, 0, 1], dtype=torch.int32, device=DEV)
    table = torch.tensor([[1]], dtype=torch.int32, device=DEV)
    kp = torch.zeros(2, nkv, PAGE, hd, device=DEV)
    vp = torch.zeros(2, nkv, PAGE, hd, device=DEV)
    q_out = torch.empty(n, nh * hd, device=DEV)
    ops.qk_norm_rope_append(qkv, None, None, 0.0, None, tok_seq, tok_pos, table, kp, vp, q_out, nh, nkv, hd)
    assert torch.equal(q_out, qkv[:, :nh * hd])                      # no norm, no rotation: a copy
    assert torch.equal(kp[1, 0, 0], qkv[0, nh * hd:(nh + 1) * hd]) and torch.equal(kp[1, 0, 1], qkv[2, 32:48])
    assert float(kp[0].abs().sum()) == 0 and float(kp[1, 0, 2:].abs().sum()) == 0   # the padded row wrote nothing


def plain_paged_attention(q, ks, vs, tok_seq, tok_pos, window):
    out = np.zeros_like(q)
    for t in range(q.shape[0]):
        b, p = tok_seq[t], tok_pos[t]
        first, last = P.attn_span(window, p)
        k, v = ks[b][first:last + 1].numpy(), vs[b][first:last + 1].numpy()
        nh, hd = q.shape[1], q.shape[2]
        for h in range(nh):
            kv = h // (nh // k.shape[1])
            s = (k[:, kv].astype(np.float64) @ q[t, h].astype(np.float64)) / math.sqrt(hd)
            w = np.exp(s - s.max())
            out[t, h] = (w @ v[:, kv].astype(np.float64)) / w.sum()
    return out


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (5, 1, 48, 0), (8, 2, 128, 0), (6, 3, 32, 50),
                                              (2, 2, 80, 7), (4, 1, 256, 130)])
@pytest.mark.parametrize("dt", DT)
def test_attention_over_pages(ops, nh, nkv, hd, window, dt):
    seqs = [300, 1, 64, 65, 129]
    kp, vp, table, ks, vs = scatter_pages(16, nkv, hd, seqs, dt, seed=hd)
    # queries: the last 3 positions of sequence 0 (a prompt's end), every position of 3 and some of the others
    tok = [(0, 297), (0, 298), (0, 299), (1, 0), (2, 63), (4, 128), (4, 64), (4, 5)] + [(3, p) for p in range(65)]
    tok_seq = torch.tensor([t[0] for t in tok], dtype=torch.int32)
    tok_pos = torch.tensor([t[1] for t in tok], dtype=torch.int32)
    g = torch.Generator().manual_seed(1)
    q = torch.randn(len(tok), nh, hd, generator=g).to(dt)
    out = torch.empty(len(tok), nh * hd, dtype=dt, device=DEV)
    ops.attention(q.view(len(tok), -1).to(DEV), kp, vp, table, tok_seq.to(DEV), tok_pos.to(DEV), out, nh, nkv, hd,
                  1.0 / math.sqrt(hd), window)
    want = plain_paged_attention(q.float().numpy(), ks, vs, tok_seq.tolist(), tok_pos.tolist(), window)
    check(out.view(len(tok), nh, hd), want, 2e-5 if dt == torch.float32 else 1.5e-2, "attention")


@pytest.mark.parametrize("dt", DT)
def test_attention_finds_one_far_key_and_respects_the_window_edge(ops, dt):
    nh, nkv, hd, n = 2, 1, 32, 700
    kp, vp, table, ks, vs = scatter_pages(12, nkv, hd, [n], dt, seed=3)
    q = torch.randn(1, nh, hd).to(dt)
    # make key 3 (far back, first page) the one that matters: aligned with q and large
    far = 3
    page, row = int(table[0, far // PAGE]), far % PAGE
    kp[page, 0, row] = (q[0, 0].float() * 4).to(dt).to(DEV)
    args = (table, torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([n - 1], dtype=torch.int32, device=DEV))
    out = torch.empty(1, nh * hd, dtype=dt, device=DEV)
    ops.attention(q.view(1, -1).to(DEV), kp, vp, *args, out, nh, nkv, hd, 1.0 / math.sqrt(hd), 0)
    assert rel_err(out.view(nh, hd)[0], vs[0][far, 0].to(dt).float()) < 2e-2      # head 0 returns that key's value
    # window n - far: key `far` is the first key inside; window one less: it is outside
    inside = torch.empty_like(out)
    ops.attention(q.view(1, -1).to(DEV), kp, vp, *args, inside, nh, nkv, hd, 1.0 / math.sqrt(hd), n - far)
    assert rel_err(inside.view(nh, hd)[0], vs[0][far, 0].to(dt).float()) < 2e-2
    outside = torch.empty_like(out)
    ops.attention(q.view(1, -1).to(DEV), kp, vp, *args, outside, nh, nkv, hd, 1.0 / math.sqrt(hd), n - far - 1)
    assert rel_err(outside.view(nh, hd)[0], vs[0][far, 0].to(dt).float()) > 0.5
    ks[0][far, 0] = (q[0, 0].float() * 4).to(dt).float()
    for w, got in ((0, out), (n - far, inside), (n - far - 1, outside)):
        want = plain_paged_attention(q.float().numpy(), ks, vs, [0], [n - 1], w)
        check(got.view(1, nh, hd), want, 2e-5 if dt == torch.float32 else 1.5e-2, f"window {w}")


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 64, 0), (8, 1, 128, 0), (32, 8, 128, 0), (16, 1, 64, 70),
                                              (3, 3, 128, 33), (12, 2, 128, 500)])
def test_attention_tensor_core_decode(ops, nh, nkv, hd, window):
    seqs = [700, 1, 64, 65, 16, 17, 300]
    kp, vp, table, ks, vs = scatter_pages(24, nkv, hd, seqs, torch.bfloat16, seed=hd + nh)
    tok_seq = torch.tensor([0, 1, 2, -1, 3, 4, 5, 6], dtype=torch.int32)
    tok_pos = torch.tensor([699, 0, 63, 5, 64, 15, 16, 299], dtype=torch.int32)
    n = len(tok_seq)
    q = torch.randn(n, nh, hd, generator=torch.Generator().manual_seed(2)).bfloat16()
    live = [i for i in range(n) if tok_seq[i] >= 0]
    want = plain_paged_attention(q.float().numpy()[live], ks, vs, tok_seq[live].tolist(), tok_pos[live].tolist(), window)
    for n_splits in (1, 2, 5, 8, 64):
        out = torch.full((n, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
        floats = ops.attention_decode_scratch_floats(n, nh, nkv, hd, n_splits)
        scratch = torch.full((floats,), float("nan"), device=DEV) if floats else None
        ops.attention_decode_mma(q.view(n, -1).to(DEV), kp, vp, table, tok_seq.to(DEV), tok_pos.to(DEV), out, scratch,
                                 nh, nkv, hd, 1.0 / math.sqrt(hd), window, n_splits)
        check(out.view(n, nh, hd)[live], want, 1.5e-2, f"decode attention, {n_splits} splits")
        assert float(out[3].float().abs().sum()) == 0.0          # the padded row
        if 1 < n_splits <= 8:                                    # the same splits merged inside a cluster
            clustered = torch.full((n, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
            ops.attention_decode_mma(q.view(n, -1).to(DEV), kp, vp, table, tok_seq.to(DEV), tok_pos.to(DEV), clustered,
                                     None, nh, nkv, hd, 1.0 / math.sqrt(hd), window, n_splits)
            assert torch.equal(clustered, out)


@pytest.mark.parametrize("nh,nkv,hd,window,with_norm,with_rope", [(4, 2, 64, 0, True, True), (8, 1, 128, 0, True, True),
                                                                  (32, 8, 128, 0, True, True), (16, 1, 64, 70, False, True),
                                                                  (3, 3, 128, 33, True, False), (12, 2, 128, 500, True, True)])
def test_attention_decode_from_the_projections(ops, nh, nkv, hd, window, with_norm, with_rope):
    """One launch (norm, rotation and append as the attention kernel's first steps) against the two it replaces:
    the same outputs and the same cache rows, bit for bit, for every number of splits, with a padding row, with
    sequences whose new token opens a page (position 64) or closes one (63), and also when the keys and values
    are another entry's (queries only, nothing appended)."""
    seqs = [700, 1, 64, 65, 16, 17, 300]
    kp0, vp0, table, _, _ = scatter_pages(24, nkv, hd, seqs, torch.bfloat16, seed=hd + nh)
    tok_seq = torch.tensor([0, 1, 2, -1, 3, 4, 5, 6], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([699, 0, 63, 5, 64, 15, 16, 299], dtype=torch.int32, device=DEV)
    n = len(tok_seq)
    g = torch.Generator().manual_seed(7)
    qkv = torch.randn(n, (nh + 2 * nkv) * hd, generator=g).to(DEV)
    qg = (1 + 0.1 * torch.randn(hd, generator=g)).bfloat16().to(DEV) if with_norm else None
    kg = (1 + 0.1 * torch.randn(hd, generator=g)).bfloat16().to(DEV) if with_norm else None
    cs = None
    if with_rope:
        inv = torch.pow(torch.tensor(1e6, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
        cs = torch.empty(n, hd // 2, 2, device=DEV)
        ops.rope_table(tok_pos, inv.float().to(DEV), cs)
    scale = 1.0 / math.sqrt(hd)
    for n_splits in (1, 3, 8, 20):
        floats = ops.attention_decode_scratch_floats(n, nh, nkv, hd, n_splits)
        for use_scratch in ([True] if n_splits > 8 else [True, False] if n_splits > 1 else [False]):
            scratch = torch.empty(floats, device=DEV) if (use_scratch and floats) else None
            kp, vp = kp0.clone(), vp0.clone()
            q = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
            ops.qk_norm_rope_append(qkv, qg, kg, 1e-6, cs, tok_seq, tok_pos, table, kp, vp, q, nh, nkv, hd)
            want = torch.full((n, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
            ops.attention_decode_mma(q, kp, vp, table, tok_seq, tok_pos, want, scratch, nh, nkv, hd, scale, window, n_splits)
            kp2, vp2 = kp0.clone(), vp0.clone()
            got = torch.full((n, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
            ops.attention_decode_mma_from_qkv(qkv, qg, kg, 1e-6, cs, kp2, vp2, True, table, tok_seq, tok_pos, got, scratch,
                                              nh, nkv, hd, scale, window, n_splits)
            assert torch.equal(got, want), (n_splits, use_scratch)
            assert torch.equal(kp2, kp) and torch.equal(vp2, vp)          # the same rows were appended, and only those
            # queries only: the cache already holds the token's key and value (another entry appended them)
            q_only = qkv[:, :nh * hd].contiguous()
            kp3, vp3 = kp.clone(), vp.clone()
            shared = torch.full((n, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
            ops.attention_decode_mma_from_qkv(q_only, qg, None, 1e-6, cs, kp3, vp3, False, table, tok_seq, tok_pos, shared,
                                              scratch, nh, nkv, hd, scale, window, n_splits)
            assert torch.equal(shared, want) and torch.equal(kp3, kp) and torch.equal(vp3, vp)


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 64, 0), (8, 1, 128, 0), (6, 3, 128, 40), (16, 1, 64, 17)])
def test_attention_tensor_core_prefill(ops, nh, nkv, hd, window):
    # sequence 0 adds 70 tokens to 130 cached ones, 1 starts with 1 token, 2 starts with 100, 3 adds 1 to 64, 4 adds 16 to 5
    old, new = [130, 0, 0, 64, 5], [70, 1, 100, 1, 16]
    seqs = [o + n for o, n in zip(old, new)]
    kp, vp, table, ks, vs = scatter_pages(16, nkv, hd, seqs, torch.bfloat16, seed=nh)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [o + i for o, n in zip(old, new) for i in range(n)]
    cu = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    n = len(tok_seq)
    q = torch.randn(n, nh, hd, generator=torch.Generator().manual_seed(5)).bfloat16()
    out = torch.full((n, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_mma(q.view(n, -1).to(DEV), kp, vp, table, torch.tensor(cu).to(DEV),
                              torch.tensor(tok_pos, dtype=torch.int32).to(DEV), out, len(new), nh, nkv, hd,
                              1.0 / math.sqrt(hd), window)
    want = plain_paged_attention(q.float().numpy(), ks, vs, tok_seq, tok_pos, window)
    check(out.view(n, nh, hd), want, 1.5e-2, "prefill attention")


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 64, 0), (8, 1, 128, 0), (6, 3, 128, 40), (16, 1, 64, 17),
                                              (3, 3, 128, 0), (5, 5, 64, 200), (8, 2, 128, 130), (10, 2, 128, 0),
                                              (3, 1, 64, 90)])
def test_attention_tcgen05_prefill(ops, nh, nkv, hd, window):
    """One and two heads per block (groups of 1, 2, 3, 4, 5, 8, 16: an odd group's last block has one head), spans that fill several 128-row tiles, start in
    the middle of a page, end one row into a tile, and windows shorter and longer than a tile."""
    old, new = [130, 0, 0, 64, 5, 0, 37], [70, 1, 100, 1, 16, 385, 129]
    seqs = [o + n for o, n in zip(old, new)]
    kp, vp, table, ks, vs = scatter_pages(32, nkv, hd, seqs, torch.bfloat16, seed=nh)
    tok_seq = [b for b, n in enumerate(new) for _ in range(n)]
    tok_pos = [o + i for o, n in zip(old, new) for i in range(n)]
    cu = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    n = len(tok_seq)
    q = torch.randn(n, nh, hd, generator=torch.Generator().manual_seed(5)).bfloat16()
    out = torch.full((n, nh * hd), 9.0, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.attention_prefill_tc(q.view(n, -1).to(DEV), kp, vp, table, torch.tensor(cu).to(DEV),
                             torch.tensor(tok_pos, dtype=torch.int32).to(DEV), out, status, len(new), nh, nkv, hd,
                             1.0 / math.sqrt(hd), window)
    assert int(status.item()) == 0
    want = plain_paged_attention(q.float().numpy(), ks, vs, tok_seq, tok_pos, window)
    check(out.view(n, nh, hd), want, 1.5e-2, "prefill attention (tcgen05)")


def test_attention_tcgen05_prefill_growing_maximum(ops):
    """Scores that grow along the keys make every page raise a row's running maximum by more than the
    rescale step (head 0); scores that fall along the keys never raise it after the first page (head 1)."""
    nh, nkv, hd, n = 2, 1, 128, 600
    kp, vp, table, ks, vs = scatter_pages(16, nkv, hd, [n], torch.bfloat16, seed=9)
    q = torch.randn(n, nh, hd, generator=torch.Generator().manual_seed(6)).bfloat16()
    d = torch.randn(hd, generator=torch.Generator().manual_seed(7))
    d = d / d.norm()
    q[:, 0] = (d * 8).bfloat16()
    q[:, 1] = (d * -8).bfloat16()
    for j in range(n):
        # score of key j for head 0: 8 * (j / 20) * sqrt(hd) / 8 / sqrt(hd) = j / 20, about 4.6 a page in log2 units
        # (twice that between the first key of one page and the last of the next)
        kj = (d * (j / 20.0) * math.sqrt(hd) / 8).bfloat16()
        kp[int(table[0, j // PAGE]), 0, j % PAGE] = kj.to(DEV)
        ks[0][j, 0] = kj.float()
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for window in (0, 150):
        out = torch.empty(n, nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_tc(q.view(n, -1).to(DEV), kp, vp, table, cu, pos, out, status, 1, nh, nkv, hd,
                                 1.0 / math.sqrt(hd), window)
        assert int(status.item()) == 0
        want = plain_paged_attention(q.float().numpy(), ks, vs, [0] * n, list(range(n)), window)
        check(out.view(n, nh, hd), want, 1.5e-2, f"prefill (tcgen05), window {window}")


def test_attention_tensor_core_far_key_and_window_edge(ops):
    nh, nkv, hd, n = 4, 1, 128, 900
    kp, vp, table, ks, vs = scatter_pages(16, nkv, hd, [n], torch.bfloat16, seed=8)
    q = torch.randn(1, nh, hd).bfloat16()
    far = 3
    page, row = int(table[0, far // PAGE]), far % PAGE
    kp[page, 0, row] = (q[0, 2].float() * 4).bfloat16().to(DEV)
    ks[0][far, 0] = (q[0, 2].float() * 4).bfloat16().float()
    z, last = torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    for window, seen in ((0, True), (n - far, True), (n - far - 1, False)):
        want = plain_paged_attention(q.float().numpy(), ks, vs, [0], [n - 1], window)
        for n_splits in (1, 7):
            out = torch.empty(1, nh * hd, dtype=torch.bfloat16, device=DEV)
            floats = ops.attention_decode_scratch_floats(1, nh, nkv, hd, n_splits)
            ops.attention_decode_mma(q.view(1, -1).to(DEV), kp, vp, table, z, last, out,
                                     torch.empty(floats, device=DEV) if floats else None, nh, nkv, hd,
                                     1.0 / math.sqrt(hd), window, n_splits)
            check(out.view(1, nh, hd), want, 1.5e-2, f"decode, window {window}")
            assert (rel_err(out.view(nh, hd)[2], vs[0][far, 0]) < 2e-2) == seen
        out = torch.empty(1, nh * hd, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_mma(q.view(1, -1).to(DEV), kp, vp, table, cu, last, out, 1, nh, nkv, hd,
                                  1.0 / math.sqrt(hd), window)
        check(out.view(1, nh, hd), want, 1.5e-2, f"prefill, window {window}")
        out = torch.empty(1, nh * hd, dtype=torch.bfloat16, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.attention_prefill_tc(q.view(1, -1).to(DEV), kp, vp, table, cu, last, out, status, 1, nh, nkv, hd,
                                 1.0 / math.sqrt(hd), window)
        check(out.view(1, nh, hd), want, 1.5e-2, f"prefill (tcgen05), window {window}")
        assert (rel_err(out.view(nh, hd)[2], vs[0][far, 0]) < 2e-2) == seen and int(status.item()) == 0


def test_attention_tensor_core_refuses_other_sizes(ops):
    assert not ops.attention_mma_supported(4, 2, 48) and not ops.attention_mma_supported(34, 1, 64)
    assert not ops.attention_mma_supported(4, 2, 64, torch.zeros(1)) and ops.attention_mma_supported(32, 8, 128)
    kp, vp, table, _, _ = scatter_pages(1, 1, 48, [4], torch.bfloat16)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = torch.zeros(1, 96, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ExtensionError, match="head size 64 or 128"):
        ops.attention_decode_mma(q, kp, vp, table, z, z, torch.empty_like(q), None, 2, 1, 48, 1.0, 0, 1)
    kp, vp, table, _, _ = scatter_pages(1, 1, 64, [4], torch.bfloat16)
    q = torch.zeros(1, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ExtensionError, match="scratch"):
        ops.attention_decode_mma(q, kp, vp, table, z, z, torch.empty_like(q), torch.empty(8, device=DEV), 2, 1, 64,
                                 1.0, 0, 4)


def test_attention_padding_row_is_zero(ops):
    kp, vp, table, _, _ = scatter_pages(2, 1, 16, [10], torch.float32)
    out = torch.full((2, 32), 5.0, device=DEV)
    ops.attention(torch.randn(2, 32, device=DEV), kp, vp, table, torch.tensor([-1, 0], dtype=torch.int32, device=DEV),
                  torch.tensor([0, 9], dtype=torch.int32, device=DEV), out, 2, 1, 16, 0.25, 0)
    assert float(out[0].abs().sum()) == 0 and float(out[1].abs().sum()) > 0


@pytest.mark.parametrize("inter", [1, 136, 1000])
@pytest.mark.parametrize("dt", DT)
def test_swiglu(ops, inter, dt):
    gu = (torch.randn(7, 2 * inter) * 4).to(dt)
    out = torch.empty(7, inter, dtype=dt, device=DEV)
    ops.swiglu(gu.to(DEV), out)
    want = P.swiglu(gu.float().numpy()[:, :inter], gu.float().numpy()[:, inter:])
    check(out, want, 2e-6 if dt == torch.float32 else 8e-3, "swiglu")


def test_gather_rows(ops):
    x = torch.randn(9, 33, device=DEV)
    out = torch.empty(3, 33, device=DEV)
    ops.gather_rows(x, torch.tensor([8, -1, 2], dtype=torch.int32, device=DEV), out)
    assert torch.equal(out[0], x[8]) and torch.equal(out[2], x[2]) and float(out[1].abs().sum()) == 0


def test_argmax_first_largest(ops):
    for vocab in (1, 31, 307, 8191, 8192, 10007, 151936):      # from 8192 on the row is searched in chunks
        logits = torch.randn(5, vocab)
        if vocab > 30:
            logits[1, 17] = logits[1, 5] = 50.0          # a tie: the lower id
            logits[2, :] = float("nan")
            logits[2, 9] = -3.0                          # NaN never wins
            logits[3, vocab - 1] = 60.0
            logits[4, :] = float("-inf")                  # nothing to choose from: the first id
        out = torch.empty(5, dtype=torch.int32, device=DEV)
        ops.argmax(logits.to(DEV), out)
        want = [P.argmax_first(np.where(np.isnan(r), -np.inf, r)) for r in logits.numpy()]
        assert out.tolist() == want


def test_topk_candidates(ops):
    rs = np.random.RandomState(3)
    for vocab, k in ((5, 5), (40, 1), (307, 40), (5000, 40), (151936, 40), (151936, 1000)):
        logits = (rs.randn(4, vocab) * 3).astype(np.float32)
        logits[1, rs.randint(vocab, size=max(1, vocab // 7))] = np.nan      # NaN ranks last
        logits[2, :] = np.round(logits[2, :])                                 # many ties: lower ids win
        logits[3, :] = 1.5                                                    # all equal: the first k ids
        vals = torch.empty(4, k, device=DEV)
        ids = torch.empty(4, k, dtype=torch.int32, device=DEV)
        ops.topk(torch.tensor(logits).to(DEV), vals, ids)
        for r in range(4):
            l = np.where(np.isnan(logits[r]), -np.inf, logits[r])
            want = np.lexsort((np.arange(vocab), -l))[:k]
            got = ids[r].cpu().numpy()
            assert sorted(got.tolist()) == sorted(want.tolist()), (vocab, k, r)
            assert np.array_equal(vals[r].cpu().numpy(), l[got])


def plain_temperature_draw(row, u, temperature):
    """The draw in token-id order: p_i = exp((l_i - max) / T) in double, first i whose running sum reaches u * total."""
    ok = ~np.isnan(row)
    mx = row[ok].max()
    p = np.where(ok, np.exp((row.astype(np.float64) - mx) / np.float32(temperature)), 0.0)
    r = u * p.sum()
    c = np.cumsum(p)
    return int(np.searchsorted(c, r, side="left"))


def test_sample_temperature(ops):
    rs = np.random.RandomState(0)
    for vocab, temp in ((5, 1.0), (307, 0.8), (5000, 1.5), (8192, 0.5), (20011, 1.2), (151936, 0.7)):
        logits = (rs.randn(6, vocab) * 2).astype(np.float32)     # from 8192 on the row is summed in chunks
        logits[1, 3 % vocab] = np.nan
        if vocab > 5000:
            logits[2, :vocab // 2] = -np.inf                     # whole chunks without weight
            logits[3, vocab // 3:] = np.nan
            logits[4, :] = -np.inf
            logits[4, vocab - 7] = 0.5                           # one id to draw
        u = rs.rand(6)
        u[0], u[5] = 0.0, 1.0 - 1e-16
        out = torch.empty(6, dtype=torch.int32, device=DEV)
        ops.sample_temperature(torch.tensor(logits).to(DEV), torch.tensor(u).to(DEV), out, temp)
        got = out.tolist()
        for r in range(6):
            want = plain_temperature_draw(logits[r], u[r], temp)
            # rounding of the running sum may move a draw that lands on a boundary by one id
            assert abs(got[r] - want) <= 1 and not np.isnan(logits[r, got[r]]), (vocab, r, got[r], want)
    # the distribution
    logits = torch.log(torch.tensor([[0.6, 0.3, 0.1]])).repeat(4000, 1).to(DEV)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops.sample_temperature(logits, torch.tensor(rs.rand(4000)).to(DEV), out, 1.0)
    freq = np.bincount(out.cpu().numpy(), minlength=3) / 4000
    assert np.abs(freq - [0.6, 0.3, 0.1]).max() < 0.03
    with pytest.raises(ExtensionError, match="temperature"):
        ops.sample_temperature(logits, torch.zeros(4000, dtype=torch.float64, device=DEV), out, 0.0)


def test_sample_chain_on_the_device(ops):
    """The whole chain in one kernel against the plain chain: the same uniform numbers give the same tokens,
    with ties at the top-k boundary, NaN, flat and peaked rows, every combination of the cuts."""
    from plain_qwen3 import PlainMt19937_64, sample_chain
    rs = np.random.RandomState(12)
    for vocab in (50, 1031, 20011):
        rows = np.stack([(rs.randn(vocab) * s).astype(np.float32) for s in (8.0, 3.0, 1.0, 0.05, 3.0, 3.0)])
        rows[4] = np.round(rows[4])                        # ties everywhere
        rows[5, rs.randint(vocab, size=vocab // 5)] = np.nan
        dev = torch.tensor(rows).to(DEV)
        for top_k, temp, top_p, min_p in ((40, 0.7, 0.95, 0.05), (1, 1.0, 1.0, 0.0), (7, 1.3, 1.0, 0.0),
                                          (40, 0.5, 0.5, 0.0), (40, 1.0, 1.0, 0.3), (min(1024, vocab - 1), 0.9, 0.9, 0.01)):
            gens = [PlainMt19937_64(77 + r) for r in range(6)]
            mine = [PlainMt19937_64(77 + r) for r in range(6)]
            for draw in range(8):
                u = torch.tensor([g.uniform(1.0) for g in mine], dtype=torch.float64).to(DEV)
                out = torch.empty(6, dtype=torch.int32, device=DEV)
                ops.sample_chain(dev, u, out, top_k, temp, top_p, min_p)
                want = [sample_chain(rows[r], gens[r], temp, top_k, top_p, min_p) for r in range(6)]
                assert out.tolist() == want, (vocab, top_k, temp, top_p, min_p, draw)
    with pytest.raises(ExtensionError, match="top-k"):
        ops.sample_chain(dev, u, out, 0, 1.0, 1.0, 0.0)


def test_row_exp_sum(ops):
    rs = np.random.RandomState(4)
    for vocab in (3, 307, 151936):
        logits = (rs.randn(3, vocab) * 4).astype(np.float32)
        logits[1, 1] = np.nan
        logits[2, 0] = -np.inf
        out = torch.empty(3, dtype=torch.float64, device=DEV)
        ops.row_exp_sum(torch.tensor(logits).to(DEV), out)
        l = np.where(np.isnan(logits), -np.inf, logits).astype(np.float64)
        want = np.exp(l - l.max(axis=1, keepdims=True)).sum(axis=1)
        assert np.allclose(out.cpu().numpy(), want, rtol=1e-6, atol=0)


def test_sampler_routes_match_the_plain_chain(ops):
    """Every route of the sampler at a vocabulary large enough for the device candidates: top-k on the
    device, candidates with the row's denominator when there is no top-k, and the whole row when a
    flat distribution puts the cut beyond the candidates."""
    from nncpu_b200.sampling import Sampler, SamplerParams
    from plain_qwen3 import PlainMt19937_64, sample_chain
    rs = np.random.RandomState(8)
    vocab = 9001
    rows = np.stack([(rs.randn(vocab) * s).astype(np.float32) for s in (6.0, 3.0, 1.0, 0.01)])
    rows[1, 5] = np.nan
    rows[2, 100:140] = rows[2].max()                      # ties at the top
    dev = torch.tensor(rows).to(DEV)
    for p in (SamplerParams(), SamplerParams(1.2, 7, 1.0, 0.0), SamplerParams(0.9, 2000, 0.99, 0.0),
              SamplerParams(0.8, 0, 0.9, 0.0), SamplerParams(1.0, 0, 1.0, 0.1), SamplerParams(0.6, 0, 0.5, 0.2)):
        sampler = Sampler(p, 21, vocab)
        plain = [PlainMt19937_64(21 + i) for i in range(4)]
        for _ in range(6):
            got = sampler.choose(dev, range(4))
            want = [sample_chain(rows[i], plain[i], p.temperature, p.top_k, p.top_p, p.min_p) for i in range(4)]
            assert got == want, p


def test_kernels_refuse_what_they_cannot_take(ops):
    with pytest.raises(ExtensionError, match="no CPU path"):
        ops.swiglu(torch.zeros(1, 2), torch.zeros(1, 1))
    kp, vp, table, _, _ = scatter_pages(1, 1, 16, [4], torch.float32)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ExtensionError, match="key/value heads"):
        ops.attention(torch.zeros(1, 48, device=DEV), kp, vp, table, z, z, torch.zeros(1, 48, device=DEV), 3, 2, 16,
                      1.0, 0)
