"""Index arithmetic of ``csrc/kernels/gpt_ops.cu`` restated on the host.

The row-normalisation backward walks its rows in groups of R with NV column pieces
per thread (shape chosen per hidden size), every CTA leaves one partial row of the
weight / bias gradients, and a second kernel sums the partial rows.  The bias +
activation backward tiles columns over ``blockIdx.x`` and rows over ``blockIdx.y`` x 8
lanes.  Here the same loops run in numpy, thread by thread and CTA by CTA, with the
launch shapes the host code picks; the results must equal autograd, which checks the
coverage (every element exactly once), the predicates at the ragged ends and the
offsets of the partial rows.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as TF


def norm_bwd_shape(H):                      # norm_bwd_shape() of gpt_ops.cu
    nvec = H // 8
    up32 = lambda v: (v + 31) // 32 * 32    # noqa: E731
    if nvec <= 640:
        return 1, 4, up32(nvec)
    if nvec <= 1024:
        return 2, 2, up32((nvec + 1) // 2)
    return 4, 1, up32((nvec + 3) // 4)


def norm_bwd_parts(rows, H):                # ft_norm_bwd_parts()
    r = norm_bwd_shape(H)[1]
    groups = (rows + r - 1) // r
    return max(1, min(groups, 148))


def emulate_norm_bwd(x, w, dy, mean, rstd, layernorm):
    rows, H = x.shape
    NV, R, threads = norm_bwd_shape(H)
    assert NV * threads * 8 >= H and threads <= 640 and threads % 32 == 0
    parts = norm_bwd_parts(rows, H)
    nvec = H // 8
    dx = np.full_like(x, np.nan)
    dw_part = np.full((parts, H), np.nan, np.float64)
    db_part = np.full((parts, H), np.nan, np.float64)
    groups = (rows + R - 1) // R
    tid = np.arange(threads)
    for cta in range(parts):
        dw_acc = np.zeros((NV, threads, 8))
        db_acc = np.zeros((NV, threads, 8))
        for g in range(cta, groups, parts):
            for r in range(R):
                row = g * R + r
                ok = row < rows
                s1 = s2 = 0.0
                cache = []
                for j in range(NV):
                    i = tid + j * threads                      # 128-bit piece owned by each thread
                    live = ok & (i < nvec)
                    cols = (i[:, None] * 8 + np.arange(8)[None, :])
                    cols = np.where(live[:, None], cols, 0)
                    xv = np.where(live[:, None], x[row if ok else 0][cols], 0.0)
                    gv = np.where(live[:, None], dy[row if ok else 0][cols], 0.0)
                    wv = np.where((i < nvec)[:, None], w[np.where((i < nvec)[:, None], cols, 0)], 0.0)
                    m = mean[row] if (ok and layernorm) else 0.0
                    rs = rstd[row] if ok else 0.0
                    xh = (xv - m) * rs
                    gw = gv * wv
                    s1 += gw.sum()
                    s2 += (gw * xh).sum()
                    dw_acc[j] += gv * xh
                    db_acc[j] += gv
                    cache.append((live, cols, xh, gw, rs))
                if ok:
                    c1 = s1 / H if layernorm else 0.0
                    c2 = s2 / H
                    for live, cols, xh, gw, rs in cache:
                        out = rs * (gw - c1 - xh * c2)
                        sel = np.nonzero(live)[0]
                        dx[row][cols[sel].reshape(-1)] = out[sel].reshape(-1)
        for j in range(NV):
            i = tid + j * threads
            sel = np.nonzero(i < nvec)[0]
            cols = (i[sel][:, None] * 8 + np.arange(8)[None, :]).reshape(-1)
            dw_part[cta][cols] = dw_acc[j][sel].reshape(-1)
            db_part[cta][cols] = db_acc[j][sel].reshape(-1)
    assert not np.isnan(dx).any() and not np.isnan(dw_part).any()
    return dx, dw_part.sum(0), db_part.sum(0)


@pytest.mark.parametrize("layernorm", [True, False])
@pytest.mark.parametrize("rows,H", [(5, 256), (9, 1024), (3, 5120), (2, 8192), (2, 12288), (150, 64), (601, 40)])
def test_row_norm_backward_walk(rows, H, layernorm):
    torch.manual_seed(rows + H)
    x = torch.randn(rows, H, dtype=torch.float64, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, dtype=torch.float64)).requires_grad_()
    b = torch.zeros(H, dtype=torch.float64, requires_grad=True)
    dy = torch.randn(rows, H, dtype=torch.float64)
    eps = 1e-5
    if layernorm:
        y = TF.layer_norm(x, (H,), w, b, eps)
        mean = x.mean(-1)
        rstd = torch.rsqrt(x.var(-1, unbiased=False) + eps)
        gx, gw, gb = torch.autograd.grad(y, (x, w, b), dy)
    else:
        rstd = torch.rsqrt(x.pow(2).mean(-1) + eps)
        mean = torch.zeros(rows, dtype=torch.float64)
        y = x * rstd[:, None] * w
        gx, gw = torch.autograd.grad(y, (x, w), dy)
        gb = dy.sum(0)
    dx, dw, db = emulate_norm_bwd(x.detach().numpy(), w.detach().numpy(), dy.numpy(), mean.detach().numpy(),
                                  rstd.detach().numpy(), layernorm)
    assert np.allclose(dx, gx.numpy(), atol=1e-9)
    assert np.allclose(dw, gw.numpy(), atol=1e-9)
    assert np.allclose(db, gb.numpy(), atol=1e-9)


def bias_act_bwd_parts(rows, N):            # ft_bias_act_bwd_parts()
    gx = (N + 255) // 256
    parts = (148 * 8 + gx - 1) // gx
    return max(1, min(parts, (rows + 7) // 8, 64))


@pytest.mark.parametrize("rows,N", [(3, 8), (100, 264), (513, 1024), (64, 20480), (7, 2048)])
def test_bias_backward_tiling(rows, N):
    """Column sums through the CTA tiling: 32 column groups x 8 row lanes per CTA."""
    rng = np.random.default_rng(rows + N)
    dy = rng.standard_normal((rows, N))
    vec = N // 8
    parts = bias_act_bwd_parts(rows, N)
    gx = (N + 255) // 256
    db_part = np.full((parts, N), np.nan)
    touched = np.zeros((rows, N), np.int32)
    for by in range(parts):
        for bx in range(gx):
            red = np.zeros((8, 256))
            for t in range(256):
                cg, rl = t & 31, t >> 5
                c = bx * 32 + cg
                if c < vec:
                    for r in range(by * 8 + rl, rows, parts * 8):
                        red[rl, cg * 8:cg * 8 + 8] += dy[r, c * 8:c * 8 + 8]
                        touched[r, c * 8:c * 8 + 8] += 1
            for t in range(256):
                col = bx * 256 + t
                if col < N:
                    db_part[by, col] = red[:, t].sum()
    assert (touched == 1).all()
    assert not np.isnan(db_part).any()
    assert np.allclose(db_part.sum(0), dy.sum(0), atol=1e-9)


@pytest.mark.parametrize("M,F", [(256, 128), (520, 384), (4096, 11008), (32768, 13824), (8192, 28672)])
def test_swiglu_gemm_tile_mapping(M, F):
    """Tile walk of ``gemm_pair_swiglu_kernel`` (csrc/kernels/gemm2_swiglu.cuh): per output
    tile the leader CTA stages gate rows and its partner the up rows of the SAME output
    columns; accumulator columns [0,128) / [128,256) of a row therefore pair up element by
    element.  Every output element must be produced exactly once."""
    assert F % 128 == 0
    mt, nt = (M + 255) // 256, F // 128
    pairs = 74
    out_cols = np.zeros(F, np.int64)
    out_rows = np.zeros(M, np.int64)
    for pair in range(min(pairs, mt * nt)):
        for t in range(pair, mt * nt, pairs):
            mb, nb = t // nt, t % nt                      # any bijection works for the check
            w_rows = {cta: nb * 128 + cta * F for cta in (0, 1)}
            assert 0 <= w_rows[0] and w_rows[0] + 128 <= F            # gate block
            assert F <= w_rows[1] and w_rows[1] + 128 <= 2 * F        # up block of the same columns
            assert w_rows[1] - F == w_rows[0]
            for c in range(4):                            # epilogue chunks of 32 columns
                col0 = nb * 128 + c * 32
                assert col0 + 32 <= F
                if mb == 0:
                    out_cols[col0:col0 + 32] += 1
            if nb == 0:
                for cta in (0, 1):
                    lo = mb * 256 + cta * 128
                    out_rows[lo:min(lo + 128, M)] += 1
    assert (out_cols == 1).all() and (out_rows == 1).all()
