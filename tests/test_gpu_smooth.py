"""The smooth-quant recipe (one scale per row after a per-column smoothing divisor):
triton_rms_norm_and_smooth_quant_forward (linghe/utils/norm.py:557) and
triton_silu_and_smooth_quant_forward (linghe/utils/silu.py:1498) against the oracle's
restatement of upstream's torch_smooth_quant and against golden vectors made by upstream's own
test functions.  Fused-variant tolerances: scales and calibration maxima within 1e-6 relative,
at most 1e-3 of the codes off by one e4m3 step."""

import pytest
import torch

from oracle import oracle as O
from tests.common import (assert_codes_close, assert_rel_close, assert_scales_close, bf16, bits, fp8, golden, record)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _status_clean():
    from linghe_b200 import _lib
    yield
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0


def check_rows(got_q, ref_q, got_s, ref_s, what, pow2, scale_rtol=1e-6):
    """Per-row scales.  With power-of-two scales a last-bit difference in a row maximum can move a
    scale by exactly 2x: rows whose scales agree meet the code rule, the others (at most 1e-3 of the
    rows) must differ by a factor of two and dequantise to the same values within one step."""
    if not pow2:
        assert_scales_close(got_s, ref_s, what + " scale", rtol=scale_rtol)
        assert_codes_close(got_q, ref_q, what + " codes")
        return
    gs, rs = got_s.detach().float().cpu(), ref_s.detach().float().cpu()
    same = gs == rs
    frac = 1.0 - same.float().mean().item()
    record(what, "pow2_scale_diff_frac", frac)
    assert frac <= 1e-3, f"{what}: {frac:.2e} of power-of-two row scales differ"
    if same.any():
        assert_codes_close(got_q[same.to(got_q.device)], ref_q[same], what + " codes")
    if (~same).any():
        ratio = gs[~same] / rs[~same]
        assert bool(((ratio == 2.0) | (ratio == 0.5)).all())
        dg = got_q.detach().float().cpu()[~same] * gs[~same, None]
        dr = ref_q.detach().float().cpu()[~same] * rs[~same, None]
        lim = 0.13 * torch.maximum(dg.abs(), dr.abs()) + 2.0 ** -8 * torch.maximum(gs, rs)[~same, None]
        assert bool(((dg - dr).abs() <= lim).all())


@pytest.mark.parametrize("rs", [0, 1])
def test_golden_smooth(rs):
    from linghe_b200.utils.norm import triton_rms_norm_and_smooth_quant_forward
    from linghe_b200.utils.silu import triton_silu_and_smooth_quant_forward
    G = golden("smooth")
    x, w, sm = bf16(G["norm_x"]).cuda(), bf16(G["norm_w"]).cuda(), torch.from_numpy(G["norm_smooth"]).cuda()
    q, s, maxs, rms = triton_rms_norm_and_smooth_quant_forward(x, w, smooth_scale=sm, calibrate=True, output_rms=True,
                                                               round_scale=bool(rs))
    check_rows(q, fp8(G[f"norm_r{rs}_q"]), s, torch.from_numpy(G[f"norm_r{rs}_s"]), "golden norm smooth", bool(rs))
    assert_scales_close(maxs, torch.from_numpy(G[f"norm_r{rs}_maxs"]), "maxs")
    assert_scales_close(rms, O.rms_recip(x.cpu()), "rms")
    xs, sm2 = bf16(G["silu_x"]).cuda(), torch.from_numpy(G["silu_smooth"]).cuda()
    q, s, maxs = triton_silu_and_smooth_quant_forward(xs, smooth_scale=sm2, calibrate=True, round_scale=bool(rs))
    check_rows(q, fp8(G[f"silu_r{rs}_q"]), s, torch.from_numpy(G[f"silu_r{rs}_s"]), "golden silu smooth", bool(rs))
    assert_scales_close(maxs, torch.from_numpy(G[f"silu_r{rs}_maxs"]), "maxs")


# upstream's own test shapes are (16384, 2048), (8192, 4096), (4096, 8192) (tests/test_norm.py:333-335)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,N", [(4096, 2048), (1000, 4096), (515, 8192), (64, 1536), (3, 8)])
def test_rms_norm_and_smooth_quant(M, N, dtype):
    from linghe_b200.utils.norm import triton_rms_norm_and_smooth_quant_forward as f
    g = torch.Generator().manual_seed(71)
    x = torch.randn((M, N), generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn((N,), generator=g)).to(dtype)
    sm = 1 + 10 * torch.rand((N,), generator=g)
    sm[::17] = 0.0           # the divisor is floored at 1e-30, as upstream's oracle does
    x[:, ::17] = 0           # ... and the columns it hits are zero, so that the row maxima stay finite
    for rs in (False, True):
        rq, rsc, rmaxs, rr = O.rms_norm_and_smooth_quant_forward(x, w, sm, 1e-6, rs)
        q, s, maxs, rms = f(x.cuda(), w.cuda(), smooth_scale=sm.cuda(), calibrate=True, output_rms=True, round_scale=rs)
        assert q.shape == (M, N) and s.shape == (M,) and maxs.shape == (N,) and rms.shape == (M,)
        check_rows(q, rq, s, rsc, "norm smooth", rs)
        assert torch.allclose(maxs.cpu(), rmaxs, rtol=1e-6, atol=0)
        assert_scales_close(rms, rr, "rms")
    # without calibration / rms: None in their places, outputs written into the buffers passed
    out = torch.empty((M, N), device="cuda", dtype=torch.float8_e4m3fn)
    sc = torch.empty((M,), device="cuda")
    r = f(x.cuda(), w.cuda(), smooth_scale=sm.cuda(), out=out, scale=sc)
    assert r[0] is out and r[1] is sc and r[2] is None and r[3] is None
    assert torch.equal(bits(out), bits(f(x.cuda(), w.cuda(), smooth_scale=sm.cuda())[0]))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,n", [(4096, 2048), (1000, 1408), (130, 8192), (16, 1536), (5, 8)])
def test_silu_and_smooth_quant(M, n, dtype):
    from linghe_b200.utils.silu import triton_silu_and_smooth_quant_forward as f
    g = torch.Generator().manual_seed(72)
    x = torch.randn((M, 2 * n), generator=g).to(dtype)
    sm = 1 + torch.rand((n,), generator=g)
    for rs in (False, True):
        rq, rsc, rmaxs = O.silu_and_smooth_quant_forward(x, sm, rs)
        q, s, maxs = f(x.cuda(), smooth_scale=sm.cuda(), calibrate=True, round_scale=rs)
        assert q.shape == (M, n) and s.shape == (M,) and maxs.shape == (n,)
        check_rows(q, rq, s, rsc, "silu smooth", rs)
        assert torch.allclose(maxs.cpu(), rmaxs, rtol=1e-6, atol=1e-30)
    r = f(x.cuda(), smooth_scale=sm.cuda())
    assert r[2] is None


def test_smooth_quant_argument_errors():
    from linghe_b200.utils.norm import triton_rms_norm_and_smooth_quant_forward as fn
    from linghe_b200.utils.silu import triton_silu_and_smooth_quant_forward as fs
    x = torch.zeros((16, 16384), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        fn(x, torch.ones(16384, device="cuda", dtype=torch.bfloat16), smooth_scale=torch.ones(16384, device="cuda"))
    with pytest.raises(AssertionError):
        fs(x[:, :64].contiguous(), smooth_scale=None)
    # empty input: nothing launched, shapes kept
    e = torch.zeros((0, 256), device="cuda", dtype=torch.bfloat16)
    q, s, maxs = fs(e, smooth_scale=torch.ones(128, device="cuda"), calibrate=True)
    assert q.shape == (0, 128) and s.shape == (0,) and float(maxs.abs().max()) == 0.0


# upstream's test: 32 experts with 512-1536 rows each (multiples of 16), N = 4096, weights randn,
# smooth scales 1 + 10 * rand (tests/test_silu.py:482-527); here also empty experts, ragged counts,
# int64 counts and the `reverse` form
@pytest.mark.parametrize("dtype,wdt", [(torch.bfloat16, torch.float32), (torch.float16, torch.float16),
                                       (torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("counts,n,it", [([512, 0, 1040, 16, 0, 333], 2048, torch.int32), ([7], 8, torch.int64),
                                         ([128] * 64, 512, torch.int64), ([0, 0, 5], 1408, torch.int32)])
def test_batch_weighted_silu_and_smooth_quant(counts, n, it, dtype, wdt):
    from linghe_b200.utils.silu import triton_batch_weighted_silu_and_smooth_quant_forward as f
    g = torch.Generator().manual_seed(73)
    R, E = sum(counts), len(counts)
    x = torch.randn((R, 2 * n), generator=g).to(dtype)
    w = torch.randn((R, 1), generator=g).to(wdt)
    sm = 1 + 10 * torch.rand((E, n), generator=g)
    cd = torch.tensor(counts, dtype=it, device="cuda")
    for rs, rev in ((False, False), (True, False), (True, True)):
        rq, rsc, rmaxs = O.batch_weighted_silu_and_smooth_quant_forward(x, w, counts, sm, rs, rev)
        q, s, maxs = f(x.cuda(), w.cuda(), cd, smooth_scale=sm.cuda(), splits=counts, round_scale=rs, reverse=rev,
                       calibrate=True)
        assert q.shape == (R, n) and s.shape == (R,) and maxs.shape == (E, n)
        check_rows(q, rq, s, rsc, "batch smooth", rs)
        assert torch.allclose(maxs.cpu(), rmaxs, rtol=1e-6, atol=1e-30)
    r = f(x.cuda(), w.cuda(), cd, smooth_scale=sm.cuda())
    assert r[2] is None


def test_batch_smooth_quant_empty():
    from linghe_b200.utils.silu import triton_batch_weighted_silu_and_smooth_quant_forward as f
    x = torch.zeros((0, 512), device="cuda", dtype=torch.bfloat16)
    w = torch.zeros((0, 1), device="cuda")
    c = torch.zeros((4,), device="cuda", dtype=torch.int32)
    q, s, maxs = f(x, w, c, smooth_scale=torch.ones((4, 256), device="cuda"))
    assert q.shape == (0, 256) and s.shape == (0,) and maxs.shape == (4, 256) and float(maxs.abs().max()) == 0.0


@pytest.mark.parametrize("rs,rev", [(0, 0), (1, 0), (1, 1)])
def test_golden_batch_smooth(rs, rev):
    from linghe_b200.utils.silu import triton_batch_weighted_silu_and_smooth_quant_forward as f
    G = golden("smooth")
    x, w, sm = bf16(G["batch_x"]).cuda(), torch.from_numpy(G["batch_w"]).cuda(), torch.from_numpy(G["batch_smooth"]).cuda()
    counts = torch.from_numpy(G["batch_counts"]).cuda()
    q, s, _ = f(x, w, counts, smooth_scale=sm, round_scale=bool(rs), reverse=bool(rev))
    check_rows(q, fp8(G[f"batch_r{rs}v{rev}_q"]), s, torch.from_numpy(G[f"batch_r{rs}v{rev}_s"]), "golden batch smooth", bool(rs))


def check_cols(got_qt, ref_qt, got_st, ref_st, what, pow2):
    """transposed copy: codes [C, M] with one scale per row of the transposed matrix"""
    check_rows(got_qt, ref_qt, got_st, ref_st, what, pow2)


# upstream's test: M = N = 4096, smooth scales 1 + rand, reverse=True, round_scale=True
# (tests/test_silu.py:332-377)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,n", [(2048, 2048), (1000, 1408), (130, 4096), (64, 8), (4096, 512)])
def test_silu_and_smooth_quant_backward(M, n, dtype):
    from linghe_b200.utils.silu import triton_silu_and_smooth_quant_backward as f
    gen = torch.Generator().manual_seed(74)
    x = torch.randn((M, 2 * n), generator=gen).to(dtype)
    g = (0.1 * torch.randn((M, n), generator=gen)).to(dtype)
    sm = 1 + torch.rand((2 * n,), generator=gen)
    tsm = 1 + torch.rand((M,), generator=gen)
    for rs, rev in ((True, True), (True, False), (False, True)):
        rq, rsc, rqt, rst = O.silu_and_smooth_quant_backward(g, x, sm, tsm, rs, rev)
        q, s, qt, st = f(g.cuda(), x.cuda(), smooth_scale=sm.cuda(), transpose_smooth_scale=tsm.cuda(), reverse=rev,
                         round_scale=rs)
        assert q.shape == (M, 2 * n) and s.shape == (M,) and qt.shape == (2 * n, M) and st.shape == (2 * n,)
        check_rows(q, rq, s, rsc, "smooth bwd dx", rs)
        check_cols(qt, rqt, st, rst, "smooth bwd dxT", rs)


@pytest.mark.parametrize("rs,rev", [(1, 1), (1, 0), (0, 1)])
def test_golden_smooth_backward(rs, rev):
    from linghe_b200.utils.silu import triton_silu_and_smooth_quant_backward as f
    G = golden("smooth")
    g, x = bf16(G["bwd_g"]).cuda(), bf16(G["bwd_x"]).cuda()
    sm, tsm = torch.from_numpy(G["bwd_smooth"]).cuda(), torch.from_numpy(G["bwd_tsmooth"]).cuda()
    q, s, qt, st = f(g, x, smooth_scale=sm, transpose_smooth_scale=tsm, reverse=bool(rev), round_scale=bool(rs))
    tag = f"bwd_r{rs}v{rev}"
    check_rows(q, fp8(G[tag + "_q"]), s, torch.from_numpy(G[tag + "_s"]), "golden smooth bwd dx", bool(rs))
    check_cols(qt, fp8(G[tag + "_qt"]), st, torch.from_numpy(G[tag + "_st"]), "golden smooth bwd dxT", bool(rs))


def _check_batch_bwd(got, ref, counts, N, rs, what):
    q, s, dw, qt, st = got
    rq, rsc, rdw, rqt, rst = ref
    check_rows(q, rq, s, rsc, what + " dx", rs)
    # dw is a sum with cancellation: bound the error against the largest entry (a handful of rows
    # cannot meet an element-wise relative bound)
    err = (dw.float().cpu().reshape(-1) - rdw.reshape(-1)).abs().max().item()
    assert err <= (1e-2 if dw.dtype != torch.float32 else 1e-4) * max(rdw.abs().max().item(), 1e-30), f"{what} dw: {err:.3e}"
    assert qt.numel() == rqt.numel() and tuple(st.shape) == tuple(rst.shape)
    off = 0
    for e, c in enumerate(counts):         # expert blocks [N, pad32(c)] of the flat transposed buffer
        cp = (c + 31) // 32 * 32
        if cp == 0:
            continue
        ge = qt[off:off + N * cp].view(N, cp)
        re_ = rqt[off:off + N * cp].view(N, cp)
        # A column maximum over a handful of rows can sit on an element whose factor 1 + x1 (1 - sigmoid)
        # cancels, which amplifies the 4e-7 error of the hardware sigmoid: such blocks get 2e-5
        check_rows(ge, re_, st[e], rst[e], f"{what} dxT expert {e}", rs, scale_rtol=1e-6 if c >= 32 else 2e-5)
        if cp > c:
            assert int(bits(ge[:, c:]).max()) == 0, "padding rows must be zero codes"
        off += N * cp


# upstream's test: 32 experts of 512-1536 rows (multiples of 16), N = 4096, smooth scales 1 + 10 rand,
# reverse=False, round_scale=True (tests/test_silu.py:482-557)
@pytest.mark.parametrize("dtype,wdt", [(torch.bfloat16, torch.float32), (torch.float16, torch.float16),
                                       (torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("counts,n,it", [([512, 0, 1040, 16, 0, 333], 1024, torch.int32), ([7], 8, torch.int64),
                                         ([96] * 24, 512, torch.int64), ([0, 0, 5], 704, torch.int32)])
def test_batch_weighted_silu_and_smooth_quant_backward(counts, n, it, dtype, wdt):
    from linghe_b200.utils.silu import triton_batch_weighted_silu_and_smooth_quant_backward as f
    gen = torch.Generator().manual_seed(75)
    R, E, N = sum(counts), len(counts), 2 * n
    x = torch.randn((R, N), generator=gen).to(dtype)
    g = (0.1 * torch.randn((R, n), generator=gen)).to(dtype)
    w = torch.randn((R, 1), generator=gen).to(wdt)
    sm = 1 + 10 * torch.rand((E, N), generator=gen)
    tsm = 1 + 10 * torch.rand((R,), generator=gen)
    cd = torch.tensor(counts, dtype=it, device="cuda")
    for rs, rev in ((True, False), (True, True), (False, False)):
        ref = O.batch_weighted_silu_and_smooth_quant_backward(g, x, w, counts, sm, tsm, rs, rev)
        got = f(g.cuda(), x.cuda(), w.cuda(), cd, smooth_scale=sm.cuda(), transpose_smooth_scale=tsm.cuda(), splits=counts,
                reverse=rev, round_scale=rs)
        assert got[0].shape == (R, N) and got[1].shape == (R,) and got[2].shape == w.shape and got[2].dtype == wdt
        assert got[4].shape == (E, N)
        _check_batch_bwd(got, ref, counts, N, rs, "batch smooth bwd")


@pytest.mark.parametrize("rs,rev", [(1, 0), (1, 1), (0, 0)])
def test_golden_batch_smooth_backward(rs, rev):
    from linghe_b200.utils.silu import triton_batch_weighted_silu_and_smooth_quant_backward as f
    G = golden("smooth")
    g, x, w = bf16(G["bbwd_g"]).cuda(), bf16(G["bbwd_x"]).cuda(), torch.from_numpy(G["bbwd_w"]).cuda()
    sm, tsm = torch.from_numpy(G["bbwd_smooth"]).cuda(), torch.from_numpy(G["bbwd_tsmooth"]).cuda()
    counts = [int(c) for c in G["bbwd_counts"]]
    got = f(g, x, w, torch.tensor(counts, device="cuda"), smooth_scale=sm, transpose_smooth_scale=tsm, splits=counts,
            reverse=bool(rev), round_scale=bool(rs))
    tag = f"bbwd_r{rs}v{rev}"
    ref = (fp8(G[tag + "_q"]), torch.from_numpy(G[tag + "_s"]), torch.from_numpy(G["bbwd_dw"]), fp8(G[tag + "_qt"]),
           torch.from_numpy(G[tag + "_st"]).view(len(counts), x.shape[1]))
    _check_batch_bwd(got, ref, counts, x.shape[1], bool(rs), "golden batch smooth bwd")


def test_batch_smooth_backward_empty():
    from linghe_b200.utils.silu import triton_batch_weighted_silu_and_smooth_quant_backward as f
    x = torch.zeros((0, 512), device="cuda", dtype=torch.bfloat16)
    g = torch.zeros((0, 256), device="cuda", dtype=torch.bfloat16)
    w = torch.zeros((0, 1), device="cuda")
    c = torch.zeros((4,), device="cuda", dtype=torch.int32)
    dx, s, dw, qt, st = f(g, x, w, c, smooth_scale=torch.ones((4, 512), device="cuda"),
                          transpose_smooth_scale=torch.ones((0,), device="cuda"), splits=[0, 0, 0, 0], round_scale=True)
    assert dx.shape == (0, 512) and qt.numel() == 0 and st.shape == (4, 512) and float(st.abs().max()) == 0.0
