"""Parity of the CUDA path (called through the Python mirror of the upstream interface,
which goes straight to the C ABI) against the CPU oracle and the golden vectors.

Rules: pure quantisers are bit-exact in codes and scales; fused variants keep scales
within 1e-6 relative and at most 0.1 % of codes one e4m3 ulp off; bf16 gradients within
1e-2 relative."""

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.common import (SILU_DENORMAL_ATOL, golden, bf16, fp8, bits, assert_bits_equal, assert_f32_equal, assert_codes_close,
                          assert_scales_close, assert_rel_close, assert_fused_pow2)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _status_clean():
    from linghe_b200 import _lib
    yield
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0, "a kernel gave up on a bounded wait"


def _cuda(t):
    return t.to(DEV)


def randn_bf16(shape, seed, power=1, coef=1.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    if power != 1:
        x = x ** power
    return (x * coef).to(torch.bfloat16)


def check_exact(got, ref, names):
    for g, r, nm in zip(got, ref, names):
        if r.dtype == torch.float8_e4m3fn:
            assert_bits_equal(g, r, nm)
        else:
            assert_f32_equal(g, r, nm)


def check_fused(got_q, ref_q, got_s, ref_s, what, round_scale=False):
    """codes / scales of a fused variant.  With power-of-two scales a last-bit difference
    in the block maximum can move a scale by a factor of two: blocks whose scales agree meet
    the code rule, the others (at most 1e-3 of them) are checked through their dequantised
    values (tests/common.py: assert_fused_pow2)."""
    if not round_scale:
        assert_scales_close(got_s, ref_s, what + " scale")
        assert_codes_close(got_q, ref_q, what + " codes")
    else:
        assert_fused_pow2(got_q, ref_q, got_s, ref_s, what)


# ------------------------------------------------------------------------------------
# e4m3 conversion: every bf16 value with |x| <= 448 through a unit scale
# ------------------------------------------------------------------------------------
def test_e4m3_cast_exhaustive():
    from linghe_b200.quant.group import triton_group_quant
    allb = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    ok = torch.isfinite(allb.float()) & (allb.float().abs() <= 448)
    vals = allb[ok]
    n = vals.numel()
    rows = (n + 126) // 127
    x = torch.zeros(rows * 127, dtype=torch.bfloat16)
    x[:n] = vals
    x = torch.cat([x.view(rows, 127), torch.full((rows, 1), 448.0, dtype=torch.bfloat16)], 1).contiguous()
    q, s = triton_group_quant(_cuda(x))
    rq, rs = O.group_quant(x)
    assert_f32_equal(s, rs, "scale")
    assert_bits_equal(q, rq, "codes")
    assert float(s.min()) == 1.0 and float(s.max()) == 1.0


# ------------------------------------------------------------------------------------
# pure quantisers: bit-exact
# ------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["n1", "n3"])
@pytest.mark.parametrize("rs", [0, 1])
def test_golden_quant(tag, rs):
    from linghe_b200.quant.block import triton_blockwise_quant
    from linghe_b200.quant.group import triton_group_quant
    G = golden("quant")
    x = _cuda(bf16(G[f"x_{tag}"]))
    q, s = triton_group_quant(x, round_scale=bool(rs))
    assert_bits_equal(q, fp8(G[f"group_{tag}_r{rs}_q"]), "group q")
    assert_f32_equal(s, torch.from_numpy(G[f"group_{tag}_r{rs}_s"]), "group s")
    out = triton_blockwise_quant(x, round_scale=bool(rs))
    p = f"blockwise_{tag}_r{rs}_"
    check_exact(out, (fp8(G[p + "q"]), torch.from_numpy(G[p + "s"]), fp8(G[p + "qt"]), torch.from_numpy(G[p + "st"])),
                ("q", "s", "qt", "st"))


def test_golden_quant_f32_block_batch():
    from linghe_b200.quant.block import triton_blockwise_quant, triton_block_quant, triton_batch_blockwise_quant
    G = golden("quant")
    out = triton_blockwise_quant(_cuda(torch.from_numpy(G["x_f32"])))
    p = "blockwise_f32_r0_"
    check_exact(out, (fp8(G[p + "q"]), torch.from_numpy(G[p + "s"]), fp8(G[p + "qt"]), torch.from_numpy(G[p + "st"])),
                ("q", "s", "qt", "st"))
    for rs in (0, 1):
        q, s = triton_block_quant(_cuda(bf16(G["w"])), round_scale=bool(rs))
        assert_bits_equal(q, fp8(G[f"block_r{rs}_q"]), "block q")
        assert_f32_equal(s, torch.from_numpy(G[f"block_r{rs}_s"]), "block s")
        counts = G["xb_counts"].tolist()
        for dt in (torch.int32, torch.int64):
            out = triton_batch_blockwise_quant(_cuda(bf16(G["xb"])), torch.tensor(counts, dtype=dt, device=DEV),
                                               counts, round_scale=bool(rs))
            p = f"batchq_r{rs}_"
            check_exact(out, (fp8(G[p + "q"]), torch.from_numpy(G[p + "s"]), fp8(G[p + "qt"]),
                              torch.from_numpy(G[p + "st"])), ("q", "s", "qt", "st"))


@pytest.mark.parametrize("shape,power,dtype", [
    ((256, 512), 3, torch.bfloat16), ((144, 384), 1, torch.bfloat16), ((4096, 2048), 3, torch.bfloat16),
    ((1040, 1536), 2, torch.float16), ((528, 640), 3, torch.float32), ((16, 128), 1, torch.bfloat16),
])
@pytest.mark.parametrize("rs", [False, True])
def test_blockwise_quant(shape, power, dtype, rs):
    from linghe_b200.quant.block import triton_blockwise_quant
    x = randn_bf16(shape, 1, power).to(dtype)
    if dtype == torch.float32:
        x = x * 1.2345
    x[3, :128] = 0
    ref = O.blockwise_quant(x, rs)
    xd = _cuda(x)
    out = triton_blockwise_quant(xd, round_scale=rs, output_mode=2)
    check_exact(out, ref, ("q", "s", "qt", "st"))
    o0 = triton_blockwise_quant(xd, round_scale=rs, output_mode=0)
    check_exact(o0[:2], ref[:2], ("q", "s"))
    o1 = triton_blockwise_quant(xd, round_scale=rs, output_mode=1)
    check_exact(o1[2:], ref[2:], ("qt", "st"))


def test_blockwise_quant_extremes():
    """tiny, huge and signed-zero inputs: scale floor, division slow path, sign of zero"""
    from linghe_b200.quant.block import triton_blockwise_quant
    g = torch.Generator().manual_seed(5)
    x = torch.randn((256, 256), generator=g)
    x[:128, :128] *= 1e-35          # below the scale floor
    x[:128, 128:] *= 1e30
    x[128:, :128] *= 3e-29          # scale just above the floor
    x[200] = 0
    x[201] = -0.0
    x[128:, 130] = -0.0
    ref = O.blockwise_quant(x, False)
    out = triton_blockwise_quant(_cuda(x))
    check_exact(out, ref, ("q", "s", "qt", "st"))
    xb = x.to(torch.bfloat16)
    check_exact(triton_blockwise_quant(_cuda(xb)), O.blockwise_quant(xb, False), ("q", "s", "qt", "st"))


@pytest.mark.parametrize("M,N", [(2049, 1024), (16, 128), (300, 2048), (3, 4224), (5, 6144), (1, 128)])
def test_group_quant(M, N):
    from linghe_b200.quant.group import triton_group_quant
    x = randn_bf16((M, N), 2, 3)
    for rs in (False, True):
        q, s = triton_group_quant(_cuda(x), round_scale=rs)
        rq, rsx = O.group_quant(x, rs)
        assert_bits_equal(q, rq, "q")
        assert_f32_equal(s, rsx, "s")
    # an input that is 16- but not 32-byte aligned takes the 128-bit loads
    buf = torch.empty(M * N + 8, dtype=torch.bfloat16, device="cuda")
    xo = buf[8:].view(M, N)
    xo.copy_(x)
    assert xo.data_ptr() % 32 == 16
    q, s = triton_group_quant(xo)
    rq, rsx = O.group_quant(x, False)
    assert_bits_equal(q, rq, "q (offset input)")
    assert_f32_equal(s, rsx, "s (offset input)")


def test_block_quant():
    from linghe_b200.quant.block import triton_block_quant
    x = randn_bf16((512, 768), 3, 3)
    for rs in (False, True):
        q, s = triton_block_quant(_cuda(x), round_scale=rs)
        rq, rsx = O.block_quant(x, rs)
        assert_bits_equal(q, rq, "q")
        assert_f32_equal(s, rsx, "s")


@pytest.mark.parametrize("counts", [[5, 0, 130, 128, 1, 257, 0, 64], [16] * 40, [0, 0, 384], [1000]])
def test_batch_blockwise_quant(counts):
    from linghe_b200.quant.block import triton_batch_blockwise_quant
    R = sum(counts)
    x = randn_bf16((R, 256), 4)
    ref = O.batch_blockwise_quant(x, counts, True)
    out = triton_batch_blockwise_quant(_cuda(x), torch.tensor(counts, dtype=torch.int64, device=DEV), counts,
                                       round_scale=True)
    check_exact(out, ref, ("q", "s", "qt", "st"))


# ------------------------------------------------------------------------------------
# RMSNorm
# ------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["n1", "n2"])
@pytest.mark.parametrize("rs", [0, 1])
def test_golden_rms_block_quant(tag, rs):
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward
    G = golden("norm")
    x, g = _cuda(bf16(G[f"x_{tag}"])), _cuda(bf16(G[f"gamma_{tag}"]))
    p = f"rmsq_{tag}_r{rs}_"
    q, s, r, qt, st = triton_rms_norm_and_block_quant_forward(x, g, round_scale=bool(rs), output_mode=2)
    assert_scales_close(r, torch.from_numpy(G[p + "r"]), "rms")
    check_fused(q, fp8(G[p + "q"]), s, torch.from_numpy(G[p + "s"]), "row", bool(rs))
    check_fused(qt, fp8(G[p + "qt"]), st, torch.from_numpy(G[p + "st"]), "col", bool(rs))


# (4200, 8192) is past the size where wide rows switch to the persistent-walk kernel; (600, 5120)
# fills the ring kernel's slab poorly and takes the one-CTA-per-row kernel at any size
@pytest.mark.parametrize("M,n", [(1000, 1536), (512, 2048), (384, 4096), (130, 8192), (64, 128), (2048, 1664),
                                 (4200, 8192), (600, 5120)])
def test_rms_block_quant_modes(M, n):
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward
    x = randn_bf16((M, n), 7, 2)
    g = randn_bf16((n,), 8)
    rq, rs, rr, rqt, rst = O.rms_norm_and_block_quant_forward(x, g, 1e-6, False)
    xd, gd = _cuda(x), _cuda(g)
    q, s, r, _, _ = triton_rms_norm_and_block_quant_forward(xd, gd, output_mode=0)
    assert_scales_close(r, rr, "rms")
    check_fused(q, rq, s, rs, "mode0 row")
    o = triton_rms_norm_and_block_quant_forward(xd, gd, rms=r, output_mode=1)
    assert o[0] is None and o[1] is None and o[2] is r
    check_fused(o[3], rqt, o[4], rst, "mode1 col")
    q, s, r2, qt, st = triton_rms_norm_and_block_quant_forward(xd, gd, output_mode=2)
    check_fused(q, rq, s, rs, "mode2 row")
    check_fused(qt, rqt, st, rst, "mode2 col")
    assert_scales_close(r2, rr, "rms2")
    # round_scale path
    rq, rs, _, rqt, rst = O.rms_norm_and_block_quant_forward(x, g, 1e-6, True)
    q, s, _, qt, st = triton_rms_norm_and_block_quant_forward(xd, gd, round_scale=True, output_mode=2)
    check_fused(q, rq, s, rs, "pow2 row", True)
    check_fused(qt, rqt, st, rst, "pow2 col", True)


# n >= 1536 takes the streaming backward kernel (one span per thread up to 2048 columns, two above;
# 2304 and 5120 leave the second span partly empty), narrower rows the ring kernel
@pytest.mark.parametrize("M,n", [(1000, 1536), (512, 2048), (4096, 4096), (130, 8192), (96, 256), (778, 2304),
                                 (2000, 5120)])
def test_rms_fwd_bwd(M, n):
    from linghe_b200.utils.norm import triton_rms_norm_forward, triton_rms_norm_backward
    x = randn_bf16((M, n), 11)
    g = (1 + 0.1 * torch.randn(n, generator=torch.Generator().manual_seed(12))).to(torch.bfloat16)
    dy = randn_bf16((M, n), 13, 1, 0.01)
    xd, gd, dyd = _cuda(x), _cuda(g), _cuda(dy)
    y, r = triton_rms_norm_forward(xd, gd)
    assert_rel_close(y, O.rms_norm_forward(x, g), "y", 1e-2)
    assert_scales_close(r, O.rms_recip(x), "rms")
    y2, r2 = triton_rms_norm_forward(xd, gd, rms=r)
    assert r2 is r and torch.equal(y2, y)
    rdx, rdw = O.rms_norm_backward(x, g, dy)
    for rms in (r, None):
        dx, dw = triton_rms_norm_backward(dyd, xd, gd, rms=rms)
        assert dw.dtype == torch.float32 and tuple(dw.shape) == (n,)
        assert_rel_close(dx, rdx, "dx", 1e-2)
        assert_rel_close(dw, rdw, "dgamma", 1e-3, 1e-5)
    # 3-D input as the facade passes it
    dx3, dw3 = triton_rms_norm_backward(dyd.view(2, M // 2, n), xd.view(2, M // 2, n), gd)
    assert dx3.shape == (2, M // 2, n) and torch.equal(dx3.view(M, n), dx)


# the two backward kernels at the same width (the crossover is a tuning value): both against the oracle,
# dx of the two identical up to the last bf16 bit of a few elements (different summation order of the row sums)
@pytest.mark.parametrize("M,n", [(1000, 1536), (777, 2048), (640, 1024), (2000, 1792)])
def test_rms_bwd_ring_and_streaming_kernels(M, n):
    from linghe_b200.utils.norm import triton_rms_norm_backward
    x = randn_bf16((M, n), 21)
    g = (1 + 0.1 * torch.randn(n, generator=torch.Generator().manual_seed(22))).to(torch.bfloat16)
    dy = randn_bf16((M, n), 23, 1, 0.01)
    xd, gd, dyd = _cuda(x), _cuda(g), _cuda(dy)
    rdx, rdw = O.rms_norm_backward(x, g, dy)
    got = {}
    for name, min_n in (("streaming", 1), ("ring", 1 << 30)):
        with tuning("rmsnorm_bwd_stream_min_n", min_n):
            dx, dw = triton_rms_norm_backward(dyd, xd, gd)
            torch.cuda.synchronize()
        assert_rel_close(dx, rdx, f"dx {name}", 1e-2)
        assert_rel_close(dw, rdw, f"dgamma {name}", 1e-3, 1e-5)
        got[name] = (dx, dw)
    differ = (got["ring"][0] != got["streaming"][0]).float().mean().item()
    assert differ < 1e-2, f"{differ:.2e} of dx differs between the two kernels"


def test_golden_rms_fwd_bwd():
    from linghe_b200.utils.norm import triton_rms_norm_forward, triton_rms_norm_backward
    G = golden("norm")
    for tag in ("n1", "n2"):
        x, g, dy = (_cuda(bf16(G[f"{k}_{tag}"])) for k in ("x", "gamma", "dy"))
        y, _ = triton_rms_norm_forward(x, g)
        assert_rel_close(y, bf16(G[f"rmsfwd_{tag}_y"]), "y", 1e-2)
        dx, dw = triton_rms_norm_backward(dy, x, g)
        assert_rel_close(dx, bf16(G[f"rmsbwd_{tag}_dx"]), "dx", 1e-2)
        assert_rel_close(dw.to(torch.bfloat16), bf16(G[f"rmsbwd_{tag}_dw"]), "dw", 1e-2)


class tuning:
    """set a dispatch option of the library for the duration of a with-block"""

    def __init__(self, key, value):
        self.key, self.value = key.encode(), value

    def __enter__(self):
        from linghe_b200 import _lib
        self.old = _lib.load().lh_tuning(self.key, self.value)
        assert self.old != _lib.LH_ERR_ARG

    def __exit__(self, *exc):
        from linghe_b200 import _lib
        _lib.load().lh_tuning(self.key, self.old)


# Both-axes RMSNorm + quant has two implementations (one kernel over a cluster band, x read from HBM
# once; or a row kernel followed by a column kernel) chosen by row width: each is checked at widths
# where the other is the default.
@pytest.mark.parametrize("M,n,force", [(1000, 1536, 0), (512, 2048, 0), (2048, 1664, 0), (384, 4096, 2), (130, 8192, 2),
                                       (4200, 8192, 2), (600, 5120, 2), (64, 128, 2), (128, 256, 0)])
def test_rms_block_quant_both_paths(M, n, force):
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward
    x = randn_bf16((M, n), 7, 2)
    g = randn_bf16((n,), 8)
    xd, gd = _cuda(x), _cuda(g)
    for rsc in (False, True):
        rq, rs, rr, rqt, rst = O.rms_norm_and_block_quant_forward(x, g, 1e-6, rsc)
        with tuning("rmsnorm_both_single_pass", force):
            q, s, r, qt, st = triton_rms_norm_and_block_quant_forward(xd, gd, round_scale=rsc, output_mode=2)
            torch.cuda.synchronize()
        assert_scales_close(r, rr, "rms")
        check_fused(q, rq, s, rs, "row", rsc)
        check_fused(qt, rqt, st, rst, "col", rsc)


# rows wider than 2048: the streaming backward also writes dy's row-wise codes and scales, the tile
# kernel only the transposed copy; (640, 2304) leaves the second span of a thread partly empty.
# The two single-pass implementations (x and dy read from HBM once) are selectable and held to the
# same checks: "band" = the cluster kernel, "two_role" = the streaming kernel whose CTAs carry a
# second role (four more warps) that writes the transposed copy tile by tile.
@pytest.mark.parametrize("path", ["default", "band", "two_role"])
@pytest.mark.parametrize("M,n", [(1024, 2048), (1024, 4096), (640, 2304), (384, 8192), (400, 2048), (4112, 1536),
                                 (128, 128)])
def test_rms_bwd_fused_dy_quant(M, n, path):
    from linghe_b200.utils.norm import rms_norm_backward_and_block_quant as fused_entry
    key, val = {"default": ("band_cluster", 0), "band": ("rmsnorm_bwd_quant_single_pass", 1),
                "two_role": ("rmsnorm_bwd_quant_two_role_min_n", 128)}[path]

    def rms_norm_backward_and_block_quant(*a, **kw):
        with tuning(key, val):
            out = fused_entry(*a, **kw)
            torch.cuda.synchronize()
        return out

    x = randn_bf16((M, n), 21)
    g = (1 + 0.1 * torch.randn(n, generator=torch.Generator().manual_seed(22))).to(torch.bfloat16)
    dy = randn_bf16((M, n), 23, 1, 0.01)
    dx, dw, q, s, qt, st = rms_norm_backward_and_block_quant(_cuda(dy), _cuda(x), _cuda(g))
    rdx, rdw = O.rms_norm_backward(x, g, dy)
    assert_rel_close(dx, rdx, "dx", 1e-2)
    assert_rel_close(dw, rdw, "dgamma", 1e-3, 1e-5)
    check_exact((q, s, qt, st), O.blockwise_quant(dy, False), ("dy q", "dy s", "dy qt", "dy st"))
    # a given 1/rms is used instead of the recomputed one
    r = _cuda(O.rms_recip(x))
    dx_r, dw_r, *_ = rms_norm_backward_and_block_quant(_cuda(dy), _cuda(x), _cuda(g), rms=r)
    assert_rel_close(dx_r, rdx, "dx with rms", 1e-2)
    assert_rel_close(dw_r, rdw, "dgamma with rms", 1e-3, 1e-5)
    # power-of-two scales, and zero / negative-zero / tiny blocks in dy
    dy2 = dy.clone()
    dy2[0, :128] = 0
    dy2[1, :128] = -0.0
    dy2[2, :256] = dy2[2, :256] * 1e-30
    _, _, q, s, qt, st = rms_norm_backward_and_block_quant(_cuda(dy2), _cuda(x), _cuda(g), round_scale=True)
    check_exact((q, s, qt, st), O.blockwise_quant(dy2, True), ("dy q", "dy s", "dy qt", "dy st"))


# ------------------------------------------------------------------------------------
# SwiGLU dense
# ------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag,rs", [("c1", 0), ("c1", 1), ("c100", 0), ("c0", 0)])
def test_golden_silu(tag, rs):
    from linghe_b200.utils.silu import triton_silu_and_block_quant_forward, triton_silu_and_block_quant_backward
    G = golden("silu")
    x, g = _cuda(bf16(G[f"x_{tag}"])), _cuda(bf16(G[f"g_{tag}"]))
    q, s, qt, st = triton_silu_and_block_quant_forward(x, round_scale=bool(rs))
    p = f"silufwd_{tag}_r{rs}_"
    check_fused(q, fp8(G[p + "q"]), s, torch.from_numpy(G[p + "s"]), "fwd row", bool(rs))
    check_fused(qt, fp8(G[p + "qt"]), st, torch.from_numpy(G[p + "st"]), "fwd col", bool(rs))
    q, s, qt, st = triton_silu_and_block_quant_backward(g, x, round_scale=bool(rs))
    p = f"silubwd_{tag}_r{rs}_"
    check_fused(q, fp8(G[p + "q"]), s, torch.from_numpy(G[p + "s"]), "bwd row", bool(rs))
    check_fused(qt, fp8(G[p + "qt"]), st, torch.from_numpy(G[p + "st"]), "bwd col", bool(rs))


@pytest.mark.parametrize("M,N,coef", [(1024, 1024, 1.0), (1000, 2816, 1.0), (512, 4096, 100.0), (256, 3072, 0.0),
                                      (72, 256, 1.0), (130, 32768, 1.0), (67, 16640, 1.0)])
def test_silu_fwd_modes(M, N, coef):
    from linghe_b200.utils.silu import triton_silu_and_block_quant_forward
    x = randn_bf16((M, N), 31, 1, coef)
    rq, rs, rqt, rst = O.silu_and_block_quant_forward(x, False)
    xd = _cuda(x)
    q, s, qt, st = triton_silu_and_block_quant_forward(xd, output_mode=2)
    check_fused(q, rq, s, rs, "mode2 row")
    check_fused(qt, rqt, st, rst, "mode2 col")
    q, s, _, _ = triton_silu_and_block_quant_forward(xd, output_mode=0)
    check_fused(q, rq, s, rs, "mode0 row")
    _, _, qt, st = triton_silu_and_block_quant_forward(xd, output_mode=1)
    check_fused(qt, rqt, st, rst, "mode1 col")
    # an input that is 16- but not 32-byte aligned takes the 128-bit loads
    buf = torch.empty(M * N + 8, dtype=torch.bfloat16, device="cuda")
    xo = buf[8:].view(M, N)
    xo.copy_(x)
    q, s, _, _ = triton_silu_and_block_quant_forward(xo, output_mode=0)
    check_fused(q, rq, s, rs, "mode0 row (offset input)")


@pytest.mark.parametrize("M,N,coef,gcoef", [(1024, 1024, 1.0, 1.0), (512, 2816, 1.0, 0.01), (256, 4096, 100.0, 100.0),
                                            (128, 512, 0.0, 0.0)])
def test_silu_bwd(M, N, coef, gcoef):
    from linghe_b200.utils.silu import triton_silu_and_block_quant_backward
    x = randn_bf16((M, N), 41, 1, coef)
    g = randn_bf16((M, N // 2), 42, 1, gcoef)
    rq, rs, rqt, rst, rdx = O.silu_and_block_quant_backward(g, x, False)
    q, s, qt, st, dx = triton_silu_and_block_quant_backward(_cuda(g), _cuda(x), return_bf16=True)
    check_fused(q, rq, s, rs, "row")
    check_fused(qt, rqt, st, rst, "col")
    assert dx.dtype == torch.bfloat16
    assert_rel_close(dx, rdx.to(torch.bfloat16), "dx bf16", 1e-2, SILU_DENORMAL_ATOL)
    out4 = triton_silu_and_block_quant_backward(_cuda(g), _cuda(x))
    assert len(out4) == 4 and torch.equal(out4[0].view(torch.uint8), q.view(torch.uint8))


@pytest.mark.parametrize("tag", ["c1", "c100", "c0"])
def test_golden_weighted_silu(tag):
    from linghe_b200.utils.silu import triton_weighted_silu_forward, triton_weighted_silu_backward
    G = golden("silu")
    x, g = _cuda(bf16(G[f"x_{tag}"])), _cuda(bf16(G[f"g_{tag}"]))
    w = _cuda(torch.from_numpy(G[f"wrow_{tag}"]))
    y = triton_weighted_silu_forward(x, w)
    assert_rel_close(y, bf16(G[f"wsilu_{tag}_y"]), "y", 1e-2, SILU_DENORMAL_ATOL)
    dx, dw = triton_weighted_silu_backward(g, x, w)
    assert_rel_close(dx, bf16(G[f"wsilubwd_{tag}_dx"]), "dx", 1e-2, SILU_DENORMAL_ATOL)
    assert dw.shape == w.shape and dw.dtype == w.dtype
    rate = 100.0 ** 1.5 if tag == "c100" else 1.0
    assert_rel_close(dw, torch.from_numpy(G[f"wsilubwd_{tag}_dw"]), "dw", 1e-3, 1e-3 * rate)
    y0 = triton_weighted_silu_forward(x)
    assert_rel_close(y0, O.weighted_silu_forward(bf16(G[f"x_{tag}"])), "y unweighted", 1e-2, SILU_DENORMAL_ATOL)
    dx0, dw0 = triton_weighted_silu_backward(g, x)
    assert dw0 is None
    assert_rel_close(dx0, O.weighted_silu_backward(bf16(G[f"g_{tag}"]), bf16(G[f"x_{tag}"]))[0].to(torch.bfloat16),
                     "dx unweighted", 1e-2, SILU_DENORMAL_ATOL)


# ------------------------------------------------------------------------------------
# SwiGLU per-expert batched
# ------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["c1", "c100"])
def test_golden_batch_silu(tag):
    from linghe_b200.utils.silu import (triton_batch_weighted_silu_and_block_quant_forward,
                                        triton_batch_weighted_silu_and_block_quant_backward)
    G = golden("batch")
    counts = G["counts"].tolist()
    x, g = _cuda(bf16(G[f"x_{tag}"])), _cuda(bf16(G[f"g_{tag}"]))
    w = _cuda(torch.from_numpy(G[f"w_{tag}"]))
    ct = torch.tensor(counts, dtype=torch.int32, device=DEV)
    q, s, qt, st = triton_batch_weighted_silu_and_block_quant_forward(x, w, ct, counts)
    check_fused(q, fp8(G[f"bfwd_{tag}_q"]), s, torch.from_numpy(G[f"bfwd_{tag}_s"]), "fwd row")
    check_fused(qt, fp8(G[f"bfwd_{tag}_qt"]), st, torch.from_numpy(G[f"bfwd_{tag}_st"]), "fwd col")
    q, s, dw, qt, st = triton_batch_weighted_silu_and_block_quant_backward(g, x, w, ct, splits=counts)
    check_fused(q, fp8(G[f"bbwd_{tag}_q"]), s, torch.from_numpy(G[f"bbwd_{tag}_s"]), "bwd row")
    check_fused(qt, fp8(G[f"bbwd_{tag}_qt"]), st, torch.from_numpy(G[f"bbwd_{tag}_st"]), "bwd col")
    rate = 100.0 ** 1.5 if tag == "c100" else 1.0
    assert_rel_close(dw, torch.from_numpy(G[f"bbwd_{tag}_dw"]), "dw", 1e-3, 1e-3 * rate)


@pytest.mark.parametrize("counts,N,cdt", [
    ([48, 0, 272, 128, 16, 0, 400, 96], 1024, torch.int32),
    ([0, 0, 0], 512, torch.int64),
    ([16] * 33, 256, torch.int64),
    ([1536], 2048, torch.int32),
])
def test_batch_silu(counts, N, cdt):
    from linghe_b200.utils.silu import (triton_batch_weighted_silu_and_block_quant_forward,
                                        triton_batch_weighted_silu_and_block_quant_backward)
    R = sum(counts)
    x = randn_bf16((R, N), 51)
    if R > 3:
        x[:3] = 0
    g = randn_bf16((R, N // 2), 52, 1, 0.01)
    w = torch.randn((R, 1), generator=torch.Generator().manual_seed(53))
    ct = torch.tensor(counts, dtype=cdt, device=DEV)
    rq, rs, rqt, rst = O.batch_weighted_silu_and_block_quant_forward(x, w, counts)
    xd, wd, gd = _cuda(x), _cuda(w), _cuda(g)
    for mode in (2, 0, 1):
        q, s, qt, st = triton_batch_weighted_silu_and_block_quant_forward(xd, wd, ct, counts, output_mode=mode)
        assert q.shape == (R, N // 2) and s.shape == (R, N // 256)
        if R == 0:
            continue
        if mode != 1:
            check_fused(q, rq, s, rs, f"fwd row m{mode}")
        if mode != 0:
            check_fused(qt, rqt, st, rst, f"fwd col m{mode}")
    rq, rs, rdw, rqt, rst = O.batch_weighted_silu_and_block_quant_backward(g, x, w, counts)
    q, s, dw, qt, st = triton_batch_weighted_silu_and_block_quant_backward(gd, xd, wd, ct, splits=counts)
    assert dw.shape == w.shape and dw.dtype == w.dtype
    if R == 0:
        return
    check_fused(q, rq, s, rs, "bwd row")
    check_fused(qt, rqt, st, rst, "bwd col")
    assert_rel_close(dw, rdw, "dw", 1e-3, 1e-3)


# ------------------------------------------------------------------------------------
# facade (autograd glue) with a duck-typed FP8 container
# ------------------------------------------------------------------------------------
class _Box:
    def __init__(self, **kw):
        self.__dict__.update(kw)


class _Quantizer:
    def __init__(self, pow2=False):
        self.force_pow_2_scales = pow2
        self.dtype = "e4m3"


def test_facade_block_rms_norm():
    from linghe_b200.facade.norm import block_rms_norm, rms_norm
    S, B, H = 8, 16, 1024
    x = randn_bf16((S, B, H), 61).to(DEV).requires_grad_()
    w = randn_bf16((H,), 62).to(DEV).requires_grad_()
    out, rms = block_rms_norm(x, w, None, _Quantizer(), _Box)
    assert out.rowwise_data.shape == (S, B, H) and out.columnwise_data.shape == (H, S, B)
    assert out.rowwise_scale_inv.shape == (H // 128, S * B) and out.columnwise_scale_inv.shape == (1, H)
    assert not rms.requires_grad and out.is_2D_scaled is False
    rq, rs, rr, rqt, rst = O.rms_norm_and_block_quant_forward(x.detach().cpu().view(S * B, H), w.detach().cpu())
    check_fused(out.rowwise_data, rq, out.rowwise_scale_inv, rs, "row")
    check_fused(out.columnwise_data, rqt, out.columnwise_scale_inv, rst, "col")
    out1, _ = block_rms_norm(x, w, rms, _Quantizer(), _Box, is_recomputing=True)
    assert out1.rowwise_data is None
    check_fused(out1.columnwise_data, rqt, out1.columnwise_scale_inv, rst, "recompute col")
    y = rms_norm(x, w)
    dy = randn_bf16((S, B, H), 63, 1, 0.01).to(DEV)
    y.backward(dy)
    rdx, rdw = O.rms_norm_backward(x.detach().cpu().view(S * B, H), w.detach().cpu(), dy.cpu().view(S * B, H))
    assert_rel_close(x.grad.view(S * B, H), rdx, "dx", 1e-2)
    assert_rel_close(w.grad.float(), rdw, "dw", 1e-2, 1e-4)


def test_facade_silu():
    from linghe_b200.facade.silu import block_silu_impl, block_batch_weighted_silu_impl
    S, B, H2 = 8, 16, 1024
    x = randn_bf16((S, B, H2), 71).to(DEV)
    out = block_silu_impl(x, _Quantizer(), _Quantizer(), _Box)
    assert out.rowwise_data.shape == (S, B, H2 // 2) and out.columnwise_data.shape == (H2 // 2, S, B)
    rq, rs, rqt, rst = O.silu_and_block_quant_forward(x.cpu().view(S * B, H2))
    check_fused(out.rowwise_data, rq, out.rowwise_scale_inv, rs, "row")
    counts = [32, 0, 160, 64]
    R = sum(counts)
    xb = randn_bf16((R, 512), 72).to(DEV)
    wb = torch.randn((R, 1), generator=torch.Generator().manual_seed(73)).to(DEV)
    ct = torch.tensor(counts, dtype=torch.int32, device=DEV)
    ob = block_batch_weighted_silu_impl(xb, wb, ct, counts, [_Quantizer()], [_Quantizer()], _Box)
    rq, rs, rqt, rst = O.batch_weighted_silu_and_block_quant_forward(xb.cpu(), wb.cpu(), counts)
    check_fused(ob.rowwise_data, rq, ob.rowwise_scale_inv, rs, "batch row")
    check_fused(ob.columnwise_data, rqt, ob.columnwise_scale_inv, rst, "batch col")


# ------------------------------------------------------------------------------------
# argument errors surface as AssertionError like upstream's bare asserts
# ------------------------------------------------------------------------------------
def test_argument_errors():
    from linghe_b200.quant.block import triton_blockwise_quant
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward
    x = torch.zeros((32, 200), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(AssertionError):
        triton_blockwise_quant(x)
    with pytest.raises(AssertionError):
        triton_blockwise_quant(torch.zeros((30, 128), dtype=torch.bfloat16, device=DEV))
    xx = torch.zeros((32, 256), dtype=torch.bfloat16, device=DEV)
    w = torch.ones((256,), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(AssertionError):
        triton_rms_norm_and_block_quant_forward(xx, w, output_mode=1)  # needs rms
    with pytest.raises(AssertionError):
        triton_rms_norm_and_block_quant_forward(xx.t(), w)  # not contiguous


# ------------------------------------------------------------------------------------
# permute + pad-to-16 + dual quant (the step before the per-expert SwiGLU)
# ------------------------------------------------------------------------------------
def _padded_indices(indices, counts, fill=0):
    """expert-major source rows -> the padded layout the kernel takes (16-row multiples)"""
    out, start = [], 0
    for c in counts:
        pc = (c + 15) // 16 * 16
        out.append(indices[start:start + c])
        out.append(torch.full((pc - c,), fill, dtype=indices.dtype))
        start += c
    return torch.cat(out) if out else indices[:0]


@pytest.mark.parametrize("rs", [0, 1])
@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
def test_golden_pad_permute(rs, idt):
    from linghe_b200.utils.gather import triton_batch_block_pad_permute_with_indices as f
    G = golden("permute")
    counts = G["counts"].tolist()
    idx = _padded_indices(torch.from_numpy(G["indices"]), counts, fill=10 ** 6).to(idt)   # pad entries are never read
    probs = torch.from_numpy(G["probs"])
    q, s, qt, st, p = f(_cuda(bf16(G["x"])), torch.tensor(counts, dtype=torch.int64, device=DEV), _cuda(idx), counts,
                        probs=_cuda(probs), round_scale=bool(rs))
    assert_bits_equal(q.view(-1), fp8(G[f"perm_r{rs}_q"]), "q")
    assert_f32_equal(s.view(-1), torch.from_numpy(G[f"perm_r{rs}_s"]), "s")
    assert_bits_equal(qt.view(-1), fp8(G[f"perm_r{rs}_qt"]), "qt")
    assert_f32_equal(st.view(-1), torch.from_numpy(G[f"perm_r{rs}_st"]), "st")
    assert_f32_equal(p, torch.from_numpy(G[f"perm_r{rs}_p"]), "probs")


@pytest.mark.parametrize("m,E,N,topk,dtype", [(2048, 32, 1024, 2, torch.bfloat16), (777, 8, 256, 3, torch.float32),
                                              (4096, 64, 512, 8, torch.bfloat16)])
def test_pad_permute(m, E, N, topk, dtype):
    from linghe_b200.utils.gather import triton_batch_block_pad_permute_with_indices as f
    g = torch.Generator().manual_seed(81)
    x = torch.randn((m, N), generator=g).to(dtype)
    logits = torch.randn((m, E), generator=g)
    logits[:, 0] -= 1000                                    # an expert nobody routes to
    top = logits.topk(topk, dim=1).indices
    route = torch.zeros((m, E), dtype=torch.bool).scatter_(1, top, True)
    probs = torch.softmax(logits, 1) * route
    counts = route.sum(0).tolist()
    tok = torch.arange(m).unsqueeze(0).expand(E, -1)
    indices = tok.masked_select(route.T.contiguous())
    ref = O.batch_block_pad_permute_with_indices(x, indices, probs, counts, False)
    idx = _padded_indices(indices, counts).to(torch.int32)
    out = f(_cuda(x), torch.tensor(counts, dtype=torch.int32, device=DEV), _cuda(idx), counts, probs=_cuda(probs))
    M = sum((c + 15) // 16 * 16 for c in counts)
    assert out[0].shape == (M, N) and out[1].shape == (M, N // 128) and out[4].shape == (M,)
    check_exact([o.view(-1) for o in out], ref, ("q", "s", "qt", "st", "probs"))
    out2 = f(_cuda(x), torch.tensor(counts, dtype=torch.int32, device=DEV), _cuda(idx), counts)
    assert out2[4] is None
    check_exact([o.view(-1) for o in out2[:4]], ref[:4], ("q", "s", "qt", "st"))


# ------------------------------------------------------------------------------------
# RMSNorm + float32 router logits + quantisation
# ------------------------------------------------------------------------------------
def _check_router(x, nw, rw, rs, golden_ref=None):
    from linghe_b200.utils.norm import triton_rms_norm_fp32_gemm_block_quant_forward
    if golden_ref is None:
        ry, rr, rl, rq, rsc, rqt, rst = O.rms_norm_fp32_gemm_block_quant_forward(x, nw, rw, 1e-6, rs)
    else:
        ry, rl, rq, rsc, rqt, rst = golden_ref
        rr = O.rms_recip(x)
    xd, nwd, rwd = _cuda(x), _cuda(nw), _cuda(rw)
    y, r, logits, q, s, qt, st = triton_rms_norm_fp32_gemm_block_quant_forward(
        xd, nwd, rwd, round_scale=rs, output_mode=0)
    assert logits.dtype == torch.float32 and tuple(logits.shape) == (x.shape[0], rw.shape[0])
    assert y.dtype == x.dtype and tuple(s.shape) == (x.shape[1] // 128, x.shape[0])
    assert_scales_close(r, rr, "rms")
    assert_rel_close(y.float(), ry.float(), "y", 1e-2, 1e-6)
    # float32 accumulation of exact products: only the summation order differs from the oracle
    err = (logits.cpu().double() - rl.double()).abs().max().item()
    mag = rl.double().abs().max().item()
    assert err <= 1e-4 * mag + 1e-6, f"logits: max abs err {err:.3e} at magnitude {mag:.3e}"
    check_fused(q, rq, s, rsc, "row", rs)
    o = triton_rms_norm_fp32_gemm_block_quant_forward(xd, nwd, rwd, rms=r, round_scale=rs, output_mode=1)
    assert o[1] is r
    check_fused(o[5], rqt, o[6], rst, "col", rs)
    return err / max(mag, 1e-30)


@pytest.mark.parametrize("rs", [0, 1])
def test_golden_rms_router_gemm(rs):
    G = golden("router")
    p = f"router_r{rs}_"
    ref = (bf16(G[p + "y"]), torch.from_numpy(G[p + "logits"]), fp8(G[p + "q"]), torch.from_numpy(G[p + "s"]),
           fp8(G[p + "qt"]), torch.from_numpy(G[p + "st"]))
    _check_router(bf16(G["x"]), bf16(G["norm_weight"]), bf16(G["route_weight"]), bool(rs), ref)


@pytest.mark.parametrize("M,K,N", [(128, 128, 128), (256, 2048, 256), (1024, 1536, 128), (384, 8192, 384)])
def test_rms_router_gemm(M, K, N):
    x = randn_bf16((M, K), 41, 2)
    nw = randn_bf16((K,), 42)
    rw = randn_bf16((N, K), 43)
    rel = _check_router(x, nw, rw, False)
    print(f"router logits max error / max magnitude: {rel:.2e}")


def test_rms_router_gemm_errors():
    from linghe_b200.utils.norm import triton_rms_norm_fp32_gemm_block_quant_forward
    x = _cuda(randn_bf16((128, 256), 1))
    nw = _cuda(randn_bf16((256,), 2))
    rw = _cuda(randn_bf16((128, 256), 3))
    with pytest.raises(AssertionError):
        triton_rms_norm_fp32_gemm_block_quant_forward(x, nw, rw, output_mode=2)
    with pytest.raises(AssertionError):
        triton_rms_norm_fp32_gemm_block_quant_forward(x, nw, rw, output_mode=1)      # needs rms
    with pytest.raises(AssertionError):
        triton_rms_norm_fp32_gemm_block_quant_forward(x[:100].contiguous(), nw, rw)  # M % 128
    with pytest.raises(AssertionError):
        triton_rms_norm_fp32_gemm_block_quant_forward(x, nw, rw[:64].contiguous())   # N % 128


# ------------------------------------------------------------------------------------
# blockwise-scaled FP8 GEMM (consumer of the quantisers' wire format)
# ------------------------------------------------------------------------------------
def _gemm_err(got, ref):
    g, r = got.detach().float().cpu().double(), ref.double()
    return (g - r).abs().max().item() / max(r.abs().max().item(), 1e-30)


@pytest.mark.parametrize("block", [128, 64])
def test_golden_fp8_gemm(block):
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
    G = golden("fp8gemm")
    a_q, b_q = _cuda(fp8(G["a_q"])), _cuda(fp8(G["b_q"]))
    a_s, b_s = _cuda(torch.from_numpy(G[f"a_s{block}"])), _cuda(torch.from_numpy(G[f"b_s{block}"]))
    y32 = triton_tt_fp8_gemm(a_q, b_q, a_s, b_s, out_dtype=torch.float32, block_size=block)
    ref = torch.from_numpy(G[f"y{block}_f32"])
    assert _gemm_err(y32, ref) <= 1e-5            # exact products, float32 sums: summation order only
    yb = triton_tt_fp8_gemm(a_q, b_q, a_s, b_s, out_dtype=torch.bfloat16, block_size=block)
    assert yb.dtype == torch.bfloat16
    assert_rel_close(yb.float(), bf16(G[f"y{block}_bf16"]).float(), "y bf16", 1e-2)
    # the same scales in the layout the quantisers of this package write
    yt = triton_tt_fp8_gemm(a_q, b_q, a_s.t().contiguous(), b_s.t().contiguous(), out_dtype=torch.float32,
                            block_size=block, scales_transposed=True)
    assert torch.equal(yt, y32)


@pytest.mark.parametrize("M,N,K,block,dt", [(512, 384, 1024, 128, torch.bfloat16), (1000, 264, 512, 64, torch.float16),
                                            (130, 8, 4096, 128, torch.float32), (128, 128, 16384, 128, torch.bfloat16),
                                            (2048, 2048, 2048, 64, torch.bfloat16),
                                            # widths the vector epilogues do not take (N % 8, odd N), a partial last
                                            # chunk of scales (10 k-blocks), several ragged tiles per persistent CTA
                                            (300, 100, 1280, 128, torch.bfloat16), (257, 77, 384, 128, torch.float32),
                                            (5000, 3000, 768, 128, torch.bfloat16), (3000, 1500, 1024, 64, torch.float16),
                                            (128, 256, 32768, 128, torch.float32)])     # 256 k-blocks: 32 chunks of scales
def test_fp8_gemm(M, N, K, block, dt):
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
    g = torch.Generator().manual_seed(51)
    a_q = torch.randn((M, K), generator=g).to(torch.float8_e4m3fn)
    b_q = torch.randn((N, K), generator=g).to(torch.float8_e4m3fn)
    a_s = torch.rand((M, K // block), generator=g) + 0.01
    b_s = torch.rand((N, K // block), generator=g) + 0.01
    ref = O.tt_fp8_gemm(a_q, b_q, a_s, b_s, torch.float32, block)
    y = triton_tt_fp8_gemm(_cuda(a_q), _cuda(b_q), _cuda(a_s), _cuda(b_s), out_dtype=dt, block_size=block)
    assert y.dtype == dt and tuple(y.shape) == (M, N)
    err = _gemm_err(y, ref)
    print(f"fp8 gemm {M}x{N}x{K} block {block}: max err / max |y| = {err:.2e}")
    assert err <= (1e-5 if dt == torch.float32 else 5e-3)


@pytest.mark.parametrize("dt,code", [(torch.bfloat16, 0), (torch.float32, 2)])
def test_fp8_gemm_output_at_16_byte_offset(dt, code):
    # through the C ABI with an output pointer that is 16- but not 32-byte aligned: the 32-byte
    # store path must step aside, the result must not change
    from linghe_b200 import _lib
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
    M, N, K = 256, 384, 512
    g = torch.Generator().manual_seed(57)
    a_q = _cuda(torch.randn((M, K), generator=g).to(torch.float8_e4m3fn))
    b_q = _cuda(torch.randn((N, K), generator=g).to(torch.float8_e4m3fn))
    a_s = _cuda(torch.rand((M, K // 128), generator=g) + 0.01)
    b_s = _cuda(torch.rand((N, K // 128), generator=g) + 0.01)
    want = triton_tt_fp8_gemm(a_q, b_q, a_s, b_s, out_dtype=dt)
    shift = 16 // want.element_size()
    flat = torch.zeros(M * N + shift, dtype=dt, device="cuda")
    out = flat[shift:]
    assert out.data_ptr() % 32 == 16
    _lib.call("lh_fp8_gemm", a_q, _lib.ptr(a_q), _lib.ptr(b_q), _lib.ptr(a_s), _lib.ptr(b_s), out.data_ptr(), M, N, K,
              128, 0, 0, code)
    torch.cuda.synchronize()
    assert torch.equal(out.view(M, N), want)
    assert float(flat[:shift].abs().max()) == 0.0


@pytest.mark.parametrize("block", [128, 64])
def test_golden_bb_fp8_gemm(block):
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_bb_fp8_gemm
    G = golden("fp8gemm_bb")
    a_q, b_q = _cuda(fp8(G["a_q"])), _cuda(fp8(G["b_q"]))
    a_s, b_s = _cuda(torch.from_numpy(G[f"a_s{block}"])), _cuda(torch.from_numpy(G[f"b_s{block}"]))
    y32 = triton_bb_fp8_gemm(a_q, b_q, a_s, b_s, out_dtype=torch.float32, block_size=block)
    assert _gemm_err(y32, torch.from_numpy(G[f"y{block}_f32"])) <= 1e-5
    yb = triton_bb_fp8_gemm(a_q, b_q, a_s, b_s, out_dtype=torch.bfloat16, block_size=block)
    assert yb.dtype == torch.bfloat16
    assert_rel_close(yb.float(), bf16(G[f"y{block}_bf16"]).float(), "y bf16", 1e-2)


# 2-D block scales (one per block x block sub-matrix): the reference's test uses block 64 at 4096^3
# (tests/test_blockwise_fp8_gemm.py:14-36); ragged M and N take the scale row of their block
@pytest.mark.parametrize("M,N,K,block,dt", [(512, 384, 1024, 128, torch.bfloat16), (1024, 256, 512, 64, torch.float16),
                                            (130, 72, 4096, 128, torch.float32), (2048, 2048, 2048, 64, torch.bfloat16),
                                            (1000, 200, 1024, 64, torch.float32)])
def test_bb_fp8_gemm(M, N, K, block, dt):
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_bb_fp8_gemm
    g = torch.Generator().manual_seed(52)
    a_q = torch.randn((M, K), generator=g).to(torch.float8_e4m3fn)
    b_q = torch.randn((N, K), generator=g).to(torch.float8_e4m3fn)
    a_s = torch.rand((-(-M // block), K // block), generator=g) + 0.01
    b_s = torch.rand((-(-N // block), K // block), generator=g) + 0.01
    ref = O.bb_fp8_gemm(a_q, b_q, a_s, b_s, torch.float32, block)
    y = triton_bb_fp8_gemm(_cuda(a_q), _cuda(b_q), _cuda(a_s), _cuda(b_s), out_dtype=dt, block_size=block)
    assert y.dtype == dt and tuple(y.shape) == (M, N)
    err = _gemm_err(y, ref)
    print(f"bb fp8 gemm {M}x{N}x{K} block {block}: max err / max |y| = {err:.2e}")
    assert err <= (1e-5 if dt == torch.float32 else 5e-3)


def test_bb_fp8_gemm_consumes_block_quant_outputs():
    """x, w -> 128 x 128 block codes and scales from triton_block_quant -> GEMM, against the float32
    product of the dequantised operands and, loosely, of the unquantised ones; and the same
    product through the 1 x 128 entry point with the block scales repeated per row, bit for bit."""
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_bb_fp8_gemm, triton_tt_fp8_gemm
    from linghe_b200.quant.block import triton_block_quant
    M, N, K = 1024, 512, 2048
    x, w = randn_bf16((M, K), 64), randn_bf16((N, K), 65)
    xq, xs = triton_block_quant(_cuda(x))
    wq, ws = triton_block_quant(_cuda(w))
    y = triton_bb_fp8_gemm(xq, wq, xs, ws, out_dtype=torch.float32, block_size=128)
    ref = O.bb_fp8_gemm(xq.cpu(), wq.cpu(), xs.cpu(), ws.cpu(), torch.float32, 128)
    assert _gemm_err(y, ref) <= 1e-5
    assert _gemm_err(y, x.float() @ w.float().t()) <= 5e-2           # the quantisation error itself
    yt = triton_tt_fp8_gemm(xq, wq, xs.repeat_interleave(128, dim=0).contiguous(),
                            ws.repeat_interleave(128, dim=0).contiguous(), out_dtype=torch.float32, block_size=128)
    assert torch.equal(y, yt)
    with pytest.raises(AssertionError):
        triton_bb_fp8_gemm(xq, wq, xs[:-1].contiguous(), ws, block_size=128)


def test_fp8_gemm_consumes_quantiser_outputs():
    """x, w -> row-wise (q, s[K/128, M]) from this package's quantisers -> GEMM; against the
    float32 product of the dequantised operands and, loosely, of the unquantised ones."""
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
    from linghe_b200.quant.block import triton_blockwise_quant
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward
    M, N, K = 1024, 512, 2048
    x = randn_bf16((M, K), 61)
    gam = randn_bf16((K,), 62)
    w = randn_bf16((N, K), 63)
    xq, xs, _, _, _ = triton_rms_norm_and_block_quant_forward(_cuda(x), _cuda(gam), output_mode=0)
    wq, ws, _, _ = triton_blockwise_quant(_cuda(w), output_mode=0)
    y = triton_tt_fp8_gemm(xq, wq, xs, ws, out_dtype=torch.bfloat16, block_size=128, scales_transposed=True)
    ref = O.tt_fp8_gemm(xq.cpu(), wq.cpu(), xs.cpu().t().contiguous(), ws.cpu().t().contiguous(), torch.float32, 128)
    assert _gemm_err(y, ref) <= 5e-3
    full = O.rms_norm_forward(x, gam).float() @ w.float().t()
    assert _gemm_err(y, full) <= 5e-2           # the quantisation error itself


def test_fp8_gemm_errors():
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
    a = _cuda(torch.zeros((128, 256)).to(torch.float8_e4m3fn))
    s = _cuda(torch.ones((128, 2)))
    with pytest.raises(AssertionError):
        triton_tt_fp8_gemm(a, a, s, s, block_size=32)
    with pytest.raises(AssertionError):
        triton_tt_fp8_gemm(a, a, s[:, :1].contiguous(), s, block_size=128)
    with pytest.raises(AssertionError):
        triton_tt_fp8_gemm(a.to(torch.bfloat16), a, s, s)


# ------------------------------------------------------------------------------------
# routing helpers and the padded-permute facade
# ------------------------------------------------------------------------------------
def _route_map(T, E, topk, seed, empty=()):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn((T, E), generator=g)
    for e in empty:
        logits[:, e] -= 1000
    top = torch.topk(logits, topk, dim=1).indices
    rm = torch.zeros((T, E), dtype=torch.bool)
    rm.scatter_(1, top, True)
    return rm


def test_golden_row_id_map():
    from linghe_b200.utils.gather import triton_make_row_id_map_and_index
    G = golden("route")
    rm = torch.from_numpy(G["route_map"]).bool()
    row_map, index = triton_make_row_id_map_and_index(_cuda(rm), int(G["counts"].sum()))
    assert torch.equal(row_map.cpu().long(), torch.from_numpy(G["row_id_map"]))
    assert torch.equal(index.cpu().long(), torch.from_numpy(G["indices"]))


@pytest.mark.parametrize("T,E,topk,mult,dt", [(4098, 32, 2, 16, torch.bool), (8192, 256, 8, 16, torch.bool),
                                              (777, 1500, 3, 1, torch.int32), (1, 8, 2, 16, torch.uint8)])
def test_row_id_map_and_index(T, E, topk, mult, dt):
    from linghe_b200.utils.gather import triton_make_row_id_map_and_index
    rm = _route_map(T, E, topk, 81, empty=(1,))
    ref_map, ref_index = O.make_row_id_map_and_index(rm, mult)
    row_map, index = triton_make_row_id_map_and_index(_cuda(rm.to(dt)), ref_index.numel(), multiple_of=mult)
    assert row_map.dtype == torch.int32 and index.dtype == torch.int32
    assert torch.equal(row_map.cpu(), ref_map)
    assert torch.equal(index.cpu(), ref_index)


@pytest.mark.parametrize("T,E,topk,n,dt,with_probs", [(1024, 32, 2, 2048, torch.bfloat16, True),
                                                      (300, 8, 3, 136, torch.float16, False),
                                                      (257, 64, 8, 512, torch.float32, True)])
def test_unpermute_with_mask_map(T, E, topk, n, dt, with_probs):
    from linghe_b200.utils.scatter import triton_unpermute_with_mask_map
    rm = _route_map(T, E, topk, 82)
    row_map, index = O.make_row_id_map_and_index(rm, 16)
    g = torch.Generator().manual_seed(83)
    grad = torch.randn((index.numel(), n), generator=g).to(dt)
    probs = torch.rand((index.numel(),), generator=g) if with_probs else None
    ref, ref_p = O.unpermute_with_mask_map(grad, row_map, probs)
    out, rp = triton_unpermute_with_mask_map(_cuda(grad), _cuda(row_map), _cuda(probs) if with_probs else None)
    assert out.dtype == dt
    assert torch.equal(out.cpu().view(torch.uint8), ref.contiguous().view(torch.uint8))   # same order of float32 sums
    if with_probs:
        assert torch.equal(rp.cpu(), ref_p)
    else:
        assert rp is None


def test_facade_block_padded_permute():
    import types
    from linghe_b200.facade import permutation as P
    T, E, topk, H = 2048, 32, 2, 1024
    rm = _route_map(T, E, topk, 84, empty=(5,))
    counts = rm.sum(0).tolist()
    x = randn_bf16((T, H), 85)
    probs = torch.rand((T, E), generator=torch.Generator().manual_seed(86)) * rm
    ct = torch.tensor(counts, dtype=torch.int32, device=DEV)
    out, pp, row_map, row_index = P.block_padded_permute(_cuda(x), _cuda(rm), ct, counts, [_Quantizer()], _Box,
                                                         probs=_cuda(probs))
    ref_map, ref_index = O.make_row_id_map_and_index(rm, 16)
    assert torch.equal(row_map.cpu(), ref_map) and torch.equal(row_index.cpu(), ref_index)
    src = torch.cat([row_index.cpu()[s:s + c] for s, c in zip(np.cumsum([0] + [(c + 15) // 16 * 16 for c in counts[:-1]]), counts)])
    rq, rs, rqt, rst, rp = O.batch_block_pad_permute_with_indices(x, src.long(), probs, counts, False)
    assert_bits_equal(out.rowwise_data.reshape(-1), rq, "q")
    assert_bits_equal(out.columnwise_data.reshape(-1)[:rqt.numel()], rqt, "qt")
    assert_f32_equal(out.rowwise_scale_inv.reshape(-1)[:rs.numel()], rs, "s")
    assert_f32_equal(pp.reshape(-1), rp, "probs")
    # backward of the permute = un-permute of the incoming gradient
    g = torch.Generator().manual_seed(87)
    go = torch.randn((ref_index.numel(), H), generator=g).to(torch.bfloat16)
    gp = torch.rand((ref_index.numel(),), generator=g)
    ctx = types.SimpleNamespace(saved_tensors=(row_map,), shape=x.shape, prob_shape=probs.shape)
    gx, gprob = P._BlockPaddedPermute.backward(ctx, _cuda(go), _cuda(gp), None, None)[:2]
    rgx, rgp = O.unpermute_with_mask_map(go, ref_map, gp)
    assert torch.equal(gx.cpu().view(torch.uint8), rgx.contiguous().view(torch.uint8)) and torch.equal(gprob.cpu(), rgp)
    # un-permute facade: forward sums the experts' rows, backward permutes + quantises the gradient
    y = P.block_padded_unpermute(_cuda(go), row_map, row_index, ct, counts, x.shape, [_Quantizer()], _Box)
    assert torch.equal(y.cpu().view(torch.uint8), rgx.contiguous().view(torch.uint8))
    ctx = types.SimpleNamespace(saved_tensors=(row_index,), tokens_per_expert=ct, splits=counts,
                                quantizers=[_Quantizer()], cls=_Box)
    gq = P._BlockPaddedUnpermute.backward(ctx, _cuda(x))[0]
    assert_bits_equal(gq.rowwise_data.reshape(-1), rq, "unpermute bwd q")
