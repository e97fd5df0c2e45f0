"""The benchmark configurations at their full sizes, checked through properties that do not
need the CPU oracle on the whole tensor:

  * sampled 128-row blocks (and, for the per-expert path, sampled experts) against the
    oracle -- exact for row-wise and column-wise blocks because block boundaries are
    multiples of 128 rows;
  * determinism (two runs, bit-identical);
  * mode consistency (row-only / column-only outputs equal the both-axes outputs);
  * dequantisation: |code * scale - value| within half an e4m3 step of the block;
  * a checksum of per-block checksums that must agree between entry points that
    produce the same codes.
"""

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.common import (SILU_DENORMAL_ATOL, assert_bits_equal, assert_f32_equal, assert_codes_close, assert_scales_close,
                          assert_rel_close, bits)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def gen_bf16(shape, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    out = torch.empty(shape, device=DEV, dtype=torch.bfloat16)
    step = max(128, (1 << 25) // shape[1] // 128 * 128)
    for r0 in range(0, shape[0], step):
        r1 = min(shape[0], r0 + step)
        out[r0:r1] = (torch.randn((r1 - r0, shape[1]), generator=g, device=DEV) * scale).to(torch.bfloat16)
    return out


def u8(t):
    return t.view(torch.uint8)


def same(a, b):
    return torch.equal(u8(a) if a.dtype == torch.float8_e4m3fn else a, u8(b) if b.dtype == torch.float8_e4m3fn else b)


def sample_blocks(M, k, seed):
    rng = np.random.default_rng(seed)
    nblk = M // 128
    idx = sorted(set([0, nblk - 1] + rng.integers(0, nblk, size=k).tolist()))
    return idx


def check_block_fused(outs, ref_fn, x_rows, blk, M):
    """outs = (q [M,n], s [nb,M], qT [n,M], sT [M/128,n]); compare 128-row block `blk`."""
    q, s, qt, st = outs
    r0 = blk * 128
    rq, rs, rqt, rst = ref_fn(x_rows)
    assert_scales_close(s[:, r0:r0 + 128], rs, f"row scale blk {blk}")
    assert_codes_close(q[r0:r0 + 128], rq, f"row codes blk {blk}")
    assert_scales_close(st[blk:blk + 1], rst, f"col scale blk {blk}")
    assert_codes_close(qt[:, r0:r0 + 128], rqt, f"col codes blk {blk}")


def checksum(codes):
    """checksum of per-row checksums of the code bytes (order-sensitive inside a row)"""
    c = u8(codes).to(torch.int64)
    w = torch.arange(1, c.shape[1] + 1, device=c.device, dtype=torch.int64) % 251
    per_row = (c * w).sum(1) % 1000003
    return int((per_row * (torch.arange(per_row.numel(), device=c.device) % 257 + 1)).sum() % 2147483647)


def dequant_error_ok(q, s_t, y_block, r0):
    """|q*s - y| <= 2^-4 * |y| + s * 2^-10 (half a step of e4m3 incl. the subnormal range)"""
    deq = q[r0:r0 + 128].float().cpu().view(128, -1, 128) * s_t[:, r0:r0 + 128].t().cpu().unsqueeze(-1)
    y = y_block.view(128, -1, 128)
    err = (deq - y).abs()
    lim = y.abs() * 2.0 ** -4 + s_t[:, r0:r0 + 128].t().cpu().unsqueeze(-1) * 2.0 ** -9
    return bool((err <= lim * 1.001).all())


# ------------------------------------------------------------------------------------
def test_cfg1_rmsnorm_quant_8192x2048():
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as f
    M, n = 8192, 2048
    x = gen_bf16((M, n), 0)
    g = (1 + 0.1 * torch.randn(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))).to(torch.bfloat16)
    q, s, r, qt, st = f(x, g, output_mode=2)
    q0, s0, r0_, _, _ = f(x, g, output_mode=0)
    _, _, _, qt1, st1 = f(x, g, rms=r, output_mode=1)
    q2, s2, r2, qt2, st2 = f(x, g, output_mode=2)
    assert same(q, q2) and same(s, s2) and same(qt, qt2) and same(st, st2) and same(r, r2), "not deterministic"
    # The single-pass both-axes kernel adds a row's squares in another order than the row-only
    # kernels, so 1/rms may differ in the last bit between the modes: fused tolerance there.  Given
    # the same 1/rms, the column-only kernel must reproduce the both-axes outputs bit for bit.
    assert_scales_close(r0_, r, "rms mode 0 vs mode 2")
    assert_scales_close(s0, s, "row scales mode 0 vs mode 2")
    assert_codes_close(q0, q, "row codes mode 0 vs mode 2")
    assert same(qt, qt1) and same(st, st1), "mode 1 (with mode 2's 1/rms) differs from mode 2"
    assert checksum(qt) == checksum(qt1)
    xc, gc = x.cpu(), g.cpu()
    for blk in sample_blocks(M, 6, 11):
        rows = xc[blk * 128:(blk + 1) * 128]
        ref = O.rms_norm_and_block_quant_forward(rows, gc)
        check_block_fused((q, s, qt, st), lambda xr: (ref[0], ref[1], ref[3], ref[4]), rows, blk, M)
        assert_scales_close(r[blk * 128:(blk + 1) * 128], ref[2], "rms")
        y = torch.nn.functional.rms_norm(rows.float(), (n,), gc.float(), 1e-6)
        assert dequant_error_ok(q, s, y, blk * 128)


def test_cfg2_swiglu_fwd_bwd_8192x2816():
    from linghe_b200.utils.silu import (triton_silu_and_block_quant_forward as fwd,
                                        triton_silu_and_block_quant_backward as bwd)
    M, N = 8192, 2816
    x = gen_bf16((M, N), 2)
    g = gen_bf16((M, N // 2), 3, 0.01)
    outs = fwd(x, output_mode=2)
    o0 = fwd(x, output_mode=0)
    o1 = fwd(x, output_mode=1)
    assert all(same(a, b) for a, b in zip(outs, fwd(x, output_mode=2))), "not deterministic"
    assert same(outs[2], o1[2]) and same(outs[3], o1[3]), "mode 1 differs from mode 2"
    # the row-only path is a different kernel (streaming rows): same scales, codes within tolerance
    assert_scales_close(o0[1], outs[1], "row scales mode 0 vs 2")
    assert_codes_close(o0[0], outs[0], "row codes mode 0 vs 2")
    b = bwd(g, x, return_bf16=True)
    assert all(same(a, c) for a, c in zip(b, bwd(g, x, return_bf16=True))), "bwd not deterministic"
    xc, gc = x.cpu(), g.cpu()
    for blk in sample_blocks(M, 5, 12):
        rows = xc[blk * 128:(blk + 1) * 128]
        check_block_fused(outs, lambda xr: O.silu_and_block_quant_forward(xr, False), rows, blk, M)
        rq, rs, rqt, rst, rdx = O.silu_and_block_quant_backward(gc[blk * 128:(blk + 1) * 128], rows, False)
        check_block_fused(b[:4], lambda xr: (rq, rs, rqt, rst), rows, blk, M)
        assert_rel_close(b[4][blk * 128:(blk + 1) * 128], rdx.to(torch.bfloat16), "bf16 dx", 1e-2)


def moe_counts(seed=0, experts=256, tokens=65536, alpha=0.3):
    rng = np.random.default_rng(seed)
    p = rng.dirichlet(np.full(experts, alpha))
    c = rng.multinomial(tokens, p)
    return ((c + 127) // 128 * 128).astype(np.int64)


def test_cfg3_batched_moe_256_experts():
    from linghe_b200.utils.silu import (triton_batch_weighted_silu_and_block_quant_forward as fwd,
                                        triton_batch_weighted_silu_and_block_quant_backward as bwd)
    counts = moe_counts()
    R, n = int(counts.sum()), 512
    assert R == 83328 and int((counts == 0).sum()) == 29
    x = gen_bf16((R, 2 * n), 4)
    g = gen_bf16((R, n), 5, 0.01)
    w = torch.randn((R, 1), device=DEV, generator=torch.Generator(device=DEV).manual_seed(6))
    ct = torch.tensor(counts, dtype=torch.int32, device=DEV)
    splits = counts.tolist()
    f = fwd(x, w, ct, splits, output_mode=2)
    assert all(same(a, b) for a, b in zip(f, fwd(x, w, ct, splits, output_mode=2))), "fwd not deterministic"
    f0 = fwd(x, w, ct, splits, output_mode=0)
    f1 = fwd(x, w, ct, splits, output_mode=1)
    assert same(f[0], f0[0]) and same(f[1], f0[1]) and same(f[2], f1[2]) and same(f[3], f1[3])
    b = bwd(g, x, w, ct, splits=splits)
    b2 = bwd(g, x, w, ct, splits=splits)
    assert all(same(a, c) for a, c in zip(b, b2)), "bwd not deterministic"
    # sampled experts against the oracle (packed per-expert layouts)
    starts = np.concatenate([[0], np.cumsum(counts)])
    blk_starts = np.concatenate([[0], np.cumsum((counts + 127) // 128)])
    rng = np.random.default_rng(7)
    nonzero = np.nonzero(counts)[0]
    big = int(np.argmax(counts))
    for e in sorted(set([int(nonzero[0]), int(nonzero[-1])] + rng.choice(nonzero, 4).tolist() + ([big] if counts[big] <= 1024 else []))):
        s0, c = int(starts[e]), int(counts[e])
        xe, we, ge = x[s0:s0 + c].cpu(), w[s0:s0 + c].cpu(), g[s0:s0 + c].cpu()
        rq, rs, rqt, rst = O.batch_weighted_silu_and_block_quant_forward(xe, we, [c])
        nb = n // 128
        assert_codes_close(f[0][s0:s0 + c], rq, f"expert {e} q")
        assert_scales_close(f[1].view(-1)[s0 * nb:(s0 + c) * nb], rs, f"expert {e} s")
        assert_codes_close(f[2].view(-1)[s0 * n:(s0 + c) * n], rqt, f"expert {e} qT")
        b0 = int(blk_starts[e])
        assert_scales_close(f[3][b0:b0 + c // 128].reshape(-1), rst, f"expert {e} sT")
        rq, rs, rdw, rqt, rst = O.batch_weighted_silu_and_block_quant_backward(ge, xe, we, [c])
        assert_codes_close(b[0][s0:s0 + c], rq, f"expert {e} dx q")
        assert_scales_close(b[1].view(-1)[s0 * 2 * nb:(s0 + c) * 2 * nb], rs, f"expert {e} dx s")
        assert_rel_close(b[2][s0:s0 + c], rdw, f"expert {e} dw", 1e-3, 1e-3)
        assert_codes_close(b[3].view(-1)[s0 * 2 * n:(s0 + c) * 2 * n], rqt, f"expert {e} dx qT")
        assert_scales_close(b[4][b0:b0 + c // 128].reshape(-1), rst, f"expert {e} dx sT")


def test_cfg4_rmsnorm_bwd_dual_quant_16384x4096():
    from linghe_b200.quant.block import triton_blockwise_quant
    from linghe_b200.utils.norm import rms_norm_backward_and_block_quant, triton_rms_norm_backward
    M, n = 16384, 4096
    x = gen_bf16((M, n), 8)
    dy = gen_bf16((M, n), 9, 0.01)
    g = (1 + 0.1 * torch.randn(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(10))).to(torch.bfloat16)
    dx, dw, q, s, qt, st = rms_norm_backward_and_block_quant(dy, x, g)
    dx2, dw2 = triton_rms_norm_backward(dy, x, g)
    # the fused entry is its own single-pass kernel: same math, another summation order
    assert_rel_close(dx, dx2.float(), "fused dx vs plain backward", 1e-2)
    assert_rel_close(dw, dw2, "fused dgamma vs plain backward", 1e-4, 1e-5)
    dx3, dw3, *_ = rms_norm_backward_and_block_quant(dy, x, g)
    assert same(dx, dx3) and same(dw, dw3), "not deterministic"
    pq = triton_blockwise_quant(dy)
    assert all(same(a, b) for a, b in zip((q, s, qt, st), pq)), "fused dy copies differ from blockwise_quant"
    assert checksum(q) == checksum(pq[0]) and checksum(qt) == checksum(pq[2])
    # pure quantiser part: bit-exact on sampled blocks
    dyc = dy.cpu()
    for blk in sample_blocks(M, 5, 13):
        r0 = blk * 128
        rq, rs, rqt, rst = O.blockwise_quant(dyc[r0:r0 + 128], False)
        assert_bits_equal(q[r0:r0 + 128], rq, "dy q")
        assert_f32_equal(s[:, r0:r0 + 128], rs, "dy s")
        assert_bits_equal(qt[:, r0:r0 + 128], rqt, "dy qT")
        assert_f32_equal(st[blk:blk + 1], rst, "dy sT")
    # dx on sampled rows (row-local), dgamma by linearity: dgamma(all) == dgamma(top) + dgamma(bottom)
    xc, gc = x.cpu(), g.cpu()
    for blk in sample_blocks(M, 3, 14):
        r0 = blk * 128
        rdx, _ = O.rms_norm_backward(xc[r0:r0 + 128], gc, dyc[r0:r0 + 128])
        assert_rel_close(dx[r0:r0 + 128], rdx, "dx", 1e-2)
    _, dw_top = triton_rms_norm_backward(dy[:M // 2].contiguous(), x[:M // 2].contiguous(), g)
    _, dw_bot = triton_rms_norm_backward(dy[M // 2:].contiguous(), x[M // 2:].contiguous(), g)
    assert_rel_close(dw, dw_top + dw_bot, "dgamma linearity", 1e-4, 1e-5)
    # dgamma over all 16384 rows against the oracle (row chunks bound the oracle's float32
    # temporaries; the chunk sums are added in float64)
    rdw = torch.zeros(n, dtype=torch.float64)
    for r0 in range(0, M, 4096):
        _, part = O.rms_norm_backward(xc[r0:r0 + 4096], gc, dyc[r0:r0 + 4096])
        rdw += part.double()
    assert_rel_close(dw, rdw.float(), "dgamma vs oracle (all rows)", 1e-3, 1e-5)


# ------------------------------------------------------------------------------------
# The reference's own stress inputs at their full widths (tests/test_norm.py:189-219,329-331:
# x = randn**2, gamma = randn, 16384 x 1536, power-of-two scales; tests/test_silu.py:405-460,
# 714-721: 4096 x 12288 with coef 1 / 100 / 0), whole tensors against the oracle.
# ------------------------------------------------------------------------------------
def test_stress_rmsnorm_quant_sq_input_16384x1536():
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as norm_q
    from tests.common import assert_fused_pow2
    M, n = 16384, 1536
    gen = torch.Generator().manual_seed(77)
    x = (torch.randn((M, n), generator=gen) ** 2).to(torch.bfloat16)
    g = torch.randn((n,), generator=gen).to(torch.bfloat16)
    xd, gd = x.to(DEV), g.to(DEV)
    for rsc in (False, True):
        rq, rs, rr, rqt, rst = O.rms_norm_and_block_quant_forward(x, g, 1e-6, rsc)
        q, s, r, _, _ = norm_q(xd, gd, round_scale=rsc, output_mode=0)
        _, _, _, qt1, st1 = norm_q(xd, gd, round_scale=rsc, rms=r, output_mode=1)
        q2, s2, r2, qt2, st2 = norm_q(xd, gd, round_scale=rsc, output_mode=2)
        assert_scales_close(r, rr, "rms")
        assert_scales_close(r2, rr, "rms mode 2")
        for (cq, cs, rq_, rs_, nm) in ((q, s, rq, rs, "mode0 row"), (qt1, st1, rqt, rst, "mode1 col"),
                                      (q2, s2, rq, rs, "mode2 row"), (qt2, st2, rqt, rst, "mode2 col")):
            if rsc:
                assert_fused_pow2(cq, rq_, cs, rs_, nm + " pow2")
            else:
                assert_scales_close(cs, rs_, nm + " scale")
                assert_codes_close(cq, rq_, nm + " codes")


@pytest.mark.parametrize("coef,gcoef", [(1.0, 1.0), (100.0, 100.0), (0.0, 0.0)])
def test_stress_swiglu_quant_4096x12288(coef, gcoef):
    from linghe_b200.utils.silu import triton_silu_and_block_quant_backward, triton_silu_and_block_quant_forward
    M, N = 4096, 12288
    gen = torch.Generator().manual_seed(78)
    x = (torch.randn((M, N), generator=gen) * coef).to(torch.bfloat16)
    gr = (torch.randn((M, N // 2), generator=gen) * gcoef).to(torch.bfloat16)
    xd, gd = x.to(DEV), gr.to(DEV)
    rq, rs, rqt, rst = O.silu_and_block_quant_forward(x, False)
    q0, s0, _, _ = triton_silu_and_block_quant_forward(xd, output_mode=0)
    _, _, qt1, st1 = triton_silu_and_block_quant_forward(xd, output_mode=1)
    q2, s2, qt2, st2 = triton_silu_and_block_quant_forward(xd, output_mode=2)
    for (cq, cs, rq_, rs_, nm) in ((q0, s0, rq, rs, "fwd mode0 row"), (qt1, st1, rqt, rst, "fwd mode1 col"),
                                  (q2, s2, rq, rs, "fwd mode2 row"), (qt2, st2, rqt, rst, "fwd mode2 col")):
        assert_scales_close(cs, rs_, nm + " scale")
        assert_codes_close(cq, rq_, nm + " codes")
    rq, rs, rqt, rst, rdx = O.silu_and_block_quant_backward(gr, x, False)
    q, s_, qt, st, dx = triton_silu_and_block_quant_backward(gd, xd, return_bf16=True)
    assert_scales_close(s_, rs, "bwd row scale")
    assert_codes_close(q, rq, "bwd row codes")
    assert_scales_close(st, rst, "bwd col scale")
    assert_codes_close(qt, rqt, "bwd col codes")
    assert_rel_close(dx, rdx, "bwd bf16 dx", 1e-2, SILU_DENORMAL_ATOL)


def test_cfg5_scaleout_shard_65536x8192():
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as norm_q
    from linghe_b200.utils.silu import triton_silu_and_block_quant_forward as silu_q
    M, n = 65536, 8192
    x = gen_bf16((M, n), 20)
    g = (1 + 0.1 * torch.randn(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(21))).to(torch.bfloat16)
    q, s, r, _, _ = norm_q(x, g, output_mode=0)
    q2, s2, r2, _, _ = norm_q(x, g, output_mode=0)
    assert same(q, q2) and same(s, s2) and same(r, r2), "not deterministic"
    # a shard is the same computation on a row slice: the slice of the big run equals a run on the slice
    lo, hi = 128 * 100, 128 * 164
    qs, ss, rs_, _, _ = norm_q(x[lo:hi].contiguous(), g, output_mode=0)
    assert same(q[lo:hi], qs) and same(s[:, lo:hi].contiguous(), ss) and same(r[lo:hi], rs_)
    xc, gc = x[:1].cpu(), g.cpu()
    for blk in sample_blocks(M, 4, 15):
        rows = x[blk * 128:(blk + 1) * 128].cpu()
        ref = O.rms_norm_and_block_quant_forward(rows, gc)
        assert_scales_close(s[:, blk * 128:(blk + 1) * 128], ref[1], "row scale")
        assert_codes_close(q[blk * 128:(blk + 1) * 128], ref[0], "row codes")
        assert_scales_close(r[blk * 128:(blk + 1) * 128], ref[2], "rms")
    del q, s, q2, s2, x
    torch.cuda.empty_cache()
    xs = gen_bf16((M, 2 * n), 22)
    q, s, _, _ = silu_q(xs, output_mode=0)
    q2, s2, _, _ = silu_q(xs, output_mode=0)
    assert same(q, q2) and same(s, s2), "not deterministic"
    for blk in sample_blocks(M, 4, 16):
        rows = xs[blk * 128:(blk + 1) * 128].cpu()
        rq, rs, _, _ = O.silu_and_block_quant_forward(rows, False)
        assert_scales_close(s[:, blk * 128:(blk + 1) * 128], rs, "row scale")
        assert_codes_close(q[blk * 128:(blk + 1) * 128], rq, "row codes")


# ------------------------------------------------------------------------------------
# blockwise-scaled FP8 GEMM at the upstream test's size: an input family whose result is exact
# ------------------------------------------------------------------------------------
def test_fp8_gemm_exact_integers_4096():
    """Codes drawn from small integers and power-of-two scales: every product, every partial sum
    and every scaled accumulation is exactly representable in float32, so the kernel must match
    an integer computation bit for bit whatever the summation order."""
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
    M = N = K = 4096
    g = torch.Generator().manual_seed(77)
    a = torch.randint(-2, 3, (M, K), generator=g, dtype=torch.int32)
    b = torch.randint(-2, 3, (N, K), generator=g, dtype=torch.int32)
    ea = torch.randint(-1, 2, (M, K // 128), generator=g)
    eb = torch.randint(-1, 2, (N, K // 128), generator=g)
    a_s, b_s = torch.exp2(ea.float()), torch.exp2(eb.float())
    dev = "cuda:0"
    y = triton_tt_fp8_gemm(a.float().to(torch.float8_e4m3fn).to(dev), b.float().to(torch.float8_e4m3fn).to(dev),
                           a_s.to(dev), b_s.to(dev), out_dtype=torch.float32, block_size=128)
    # exact reference on the same device in float64 (|partial| <= 512, scale products 2^-2..2^2, 32 blocks:
    # every value is a multiple of 1/4 below 2^16, far inside float32's 24 bits)
    ad = (a.double().view(M, K // 128, 128) * a_s.double()[:, :, None]).view(M, K).to(dev)
    bd = (b.double().view(N, K // 128, 128) * b_s.double()[:, :, None]).view(N, K).to(dev)
    ref = ad @ bd.t()
    assert torch.equal(y.double(), ref), f"max abs diff {(y.double() - ref).abs().max().item()}"
    # transposed-scale entry gives the identical result
    yt = triton_tt_fp8_gemm(a.float().to(torch.float8_e4m3fn).to(dev), b.float().to(torch.float8_e4m3fn).to(dev),
                            a_s.t().contiguous().to(dev), b_s.t().contiguous().to(dev), out_dtype=torch.float32,
                            block_size=128, scales_transposed=True)
    assert torch.equal(yt, y)
