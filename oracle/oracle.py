"""CPU oracle for the fused norm / SwiGLU + FP8 e4m3 blockwise-quantisation path.

TEST INFRASTRUCTURE ONLY.  This module restates, with torch CPU float32 ops, the
PyTorch reference math that the upstream project (inclusionAI/linghe) uses as its
own test oracle.  It is imported by the test-suite, by the smoke check and by the
CPU-baseline leg of the benchmark -- never by the product path, which runs only
hand-written CUDA and fails loudly when the CUDA library is missing.

Parity pin: every function here is compared bit-for-bit (pure quantisers) or
code-for-code (fused variants) against outputs of the upstream functions that were
produced by importing the upstream Python on CPU; the vectors and the script that
made them live in ``tests/golden/``.

Each function cites the upstream file:line it follows (paths inside the upstream
project).  Shapes / layouts returned are the *kernel* layouts (transposed row
scales and so on), so tests compare buffers directly.
"""

from __future__ import annotations

import torch

E4M3_MAX = 448.0
SCALE_FLOOR = 1e-30
BLOCK = 128


# --------------------------------------------------------------------------- #
# quantisation primitives
# --------------------------------------------------------------------------- #
def _pow2_ceil(scale: torch.Tensor) -> torch.Tensor:
    """exp2(ceil(log2(s))) in float32 -- linghe/tools/util.py:61-62."""
    return torch.exp2(torch.ceil(torch.log2(scale)))


def quant_rows_1x128(v: torch.Tensor, round_scale: bool = False):
    """Quantise every 1x128 block along the last dim of a 2-D float matrix.

    Follows ``torch_group_quant`` (linghe/tools/util.py:46-66): the last dim is
    zero-padded to a multiple of 128, scale = max(amax/448, 1e-30) in float32,
    optional power-of-two round-up, code = e4m3fn(v / scale) with IEEE division
    and round-to-nearest-even.  Returns (codes [M,K] e4m3fn, scales [M, ceil(K/128)]).
    """
    assert v.dim() == 2
    m, k = v.shape
    v = v.float()
    pad = (-k) % BLOCK
    if pad:
        v = torch.nn.functional.pad(v, (0, pad))
    blocks = v.contiguous().view(m, (k + pad) // BLOCK, BLOCK)
    scale = blocks.abs().amax(dim=2) / E4M3_MAX
    scale = torch.clamp_min(scale, SCALE_FLOOR)
    if round_scale:
        scale = _pow2_ceil(scale)
    codes = (blocks / scale.unsqueeze(-1)).to(torch.float8_e4m3fn)
    codes = codes.view(m, k + pad)[:, :k].contiguous()
    return codes, scale


def blockwise_quant(x: torch.Tensor, round_scale: bool = False):
    """Dual-axis activation quantiser (1x128 rows + 128x1 columns).

    Follows ``torch_blockwise_quant`` (linghe/tools/util.py:69-82, padding=False) and
    the kernel layouts of ``triton_blockwise_quant`` (linghe/quant/block.py:129-170):
    returns (q [M,N], s [N/128, M], qT [N, M], sT [ceil(M/128), N]).
    """
    x = x.float()
    q, s = quant_rows_1x128(x, round_scale)
    qt, st = quant_rows_1x128(x.t(), round_scale)
    return q, s.t().contiguous(), qt, st.t().contiguous()


def group_quant(x: torch.Tensor, round_scale: bool = False):
    """Row-only 1x128 quantiser with untransposed scales [M, N/128].

    linghe/tools/util.py:46-66 as used by tests/test_group_quant.py:14-32 and the
    layout of ``triton_group_quant`` (linghe/quant/group.py:40-63).
    """
    return quant_rows_1x128(x.float(), round_scale)


def block_quant(w: torch.Tensor, round_scale: bool = False):
    """128x128 2-D block quantiser for weights; one scale per block, no floor.

    Follows ``torch_block_quant`` (linghe/tools/util.py:85-98).  Returns
    (codes [N,K], scales [N/128, K/128]).
    """
    n, k = w.shape
    assert n % BLOCK == 0 and k % BLOCK == 0
    tiles = w.view(n // BLOCK, BLOCK, k // BLOCK, BLOCK).permute(0, 2, 1, 3)
    scale = tiles.abs().float().amax(dim=(2, 3)) / E4M3_MAX
    if round_scale:
        scale = _pow2_ceil(scale)
    codes = (tiles / scale[:, :, None, None]).to(torch.float8_e4m3fn)
    codes = codes.permute(0, 2, 1, 3).reshape(n, k).contiguous()
    return codes, scale


def batch_blockwise_quant(x: torch.Tensor, counts, round_scale: bool = False):
    """Per-expert dual-axis quantiser with flat packed outputs.

    Follows ``torch_batch_blockwise_quant`` (tests/test_blockwise_quant.py:17-43) and
    the packing of ``triton_batch_blockwise_quant`` (linghe/quant/block.py:251-297):
    for expert e (rows [S_e, S_e+c_e)) the flat outputs hold q [c_e,N], s [N/128,c_e],
    qT [N,c_e], sT [ceil(c_e/128),N] back to back.
    Returns flat tensors (q, s, qT, sT).
    """
    counts = [int(c) for c in counts]
    qs, ss, qts, sts = [], [], [], []
    start = 0
    for c in counts:
        if c == 0:
            continue
        q, s, qt, st = blockwise_quant(x[start:start + c], round_scale)
        qs.append(q.reshape(-1))
        ss.append(s.reshape(-1))
        qts.append(qt.reshape(-1))
        sts.append(st.reshape(-1))
        start += c
    if not qs:
        e = torch.empty(0)
        return (e.to(torch.float8_e4m3fn), e.float(), e.to(torch.float8_e4m3fn), e.float())
    return torch.cat(qs), torch.cat(ss), torch.cat(qts), torch.cat(sts)


# --------------------------------------------------------------------------- #
# RMSNorm
# --------------------------------------------------------------------------- #
def rms_recip(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """r = rsqrt(sum(x^2)/n + eps) per row -- tests/test_norm.py:80."""
    x = x.float()
    return torch.rsqrt(torch.sum(x * x, dim=1) / x.shape[1] + eps)


def _rms_norm_f32(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """float32 RMSNorm through torch.nn.functional.rms_norm, the same operator
    ``torch.nn.RMSNorm`` dispatches to in tests/test_norm.py:22-32,70-79
    (numerically (x * r) * gamma)."""
    x = x.float()
    return torch.nn.functional.rms_norm(x, (x.shape[-1],), weight.float(), eps)


def rms_norm_forward(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """Plain RMSNorm, output in x.dtype -- ``torch_rms_forward`` tests/test_norm.py:22-32."""
    return _rms_norm_f32(x, weight, eps).to(x.dtype)


def rms_norm_backward(x: torch.Tensor, weight: torch.Tensor, dy: torch.Tensor, eps: float = 1e-6):
    """RMSNorm backward by autograd in float32 -- ``torch_rms_backward``
    tests/test_norm.py:35-49.  Returns (dx in x.dtype, dgamma float32)."""
    xf = x.float().clone().requires_grad_()
    wf = weight.float().clone().requires_grad_()
    y = torch.nn.functional.rms_norm(xf, (xf.shape[-1],), wf, eps)
    y.backward(dy.float())
    return xf.grad.to(x.dtype), wf.grad


def rms_norm_and_block_quant_forward(x, weight, eps: float = 1e-6, round_scale: bool = False):
    """RMSNorm then dual-axis quantisation of the float32 result.

    Follows ``torch_rms_and_block_quant_forward`` (tests/test_norm.py:70-84) with the
    output layouts of ``triton_rms_norm_and_block_quant_forward``
    (linghe/utils/norm.py:343-502): (q [M,n], s [n/128,M], r [M], qT [n,M],
    sT [ceil(M/128), n]).
    """
    y = _rms_norm_f32(x, weight, eps)
    q, s, qt, st = blockwise_quant(y, round_scale)
    return q, s, rms_recip(x, eps), qt, st


def rms_norm_fp32_gemm_block_quant_forward(x, norm_weight, route_weight, eps: float = 1e-6,
                                           round_scale: bool = False):
    """RMSNorm, float32 router logits of the normalised rows and dual-axis quantisation.

    Follows ``torch_rms_gemm_block_quant_forward`` (tests/test_norm.py:86-103) with the
    output order and layouts of ``triton_rms_norm_fp32_gemm_block_quant_forward``
    (linghe/utils/norm.py:688-784): (y [M,K] x.dtype, r [M], logits [M,N] f32,
    q [M,K], s [K/128,M], qT [K,M], sT [M/128,K]).  The logits are the float32 matmul
    of the unrounded float32 y with the router weight [N,K].
    """
    y = _rms_norm_f32(x, norm_weight, eps)
    logits = y @ route_weight.float().t()
    q, s, qt, st = blockwise_quant(y, round_scale)
    return y.to(x.dtype), rms_recip(x, eps), logits, q, s, qt, st


def tt_fp8_gemm(a_q, b_q, a_s, b_s, out_dtype=torch.bfloat16, block_size: int = 128):
    """Blockwise-scaled FP8 GEMM: dequantise both operands and multiply in float32.

    The reference's own check for ``triton_tt_fp8_gemm`` (tests/test_blockwise_fp8_gemm.py:56-74):
    x_dq = x_q.float().view(M, K/B, B) * x_scales[:, :, None], same for w, y = x_dq @ w_dq.T.
    a_s [M, K/B], b_s [N, K/B] (the reference's scale layout).
    """
    M, K = a_q.shape
    N = b_q.shape[0]
    B = block_size
    a_dq = (a_q.float().view(M, K // B, B) * a_s[:, :, None]).view(M, K)
    b_dq = (b_q.float().view(N, K // B, B) * b_s[:, :, None]).view(N, K)
    return (a_dq @ b_dq.t()).to(out_dtype)


def bb_fp8_gemm(a_q, b_q, a_s, b_s, out_dtype=torch.bfloat16, block_size: int = 128):
    """FP8 GEMM with 2-D block scales: dequantise both operands and multiply in float32.

    The reference's own check for ``triton_bb_fp8_gemm`` (tests/test_blockwise_fp8_gemm.py:14-36):
    x_dq = x_q.float().view(M/B, B, K/B, B) * x_scales[:, None, :, None], same for w,
    y = x_dq @ w_dq.T.  a_s [ceil(M/B), K/B], b_s [ceil(N/B), K/B]; a ragged last row block
    (which the reference's kernel masks, linghe/gemm/blockwise_fp8_gemm.py:30-31,53-55) takes the
    scale row of its block.
    """
    M, K = a_q.shape
    N = b_q.shape[0]
    B = block_size
    a_dq = a_q.float() * a_s.repeat_interleave(B, dim=0)[:M].repeat_interleave(B, dim=1)
    b_dq = b_q.float() * b_s.repeat_interleave(B, dim=0)[:N].repeat_interleave(B, dim=1)
    return (a_dq @ b_dq.t()).to(out_dtype)


# --------------------------------------------------------------------------- #
# smooth-quant recipe: one scale per row after a per-column smoothing divisor
# --------------------------------------------------------------------------- #
def smooth_quant(x: torch.Tensor, smooth_scale: torch.Tensor, reverse: bool = False, round_scale: bool = False):
    """``torch_smooth_quant`` (linghe/tools/util.py:127-141): column maxima of |x|, then
    x / max(smooth, 1e-30) (x * smooth when `reverse`), one scale per row =
    max(amax/448, 1e-30) [power of two], codes = e4m3(x_smooth / scale).
    Returns (codes [M,N], scale [M], maxs [N])."""
    x = x.float()
    smooth_scale = smooth_scale.float()
    maxs = x.abs().amax(0) if x.shape[0] > 0 else torch.zeros(x.shape[1])
    if reverse:
        xs = x * smooth_scale
    else:
        xs = x / torch.clamp_min(smooth_scale, SCALE_FLOOR)
    if x.shape[0] == 0:
        return xs.to(torch.float8_e4m3fn), torch.zeros(0), maxs
    scale = torch.clamp_min(xs.abs().amax(1) / E4M3_MAX, SCALE_FLOOR)
    if round_scale:
        scale = _pow2_ceil(scale)
    return (xs / scale[:, None]).to(torch.float8_e4m3fn), scale, maxs


def rms_norm_and_smooth_quant_forward(x, weight, smooth_scale, eps: float = 1e-6, round_scale: bool = False):
    """``torch_rms_and_smooth_quant_forward`` (tests/test_norm.py:52-67): float32 RMSNorm, then
    smooth_quant.  Returns (codes, scale [M], maxs [N], 1/rms [M])."""
    q, s, maxs = smooth_quant(_rms_norm_f32(x, weight, eps), smooth_scale, False, round_scale)
    return q, s, maxs, rms_recip(x, eps)


def silu_and_smooth_quant_forward(x, smooth_scale, round_scale: bool = False):
    """``torch_silu_and_smooth_quant_forward`` (tests/test_silu.py:56-72): SwiGLU in float32, then
    smooth_quant.  Returns (codes [M,n], scale [M], maxs [n])."""
    return smooth_quant(_swiglu_f32(x), smooth_scale, False, round_scale)


def silu_and_smooth_quant_backward(g, x, smooth_scale, transpose_smooth_scale, round_scale: bool = True,
                                   reverse: bool = True):
    """``torch_silu_and_smooth_quant_backward`` (tests/test_silu.py:87-110): dx by autograd in
    float32, smooth_quant of dx with `smooth_scale` and of dx.T with `transpose_smooth_scale`.
    Returns (dx codes [M,2n], dx scale [M], dx.T codes [2n,M], dx.T scale [2n])."""
    dx, _ = weighted_silu_backward(g, x, None)
    q, s, _ = smooth_quant(dx, smooth_scale, reverse, round_scale)
    qt, st, _ = smooth_quant(dx.t().contiguous(), transpose_smooth_scale, reverse, round_scale)
    return q, s, qt, st


def batch_weighted_silu_and_smooth_quant_backward(g, x, weight, counts, smooth_scales, transpose_smooth_scale,
                                                  round_scale: bool = True, reverse: bool = False):
    """``torch_batch_weighted_silu_and_smooth_quant_backward`` (tests/test_silu.py:202-256): dx and
    dw by autograd in float32; per expert smooth_quant of its rows with smooth_scales[e] and of its
    transposed block, zero-padded to a multiple of 32 rows, with its slice of
    transpose_smooth_scale.  Returns (dx codes [R,2n], dx scale [R], dw float32 [R,1], flat
    transposed codes, transposed scales [E, 2n]).  An expert without rows contributes no codes and
    the floor scale."""
    counts = [int(c) for c in (counts.tolist() if hasattr(counts, "tolist") else counts)]
    dx, dw = weighted_silu_backward(g, x, weight)
    N = x.shape[1]
    qs, scales, qts, qtscales = [], [], [], []
    s = 0
    for e, c in enumerate(counts):
        q, sc, _ = smooth_quant(dx[s:s + c], smooth_scales[e], reverse, round_scale)
        qs.append(q)
        scales.append(sc)
        if c > 0:
            dxt = dx[s:s + c].t().contiguous()
            ts = transpose_smooth_scale[s:s + c].float()
            pad = (c + 31) // 32 * 32 - c
            if pad:
                dxt = torch.nn.functional.pad(dxt, (0, pad, 0, 0))
                ts = torch.nn.functional.pad(ts, (0, pad))
            qt, tsc, _ = smooth_quant(dxt, ts, reverse, round_scale)
            qts.append(qt.reshape(-1))
            qtscales.append(tsc)
        else:
            floor = torch.full((N,), SCALE_FLOOR)
            qtscales.append(_pow2_ceil(floor) if round_scale else floor)
        s += c
    qt_flat = torch.cat(qts, 0) if qts else torch.empty((0,), dtype=torch.float8_e4m3fn)
    return torch.cat(qs, 0), torch.cat(scales, 0), dw, qt_flat, torch.stack(qtscales, 0)


def batch_weighted_silu_and_smooth_quant_forward(x, weight, counts, smooth_scales, round_scale: bool = False,
                                                 reverse: bool = False):
    """``torch_batch_weighted_silu_and_smooth_quant_forward`` (tests/test_silu.py:126-160): per
    expert, weighted SwiGLU then smooth_quant with that expert's smoothing vector.  Returns
    (codes [R,n], scale [R], maxs [E,n]).  The calibration maxima follow the reference KERNEL
    (linghe/utils/silu.py:1803-1809): column maxima of |silu(x1) * x2| before the row weight
    (upstream's test helper takes them after the weight and does not compare them)."""
    counts = [int(c) for c in (counts.tolist() if hasattr(counts, "tolist") else counts)]
    n = x.shape[1] // 2
    qs, scales, maxs = [], [], []
    s = 0
    for e, c in enumerate(counts):
        xe = x[s:s + c]
        y = _swiglu_f32(xe, weight.reshape(-1)[s:s + c])
        q, sc, _ = smooth_quant(y, smooth_scales[e], reverse, round_scale)
        qs.append(q)
        scales.append(sc)
        maxs.append(_swiglu_f32(xe).abs().amax(0) if c > 0 else torch.zeros(n))
        s += c
    return torch.cat(qs, 0), torch.cat(scales, 0), torch.stack(maxs, 0)


# --------------------------------------------------------------------------- #
# SwiGLU (dense)
# --------------------------------------------------------------------------- #
def _swiglu_f32(x: torch.Tensor, weight: torch.Tensor | None = None) -> torch.Tensor:
    """y = sigmoid(x1) * x1 * x2 [* w_row], x1/x2 the left/right column halves.
    tests/test_silu.py:29-43."""
    x = x.float()
    x1, x2 = x.chunk(2, dim=1)
    y = torch.sigmoid(x1) * x1 * x2
    if weight is not None:
        y = y * weight.float().view(-1, 1)
    return y


def weighted_silu_forward(x, weight=None):
    """bf16 SwiGLU with optional per-row weight -- ``torch_weighted_silu``
    tests/test_silu.py:36-43."""
    return _swiglu_f32(x, weight).to(x.dtype)


def weighted_silu_backward(dy, x, weight=None):
    """autograd of the above -- ``torch_weighted_silu_backward`` tests/test_silu.py:46-53.
    Returns (dx float32, dw float32 or None); callers cast as needed."""
    xf = x.float().clone().requires_grad_()
    wf = None if weight is None else weight.float().clone().requires_grad_()
    y = _swiglu_f32(xf, wf)
    y.backward(dy.float())
    return xf.grad, (None if wf is None else wf.grad)


def silu_and_block_quant_forward(x, round_scale: bool = False):
    """SwiGLU then dual-axis quantisation -- ``torch_silu_and_block_quant_forward``
    tests/test_silu.py:75-84; layouts of ``triton_silu_and_block_quant_forward``
    (linghe/utils/silu.py:279-335): (q [M,n], s [n/128,M], qT [n,M], sT [ceil(M/128),n])."""
    return blockwise_quant(_swiglu_f32(x), round_scale)


def silu_and_block_quant_backward(g, x, round_scale: bool = False):
    """SwiGLU backward (autograd, float32) then dual-axis quantisation of dx [M,2n].

    ``torch_silu_and_block_quant_backward`` tests/test_silu.py:113-123; layouts of
    ``triton_silu_and_block_quant_backward`` (linghe/utils/silu.py:424-465).
    Returns (dx_q [M,2n], dx_s [2n/128,M], dxT_q [2n,M], dxT_s [M/128,2n], dx float32).
    """
    dx, _ = weighted_silu_backward(g, x, None)
    q, s, qt, st = blockwise_quant(dx, round_scale)
    return q, s, qt, st, dx


# --------------------------------------------------------------------------- #
# SwiGLU (per-expert batched)
# --------------------------------------------------------------------------- #
def _pack_segments(y: torch.Tensor, counts, round_scale: bool):
    """Quantise each expert segment separately and pack like the kernels do:
    q row-major global; per expert s [nb,c] / qT [n,c] / sT [ceil(c/128),n] flattened
    and concatenated (tests/test_silu.py:180-198)."""
    qs, ss, qts, sts = [], [], [], []
    start = 0
    for c in counts:
        seg = y[start:start + c]
        q, s, qt, st = blockwise_quant(seg, round_scale)
        qs.append(q)
        ss.append(s.reshape(-1))
        qts.append(qt.reshape(-1))
        sts.append(st.reshape(-1))
        start += c
    return torch.cat(qs, 0), torch.cat(ss), torch.cat(qts), torch.cat(sts)


def batch_weighted_silu_and_block_quant_forward(x, weight, counts, round_scale: bool = False):
    """Per-expert weighted SwiGLU + dual quant --
    ``torch_batch_weighted_silu_and_block_quant_forward`` tests/test_silu.py:163-199.
    Returns (q [R,n], s flat, qT flat, sT flat)."""
    counts = [int(c) for c in counts]
    n = x.shape[1] // 2
    if sum(counts) == 0:
        return (torch.empty((0, n), dtype=torch.float8_e4m3fn), torch.empty(0),
                torch.empty(0, dtype=torch.float8_e4m3fn), torch.empty(0))
    y = _swiglu_f32(x, weight)
    return _pack_segments(y, counts, round_scale)


def batch_weighted_silu_and_block_quant_backward(g, x, weight, counts, round_scale: bool = False):
    """Per-expert weighted SwiGLU backward + dual quant of dx --
    ``torch_batch_weighted_silu_and_block_quant_backward`` tests/test_silu.py:260-296.
    Returns (dx_q [R,2n], dx_s flat, dw [R,1] float32, dxT_q flat, dxT_s flat)."""
    counts = [int(c) for c in counts]
    two_n = x.shape[1]
    if sum(counts) == 0:
        return (torch.empty((0, two_n), dtype=torch.float8_e4m3fn), torch.empty(0),
                torch.empty_like(weight, dtype=torch.float32),
                torch.empty(0, dtype=torch.float8_e4m3fn), torch.empty(0))
    dx, dw = weighted_silu_backward(g, x, weight)
    q, s, qt, st = _pack_segments(dx, counts, round_scale)
    return q, s, dw.view(weight.shape), qt, st


# --------------------------------------------------------------------------- #
# helpers for large shapes
# --------------------------------------------------------------------------- #
def chunked(fn, row_args, other_args=(), rows_per_chunk: int = 4096, **kw):
    """Run a row-local oracle ``fn(*row_args_chunk, *other_args, **kw)`` over
    128-row-aligned chunks and return the list of per-chunk results.  Exact for
    1x128 and 128x1 blocks because chunk boundaries are multiples of 128 rows."""
    assert rows_per_chunk % BLOCK == 0
    m = row_args[0].shape[0]
    out = []
    for r0 in range(0, m, rows_per_chunk):
        sl = [a[r0:r0 + rows_per_chunk] for a in row_args]
        out.append(fn(*sl, *other_args, **kw))
    return out


# --------------------------------------------------------------------------- #
# permute + pad + quantise (the step before the per-expert SwiGLU)
# --------------------------------------------------------------------------- #
def batch_block_pad_permute_with_indices(x, indices, probs, counts, round_scale: bool = False):
    """Gather rows per expert, zero-pad every expert to a multiple of 16 rows, dual-axis
    quantise.  Follows ``torch_batch_block_pad_permute_with_indices``
    (tests/test_gather.py:150-197): `indices` is the UNPADDED concatenation of the source
    rows of every expert; experts with zero rows contribute nothing.  Returns flat
    (q, s, qT, sT, probs) with the per-expert packing of the kernel."""
    counts = [int(c) for c in counts]
    qs, ss, qts, sts, ps = [], [], [], [], []
    start = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        idx = indices[start:start + c]
        y = x[idx].float()
        pad = (-c) % 16
        if pad:
            y = torch.nn.functional.pad(y, (0, 0, 0, pad))
        q, s, qt, st = blockwise_quant(y, round_scale)
        qs.append(q.reshape(-1)); ss.append(s.reshape(-1)); qts.append(qt.reshape(-1)); sts.append(st.reshape(-1))
        if probs is not None:
            pe = probs[:, e][idx]
            ps.append(torch.nn.functional.pad(pe, (0, pad)) if pad else pe)
        start += c
    if not qs:
        z8 = torch.empty(0, dtype=torch.float8_e4m3fn)
        return z8, torch.empty(0), z8.clone(), torch.empty(0), torch.empty(0)
    return (torch.cat(qs), torch.cat(ss), torch.cat(qts), torch.cat(sts),
            torch.cat(ps) if probs is not None else None)


# --------------------------------------------------------------------------- #
# routing helpers around the permute step
# --------------------------------------------------------------------------- #
def make_row_id_map_and_index(route_map: torch.Tensor, multiple_of: int = 1):
    """Destination row of every routed (token, expert) pair, experts padded to `multiple_of` rows.

    For multiple_of = 1 this is ``torch_make_indices`` (linghe/tools/util.py:182-194): the
    cumulative count over the expert-major flattening of the routing map, minus one, -1 where
    not routed, and the expert-major list of routed tokens.  With padding each expert's first
    row moves to the sum of the padded counts before it, as
    ``make_row_id_map_and_index_kernel`` does (linghe/utils/gather.py:133-158); padding rows of
    the index list stay 0.  Returns (row_id_map [T,E] int32, row_indices [sum padded] int32).
    """
    T, E = route_map.shape
    rm = route_map.bool()
    counts = rm.sum(0)
    padded = (counts + multiple_of - 1) // multiple_of * multiple_of
    starts = torch.cumsum(padded, 0) - padded
    rank = torch.cumsum(rm.t().contiguous().int(), dim=1) - 1            # [E, T] rank inside the expert
    row_map = (starts[:, None] + rank).t().contiguous()
    row_map[~rm] = -1
    index = torch.zeros(int(padded.sum().item()), dtype=torch.int32)
    tok = torch.arange(T).unsqueeze(1).expand(T, E)
    index[row_map[rm].long()] = tok[rm].int()
    return row_map.int(), index


def unpermute_with_mask_map(grad: torch.Tensor, row_id_map: torch.Tensor, probs=None):
    """out[t] = float32 sum over the experts of token t of grad[row_id_map[t, e]] cast to grad.dtype,
    restore_probs[t, e] = probs[row_id_map[t, e]] or 0 -- what ``unpermute_with_mask_map_kernel``
    computes (linghe/utils/scatter.py:152-190)."""
    T, E = row_id_map.shape
    valid = row_id_map >= 0
    idx = row_id_map.clamp_min(0).long()
    g = grad.float()[idx] * valid[:, :, None]                            # [T, E, n]
    out = torch.zeros((T, grad.shape[1]), dtype=torch.float32)
    for e in range(E):                                                   # expert order, as the kernel
        out += g[:, e]
    rp = None
    if probs is not None:
        rp = torch.where(valid, probs[idx], torch.zeros((), dtype=probs.dtype))
    return out.to(grad.dtype), rp
