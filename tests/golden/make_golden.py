"""Generate golden vectors by running the UPSTREAM PyTorch reference math on CPU.

Run once, in a container that has the upstream checkout (read-only) available:

    python tests/golden/make_golden.py --reference /path/to/linghe

It imports the upstream oracle functions (linghe/tools/util.py and the helper
functions inside upstream tests/test_norm.py, tests/test_silu.py,
tests/test_blockwise_quant.py), feeds them small seeded inputs and stores inputs and
outputs as raw integer views in ``tests/golden/*.npz``.  The repository's own oracle
(``oracle/oracle.py``) and CUDA kernels are then checked against these files without
needing the upstream checkout.
"""

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def u16(t):  # bf16 -> raw bits
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def u8(t):  # fp8 -> raw bits
    return t.contiguous().view(torch.uint8).numpy()


def f32(t):
    return t.detach().contiguous().float().numpy()


def bf16_randn(gen, shape, power=1, coef=1.0):
    x = torch.randn(shape, generator=gen, dtype=torch.float32)
    if power != 1:
        x = x ** power
    return (x * coef).to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the upstream linghe checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.path.insert(0, os.path.join(args.reference, "tests"))
    from linghe.tools import util as U
    import test_norm as TN
    import test_silu as TS
    import test_blockwise_quant as TB

    gen = torch.Generator().manual_seed(20240607)

    # ---- pure quantisers --------------------------------------------------- #
    out = {}
    for tag, power in (("n1", 1), ("n3", 3)):
        x = bf16_randn(gen, (144, 256), power)
        x[5, 128:256] = 0  # an all-zero 1x128 block -> scale floor
        x[:, 200] = 0      # an all-zero column
        out[f"x_{tag}"] = u16(x)
        for rs in (False, True):
            q, s = U.torch_group_quant(x, round_scale=rs)
            out[f"group_{tag}_r{int(rs)}_q"] = u8(q)
            out[f"group_{tag}_r{int(rs)}_s"] = f32(s)
            q, s, qt, st = U.torch_blockwise_quant(x, round_scale=rs, padding=False)
            for k, v in (("q", u8(q)), ("s", f32(s)), ("qt", u8(qt)), ("st", f32(st))):
                out[f"blockwise_{tag}_r{int(rs)}_{k}"] = v
    xf = torch.randn((48, 256), generator=gen, dtype=torch.float32) * 7.5
    out["x_f32"] = xf.numpy()
    q, s, qt, st = U.torch_blockwise_quant(xf, round_scale=False, padding=False)
    for k, v in (("q", u8(q)), ("s", f32(s)), ("qt", u8(qt)), ("st", f32(st))):
        out[f"blockwise_f32_r0_{k}"] = v
    w = bf16_randn(gen, (128, 256), 3)
    out["w"] = u16(w)
    for rs in (False, True):
        q, s = U.torch_block_quant(w, round_scale=rs)
        out[f"block_r{int(rs)}_q"] = u8(q)
        out[f"block_r{int(rs)}_s"] = f32(s)
    counts = [0, 48, 130, 7, 128, 0, 16]
    xb = bf16_randn(gen, (sum(counts), 128))
    out["xb"] = u16(xb)
    out["xb_counts"] = np.asarray(counts, dtype=np.int64)
    for rs in (False, True):
        q, s, qt, st = TB.torch_batch_blockwise_quant(xb, counts, round_scale=rs)
        for k, v in (("q", u8(q)), ("s", f32(s)), ("qt", u8(qt)), ("st", f32(st))):
            out[f"batchq_r{int(rs)}_{k}"] = v
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **out)

    # ---- RMSNorm ----------------------------------------------------------- #
    out = {}
    for tag, power in (("n1", 1), ("n2", 2)):
        x = bf16_randn(gen, (144, 256), power)
        g = (1 + 0.1 * torch.randn(256, generator=gen)).to(torch.bfloat16) if tag == "n1" \
            else bf16_randn(gen, (256,))
        out[f"x_{tag}"] = u16(x)
        out[f"gamma_{tag}"] = u16(g)
        for rs in (False, True):
            q, s, r, qt, st = TN.torch_rms_and_block_quant_forward(x, g, round_scale=rs)
            for k, v in (("q", u8(q)), ("s", f32(s)), ("r", f32(r)), ("qt", u8(qt)), ("st", f32(st))):
                out[f"rmsq_{tag}_r{int(rs)}_{k}"] = v
        out[f"rmsfwd_{tag}_y"] = u16(TN.torch_rms_forward(x, g))
        dy = bf16_randn(gen, (144, 256), 1, 0.01)
        out[f"dy_{tag}"] = u16(dy)
        dx, dw = TN.torch_rms_backward(x, g, dy)
        out[f"rmsbwd_{tag}_dx"] = u16(dx)
        out[f"rmsbwd_{tag}_dw"] = u16(dw)
    np.savez_compressed(os.path.join(HERE, "norm.npz"), **out)

    # ---- SwiGLU dense ------------------------------------------------------ #
    out = {}
    for tag, coef, gcoef in (("c1", 1.0, 1.0), ("c100", 100.0, 100.0), ("c0", 0.0, 0.0)):
        x = bf16_randn(gen, (128, 512), 1, coef)
        g = bf16_randn(gen, (128, 256), 1, gcoef)
        out[f"x_{tag}"] = u16(x)
        out[f"g_{tag}"] = u16(g)
        for rs in ((False, True) if tag == "c1" else (False,)):
            q, s, qt, st = TS.torch_silu_and_block_quant_forward(x, round_scale=rs)
            # upstream returns scales untransposed here; store kernel layout
            for k, v in (("q", u8(q)), ("s", f32(s.t())), ("qt", u8(qt)), ("st", f32(st.t()))):
                out[f"silufwd_{tag}_r{int(rs)}_{k}"] = v
            q, s, qt, st = TS.torch_silu_and_block_quant_backward(g, x, round_scale=rs)
            for k, v in (("q", u8(q)), ("s", f32(s.t())), ("qt", u8(qt)), ("st", f32(st.t()))):
                out[f"silubwd_{tag}_r{int(rs)}_{k}"] = v
        wrow = torch.randn((128, 1), generator=gen, dtype=torch.float32)
        out[f"wrow_{tag}"] = wrow.numpy()
        out[f"wsilu_{tag}_y"] = u16(TS.torch_weighted_silu(x, wrow))
        dxw, dww = TS.torch_weighted_silu_backward(g.float(), x, wrow)
        out[f"wsilubwd_{tag}_dx"] = u16(dxw)
        out[f"wsilubwd_{tag}_dw"] = f32(dww)
    np.savez_compressed(os.path.join(HERE, "silu.npz"), **out)

    # ---- SwiGLU per-expert batched ---------------------------------------- #
    out = {}
    counts = [0, 32, 144, 16, 128, 0, 48]
    R = sum(counts)
    for tag, coef, gcoef in (("c1", 1.0, 1.0), ("c100", 100.0, 100.0)):
        x = bf16_randn(gen, (R, 256), 1, coef)
        x[:3] = 0
        wrow = torch.randn((R, 1), generator=gen, dtype=torch.float32)
        g = bf16_randn(gen, (R, 128), 1, gcoef)
        out[f"x_{tag}"] = u16(x)
        out[f"w_{tag}"] = wrow.numpy()
        out[f"g_{tag}"] = u16(g)
        ct = torch.tensor(counts, dtype=torch.int32)
        q, s, qt, st = TS.torch_batch_weighted_silu_and_block_quant_forward(x, wrow, ct, round_scale=False)
        for k, v in (("q", u8(q)), ("s", f32(s)), ("qt", u8(qt)), ("st", f32(st))):
            out[f"bfwd_{tag}_{k}"] = v
        q, s, dw, qt, st = TS.torch_batch_weighted_silu_and_block_quant_backward(
            g, x, wrow, counts, round_scale=False)
        for k, v in (("q", u8(q)), ("s", f32(s)), ("dw", f32(dw)), ("qt", u8(qt)), ("st", f32(st))):
            out[f"bbwd_{tag}_{k}"] = v
    out["counts"] = np.asarray(counts, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "batch.npz"), **out)
    # ---- permute + pad-to-16 + dual quant (the step before the per-expert SwiGLU) ----
    import test_gather as TG
    out = {}
    m, E, N = 96, 6, 256
    x = bf16_randn(gen, (m, N))
    route = torch.rand((m, E), generator=gen) < 0.3
    route[:, 1] = False          # an expert with no tokens
    route[:5, 4] = True
    probs = torch.rand((m, E), generator=gen) * route
    counts = route.sum(0).tolist()
    tok = torch.arange(m).unsqueeze(0).expand(E, -1)
    indices = tok.masked_select(route.T.contiguous())      # unpadded, expert-major (as torch_make_indices)
    out["x"] = u16(x)
    out["probs"] = probs.numpy()
    out["counts"] = np.asarray(counts, dtype=np.int64)
    out["indices"] = indices.numpy()
    for rs in (False, True):
        q, s, qt, st, pr = TG.torch_batch_block_pad_permute_with_indices(x, indices, probs, counts, round_scale=rs)
        for k, v in (("q", u8(q)), ("s", f32(s)), ("qt", u8(qt)), ("st", f32(st)), ("p", f32(pr))):
            out[f"perm_r{int(rs)}_{k}"] = v
    np.savez_compressed(os.path.join(HERE, "permute.npz"), **out)
    # ---- RMSNorm + float32 router logits + quant (the step beside the norm in the MoE block) ----
    out = {}
    M, K, N = 128, 512, 128
    x = bf16_randn(gen, (M, K), 2)
    nw = bf16_randn(gen, (K,))
    rw = bf16_randn(gen, (N, K))
    out["x"] = u16(x)
    out["norm_weight"] = u16(nw)
    out["route_weight"] = u16(rw)
    for rs in (False, True):
        y, logits, q, s, qt, st = TN.torch_rms_gemm_block_quant_forward(x, nw, rw, round_scale=rs)
        # upstream returns the scales untransposed here; store the kernel layouts
        for k, v in (("y", u16(y)), ("logits", f32(logits)), ("q", u8(q)), ("s", f32(s.t())),
                     ("qt", u8(qt)), ("st", f32(st.t()))):
            out[f"router_r{int(rs)}_{k}"] = v
    np.savez_compressed(os.path.join(HERE, "router.npz"), **out)
    # ---- blockwise-scaled FP8 GEMM (consumer of the wire format) ----
    # upstream has no oracle function for it: the expected value is computed inline in
    # tests/test_blockwise_fp8_gemm.py:56-72 (dequantise, float32 matmul); the same lines are
    # applied here to codes produced by upstream's torch_group_quant.
    out = {}
    M, N, K = 96, 160, 256
    xa = bf16_randn(gen, (M, K))
    wb = bf16_randn(gen, (N, K), 3)
    a_q, a_s = U.torch_group_quant(xa, round_scale=False)      # scales [M, K/128]
    b_q, b_s = U.torch_group_quant(wb, round_scale=False)
    out["a_q"], out["b_q"] = u8(a_q), u8(b_q)
    out["a_s128"], out["b_s128"] = f32(a_s), f32(b_s)
    a_s64 = torch.rand((M, K // 64), generator=gen) * 0.1
    b_s64 = torch.rand((N, K // 64), generator=gen) * 0.1
    out["a_s64"], out["b_s64"] = f32(a_s64), f32(b_s64)
    for B, sa, sb in ((128, a_s, b_s), (64, a_s64, b_s64)):
        x_dq = (a_q.float().view(M, K // B, B) * sa[:, :, None]).view(M, K)
        w_dq = (b_q.float().view(N, K // B, B) * sb[:, :, None]).view(N, K)
        y = x_dq @ w_dq.t()
        out[f"y{B}_f32"] = f32(y)
        out[f"y{B}_bf16"] = u16(y.to(torch.bfloat16))
    np.savez_compressed(os.path.join(HERE, "fp8gemm.npz"), **out)
    # ---- routing map -> destination rows and source-token list (upstream torch_make_indices) ----
    out = {}
    logits = torch.randn((200, 8), generator=gen, dtype=torch.float32)
    logits[:, 3] -= 1000                                  # an expert nobody picks
    probs, route_map, counts, indices, row_id_map = U.torch_make_indices(logits, topk=2, bias=-0.01)
    out["route_map"] = route_map.numpy().astype(np.uint8)
    out["counts"] = counts.numpy().astype(np.int64)
    out["indices"] = indices.numpy().astype(np.int64)
    out["row_id_map"] = row_id_map.numpy().astype(np.int64)
    np.savez_compressed(os.path.join(HERE, "route.npz"), **out)
    # ---- FP8 GEMM with 2-D block scales: upstream computes the expected value inline in
    # tests/test_blockwise_fp8_gemm.py:14-36 (dequantise with a_s[:, None, :, None], float32
    # matmul); the same lines on codes and scales from upstream's torch_block_quant (B = 128) and
    # on random scales (B = 64, as in that test).  Its own generator: the files above stay as they are.
    out = {}
    gbb = torch.Generator().manual_seed(20240608)
    M, N, K = 256, 128, 512
    xa = bf16_randn(gbb, (M, K))
    wb = bf16_randn(gbb, (N, K), 3)
    a_q, a_s = U.torch_block_quant(xa, B=128, round_scale=False)      # scales [M/128, K/128]
    b_q, b_s = U.torch_block_quant(wb, B=128, round_scale=False)
    out["a_q"], out["b_q"] = u8(a_q), u8(b_q)
    out["a_s128"], out["b_s128"] = f32(a_s), f32(b_s)
    a_s64 = torch.rand((M // 64, K // 64), generator=gbb)
    b_s64 = torch.rand((N // 64, K // 64), generator=gbb)
    out["a_s64"], out["b_s64"] = f32(a_s64), f32(b_s64)
    for B, sa, sb in ((128, a_s, b_s), (64, a_s64, b_s64)):
        x_dq = (a_q.float().view(M // B, B, K // B, B) * sa[:, None, :, None]).view(M, K)
        w_dq = (b_q.float().view(N // B, B, K // B, B) * sb[:, None, :, None]).view(N, K)
        y = x_dq @ w_dq.t()
        out[f"y{B}_f32"] = f32(y)
        out[f"y{B}_bf16"] = u16(y.to(torch.bfloat16))
    np.savez_compressed(os.path.join(HERE, "fp8gemm_bb.npz"), **out)
    # ---- smooth-quant recipe (one scale per row after a per-column smoothing divisor): upstream's
    # torch_rms_and_smooth_quant_forward (tests/test_norm.py:52-67) and
    # torch_silu_and_smooth_quant_forward (tests/test_silu.py:56-72), inputs as in their tests
    # (smooth scales 1 + 10 * rand for the norm, tests/test_norm.py:153-156; 1 + rand for SwiGLU,
    # tests/test_silu.py:338).  Its own generator: the files above stay as they are.
    out = {}
    gs = torch.Generator().manual_seed(20240609)
    x = bf16_randn(gs, (96, 512))
    w = (1 + 0.1 * torch.randn((512,), generator=gs)).to(torch.bfloat16)
    sm = 1 + 10 * torch.rand((512,), generator=gs)
    out["norm_x"], out["norm_w"], out["norm_smooth"] = u16(x), u16(w), f32(sm)
    for rs in (False, True):
        q, sc, maxs = TN.torch_rms_and_smooth_quant_forward(x, w, smooth_scale=sm, round_scale=rs)
        out[f"norm_r{int(rs)}_q"], out[f"norm_r{int(rs)}_s"], out[f"norm_r{int(rs)}_maxs"] = u8(q), f32(sc), f32(maxs)
    xs = bf16_randn(gs, (80, 768))
    sm2 = 1 + torch.rand((384,), generator=gs)
    out["silu_x"], out["silu_smooth"] = u16(xs), f32(sm2)
    for rs in (False, True):
        q, sc, maxs = TS.torch_silu_and_smooth_quant_forward(xs, smooth_scale=sm2, round_scale=rs)
        out[f"silu_r{int(rs)}_q"], out[f"silu_r{int(rs)}_s"], out[f"silu_r{int(rs)}_maxs"] = u8(q), f32(sc), f32(maxs)
    # per-expert form: upstream's torch_batch_weighted_silu_and_smooth_quant_forward
    # (tests/test_silu.py:126-160); its maxima (taken after the row weight, unlike the kernel's)
    # are not stored
    counts = [24, 8, 40, 16]          # upstream's helper cannot take an empty expert
    xb = bf16_randn(gs, (sum(counts), 512))
    wb = torch.randn((sum(counts), 1), generator=gs)
    smb = 1 + 10 * torch.rand((len(counts), 256), generator=gs)
    out["batch_x"], out["batch_w"], out["batch_smooth"] = u16(xb), f32(wb), f32(smb)
    out["batch_counts"] = np.asarray(counts, dtype=np.int64)
    for rs, rev in ((False, False), (True, False), (True, True)):
        q, sc, _ = TS.torch_batch_weighted_silu_and_smooth_quant_forward(
            xb, wb, torch.tensor(counts), smooth_scales=smb, round_scale=rs, reverse=rev)
        out[f"batch_r{int(rs)}v{int(rev)}_q"], out[f"batch_r{int(rs)}v{int(rev)}_s"] = u8(q), f32(sc)
    # backward: upstream's torch_silu_and_smooth_quant_backward (tests/test_silu.py:87-110), smooth
    # scales 1 + rand as in tests/test_silu.py:339-342, gradients 0.1 * randn
    gbk = (0.1 * torch.randn((64, 192), generator=gs)).to(torch.bfloat16)
    xbk = bf16_randn(gs, (64, 384))
    sbk = 1 + torch.rand((384,), generator=gs)
    tsbk = 1 + torch.rand((64,), generator=gs)
    out["bwd_g"], out["bwd_x"], out["bwd_smooth"], out["bwd_tsmooth"] = u16(gbk), u16(xbk), f32(sbk), f32(tsbk)
    for rs, rev in ((True, True), (True, False), (False, True)):
        q, sc, qt, sct = TS.torch_silu_and_smooth_quant_backward(gbk, xbk, smooth_scale=sbk, transpose_smooth_scale=tsbk,
                                                                 round_scale=rs, reverse=rev)
        tag = f"bwd_r{int(rs)}v{int(rev)}"
        out[tag + "_q"], out[tag + "_s"], out[tag + "_qt"], out[tag + "_st"] = u8(q), f32(sc), u8(qt), f32(sct)
    # per-expert backward: upstream's torch_batch_weighted_silu_and_smooth_quant_backward
    # (tests/test_silu.py:202-256); counts that are not multiples of 32 exercise the padding
    bc = [24, 8, 40, 16]
    gbb_ = (0.1 * torch.randn((sum(bc), 128), generator=gs)).to(torch.bfloat16)
    xbb_ = bf16_randn(gs, (sum(bc), 256))
    wbb_ = torch.randn((sum(bc), 1), generator=gs)
    sbb_ = 1 + 10 * torch.rand((len(bc), 256), generator=gs)
    tbb_ = 1 + 10 * torch.rand((sum(bc),), generator=gs)
    out["bbwd_g"], out["bbwd_x"], out["bbwd_w"] = u16(gbb_), u16(xbb_), f32(wbb_)
    out["bbwd_smooth"], out["bbwd_tsmooth"] = f32(sbb_), f32(tbb_)
    out["bbwd_counts"] = np.asarray(bc, dtype=np.int64)
    for rs, rev in ((True, False), (True, True), (False, False)):
        q, sc, dw, qt, sct = TS.torch_batch_weighted_silu_and_smooth_quant_backward(
            gbb_, xbb_, wbb_, bc, smooth_scales=sbb_, transpose_smooth_scale=tbb_, round_scale=rs, reverse=rev)
        tag = f"bbwd_r{int(rs)}v{int(rev)}"
        out[tag + "_q"], out[tag + "_s"], out[tag + "_qt"], out[tag + "_st"] = u8(q), f32(sc), u8(qt), f32(sct)
        out["bbwd_dw"] = f32(dw)
    np.savez_compressed(os.path.join(HERE, "smooth.npz"), **out)
    for f in ("quant", "norm", "silu", "batch", "permute", "router", "fp8gemm", "route", "fp8gemm_bb", "smooth"):
        p = os.path.join(HERE, f + ".npz")
        print(p, os.path.getsize(p))


if __name__ == "__main__":
    main()
