// Shared pieces of the one-CTA-per-row kernels: their parameter block, and the two device routines
// of the streaming RMSNorm backward that are used by more than one translation unit.
#pragma once
#include "lh_common.cuh"

namespace lh {

struct SmallParams {
    const uint8_t* x;
    const uint8_t* gamma;
    int64_t M;
    int n;              // output columns
    float eps, inv_n;
    uint8_t* q;         // [M, n] codes
    float* s;           // scales: [M, n/128] when scale_rowmajor, else [n/128, M]
    float* rms;         // SOP_NORM: [M] 1/rms (written, or read when reuse_rms)
    uint8_t* y;         // plain norm: [M, n] bf16 output
    int reuse_rms;
    int scale_rowmajor;
    int round_scale;
    uint8_t* qt;        // backward with COLQ: transposed codes of dy [n, M]
    float* st;          // backward with COLQ: column scales of dy [ceil(M/128), n]
};

template <typename InT>
__device__ __forceinline__ void unpack8(const uint4& r, float2* v) {
    if constexpr (std::is_same<InT, __half>::value) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    } else {
        v[0] = bf16x2_to_f2(r.x); v[1] = bf16x2_to_f2(r.y); v[2] = bf16x2_to_f2(r.z); v[3] = bf16x2_to_f2(r.w);
    }
}

// Transposed 128x1 quantisation of one 128 x 128 tile of dy by the NT threads of a CTA (bit-exact:
// block maxima on the packed 16-bit words, exact quotients on negated values).  Thread t owns the
// 8 columns of column group t & 15 and the RG = 2048 / NT consecutive rows of row group t >> 4.
// Two sweeps over the tile: maxima first, then -- after the 128 column scales went through shared
// memory -- the codes; the second sweep reads the tile again from L1.  A thread's RG codes of one
// column are RG consecutive bytes of the transposed output: one 16-byte (8-byte) store per column.
// M is a multiple of 16, so a row group is either complete or empty.
// Barrier of one role: the whole CTA (ID 0) or the N threads that share named barrier ID.
template <int ID, int N>
__device__ __forceinline__ void role_sync() {
    if constexpr (ID == 0) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(N) : "memory");
}

template <int NT, int BAR>
__device__ __forceinline__ void col_quant_tile(const SmallParams& p, const uint8_t* __restrict__ dy, int band, int ct, int t,
                                               float* cmax /* [NT/16][128] */, float* cs, float* cy) {
    constexpr int RG = 2048 / NT;            // rows per thread: 16 (128 threads) or 8 (256 threads)
    const int l16 = t & 15, rg = t >> 4;
    const int64_t r0 = int64_t(band) * 128 + rg * RG;
    const int c0 = ct * 128 + l16 * 8;
    const bool live = r0 < p.M;              // whole row group inside the matrix
    const int64_t pitch = int64_t(p.n) * 2;
    const uint8_t* base = dy + r0 * pitch + int64_t(c0) * 2;
    uint32_t m[4] = {0u, 0u, 0u, 0u};
    if (live) {
#pragma unroll
        for (int i = 0; i < RG; ++i) {
            const uint4 w = *reinterpret_cast<const uint4*>(base + i * pitch);
            asm("max.bf16x2 %0, %0, %1;" : "+r"(m[0]) : "r"(w.x & 0x7fff7fffu));
            asm("max.bf16x2 %0, %0, %1;" : "+r"(m[1]) : "r"(w.y & 0x7fff7fffu));
            asm("max.bf16x2 %0, %0, %1;" : "+r"(m[2]) : "r"(w.z & 0x7fff7fffu));
            asm("max.bf16x2 %0, %0, %1;" : "+r"(m[3]) : "r"(w.w & 0x7fff7fffu));
        }
    }
    {
        float4* dst = reinterpret_cast<float4*>(cmax + rg * 128 + l16 * 8);
        dst[0] = make_float4(__uint_as_float(m[0] << 16), __uint_as_float(m[0] & 0xffff0000u),
                             __uint_as_float(m[1] << 16), __uint_as_float(m[1] & 0xffff0000u));
        dst[1] = make_float4(__uint_as_float(m[2] << 16), __uint_as_float(m[2] & 0xffff0000u),
                             __uint_as_float(m[3] << 16), __uint_as_float(m[3] & 0xffff0000u));
    }
    role_sync<BAR, NT>();
    if (t < 128) {
        float mx = cmax[t];
#pragma unroll
        for (int g = 1; g < NT / 16; ++g) mx = fmaxf(mx, cmax[g * 128 + t]);
        const float sc = scale_from_amax(mx, p.round_scale != 0);
        cs[t] = sc;
        cy[t] = (sc < 8.0e-28f && mx > 0.f) ? 1.f : -__frcp_rn(sc);   // +1 marks "take IEEE division"
        p.st[int64_t(band) * p.n + ct * 128 + t] = sc;
    }
    role_sync<BAR, NT>();
    if (live) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float4 s4 = *reinterpret_cast<const float4*>(cs + l16 * 8 + 4 * h);
            const float4 y4 = *reinterpret_cast<const float4*>(cy + l16 * 8 + 4 * h);
            const float2 sc2[2] = {make_float2(s4.x, s4.y), make_float2(s4.z, s4.w)};
            const float2 y2[2] = {make_float2(y4.x, y4.y), make_float2(y4.z, y4.w)};
            const bool slow = y4.x > 0.f || y4.y > 0.f || y4.z > 0.f || y4.w > 0.f;   // rare
            uint32_t acc[4][RG / 4];
#pragma unroll
            for (int grp = 0; grp < RG / 4; ++grp) {
                float2 q[4][2];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const uint2 w = *reinterpret_cast<const uint2*>(base + (grp * 4 + r) * pitch + 8 * h);
                    const float2 nd0 = bf16x2_to_neg_f2(w.x), nd1 = bf16x2_to_neg_f2(w.y);
                    q[r][0] = quot_exact2(nd0, sc2[0], y2[0]);
                    q[r][1] = quot_exact2(nd1, sc2[1], y2[1]);
                    if (slow) {
                        if (y2[0].x > 0.f) q[r][0].x = __fdiv_rn(-nd0.x, sc2[0].x);
                        if (y2[0].y > 0.f) q[r][0].y = __fdiv_rn(-nd0.y, sc2[0].y);
                        if (y2[1].x > 0.f) q[r][1].x = __fdiv_rn(-nd1.x, sc2[1].x);
                        if (y2[1].y > 0.f) q[r][1].y = __fdiv_rn(-nd1.y, sc2[1].y);
                    }
                }
                acc[0][grp] = cvt_e4m3x4(q[0][0].x, q[1][0].x, q[2][0].x, q[3][0].x);
                acc[1][grp] = cvt_e4m3x4(q[0][0].y, q[1][0].y, q[2][0].y, q[3][0].y);
                acc[2][grp] = cvt_e4m3x4(q[0][1].x, q[1][1].x, q[2][1].x, q[3][1].x);
                acc[3][grp] = cvt_e4m3x4(q[0][1].y, q[1][1].y, q[2][1].y, q[3][1].y);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint8_t* dst = p.qt + int64_t(c0 + 4 * h + c) * p.M + r0;
                if constexpr (RG == 16) *reinterpret_cast<uint4*>(dst) = make_uint4(acc[c][0], acc[c][1], acc[c][2], acc[c][3]);
                else *reinterpret_cast<uint2*>(dst) = make_uint2(acc[c][0], acc[c][1]);
            }
        }
    }
    // cmax / cs / cy are rewritten only behind the next tile's barriers
}

// RMSNorm backward, streaming: dx = r*g*gamma - r^3 * x * sum(x*g*gamma)/n, dgamma += x*g*r.
// A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; thread t owns 16 consecutive elements
// of every span of 16*NT elements and keeps their dgamma sums in registers for the whole walk.
// The loads of the next row are issued before the second pass over the current one, so every
// resident CTA always has a row in flight.  Per-CTA sums go to partial[blockIdx.x][n]; a second
// kernel adds them in a fixed order.
// The walk of one CTA's rows by its first NT threads.  BAR names the barrier of those threads (0 =
// the whole CTA).  walk_band, when given, receives the band (row / 128) the walk has reached.
// FULL: n is exactly SPANS * 16 * NT, so no thread ever has an empty span: the column tests and the
// zero-fill of the load registers go away.  The two row sums travel as one float2 (packed adds,
// 16-byte shared-memory reads), in the same order as two scalar reductions would take.
// gam_s: 4 * SPANS * NT float4 of shared memory.  gamma sits there as float32 for the whole walk, laid
// out so that a warp's 16-byte reads are 512 consecutive bytes: both passes read it with two
// conflict-free LDS.128 per 8 elements instead of a global load and eight unpack operations (the
// opcode counter showed 1.0 of the kernel's instructions per element and pass going into that).
template <int SPANS, int NT, bool WIDE, bool QDY, int BAR, bool FULL = false>
__device__ __forceinline__ void norm_bwd_walk(const SmallParams& p, const uint8_t* __restrict__ dy, float* __restrict__ partial,
                                              float2 (*wsum)[NT / 32], volatile int* walk_band, float4* gam_s) {
    // L2 prefetch of the row after next: the plain backward waits on its own loads (issue 29 % active, long-scoreboard
    // stalls) and gains 9-18 % from it; with the row codes of dy the kernel is busier and measured 1 % slower with it
    constexpr bool L2PF = !QDY;
    constexpr int SPAN = 16 * NT, NW = NT / 32;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    uint4 xr[2 * SPANS], gr[2 * SPANS];
    float2 acc[8 * SPANS];
#pragma unroll
    for (int i = 0; i < 8 * SPANS; ++i) acc[i] = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 2 * SPANS; ++i) {     // this thread's gamma: chunk i = 8 elements = float4 2 i and 2 i + 1
        const int col = (i >> 1) * SPAN + t * 16 + (i & 1) * 8;
        float2 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = make_float2(0.f, 0.f);
        if (FULL || col < p.n) unpack8<__nv_bfloat16>(__ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2)), v);
        gam_s[(2 * i) * NT + t] = make_float4(v[0].x, v[0].y, v[1].x, v[1].y);
        gam_s[(2 * i + 1) * NT + t] = make_float4(v[2].x, v[2].y, v[3].x, v[3].y);
    }
    // every thread reads back only what it wrote itself: no barrier is needed
    auto gamma_at = [&](int i, float2* w) {   // i-th 8-element chunk of this thread's gamma
        const float4 a = gam_s[(2 * i) * NT + t], b = gam_s[(2 * i + 1) * NT + t];
        w[0] = make_float2(a.x, a.y); w[1] = make_float2(a.z, a.w);
        w[2] = make_float2(b.x, b.y); w[3] = make_float2(b.z, b.w);
    };
    auto fetch = [&](int64_t row) {
#pragma unroll
        for (int i = 0; i < SPANS; ++i) {
            const int col = i * SPAN + t * 16;
            if constexpr (!FULL) xr[2 * i] = xr[2 * i + 1] = gr[2 * i] = gr[2 * i + 1] = make_uint4(0, 0, 0, 0);
            if (row < p.M && (FULL || col < p.n)) {   // past the last row nothing is loaded and nothing is used
                const int64_t off = (row * p.n + col) * 2;
                if constexpr (WIDE) {   // x, dy and dx are 32-byte aligned
                    ld_global_256(p.x + off, xr[2 * i], xr[2 * i + 1]);
                    ld_global_256(dy + off, gr[2 * i], gr[2 * i + 1]);
                } else {
                    xr[2 * i] = *reinterpret_cast<const uint4*>(p.x + off);
                    xr[2 * i + 1] = *reinterpret_cast<const uint4*>(p.x + off + 16);
                    gr[2 * i] = *reinterpret_cast<const uint4*>(dy + off);
                    gr[2 * i + 1] = *reinterpret_cast<const uint4*>(dy + off + 16);
                }
            }
        }
    };
    int64_t row = blockIdx.x;
    fetch(row);
    int par = 0;
    for (; row < p.M; row += gridDim.x, par ^= 1) {
        if (walk_band != nullptr && t == 0) *walk_band = int(row >> 7);
        // pass 1: sum x^2 and sum x*g*gamma; keep the packed words, the floats are rebuilt in pass 2
        float2 sc = make_float2(0.f, 0.f), ss = sc;
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) {
            float2 x[4], g[4], w[4];
            unpack8<__nv_bfloat16>(xr[i], x);
            unpack8<__nv_bfloat16>(gr[i], g);
            gamma_at(i, w);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sc = fma2(x[j], mul2(g[j], w[j]), sc);
                ss = fma2(x[j], x[j], ss);
            }
        }
        float2 cs = make_float2(sc.x + sc.y, ss.x + ss.y);
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1)
            cs = add2(cs, make_float2(__shfl_xor_sync(0xffffffffu, cs.x, d), __shfl_xor_sync(0xffffffffu, cs.y, d)));
        if (lane == 0) wsum[par][warp] = cs;
        role_sync<BAR, NT>();   // the buffer of the other parity was last read before the previous barrier
        float2 tot = wsum[par][0];
#pragma unroll
        for (int w = 1; w < NW; ++w) tot = add2(tot, wsum[par][w]);
        const float ctot = tot.x, stot = tot.y;
        const float r = p.reuse_rms ? p.rms[row] : rsqrt_nr(fmaf(stot, p.inv_n, p.eps));
        const float2 ncoef = splat2(-(r * r * r * ctot * p.inv_n));
        // QDY: dy is unpacked NEGATED in the second pass (the exact quotient wants -dy, and the sign
        // flip is free in the widening); the dx and dgamma terms then take -r, which gives the same
        // bits: (-r) * ((-g) * w) == r * (g * w) and ((x * (-g)) * (-r) == (x * g) * r exactly
        const float2 r2 = splat2(QDY ? -r : r);
        // pass 2 on copies, so that the next row's loads can already land in xr / gr
        uint4 xc[2 * SPANS], gc[2 * SPANS];
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) { xc[i] = xr[i]; gc[i] = gr[i]; }
        fetch(row + gridDim.x);
        if constexpr (L2PF) {
            // a row two or three ahead: pulled into L2 now, so that its register loads find it there; a thread covers 32 bytes per span, every fourth thread asks for the 128-byte line
            // distance in rows of this CTA: 3 measured best for one span per thread and for 256 threads (65536 x 2048:
            // 123 vs 135 us at distance 2; 32768 x 8192: 234 vs 255 us), 2 for two spans of 128 threads (16384 x 4096:
            // 67.7 vs 70.1 us at distance 3)
            constexpr int AHEAD = (SPANS == 2 && NT == 128) ? 2 : 3;
            const int64_t prow = row + AHEAD * int64_t(gridDim.x);
            if (prow < p.M && (t & 3) == 0) {
#pragma unroll
                for (int i = 0; i < SPANS; ++i) {
                    const int col = i * SPAN + t * 16;
                    if (FULL || col < p.n) {
                        const int64_t off = (prow * p.n + col) * 2;
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x + off));
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(dy + off));
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < SPANS; ++i) {
            const int col = i * SPAN + t * 16;
            uint32_t o[8];
            // QDY: the row-wise 1x128 codes and scales of dy from the same registers (bit-exact):
            // block maximum on the packed words (8 lanes = one block), then exact quotients
            float qs = 0.f, qny = 0.f;
            bool qtiny = false;
            uint32_t qc[4];
            if constexpr (QDY) {
                const uint32_t w8[8] = {gc[2 * i].x, gc[2 * i].y, gc[2 * i].z, gc[2 * i].w,
                                        gc[2 * i + 1].x, gc[2 * i + 1].y, gc[2 * i + 1].z, gc[2 * i + 1].w};
                uint32_t m0 = w8[0] & 0x7fff7fffu, m1 = w8[1] & 0x7fff7fffu;
#pragma unroll
                for (int j = 2; j < 8; j += 2) {
                    asm("max.bf16x2 %0, %0, %1;" : "+r"(m0) : "r"(w8[j] & 0x7fff7fffu));
                    asm("max.bf16x2 %0, %0, %1;" : "+r"(m1) : "r"(w8[j + 1] & 0x7fff7fffu));
                }
                asm("max.bf16x2 %0, %0, %1;" : "+r"(m0) : "r"(m1));
                float amax = fmaxf(__uint_as_float(m0 << 16), __uint_as_float(m0 & 0xffff0000u));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                qs = scale_from_amax(amax, p.round_scale != 0);
                qtiny = qs < 8.0e-28f && amax > 0.f;      // residual of the exact quotient could underflow
                qny = -__frcp_rn(qs);
                if ((t & 7) == 0 && (FULL || col < p.n)) p.s[int64_t(col >> 7) * p.M + row] = qs;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float2 x[4], g[4], w[4];
                unpack8<__nv_bfloat16>(xc[2 * i + h], x);
                if constexpr (QDY) {
                    g[0] = bf16x2_to_neg_f2(gc[2 * i + h].x); g[1] = bf16x2_to_neg_f2(gc[2 * i + h].y);
                    g[2] = bf16x2_to_neg_f2(gc[2 * i + h].z); g[3] = bf16x2_to_neg_f2(gc[2 * i + h].w);
                } else {
                    unpack8<__nv_bfloat16>(gc[2 * i + h], g);
                }
                gamma_at(2 * i + h, w);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 d = fma2(ncoef, x[j], mul2(r2, mul2(g[j], w[j])));
                    acc[8 * i + 4 * h + j] = fma2(mul2(x[j], g[j]), r2, acc[8 * i + 4 * h + j]);
                    o[4 * h + j] = pack_bf16x2(d.x, d.y);
                }
                if constexpr (QDY) {
                    float2 q[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) q[j] = quot_exact2(g[j], splat2(qs), splat2(qny));   // g holds -dy
                    if (qtiny) {   // rare
#pragma unroll
                        for (int j = 0; j < 4; ++j) q[j] = make_float2(__fdiv_rn(-g[j].x, qs), __fdiv_rn(-g[j].y, qs));
                    }
                    qc[2 * h] = cvt_e4m3x4(q[0].x, q[0].y, q[1].x, q[1].y);
                    qc[2 * h + 1] = cvt_e4m3x4(q[2].x, q[2].y, q[3].x, q[3].y);
                }
            }
            if constexpr (QDY) {
                if (FULL || col < p.n) *reinterpret_cast<uint4*>(p.q + row * p.n + col) = make_uint4(qc[0], qc[1], qc[2], qc[3]);
            }
            if (FULL || col < p.n) {
                uint8_t* dst = p.y + (row * p.n + col) * 2;
                if constexpr (WIDE) {
                    st_global_256(dst, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
                } else {
                    *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(dst + 16) = make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
        }
    }
    if (walk_band != nullptr && t == 0) *walk_band = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < SPANS; ++i) {
        const int col = i * SPAN + t * 16;
        if (FULL || col < p.n) {
            float4* dst = reinterpret_cast<float4*>(partial + int64_t(blockIdx.x) * p.n + col);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                dst[k] = make_float4(acc[8 * i + 2 * k].x, acc[8 * i + 2 * k].y, acc[8 * i + 2 * k + 1].x, acc[8 * i + 2 * k + 1].y);
        }
    }
}

// Launches the two-role kernel (lh_duo.cu: compiled without relocatable device code, which
// setmaxnreg needs).  p.q / p.s / p.qt / p.st set, M % 16 == 0.  Returns LH_ERR_ARG - 1000 when the
// register split does not fit, in which case nothing was enqueued.
int small_norm_bwd_duo(const SmallParams& p, const uint8_t* dy, float* partial, unsigned grid, bool wide, cudaStream_t stream);

}  // namespace lh
