// One-CTA-per-row kernels for the row-only outputs of small and medium problems.
//
// A persistent TMA ring (lh_rows.cu) reaches the copy bandwidth once every CTA streams dozens
// of slabs, but a problem of a few tens of megabytes is over before the ring is in steady
// state.  Here the grid is one small CTA (128 threads) per row: the hardware block scheduler
// keeps up to 16 CTAs per SM in flight, each thread issues its loads at once, and nothing
// is staged through shared memory.  Thread t owns 16 consecutive elements (two 16-byte
// chunks) of every 2048-element span of its row, so a 1x128 block is 8 consecutive lanes.
#include "lh_common.cuh"

namespace lh {

namespace {

enum : int { SOP_GROUP = 0, SOP_NORM = 1, SOP_SILU = 2 };

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

// 32 contiguous bytes of a thread's span: one 256-bit load when the tensor is 32-byte aligned
template <bool WIDE>
__device__ __forceinline__ void load32(const uint8_t* src, uint4& a, uint4& b) {
    if constexpr (WIDE) {
        ld_global_256(src, a, b);
    } else {
        a = *reinterpret_cast<const uint4*>(src);
        b = *reinterpret_cast<const uint4*>(src + 16);
    }
}
template <bool WIDE>
__device__ __forceinline__ void store32(uint8_t* dst, const uint4& a, const uint4& b) {
    if constexpr (WIDE) {
        st_global_256(dst, a, b);
    } else {
        *reinterpret_cast<uint4*>(dst) = a;
        *reinterpret_cast<uint4*>(dst + 16) = b;
    }
}

// 16 values of one thread (half... an eighth of a 1x128 block) -> block scale -> 16 codes, stored
template <bool EXACT>
__device__ __forceinline__ void quant16(const SmallParams& p, int64_t row, int col, bool valid, float2* v) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
        a0 = max3abs(v[j].x, v[j].y, a0);
        a1 = max3abs(v[j + 1].x, v[j + 1].y, a1);
    }
    float amax = valid ? fmaxf(a0, a1) : 0.f;
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const float scale = scale_from_amax(amax, p.round_scale != 0);
    if (!valid) return;
    if constexpr (EXACT) {
        if (scale < 8.0e-28f && amax > 0.f) {          // rare: residual of the exact quotient could underflow
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = make_float2(__fdiv_rn(v[j].x, scale), __fdiv_rn(v[j].y, scale));
        } else {
            const float y = __frcp_rn(scale);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float q0 = v[j].x * y, q1 = v[j].y * y;
                v[j] = make_float2(fmaf(fmaf(scale, q0, -v[j].x), -y, q0), fmaf(fmaf(scale, q1, -v[j].y), -y, q1));
            }
        }
    } else {
        const float2 y2 = splat2(rcp_approx(scale));
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = mul2(v[j], y2);
    }
    *reinterpret_cast<uint4*>(p.q + row * p.n + col) =
        make_uint4(cvt_e4m3x4(v[0].x, v[0].y, v[1].x, v[1].y), cvt_e4m3x4(v[2].x, v[2].y, v[3].x, v[3].y),
                   cvt_e4m3x4(v[4].x, v[4].y, v[5].x, v[5].y), cvt_e4m3x4(v[6].x, v[6].y, v[7].x, v[7].y));
    if ((threadIdx.x & 7) == 0) {
        const int b = col >> 7;
        if (p.scale_rowmajor) p.s[row * (p.n >> 7) + b] = scale;
        else p.s[int64_t(b) * p.M + row] = scale;
    }
}

// SOP_GROUP / SOP_SILU: spans of 2048 output elements are independent
template <int SOP, typename InT, bool WIDE>
__global__ void __launch_bounds__(128)
small_stream_kernel(const __grid_constant__ SmallParams p) {
    const int64_t row = blockIdx.x;
    const int64_t in_row = SOP == SOP_SILU ? 2 * int64_t(p.n) : int64_t(p.n);
    const uint8_t* xr = p.x + row * in_row * 2;
    for (int c0 = 0; c0 < p.n; c0 += 2048) {
        const int col = c0 + threadIdx.x * 16;
        const bool valid = col < p.n;
        uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0, b0 = a0, b1 = a0;
        if (valid) {
            load32<WIDE>(xr + int64_t(col) * 2, a0, a1);
            if constexpr (SOP == SOP_SILU) load32<WIDE>(xr + (int64_t(p.n) + col) * 2, b0, b1);
        }
        float2 v[8];
        unpack8<InT>(a0, v);
        unpack8<InT>(a1, v + 4);
        if constexpr (SOP == SOP_SILU) {
            float2 g[8];
            unpack8<InT>(b0, g);
            unpack8<InT>(b1, g + 4);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = mul2(mul2(sigmoid_fast2(v[j]), v[j]), g[j]);
        }
        quant16<SOP == SOP_GROUP>(p, row, col, valid, v);
    }
}

// Pure 1x128 quantiser (bit-exact).  A unit is one 2048-element span of one row; a CTA takes U
// consecutive units and every thread issues the loads of all of them before it touches the
// first, which is what keeps enough bytes in flight per SM when the whole problem is a few
// waves of CTAs.  Values are held negated so that the exact quotients are packed instructions.
template <typename InT>
__device__ __forceinline__ void unpack8_neg(const uint4& r, float2* v) {
    if constexpr (std::is_same<InT, __half>::value) {
        const uint32_t w[4] = {r.x ^ 0x80008000u, r.y ^ 0x80008000u, r.z ^ 0x80008000u, r.w ^ 0x80008000u};
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    } else {
        v[0] = bf16x2_to_neg_f2(r.x); v[1] = bf16x2_to_neg_f2(r.y);
        v[2] = bf16x2_to_neg_f2(r.z); v[3] = bf16x2_to_neg_f2(r.w);
    }
}

// FLAT: the 1x128 blocks of the row-major output are numbered through (block b = row * n/128 + column
// block) and a unit is 16 consecutive blocks whatever rows they fall in, so that every thread has
// work for any n (n = 1408 fills 69 % of a 2048-element span); `spans` is then n/128.  The price is
// one integer division per thread and unit.
// FULL (span form only): the row is a whole number of spans and the grid covers the units exactly, so
// every thread of every CTA has U units of work: no bounds tests, no zero-fill of the load registers.
template <int SOP, typename InT, int U, bool WIDE, bool FLAT = false, bool FULL = false>
__global__ void __launch_bounds__(128)
small_units_kernel(const __grid_constant__ SmallParams p, int spans, int64_t units) {
    static_assert(!(FLAT && FULL), "FULL is a property of the span form");
    constexpr bool SILU = SOP == SOP_SILU;
    const int64_t u0 = int64_t(blockIdx.x) * U;
    int64_t row = FLAT ? 0 : u0 / spans;
    int span = FLAT ? 0 : int(u0 - row * spans);
    const int64_t in_row = SILU ? 2 * int64_t(p.n) : int64_t(p.n);
    uint4 raw[2 * U], rawb[SILU ? 2 * U : 1];
    int64_t rows[U];
    int cols[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
        if constexpr (FLAT) {
            const int64_t b = (u0 + k) * 16 + (threadIdx.x >> 3);
            row = b / spans;
            cols[k] = row < p.M ? int(b - row * spans) * 128 + int(threadIdx.x & 7) * 16 : p.n;
        } else {
            cols[k] = span * 2048 + threadIdx.x * 16;
        }
        rows[k] = row;
        if constexpr (!FULL) {
            raw[2 * k] = raw[2 * k + 1] = make_uint4(0, 0, 0, 0);
            if constexpr (SILU) rawb[2 * k] = rawb[2 * k + 1] = make_uint4(0, 0, 0, 0);
        }
        if (FULL || (u0 + k < units && cols[k] < p.n)) {
            const uint8_t* src = p.x + (row * in_row + cols[k]) * 2;
            if constexpr (WIDE) {   // x is 32-byte aligned: one 256-bit load per 16 elements
                ld_global_256(src, raw[2 * k], raw[2 * k + 1]);
                if constexpr (SILU) ld_global_256(src + int64_t(p.n) * 2, rawb[2 * k], rawb[2 * k + 1]);
            } else {
                raw[2 * k] = *reinterpret_cast<const uint4*>(src);
                raw[2 * k + 1] = *reinterpret_cast<const uint4*>(src + 16);
                if constexpr (SILU) {
                    rawb[2 * k] = *reinterpret_cast<const uint4*>(src + int64_t(p.n) * 2);
                    rawb[2 * k + 1] = *reinterpret_cast<const uint4*>(src + int64_t(p.n) * 2 + 16);
                }
            }
        } else {
            cols[k] = p.n;   // nothing to do for this unit
        }
        if constexpr (!FLAT) {
            if (++span == spans) { span = 0; ++row; }
        }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
        float2 v[8];
        const bool valid = FULL || cols[k] < p.n;
        if constexpr (SILU) {
            float2 g[8];
            unpack8<InT>(raw[2 * k], v);
            unpack8<InT>(raw[2 * k + 1], v + 4);
            unpack8<InT>(rawb[2 * k], g);
            unpack8<InT>(rawb[2 * k + 1], g + 4);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = mul2(mul2(sigmoid_fast2(v[j]), v[j]), g[j]);
            quant16<false>(p, rows[k], cols[k], valid, v);
        } else {
            unpack8_neg<InT>(raw[2 * k], v);
            unpack8_neg<InT>(raw[2 * k + 1], v + 4);
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                a0 = max3abs(v[j].x, v[j].y, a0);
                a1 = max3abs(v[j + 1].x, v[j + 1].y, a1);
            }
            float amax = fmaxf(a0, a1);                   // zeros where there is nothing
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            const float scale = scale_from_amax(amax, p.round_scale != 0);
            if (!valid) continue;
            if (scale < 8.0e-28f && amax > 0.f) {          // rare: residual of the exact quotient could underflow
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = make_float2(__fdiv_rn(-v[j].x, scale), __fdiv_rn(-v[j].y, scale));
            } else {
                const float2 s2 = splat2(scale), ny2 = splat2(-__frcp_rn(scale));
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = quot_exact2(v[j], s2, ny2);
            }
            *reinterpret_cast<uint4*>(p.q + rows[k] * p.n + cols[k]) =
                make_uint4(cvt_e4m3x4(v[0].x, v[0].y, v[1].x, v[1].y), cvt_e4m3x4(v[2].x, v[2].y, v[3].x, v[3].y),
                           cvt_e4m3x4(v[4].x, v[4].y, v[5].x, v[5].y), cvt_e4m3x4(v[6].x, v[6].y, v[7].x, v[7].y));
            if ((threadIdx.x & 7) == 0) {
                const int b = cols[k] >> 7;
                if (p.scale_rowmajor) p.s[rows[k] * (p.n >> 7) + b] = scale;
                else p.s[int64_t(b) * p.M + rows[k]] = scale;
            }
        }
    }
}

// SOP_NORM: the row (n <= 2048 * SPANS) stays in registers as packed 16-bit words
// QUANT: codes + scales; otherwise the 16-bit y itself (plain RMSNorm forward).  NT threads
// per row, thread t owns 16 consecutive elements of every span of 16*NT elements.
template <int SPANS, bool QUANT, int NT, bool WIDE>
__global__ void __launch_bounds__(NT, (SPANS == 1 && NT == 128) ? 8 : 1)
small_norm_kernel(const __grid_constant__ SmallParams p) {
    constexpr int SPAN = 16 * NT;
    __shared__ float wsum[NT / 32];
    const int64_t row = blockIdx.x;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint8_t* xr = p.x + row * int64_t(p.n) * 2;
    // gamma is fetched up front for narrow rows; for wide rows (4 spans) that would cost 32 more
    // registers and a fifth of the resident warps, so it is read (from L1) when it is needed
    constexpr bool GAMMA_EARLY = SPANS < 4;
    // Wide rows with the quantising epilogue: keeping the row in registers leaves room for only
    // five CTAs per SM and the kernel waits on its own latency chain.  Instead the sum pass streams
    // the row and the second pass reads it again -- the 16 KB row is still in L1 (no shared memory
    // is used, so the whole 256 KB is cache) -- which halves the registers.
    constexpr bool REREAD = QUANT && SPANS >= 4;
    uint4 raw[REREAD ? 2 : 2 * SPANS], graw[GAMMA_EARLY ? 2 * SPANS : 2];
    float2 s0 = make_float2(0.f, 0.f), s1 = s0;
    if constexpr (REREAD) {
        uint4 tmp[2 * SPANS];
#pragma unroll
        for (int i = 0; i < SPANS; ++i) {
            const int col = i * SPAN + t * 16;
            tmp[2 * i] = tmp[2 * i + 1] = make_uint4(0, 0, 0, 0);
            if (col < p.n) {
                load32<WIDE>(xr + int64_t(col) * 2, tmp[2 * i], tmp[2 * i + 1]);
            }
        }
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) {
            float2 v[4];
            unpack8<__nv_bfloat16>(tmp[i], v);
            s0 = fma2(v[0], v[0], s0); s1 = fma2(v[1], v[1], s1);
            s0 = fma2(v[2], v[2], s0); s1 = fma2(v[3], v[3], s1);
        }
    } else {
#pragma unroll
        for (int i = 0; i < SPANS; ++i) {
            const int col = i * SPAN + t * 16;
            raw[2 * i] = raw[2 * i + 1] = make_uint4(0, 0, 0, 0);
            if constexpr (GAMMA_EARLY) graw[2 * i] = graw[2 * i + 1] = make_uint4(0, 0, 0, 0);
            if (col < p.n) {
                load32<WIDE>(xr + int64_t(col) * 2, raw[2 * i], raw[2 * i + 1]);
                if constexpr (GAMMA_EARLY) {
                    graw[2 * i] = __ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2));
                    graw[2 * i + 1] = __ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2 + 16));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) {
            float2 v[4];
            unpack8<__nv_bfloat16>(raw[i], v);
            s0 = fma2(v[0], v[0], s0); s1 = fma2(v[1], v[1], s1);
            s0 = fma2(v[2], v[2], s0); s1 = fma2(v[3], v[3], s1);
        }
    }
    s0 = add2(s0, s1);
    float ss = s0.x + s0.y;
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    if (lane == 0) wsum[warp] = ss;
    __syncthreads();
    // four warps: the same pairing as the persistent walk kernel, so that both give the same bits
    // for a row and a result does not depend on which of the two a problem size selects
    float tot = 0.f;
    if constexpr (NT == 128) {
        tot = (wsum[0] + wsum[1]) + (wsum[2] + wsum[3]);
    } else {
#pragma unroll
        for (int w = 0; w < NT / 32; ++w) tot += wsum[w];
    }
    float r;
    if (!QUANT && p.reuse_rms) {
        r = p.rms[row];
    } else {
        r = rsqrt_nr(fmaf(tot, p.inv_n, p.eps));
        if (t == 0 && p.rms != nullptr) p.rms[row] = r;
    }
    const float2 r2 = splat2(r);
#pragma unroll
    for (int i = 0; i < SPANS; ++i) {
        const int col = i * SPAN + t * 16;
        if (i * SPAN >= p.n) break;                       // uniform
        float2 v[8], g[8];
        if constexpr (REREAD) {
            raw[0] = raw[1] = make_uint4(0, 0, 0, 0);
            if (col < p.n) {
                load32<WIDE>(xr + int64_t(col) * 2, raw[0], raw[1]);
            }
            unpack8<__nv_bfloat16>(raw[0], v);
            unpack8<__nv_bfloat16>(raw[1], v + 4);
        } else {
            unpack8<__nv_bfloat16>(raw[2 * i], v);
            unpack8<__nv_bfloat16>(raw[2 * i + 1], v + 4);
        }
        if constexpr (GAMMA_EARLY) {
            unpack8<__nv_bfloat16>(graw[2 * i], g);
            unpack8<__nv_bfloat16>(graw[2 * i + 1], g + 4);
        } else {
            uint4 g0 = make_uint4(0, 0, 0, 0), g1 = g0;
            if (col < p.n) {
                g0 = __ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2));
                g1 = __ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2 + 16));
            }
            unpack8<__nv_bfloat16>(g0, g);
            unpack8<__nv_bfloat16>(g1, g + 4);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = mul2(mul2(v[j], r2), g[j]);
        if constexpr (QUANT) {
            if (p.y != nullptr && col < p.n) {           // the 16-bit y as well (RMSNorm + router logits + quant)
                store32<WIDE>(p.y + (row * p.n + col) * 2,
                              make_uint4(pack_bf16x2(v[0].x, v[0].y), pack_bf16x2(v[1].x, v[1].y),
                                         pack_bf16x2(v[2].x, v[2].y), pack_bf16x2(v[3].x, v[3].y)),
                              make_uint4(pack_bf16x2(v[4].x, v[4].y), pack_bf16x2(v[5].x, v[5].y),
                                         pack_bf16x2(v[6].x, v[6].y), pack_bf16x2(v[7].x, v[7].y)));
            }
            quant16<false>(p, row, col, col < p.n, v);
        } else if (col < p.n) {
            store32<WIDE>(p.y + (row * p.n + col) * 2,
                          make_uint4(pack_bf16x2(v[0].x, v[0].y), pack_bf16x2(v[1].x, v[1].y),
                                     pack_bf16x2(v[2].x, v[2].y), pack_bf16x2(v[3].x, v[3].y)),
                          make_uint4(pack_bf16x2(v[4].x, v[4].y), pack_bf16x2(v[5].x, v[5].y),
                                     pack_bf16x2(v[6].x, v[6].y), pack_bf16x2(v[7].x, v[7].y)));
        }
    }
}

// RMSNorm backward, streaming: dx = r*g*gamma - r^3 * x * sum(x*g*gamma)/n, dgamma += x*g*r.
// A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; thread t owns 16 consecutive elements
// of every span of 16*NT elements and keeps their dgamma sums in registers for the whole walk.
// The loads of the next row are issued before the second pass over the current one, so every
// resident CTA always has a row in flight.  Per-CTA sums go to partial[blockIdx.x][n]; a second
// kernel adds them in a fixed order.
// Transposed 128x1 quantisation of one 128 x 128 tile of dy by the NT threads of a CTA (bit-exact:
// block maxima on the packed 16-bit words, exact quotients on negated values).  Thread t owns the
// 8 columns of column group t & 15 and the RG = 2048 / NT consecutive rows of row group t >> 4.
// Two sweeps over the tile: maxima first, then -- after the 128 column scales went through shared
// memory -- the codes; the second sweep reads the tile again from L1.  A thread's RG codes of one
// column are RG consecutive bytes of the transposed output: one 16-byte (8-byte) store per column.
// M is a multiple of 16, so a row group is either complete or empty.
template <int NT>
__device__ __forceinline__ void col_quant_tile(const SmallParams& p, const uint8_t* __restrict__ dy, int band, int ct,
                                               float* cmax /* [NT/16][128] */, float* cs, float* cy) {
    constexpr int RG = 2048 / NT;            // rows per thread: 16 (128 threads) or 8 (256 threads)
    const int t = threadIdx.x, l16 = t & 15, rg = t >> 4;
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
    __syncthreads();
    if (t < 128) {
        float mx = cmax[t];
#pragma unroll
        for (int g = 1; g < NT / 16; ++g) mx = fmaxf(mx, cmax[g * 128 + t]);
        const float sc = scale_from_amax(mx, p.round_scale != 0);
        cs[t] = sc;
        cy[t] = (sc < 8.0e-28f && mx > 0.f) ? 1.f : -__frcp_rn(sc);   // +1 marks "take IEEE division"
        p.st[int64_t(band) * p.n + ct * 128 + t] = sc;
    }
    __syncthreads();
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

// COLQ: the kernel also writes the transposed 128x1 codes and scales of dy.  The column work is
// cut into 128 x 128 tiles dealt round-robin to the CTAs; a CTA takes its next tile once the walk
// has passed the tile's band, when the band's rows of dy are still in L2 (nothing depends on the
// order: read early, the tile comes from HBM and the walk's read hits L2 instead), so dy crosses
// the HBM interface once.
template <int SPANS, int NT, int MINB, bool WIDE, bool QDY, bool COLQ = false>
__global__ void __launch_bounds__(NT, MINB)
small_norm_bwd_kernel(const __grid_constant__ SmallParams p, const uint8_t* __restrict__ dy, float* __restrict__ partial) {
    constexpr int SPAN = 16 * NT, NW = NT / 32;
    __shared__ float wsum[2][2][NW];
    __shared__ __align__(16) float cq_cmax[COLQ ? (NT / 16) * 128 : 4];
    __shared__ __align__(16) float cq_cs[COLQ ? 128 : 4], cq_cy[COLQ ? 128 : 4];
    const int nct = p.n >> 7;
    const int64_t col_tiles = COLQ ? ((p.M + 127) >> 7) * nct : 0;
    int64_t next_tile = blockIdx.x;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    // gamma stays in registers for one span per thread; with two it is re-read (L1 hits) so that
    // three CTAs fit an SM without spills
    constexpr bool GAM_REG = SPANS == 1;
    uint4 xr[2 * SPANS], gr[2 * SPANS], gam[GAM_REG ? 2 * SPANS : 1];
    float2 acc[8 * SPANS];
#pragma unroll
    for (int i = 0; i < 8 * SPANS; ++i) acc[i] = make_float2(0.f, 0.f);
    auto gamma_at = [&](int i) -> uint4 {     // i-th 16-byte chunk of this thread's gamma
        if constexpr (GAM_REG) {
            return gam[i];
        } else {
            const int col = (i >> 1) * SPAN + t * 16 + (i & 1) * 8;
            return col < p.n ? __ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2)) : make_uint4(0, 0, 0, 0);
        }
    };
    if constexpr (GAM_REG) {
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) {
            const int col = (i >> 1) * SPAN + t * 16 + (i & 1) * 8;
            gam[i] = col < p.n ? __ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2)) : make_uint4(0, 0, 0, 0);
        }
    }
    auto fetch = [&](int64_t row) {
#pragma unroll
        for (int i = 0; i < SPANS; ++i) {
            const int col = i * SPAN + t * 16;
            xr[2 * i] = xr[2 * i + 1] = gr[2 * i] = gr[2 * i + 1] = make_uint4(0, 0, 0, 0);
            if (row < p.M && col < p.n) {
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
        // pass 1: sum x^2 and sum x*g*gamma; keep the packed words, the floats are rebuilt in pass 2
        float2 sc = make_float2(0.f, 0.f), ss = sc;
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) {
            float2 x[4], g[4], w[4];
            unpack8<__nv_bfloat16>(xr[i], x);
            unpack8<__nv_bfloat16>(gr[i], g);
            unpack8<__nv_bfloat16>(gamma_at(i), w);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sc = fma2(x[j], mul2(g[j], w[j]), sc);
                ss = fma2(x[j], x[j], ss);
            }
        }
        float c = sc.x + sc.y, s = ss.x + ss.y;
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) {
            c += __shfl_xor_sync(0xffffffffu, c, d);
            s += __shfl_xor_sync(0xffffffffu, s, d);
        }
        if (lane == 0) { wsum[par][0][warp] = c; wsum[par][1][warp] = s; }
        __syncthreads();   // the buffer of the other parity was last read before the previous barrier
        float ctot = 0.f, stot = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) { ctot += wsum[par][0][w]; stot += wsum[par][1][w]; }
        const float r = p.reuse_rms ? p.rms[row] : rsqrt_nr(fmaf(stot, p.inv_n, p.eps));
        const float2 ncoef = splat2(-(r * r * r * ctot * p.inv_n));
        const float2 r2 = splat2(r);
        // pass 2 on copies, so that the next row's loads can already land in xr / gr
        uint4 xc[2 * SPANS], gc[2 * SPANS];
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) { xc[i] = xr[i]; gc[i] = gr[i]; }
        fetch(row + gridDim.x);
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
                if ((t & 7) == 0 && col < p.n) p.s[int64_t(col >> 7) * p.M + row] = qs;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float2 x[4], g[4], w[4];
                unpack8<__nv_bfloat16>(xc[2 * i + h], x);
                unpack8<__nv_bfloat16>(gc[2 * i + h], g);
                unpack8<__nv_bfloat16>(gamma_at(2 * i + h), w);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 d = fma2(ncoef, x[j], mul2(r2, mul2(g[j], w[j])));
                    acc[8 * i + 4 * h + j] = fma2(mul2(x[j], g[j]), r2, acc[8 * i + 4 * h + j]);
                    o[4 * h + j] = pack_bf16x2(d.x, d.y);
                }
                if constexpr (QDY) {
                    float2 q[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) q[j] = quot_exact2(mul2(g[j], splat2(-1.f)), splat2(qs), splat2(qny));
                    if (qtiny) {   // rare
#pragma unroll
                        for (int j = 0; j < 4; ++j) q[j] = make_float2(__fdiv_rn(g[j].x, qs), __fdiv_rn(g[j].y, qs));
                    }
                    qc[2 * h] = cvt_e4m3x4(q[0].x, q[0].y, q[1].x, q[1].y);
                    qc[2 * h + 1] = cvt_e4m3x4(q[2].x, q[2].y, q[3].x, q[3].y);
                }
            }
            if constexpr (QDY) {
                if (col < p.n) *reinterpret_cast<uint4*>(p.q + row * p.n + col) = make_uint4(qc[0], qc[1], qc[2], qc[3]);
            }
            if (col < p.n) {
                uint8_t* dst = p.y + (row * p.n + col) * 2;
                if constexpr (WIDE) {
                    st_global_256(dst, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
                } else {
                    *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(dst + 16) = make_uint4(o[4], o[5], o[6], o[7]);
                }
            }
        }
        if constexpr (COLQ) {
            // bands the walk has passed: every CTA has finished the rows below row - blockIdx.x + gridDim.x or is about to
            const int64_t walked = (row - blockIdx.x + gridDim.x) >> 7;
            while (next_tile < col_tiles && next_tile / nct < walked) {
                col_quant_tile<NT>(p, dy, int(next_tile / nct), int(next_tile % nct), cq_cmax, cq_cs, cq_cy);
                next_tile += gridDim.x;
            }
        }
    }
    if constexpr (COLQ) {
        for (; next_tile < col_tiles; next_tile += gridDim.x)
            col_quant_tile<NT>(p, dy, int(next_tile / nct), int(next_tile % nct), cq_cmax, cq_cs, cq_cy);
    }
#pragma unroll
    for (int i = 0; i < SPANS; ++i) {
        const int col = i * SPAN + t * 16;
        if (col < p.n) {
            float4* dst = reinterpret_cast<float4*>(partial + int64_t(blockIdx.x) * p.n + col);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                dst[k] = make_float4(acc[8 * i + 2 * k].x, acc[8 * i + 2 * k].y, acc[8 * i + 2 * k + 1].x, acc[8 * i + 2 * k + 1].y);
        }
    }
}

// RMSNorm + 1x128 quantisation for long runs of wide rows: a persistent walk.  A CTA of 128
// threads takes rows blockIdx.x, blockIdx.x + gridDim.x, ... with the whole row in registers as
// packed words; the loads of the next row are issued as soon as the row sum is known, before
// the normalise + quantise pass over the current one, so each of the four resident CTAs per SM
// always has a row (up to 16 KB) in flight and only pays its own barrier.
// The kernel's time follows the SM clock (254 us at 1965 MHz, 301 us at 1710 MHz before the change
// below): it is bound by instruction issue and the latency chain of a row, not by HBM.  So gamma
// sits in shared memory as float32 for the whole walk -- four conflict-free 16-byte shared loads
// per 16 elements instead of two global loads and sixteen unpack operations (254 -> 248 us).
// FULL: n is exactly SPANS * 2048, so no thread ever has an empty span: the column tests and the
// zero-fill of the load registers go away.
template <int SPANS, bool WIDE, bool FULL>
__global__ void __launch_bounds__(128, 4)
small_norm_walk_kernel(const __grid_constant__ SmallParams p) {
    constexpr int SPAN = 2048;
    // gamma as float32, laid out for conflict-free 16-byte reads: the k-th quad of thread t's 16 columns
    // of span i is float4 number (4 i + k) * 128 + t, so a warp's read is 512 consecutive bytes
    extern __shared__ __align__(16) float4 gam_s[];
    __shared__ float wsum[2][4];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
#pragma unroll
    for (int i = 0; i < SPANS; ++i) {
        const int col = i * SPAN + t * 16;
        float2 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = make_float2(0.f, 0.f);
        if (col < p.n) {
            unpack8<__nv_bfloat16>(__ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2)), v);
            unpack8<__nv_bfloat16>(__ldg(reinterpret_cast<const uint4*>(p.gamma + int64_t(col) * 2 + 16)), v + 4);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) gam_s[(4 * i + k) * 128 + t] = make_float4(v[2 * k].x, v[2 * k].y, v[2 * k + 1].x, v[2 * k + 1].y);
    }
    __syncthreads();
    auto fetch = [&](uint4* xr, int64_t row) {
#pragma unroll
        for (int i = 0; i < SPANS; ++i) {
            const int col = i * SPAN + t * 16;
            if constexpr (!FULL) xr[2 * i] = xr[2 * i + 1] = make_uint4(0, 0, 0, 0);
            if (row < p.M && (FULL || col < p.n)) {   // past the last row nothing is loaded and nothing is used
                const uint8_t* src = p.x + (row * p.n + col) * 2;
                if constexpr (WIDE) {   // x is 32-byte aligned
                    ld_global_256(src, xr[2 * i], xr[2 * i + 1]);
                } else {
                    xr[2 * i] = *reinterpret_cast<const uint4*>(src);
                    xr[2 * i + 1] = *reinterpret_cast<const uint4*>(src + 16);
                }
            }
        }
    };
    // one row: `cur` holds it, `nxt` receives the loads of the row one grid stride further
    auto do_row = [&](uint4* cur, uint4* nxt, int64_t row, int par) {
        float2 s0 = make_float2(0.f, 0.f), s1 = s0;
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) {
            float2 v[4];
            unpack8<__nv_bfloat16>(cur[i], v);
            s0 = fma2(v[0], v[0], s0); s1 = fma2(v[1], v[1], s1);
            s0 = fma2(v[2], v[2], s0); s1 = fma2(v[3], v[3], s1);
        }
        s0 = add2(s0, s1);
        float ss = s0.x + s0.y;
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
        if (lane == 0) wsum[par][warp] = ss;
        __syncthreads();   // the buffer of the other parity was last read before the previous barrier
        const float tot = (wsum[par][0] + wsum[par][1]) + (wsum[par][2] + wsum[par][3]);
        const float r = rsqrt_nr(fmaf(tot, p.inv_n, p.eps));
        if (t == 0 && p.rms != nullptr) p.rms[row] = r;
        const float2 r2 = splat2(r);
        fetch(nxt, row + gridDim.x);
#pragma unroll
        for (int i = 0; i < SPANS; ++i) {
            const int col = i * SPAN + t * 16;
            if (!FULL && i * SPAN >= p.n) break;              // uniform
            const bool valid = FULL || col < p.n;
            float2 v[8];
            unpack8<__nv_bfloat16>(cur[2 * i], v);
            unpack8<__nv_bfloat16>(cur[2 * i + 1], v + 4);
            {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float4 w = gam_s[(4 * i + k) * 128 + t];   // zeros past n
                    v[2 * k] = mul2(mul2(v[2 * k], r2), make_float2(w.x, w.y));
                    v[2 * k + 1] = mul2(mul2(v[2 * k + 1], r2), make_float2(w.z, w.w));
                }
            }
            if (p.y != nullptr && valid) {
                uint8_t* yo = p.y + (row * p.n + col) * 2;
                *reinterpret_cast<uint4*>(yo) = make_uint4(pack_bf16x2(v[0].x, v[0].y), pack_bf16x2(v[1].x, v[1].y),
                                                           pack_bf16x2(v[2].x, v[2].y), pack_bf16x2(v[3].x, v[3].y));
                *reinterpret_cast<uint4*>(yo + 16) = make_uint4(pack_bf16x2(v[4].x, v[4].y), pack_bf16x2(v[5].x, v[5].y),
                                                                pack_bf16x2(v[6].x, v[6].y), pack_bf16x2(v[7].x, v[7].y));
            }
            quant16<false>(p, row, col, valid, v);
        }
    };
    uint4 xa[2 * SPANS], xb[2 * SPANS];
    int64_t row = blockIdx.x;
    fetch(xa, row);
    int par = 0;
    for (; row < p.M; row += gridDim.x, par ^= 1) {
        do_row(xa, xb, row, par);
#pragma unroll
        for (int i = 0; i < 2 * SPANS; ++i) xa[i] = xb[i];   // (writing the loop out for two register sets that swap roles spills: 315 vs 248 us)
    }
}

template <bool QUANT>
static void launch_small_norm(const SmallParams& p, cudaStream_t stream) {
    const unsigned grid = unsigned(p.M);
    // 128 threads per row at every width: fewer, fatter threads beat 256 (measured: 331 vs 381 us
    // for the plain norm at 65536 x 8192)
    const bool wide = ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.y)) & 31) == 0;
    if (wide) {
        if (p.n <= 2048) small_norm_kernel<1, QUANT, 128, true><<<grid, 128, 0, stream>>>(p);
        else if (p.n <= 4096) small_norm_kernel<2, QUANT, 128, true><<<grid, 128, 0, stream>>>(p);
        else small_norm_kernel<4, QUANT, 128, true><<<grid, 128, 0, stream>>>(p);
    } else {
        if (p.n <= 2048) small_norm_kernel<1, QUANT, 128, false><<<grid, 128, 0, stream>>>(p);
        else if (p.n <= 4096) small_norm_kernel<2, QUANT, 128, false><<<grid, 128, 0, stream>>>(p);
        else small_norm_kernel<4, QUANT, 128, false><<<grid, 128, 0, stream>>>(p);
    }
}

// WIDE (256-bit loads) needs a 32-byte aligned input
template <int SOP, typename InT, int U>
static void launch_units(const SmallParams& p, int spans, int64_t units, unsigned grid, bool wide, cudaStream_t stream) {
    const bool full = (p.n % 2048) == 0 && (units % U) == 0;
    if (wide && full) small_units_kernel<SOP, InT, U, true, false, true><<<grid, 128, 0, stream>>>(p, spans, units);
    else if (wide) small_units_kernel<SOP, InT, U, true><<<grid, 128, 0, stream>>>(p, spans, units);
    else small_units_kernel<SOP, InT, U, false><<<grid, 128, 0, stream>>>(p, spans, units);
}

}  // namespace

int small_group_quant(const void* x, int dtype, int64_t M, int64_t n, void* q, float* s, int scale_rowmajor,
                      int round_scale, cudaStream_t stream) {
    if (M > 0x7fffffff) return fail_arg("too many rows");
    SmallParams p{};
    p.x = static_cast<const uint8_t*>(x); p.M = M; p.n = int(n);
    p.q = static_cast<uint8_t*>(q); p.s = s; p.scale_rowmajor = scale_rowmajor; p.round_scale = round_scale;
    const bool wide = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    if ((n % 2048) != 0) {   // any width: 16 consecutive 1x128 blocks per unit (see small_units_kernel)
        const int nb = int(n / 128);
        const int64_t funits = (M * nb + 15) / 16;
        const int64_t fgrid = (funits + 1) / 2;
        if (fgrid > 0x7fffffff) return fail_arg("too many rows");
        const unsigned fg = unsigned(fgrid);
        if (dtype == LH_F16) {
            if (wide) small_units_kernel<SOP_GROUP, __half, 2, true, true><<<fg, 128, 0, stream>>>(p, nb, funits);
            else small_units_kernel<SOP_GROUP, __half, 2, false, true><<<fg, 128, 0, stream>>>(p, nb, funits);
        } else {
            if (wide) small_units_kernel<SOP_GROUP, __nv_bfloat16, 2, true, true><<<fg, 128, 0, stream>>>(p, nb, funits);
            else small_units_kernel<SOP_GROUP, __nv_bfloat16, 2, false, true><<<fg, 128, 0, stream>>>(p, nb, funits);
        }
        return check_launch("small_units_kernel");
    }
    const int spans = int((n + 2047) / 2048);
    const int64_t units = M * spans;
    // three units per CTA once the problem is many waves long (measured: 251 vs 259 us at
    // 65536 x 8192), two below that (10.1 vs 10.8 us with one at 8192 x 2048)
    const int U = M * n > (int64_t(96) << 20) ? 3 : 2;
    const int64_t grid = (units + U - 1) / U;
    if (grid > 0x7fffffff) return fail_arg("too many rows");
    const unsigned g = unsigned(grid);
    if (dtype == LH_F16) {
        if (U == 3) launch_units<SOP_GROUP, __half, 3>(p, spans, units, g, wide, stream);
        else launch_units<SOP_GROUP, __half, 2>(p, spans, units, g, wide, stream);
    } else {
        if (U == 3) launch_units<SOP_GROUP, __nv_bfloat16, 3>(p, spans, units, g, wide, stream);
        else launch_units<SOP_GROUP, __nv_bfloat16, 2>(p, spans, units, g, wide, stream);
    }
    return check_launch("small_units_kernel");
}

int small_silu_quant(const void* x, int64_t M, int64_t n, void* q, float* s, int round_scale, cudaStream_t stream) {
    if (M > 0x7fffffff) return fail_arg("too many rows");
    SmallParams p{};
    p.x = static_cast<const uint8_t*>(x); p.M = M; p.n = int(n);
    p.q = static_cast<uint8_t*>(q); p.s = s; p.round_scale = round_scale;
    const bool wide = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    // Long runs over whole spans: two spans per CTA with all four loads of both issued up front
    // (384 vs 393 us at 65536 x 16384).  Short runs and partly filled spans are faster with one
    // CTA per row walking its spans (12.0 vs 13.0 us at 8192 x 2816).
    if ((n % 2048) == 0 && M * n >= (int64_t(64) << 20)) {
        const int spans = int(n / 2048);
        const int64_t units = M * spans;
        const int64_t grid = (units + 1) / 2;
        if (grid > 0x7fffffff) return fail_arg("too many rows");
        launch_units<SOP_SILU, __nv_bfloat16, 2>(p, spans, units, unsigned(grid), wide, stream);
        return check_launch("small_units_kernel");
    }
    // Rows that are not a whole number of spans: 16 consecutive 1x128 blocks per unit whatever rows
    // they fall in, two units per CTA (11.3 vs 11.8 us at 8192 x 2816, 74 vs 81 us at 65536 x 2816 for
    // the ring kernel, 142 vs 145 us at 32768 x 11264).
    if ((n % 2048) != 0) {
        const int nb = int(n / 128);
        const int64_t units = (M * nb + 15) / 16;
        const int64_t grid = (units + 1) / 2;
        if (grid > 0x7fffffff) return fail_arg("too many rows");
        if (wide) small_units_kernel<SOP_SILU, __nv_bfloat16, 2, true, true><<<unsigned(grid), 128, 0, stream>>>(p, nb, units);
        else small_units_kernel<SOP_SILU, __nv_bfloat16, 2, false, true><<<unsigned(grid), 128, 0, stream>>>(p, nb, units);
        return check_launch("small_units_kernel");
    }
    if (wide) small_stream_kernel<SOP_SILU, __nv_bfloat16, true><<<unsigned(M), 128, 0, stream>>>(p);
    else small_stream_kernel<SOP_SILU, __nv_bfloat16, false><<<unsigned(M), 128, 0, stream>>>(p);
    return check_launch("small_stream_kernel");
}

// y (optional, bf16 [M, n]) is written next to the codes when given
int small_norm_quant(const void* x, const void* gamma, int64_t M, int64_t n, float eps, void* q, float* s, float* rms,
                     int round_scale, cudaStream_t stream, void* y) {
    if (M > 0x7fffffff || n > 8192) return fail_arg("small_norm_quant: size out of range");
    SmallParams p{};
    p.x = static_cast<const uint8_t*>(x); p.gamma = static_cast<const uint8_t*>(gamma); p.M = M; p.n = int(n);
    p.eps = eps; p.inv_n = 1.0f / float(n);
    p.q = static_cast<uint8_t*>(q); p.s = s; p.rms = rms; p.round_scale = round_scale; p.y = static_cast<uint8_t*>(y);
    // Long runs of wide rows: the persistent walk (263 vs 271 us at 65536 x 8192, and 266 us for
    // the TMA ring); everything else one CTA per row.
    if (p.n > 4096 && M * n > (int64_t(24) << 20)) {
        const int sms = sm_count();
        const size_t gsm = size_t(4) * 2048 * 4;   // gamma as float32 in shared memory for four spans (32 KB: four CTAs per SM fit)
        const bool wide = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
        const unsigned wg = unsigned(4 * sms);
        if (p.n == 8192) {
            if (wide) small_norm_walk_kernel<4, true, true><<<wg, 128, gsm, stream>>>(p);
            else small_norm_walk_kernel<4, false, true><<<wg, 128, gsm, stream>>>(p);
        } else {
            if (wide) small_norm_walk_kernel<4, true, false><<<wg, 128, gsm, stream>>>(p);
            else small_norm_walk_kernel<4, false, false><<<wg, 128, gsm, stream>>>(p);
        }
        return check_launch("small_norm_walk_kernel");
    }
    launch_small_norm<true>(p, stream);
    return check_launch("small_norm_kernel");
}

// plain RMSNorm forward, bf16 in and out
int small_norm_y(const void* x, const void* gamma, int64_t M, int64_t n, float eps, void* y, float* rms, int reuse_rms,
                 cudaStream_t stream) {
    if (M > 0x7fffffff || n > 8192) return fail_arg("small_norm_y: size out of range");
    SmallParams p{};
    p.x = static_cast<const uint8_t*>(x); p.gamma = static_cast<const uint8_t*>(gamma); p.M = M; p.n = int(n);
    p.eps = eps; p.inv_n = 1.0f / float(n);
    p.y = static_cast<uint8_t*>(y); p.rms = rms; p.reuse_rms = reuse_rms;
    launch_small_norm<false>(p, stream);
    return check_launch("small_norm_kernel");
}

// dx as bf16 [M, n]; partial: [grid, n] fp32 scratch rows (grid <= max_parts); returns the grid
// in *parts.  n <= 8192, 16-byte aligned pointers, bf16 inputs.
int small_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int64_t M, int64_t n, float eps,
                   void* dx, float* partial, int max_parts, int* parts, void* dy_q, float* dy_s, int round_scale,
                   cudaStream_t stream, void* dy_qt, float* dy_st) {
    SmallParams p{};
    p.x = static_cast<const uint8_t*>(x); p.gamma = static_cast<const uint8_t*>(gamma); p.M = M; p.n = int(n);
    p.eps = eps; p.inv_n = 1.0f / float(n); p.rms = const_cast<float*>(rms); p.reuse_rms = rms != nullptr;
    p.y = static_cast<uint8_t*>(dx);
    p.q = static_cast<uint8_t*>(dy_q); p.s = dy_s; p.round_scale = round_scale;
    p.qt = static_cast<uint8_t*>(dy_qt); p.st = dy_st;
    const uint8_t* g = static_cast<const uint8_t*>(dy);
    const int sms = sm_count();
    int64_t grid = int64_t(sms) * (n <= 4096 ? 3 : 1);
    if (grid > max_parts) grid = max_parts;
    if (grid > M) grid = M;
    *parts = int(grid);
    const bool wide = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 31) == 0;
    const unsigned gd = unsigned(grid);
    const bool qdy = dy_q != nullptr;
    const bool colq = qdy && dy_qt != nullptr && dy_st != nullptr && (M % 16) == 0;
#define LH_BWD_LAUNCH(S, NT_, MB, W, Q, CQ) small_norm_bwd_kernel<S, NT_, MB, W, Q, CQ><<<gd, NT_, 0, stream>>>(p, g, partial)
#define LH_BWD_PICK(W, Q, CQ)                                          \
    do {                                                               \
        if (n <= 2048) LH_BWD_LAUNCH(1, 128, 3, W, Q, CQ);             \
        else if (n <= 4096) LH_BWD_LAUNCH(2, 128, 3, W, Q, CQ);        \
        else LH_BWD_LAUNCH(2, 256, 1, W, Q, CQ);                       \
    } while (0)
    if (wide && colq) LH_BWD_PICK(true, true, true);
    else if (colq) LH_BWD_PICK(false, true, true);
    else if (wide && qdy) LH_BWD_PICK(true, true, false);
    else if (wide) LH_BWD_PICK(true, false, false);
    else if (qdy) LH_BWD_PICK(false, true, false);
    else LH_BWD_PICK(false, false, false);
#undef LH_BWD_PICK
#undef LH_BWD_LAUNCH
    return check_launch("small_norm_bwd_kernel");
}

}  // namespace lh
