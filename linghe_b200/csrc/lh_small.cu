// One-CTA-per-row kernels for the row-only outputs of small and medium problems.
//
// A persistent TMA ring (lh_rows.cu) reaches the copy bandwidth once every CTA streams dozens
// of slabs, but a problem of a few tens of megabytes is over before the ring is in steady
// state.  Here the grid is one small CTA (128 threads) per row: the hardware block scheduler
// keeps up to 16 CTAs per SM in flight, each thread issues its loads at once, and nothing
// is staged through shared memory.  Thread t owns 16 consecutive elements (two 16-byte
// chunks) of every 2048-element span of its row, so a 1x128 block is 8 consecutive lanes.
#include "lh_small.cuh"

namespace lh {

namespace {

enum : int { SOP_GROUP = 0, SOP_NORM = 1, SOP_SILU = 2 };

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


template <int SPANS, int NT, int MINB, bool WIDE, bool QDY, bool FULL = false>
__global__ void __launch_bounds__(NT, MINB)
small_norm_bwd_kernel(const __grid_constant__ SmallParams p, const uint8_t* __restrict__ dy, float* __restrict__ partial) {
    __shared__ __align__(16) float2 wsum[2][NT / 32];
    __shared__ float4 gam_s[4 * SPANS * NT];
    norm_bwd_walk<SPANS, NT, WIDE, QDY, 0, FULL>(p, dy, partial, wsum, nullptr, gam_s);
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
    __shared__ __align__(16) float wsum[2][4];
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
        const float4 w4 = *reinterpret_cast<const float4*>(wsum[par]);   // one 16-byte read of the four warp sums
        const float tot = (w4.x + w4.y) + (w4.z + w4.w);
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
    const bool wide = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 31) == 0;
    const bool qdy = dy_q != nullptr;
    const bool colq = qdy && dy_qt != nullptr && dy_st != nullptr && (M % 16) == 0;
    int64_t grid = int64_t(sms) * (n <= 4096 ? (colq ? 2 : 3) : 1);
    if (grid > max_parts) grid = max_parts;
    if (grid > M) grid = M;
    *parts = int(grid);
    const unsigned gd = unsigned(grid);
    if (colq)
        return small_norm_bwd_duo(p, g, partial, gd, wide, stream);
#define LH_BWD_LAUNCH(S, NT_, MB, W, Q, F) small_norm_bwd_kernel<S, NT_, MB, W, Q, F><<<gd, NT_, 0, stream>>>(p, g, partial)
#define LH_BWD_PICK(W, Q)                                                                   \
    do {                                                                                    \
        /* whole spans, no row-wise codes of dy: the instantiation without bounds tests (with the     \
           codes it measures no faster: 124.3 vs 123.2 us for the fused call at 16384 x 4096) */    \
        if (!Q && n == 4096 && W) LH_BWD_LAUNCH(2, 128, 3, W, Q, true);                             \
        else if (!Q && n == 8192 && W) LH_BWD_LAUNCH(2, 256, 1, W, Q, true);                        \
        else if (n <= 2048) LH_BWD_LAUNCH(1, 128, 3, W, Q, false);                          \
        else if (n <= 4096) LH_BWD_LAUNCH(2, 128, 3, W, Q, false);                          \
        else LH_BWD_LAUNCH(2, 256, 1, W, Q, false);                                         \
    } while (0)
    if (wide && qdy) LH_BWD_PICK(true, true);
    else if (wide) LH_BWD_PICK(true, false);
    else if (qdy) LH_BWD_PICK(false, true);
    else LH_BWD_PICK(false, false);
#undef LH_BWD_PICK
#undef LH_BWD_LAUNCH
    return check_launch("small_norm_bwd_kernel");
}

}  // namespace lh
