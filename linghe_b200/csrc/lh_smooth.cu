// The smooth-quant recipe of the fused producers: one scale per ROW (the whole row is one
// quantisation group) after a per-column smoothing divisor.
//
//   y        = RMSNorm(x) * gamma            (lh_rmsnorm_smoothquant_fwd, linghe/utils/norm.py:557)
//            | silu(x1) * x2                 (lh_silu_smoothquant_fwd,    linghe/utils/silu.py:1498)
//   maxs[c]  = max over rows |y[:, c]|       (calibration, optional)
//   ys       = y / max(smooth_scale, 1e-30)
//   scale[r] = max(max_c |ys[r, c]| / 448, 1e-30)  [rounded up to a power of two]
//   q        = e4m3(ys / scale[r])
//
// A second recipe beside the 1x128 / 128x1 block format, not on the benchmarked path: plain
// kernels, one CTA of 256 threads walks rows, every thread owns the 8-element vectors
// t, t + 256, ... of a row (at most four: n <= 8192), float32 math as in the block-format kernels
// (fused variants: hardware reciprocal for the quotient, ex2 / rcp for the sigmoid).
#include "lh_common.cuh"

#include <type_traits>

namespace lh {

namespace {

constexpr int SNT = 256;
constexpr int SMAXV = 4;             // 4 * 256 * 8 = 8192 columns
constexpr int kSmoothMaxCtas = 1184; // rows of the calibration scratch

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float* f) {
    if constexpr (sizeof(T) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        const float4 b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        Elem<T>::unpack8(*reinterpret_cast<const uint4*>(p), f);
    }
}

// sum (SUM) or maximum of `a` over the CTA; every thread gets the result
template <bool SUM>
__device__ __forceinline__ float block_reduce(float a, float* red) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, a, d);
        a = SUM ? a + o : fmaxf(a, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();   // red[] of the previous use has been read
    if (lane == 0) red[warp] = a;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < SNT / 32; ++w) r = SUM ? r + red[w] : fmaxf(r, red[w]);
    return r;
}

__device__ __forceinline__ float sigmoid_fast1(float x) {
    return rcp_approx(1.0f + ex2_approx(x * -1.4426950408889634f));
}

template <typename T, bool SILU, bool CALIB>
__global__ void __launch_bounds__(SNT)
smooth_rows_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const float* __restrict__ smooth, int64_t M, int n,
                   float eps, float inv_n, uint8_t* __restrict__ q, float* __restrict__ scale, float* __restrict__ rms_out,
                   float* __restrict__ colmax, int round_scale) {
    __shared__ float red[SNT / 32];
    const int t = threadIdx.x;
    float cm[CALIB ? SMAXV : 1][8];
    if constexpr (CALIB) {
#pragma unroll
        for (int k = 0; k < SMAXV; ++k)
#pragma unroll
            for (int j = 0; j < 8; ++j) cm[k][j] = 0.f;
    }
    const int64_t ld = SILU ? 2 * int64_t(n) : int64_t(n);
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
        float v[SMAXV][8];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < SMAXV; ++k) {
            const int col = (k * SNT + t) * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[k][j] = 0.f;
            if (col < n) {
                if constexpr (SILU) {
                    float a[8], b[8];
                    ld8(x + row * ld + col, a);
                    ld8(x + row * ld + n + col, b);
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[k][j] = (sigmoid_fast1(a[j]) * a[j]) * b[j];
                } else {
                    ld8(x + row * ld + col, v[k]);
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss = fmaf(v[k][j], v[k][j], ss);
                }
            }
        }
        if constexpr (!SILU) {
            const float r = rsqrt_nr(fmaf(block_reduce<true>(ss, red), inv_n, eps));
            if (t == 0 && rms_out != nullptr) rms_out[row] = r;
#pragma unroll
            for (int k = 0; k < SMAXV; ++k) {
                const int col = (k * SNT + t) * 8;
                if (col < n) {
                    float g[8];
                    ld8(gamma + col, g);
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[k][j] = (v[k][j] * r) * g[j];
                }
            }
        }
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < SMAXV; ++k) {
            const int col = (k * SNT + t) * 8;
            if (col < n) {
                float s[8];
                ld8(smooth + col, s);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if constexpr (CALIB) cm[k][j] = fmaxf(cm[k][j], fabsf(v[k][j]));
                    v[k][j] = __fdiv_rn(v[k][j], fmaxf(s[j], kScaleFloor));
                    amax = fmaxf(amax, fabsf(v[k][j]));
                }
            }
        }
        amax = block_reduce<false>(amax, red);
        const float sc = scale_from_amax(amax, round_scale != 0);
        if (t == 0) scale[row] = sc;
        const float y = rcp_approx(sc);
#pragma unroll
        for (int k = 0; k < SMAXV; ++k) {
            const int col = (k * SNT + t) * 8;
            if (col < n) {
                const uint32_t lo = cvt_e4m3x4(v[k][0] * y, v[k][1] * y, v[k][2] * y, v[k][3] * y);
                const uint32_t hi = cvt_e4m3x4(v[k][4] * y, v[k][5] * y, v[k][6] * y, v[k][7] * y);
                *reinterpret_cast<uint2*>(q + row * n + col) = make_uint2(lo, hi);
            }
        }
    }
    if constexpr (CALIB) {
#pragma unroll
        for (int k = 0; k < SMAXV; ++k) {
            const int col = (k * SNT + t) * 8;
            if (col < n) {
                float4* dst = reinterpret_cast<float4*>(colmax + int64_t(blockIdx.x) * n + col);
                dst[0] = make_float4(cm[k][0], cm[k][1], cm[k][2], cm[k][3]);
                dst[1] = make_float4(cm[k][4], cm[k][5], cm[k][6], cm[k][7]);
            }
        }
    }
}

// The per-expert form (linghe/utils/silu.py:1757-1818): rows are grouped by expert (counts[e] rows
// each, in order), expert e has its own smoothing vector smooth[e, :], every row its own weight:
//   y = silu(x1) * x2;  emax[e, c] = max over the expert's rows of |y|  (calibration, before the weight);
//   ys = (y * w[row]) / max(smooth[e], 1e-30)   (reverse: * smooth[e]);  one scale per row.
// The expert of a row comes from a binary search in the prefix sums (shared memory, warp-uniform).
// Calibration maxima are kept in registers while the walk stays inside one expert and merged into
// emax with atomicMax on the bit patterns (non-negative floats order like integers; the result
// does not depend on the order of the merges).
template <typename T, bool CALIB>
__global__ void __launch_bounds__(SNT)
smooth_batch_kernel(const T* __restrict__ x, const void* __restrict__ w, int w_dtype, const float* __restrict__ smooth,
                    const void* __restrict__ counts, int counts_i64, int E, int64_t M, int n, uint8_t* __restrict__ q,
                    float* __restrict__ scale, float* __restrict__ emax, int round_scale, int reverse) {
    extern __shared__ int64_t seg[];   // [E + 1] prefix sums of the counts
    __shared__ float red[SNT / 32];
    const int t = threadIdx.x;
    if (t == 0) {
        int64_t acc = 0;
        seg[0] = 0;
        for (int e = 0; e < E; ++e) {
            acc += counts_i64 ? reinterpret_cast<const int64_t*>(counts)[e] : int64_t(reinterpret_cast<const int32_t*>(counts)[e]);
            seg[e + 1] = acc;
        }
    }
    __syncthreads();
    const int64_t total = seg[E] < M ? seg[E] : M;
    float cm[CALIB ? SMAXV : 1][8];
    int cur_e = -1;
    auto flush = [&]() {
        if constexpr (CALIB) {
            if (cur_e >= 0) {
#pragma unroll
                for (int k = 0; k < SMAXV; ++k) {
                    const int col = (k * SNT + t) * 8;
                    if (col < n) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            atomicMax(reinterpret_cast<unsigned int*>(emax + int64_t(cur_e) * n + col + j), __float_as_uint(cm[k][j]));
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < SMAXV; ++k)
#pragma unroll
                for (int j = 0; j < 8; ++j) cm[k][j] = 0.f;
        }
    };
    flush();
    for (int64_t row = blockIdx.x; row < total; row += gridDim.x) {
        int lo = 0, hi = E - 1;            // smallest e with seg[e + 1] > row
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (seg[mid + 1] > row) hi = mid; else lo = mid + 1;
        }
        if (lo != cur_e) { flush(); cur_e = lo; }
        const float* sm = smooth + int64_t(lo) * n;
        const float wr = w_dtype == LH_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[row])
                         : w_dtype == LH_F16 ? __half2float(reinterpret_cast<const __half*>(w)[row])
                                             : reinterpret_cast<const float*>(w)[row];
        float v[SMAXV][8];
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < SMAXV; ++k) {
            const int col = (k * SNT + t) * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[k][j] = 0.f;
            if (col < n) {
                float a[8], b[8], s[8];
                ld8(x + row * 2 * int64_t(n) + col, a);
                ld8(x + row * 2 * int64_t(n) + n + col, b);
                ld8(sm + col, s);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float y = (sigmoid_fast1(a[j]) * a[j]) * b[j];
                    if constexpr (CALIB) cm[k][j] = fmaxf(cm[k][j], fabsf(y));
                    const float yw = y * wr;
                    v[k][j] = reverse ? yw * s[j] : __fdiv_rn(yw, fmaxf(s[j], kScaleFloor));
                    amax = fmaxf(amax, fabsf(v[k][j]));
                }
            }
        }
        amax = block_reduce<false>(amax, red);
        const float sc = scale_from_amax(amax, round_scale != 0);
        if (t == 0) scale[row] = sc;
        const float y = rcp_approx(sc);
#pragma unroll
        for (int k = 0; k < SMAXV; ++k) {
            const int col = (k * SNT + t) * 8;
            if (col < n) {
                const uint32_t c0 = cvt_e4m3x4(v[k][0] * y, v[k][1] * y, v[k][2] * y, v[k][3] * y);
                const uint32_t c1 = cvt_e4m3x4(v[k][4] * y, v[k][5] * y, v[k][6] * y, v[k][7] * y);
                *reinterpret_cast<uint2*>(q + row * n + col) = make_uint2(c0, c1);
            }
        }
    }
    flush();
}

// ---- SwiGLU backward + smooth quantisation (linghe/utils/silu.py:1705) -----------------------
// dx = [dx1 | dx2] with dx1 = g x2 s (1 + x1 (1 - s)), dx2 = g x1 s, s = sigmoid(x1).
// Row-wise copy: dx * smooth[c] (reverse) or dx / max(smooth[c], 1e-30), one scale per row.
// Transposed copy: dx[r, c] * tsmooth[r] (reverse) or / max(tsmooth[r], 1e-30), one scale per
// COLUMN of dx over all M rows, so it takes two launches: this one also collects the column
// maxima of the smoothed values per CTA (scratch [grid, 2n]); after their reduction to column
// scales the second kernel recomputes dx and writes the transposed codes.  (Upstream quantises
// 32-row groups locally and requantises the codes, linghe/utils/silu.py:1686-1754; the values here
// are quantised once, with the final scale, as upstream's oracle does.)
__device__ __forceinline__ void swiglu_grad8(const float* g, const float* x1, const float* x2, float* d1, float* d2) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float sg = sigmoid_fast1(x1[j]);
        const float sgg = sg * g[j];
        d2[j] = sgg * x1[j];
        d1[j] = (sgg * x2[j]) * fmaf(x1[j], 1.0f - sg, 1.0f);
    }
}

// rows: thread owns vectors t, t + 256 of each half (n <= 4096 per half: two vectors of 8 per half)
template <typename T>
__global__ void __launch_bounds__(SNT)
smooth_bwd_rows_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ smooth,
                       const float* __restrict__ tsmooth, int64_t M, int n, uint8_t* __restrict__ q,
                       float* __restrict__ scale, float* __restrict__ colmax, int round_scale, int reverse) {
    __shared__ float red[SNT / 32];
    const int t = threadIdx.x;
    constexpr int HV = SMAXV / 2;     // vectors per half and thread
    float cm[2][HV][8];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int k = 0; k < HV; ++k)
#pragma unroll
            for (int j = 0; j < 8; ++j) cm[h][k][j] = 0.f;
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
        const float ts = tsmooth[row];
        const float tmul = reverse ? ts : __frcp_rn(fmaxf(ts, kScaleFloor));
        float v[2][HV][8];
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < HV; ++k) {
            const int col = (k * SNT + t) * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[0][k][j] = v[1][k][j] = 0.f;
            if (col < n) {
                float gg[8], x1[8], x2[8], s1[8], s2[8];
                ld8(g + row * n + col, gg);
                ld8(x + row * 2 * int64_t(n) + col, x1);
                ld8(x + row * 2 * int64_t(n) + n + col, x2);
                swiglu_grad8(gg, x1, x2, v[0][k], v[1][k]);
                ld8(smooth + col, s1);
                ld8(smooth + n + col, s2);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    cm[0][k][j] = fmaxf(cm[0][k][j], fabsf(reverse ? v[0][k][j] * tmul : __fdiv_rn(v[0][k][j], fmaxf(ts, kScaleFloor))));
                    cm[1][k][j] = fmaxf(cm[1][k][j], fabsf(reverse ? v[1][k][j] * tmul : __fdiv_rn(v[1][k][j], fmaxf(ts, kScaleFloor))));
                    v[0][k][j] = reverse ? v[0][k][j] * s1[j] : __fdiv_rn(v[0][k][j], fmaxf(s1[j], kScaleFloor));
                    v[1][k][j] = reverse ? v[1][k][j] * s2[j] : __fdiv_rn(v[1][k][j], fmaxf(s2[j], kScaleFloor));
                    amax = fmaxf(amax, fmaxf(fabsf(v[0][k][j]), fabsf(v[1][k][j])));
                }
            }
        }
        amax = block_reduce<false>(amax, red);
        const float sc = scale_from_amax(amax, round_scale != 0);
        if (t == 0) scale[row] = sc;
        const float y = rcp_approx(sc);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int k = 0; k < HV; ++k) {
                const int col = (k * SNT + t) * 8;
                if (col < n) {
                    const float* vv = v[h][k];
                    *reinterpret_cast<uint2*>(q + row * 2 * int64_t(n) + h * n + col) =
                        make_uint2(cvt_e4m3x4(vv[0] * y, vv[1] * y, vv[2] * y, vv[3] * y),
                                   cvt_e4m3x4(vv[4] * y, vv[5] * y, vv[6] * y, vv[7] * y));
                }
            }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int k = 0; k < HV; ++k) {
            const int col = (k * SNT + t) * 8;
            if (col < n) {
                float4* dst = reinterpret_cast<float4*>(colmax + int64_t(blockIdx.x) * 2 * n + h * n + col);
                dst[0] = make_float4(cm[h][k][0], cm[h][k][1], cm[h][k][2], cm[h][k][3]);
                dst[1] = make_float4(cm[h][k][4], cm[h][k][5], cm[h][k][6], cm[h][k][7]);
            }
        }
}

// column scales from the per-CTA maxima: tscale[c] = max(max / 448, 1e-30) [power of two]
__global__ void __launch_bounds__(256)
colscale_reduce_kernel(const float* __restrict__ partial, int parts, int n2, float* __restrict__ tscale, int round_scale) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= n2) return;
    float m = 0.f;
    for (int p = 0; p < parts; ++p) m = fmaxf(m, partial[int64_t(p) * n2 + c]);
    tscale[c] = scale_from_amax(m, round_scale != 0);
}

// transposed codes: CTA = 128 consecutive rows x 8 columns of each half; thread = one row
template <typename T>
__global__ void __launch_bounds__(128)
smooth_bwd_cols_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ tsmooth,
                       const float* __restrict__ tscale, int64_t M, int n, uint8_t* __restrict__ qt, int reverse) {
    const int64_t row = int64_t(blockIdx.x) * 128 + threadIdx.x;
    const int col = int(blockIdx.y) * 8;
    if (row >= M) return;
    float gg[8], x1[8], x2[8], d1[8], d2[8];
    ld8(g + row * n + col, gg);
    ld8(x + row * 2 * int64_t(n) + col, x1);
    ld8(x + row * 2 * int64_t(n) + n + col, x2);
    swiglu_grad8(gg, x1, x2, d1, d2);
    const float ts = tsmooth[row];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float a = reverse ? d1[j] * ts : __fdiv_rn(d1[j], fmaxf(ts, kScaleFloor));
        const float b = reverse ? d2[j] * ts : __fdiv_rn(d2[j], fmaxf(ts, kScaleFloor));
        const uint32_t c2 = cvt_e4m3x2(a * rcp_approx(tscale[col + j]), b * rcp_approx(tscale[n + col + j]));
        qt[int64_t(col + j) * M + row] = uint8_t(c2);
        qt[int64_t(n + col + j) * M + row] = uint8_t(c2 >> 8);
    }
}

// ---- per-expert weighted SwiGLU backward + smooth quantisation (linghe/utils/silu.py:2126) ----
// Rows grouped by expert; dx1 = s g x2 w (1 + x1 (1 - s)), dx2 = s g x1 w, dw[row] = sum_j s x1 x2 g.
// Row-wise copy: smoothed by smooth[e, :] ([E, 2n]), one scale per row.  Transposed copy, per
// expert: dx[r, c] smoothed by tsmooth[r], one scale per (expert, column); expert e's codes are a
// [2n, pad32(c_e)] block (rows past c_e are zero codes) at offset 2n * sum_{e' < e} pad32(c_e').
// Same three steps as the dense form, with the column maxima merged per expert by atomicMax.
__device__ __forceinline__ int find_seg(const int64_t* seg, int E, int64_t row) {
    int lo = 0, hi = E - 1;            // smallest e with seg[e + 1] > row
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (seg[mid + 1] > row) hi = mid; else lo = mid + 1;
    }
    return lo;
}

__device__ __forceinline__ float load_scalar(const void* w, int w_dtype, int64_t i) {
    return w_dtype == LH_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i])
           : w_dtype == LH_F16 ? __half2float(reinterpret_cast<const __half*>(w)[i])
                               : reinterpret_cast<const float*>(w)[i];
}

__device__ __forceinline__ void fill_prefix(int64_t* seg, const void* counts, int counts_i64, int E, int pad) {
    int64_t acc = 0;
    seg[0] = 0;
    for (int e = 0; e < E; ++e) {
        int64_t c = counts_i64 ? reinterpret_cast<const int64_t*>(counts)[e] : int64_t(reinterpret_cast<const int32_t*>(counts)[e]);
        if (pad > 1) c = (c + pad - 1) / pad * pad;
        acc += c;
        seg[e + 1] = acc;
    }
}

template <typename T>
__global__ void __launch_bounds__(SNT)
smooth_batch_bwd_rows_kernel(const T* __restrict__ g, const T* __restrict__ x, const void* __restrict__ w, int w_dtype,
                             const float* __restrict__ smooth, const float* __restrict__ tsmooth,
                             const void* __restrict__ counts, int counts_i64, int E, int64_t M, int n,
                             uint8_t* __restrict__ q, float* __restrict__ scale, void* __restrict__ dw,
                             float* __restrict__ emax, int round_scale, int reverse) {
    extern __shared__ int64_t seg[];
    __shared__ float red[SNT / 32];
    const int t = threadIdx.x;
    if (t == 0) fill_prefix(seg, counts, counts_i64, E, 1);
    __syncthreads();
    const int64_t total = seg[E] < M ? seg[E] : M;
    constexpr int HV = SMAXV / 2;
    float cm[2][HV][8];
    int cur_e = -1;
    auto flush = [&]() {
        if (cur_e >= 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int k = 0; k < HV; ++k) {
                    const int col = (k * SNT + t) * 8;
                    if (col < n) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            atomicMax(reinterpret_cast<unsigned int*>(emax + int64_t(cur_e) * 2 * n + h * n + col + j),
                                      __float_as_uint(cm[h][k][j]));
                    }
                }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int k = 0; k < HV; ++k)
#pragma unroll
                for (int j = 0; j < 8; ++j) cm[h][k][j] = 0.f;
    };
    flush();
    for (int64_t row = blockIdx.x; row < total; row += gridDim.x) {
        const int e = find_seg(seg, E, row);
        if (e != cur_e) { flush(); cur_e = e; }
        const float* sm = smooth + int64_t(e) * 2 * n;
        const float wr = load_scalar(w, w_dtype, row);
        const float ts = tsmooth[row];
        float v[2][HV][8];
        float amax = 0.f, dwp = 0.f;
#pragma unroll
        for (int k = 0; k < HV; ++k) {
            const int col = (k * SNT + t) * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[0][k][j] = v[1][k][j] = 0.f;
            if (col < n) {
                float gg[8], x1[8], x2[8], s1[8], s2[8];
                ld8(g + row * n + col, gg);
                ld8(x + row * 2 * int64_t(n) + col, x1);
                ld8(x + row * 2 * int64_t(n) + n + col, x2);
                swiglu_grad8(gg, x1, x2, v[0][k], v[1][k]);
                ld8(sm + col, s1);
                ld8(sm + n + col, s2);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    dwp = fmaf(v[1][k][j], x2[j], dwp);          // (s g x1) x2
                    const float d1 = v[0][k][j] * wr, d2 = v[1][k][j] * wr;
                    cm[0][k][j] = fmaxf(cm[0][k][j], fabsf(reverse ? d1 * ts : __fdiv_rn(d1, fmaxf(ts, kScaleFloor))));
                    cm[1][k][j] = fmaxf(cm[1][k][j], fabsf(reverse ? d2 * ts : __fdiv_rn(d2, fmaxf(ts, kScaleFloor))));
                    v[0][k][j] = reverse ? d1 * s1[j] : __fdiv_rn(d1, fmaxf(s1[j], kScaleFloor));
                    v[1][k][j] = reverse ? d2 * s2[j] : __fdiv_rn(d2, fmaxf(s2[j], kScaleFloor));
                    amax = fmaxf(amax, fmaxf(fabsf(v[0][k][j]), fabsf(v[1][k][j])));
                }
            }
        }
        amax = block_reduce<false>(amax, red);
        dwp = block_reduce<true>(dwp, red);
        const float sc = scale_from_amax(amax, round_scale != 0);
        if (t == 0) {
            scale[row] = sc;
            if (w_dtype == LH_BF16) reinterpret_cast<__nv_bfloat16*>(dw)[row] = __float2bfloat16_rn(dwp);
            else if (w_dtype == LH_F16) reinterpret_cast<__half*>(dw)[row] = __float2half_rn(dwp);
            else reinterpret_cast<float*>(dw)[row] = dwp;
        }
        const float y = rcp_approx(sc);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int k = 0; k < HV; ++k) {
                const int col = (k * SNT + t) * 8;
                if (col < n) {
                    const float* vv = v[h][k];
                    *reinterpret_cast<uint2*>(q + row * 2 * int64_t(n) + h * n + col) =
                        make_uint2(cvt_e4m3x4(vv[0] * y, vv[1] * y, vv[2] * y, vv[3] * y),
                                   cvt_e4m3x4(vv[4] * y, vv[5] * y, vv[6] * y, vv[7] * y));
                }
            }
    }
    flush();
}

// emax [E, 2n] (column maxima) -> column scales in place
__global__ void __launch_bounds__(256)
scale_from_max_kernel(float* __restrict__ m, int64_t count, int round_scale) {
    const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
    if (i < count) m[i] = scale_from_amax(m[i], round_scale != 0);
}

// transposed codes: thread = one padded row (expert e, local row j < pad32(c_e)), 8 columns of each half
template <typename T>
__global__ void __launch_bounds__(128)
smooth_batch_bwd_cols_kernel(const T* __restrict__ g, const T* __restrict__ x, const void* __restrict__ w, int w_dtype,
                             const float* __restrict__ tsmooth, const float* __restrict__ tscale,
                             const void* __restrict__ counts, int counts_i64, int E, int n, uint8_t* __restrict__ qt,
                             int reverse) {
    extern __shared__ int64_t segs[];      // [E + 1] prefix of the counts, then [E + 1] of the padded counts
    int64_t* seg = segs;
    int64_t* pseg = segs + E + 1;
    if (threadIdx.x == 0) {
        fill_prefix(seg, counts, counts_i64, E, 1);
        fill_prefix(pseg, counts, counts_i64, E, 32);
    }
    __syncthreads();
    const int64_t p = int64_t(blockIdx.x) * 128 + threadIdx.x;
    if (p >= pseg[E]) return;
    const int e = find_seg(pseg, E, p);
    const int64_t j = p - pseg[e];                 // local row, may be padding
    const int64_t ce = seg[e + 1] - seg[e], cpad = pseg[e + 1] - pseg[e];
    const int col = int(blockIdx.y) * 8;
    uint8_t* base = qt + 2 * int64_t(n) * pseg[e];
    uint32_t codes[8];
    if (j < ce) {
        const int64_t row = seg[e] + j;
        float gg[8], x1[8], x2[8], d1[8], d2[8];
        ld8(g + row * n + col, gg);
        ld8(x + row * 2 * int64_t(n) + col, x1);
        ld8(x + row * 2 * int64_t(n) + n + col, x2);
        swiglu_grad8(gg, x1, x2, d1, d2);
        const float wr = load_scalar(w, w_dtype, row);
        const float ts = tsmooth[row];
        const float* tsc = tscale + int64_t(e) * 2 * n;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float a0 = d1[k] * wr, b0 = d2[k] * wr;
            const float a = reverse ? a0 * ts : __fdiv_rn(a0, fmaxf(ts, kScaleFloor));
            const float b = reverse ? b0 * ts : __fdiv_rn(b0, fmaxf(ts, kScaleFloor));
            codes[k] = cvt_e4m3x2(a * rcp_approx(tsc[col + k]), b * rcp_approx(tsc[n + col + k]));
        }
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) codes[k] = 0u;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        base[int64_t(col + k) * cpad + j] = uint8_t(codes[k]);
        base[int64_t(n + col + k) * cpad + j] = uint8_t(codes[k] >> 8);
    }
}

// maxs[c] = max over the per-CTA rows of the calibration scratch
__global__ void __launch_bounds__(256)
colmax_reduce_kernel(const float* __restrict__ partial, int parts, int n, float* __restrict__ maxs) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= n) return;
    float m = 0.f;
    for (int p = 0; p < parts; ++p) m = fmaxf(m, partial[int64_t(p) * n + c]);
    maxs[c] = m;
}

template <typename T, bool SILU>
int launch_smooth(const void* x, const void* gamma, const float* smooth, int64_t M, int64_t n, float eps, void* q,
                  float* scale, float* rms, float* maxs, float* scratch, int round_scale, cudaStream_t stream) {
    int64_t grid = int64_t(sm_count()) * 8;
    if (grid > kSmoothMaxCtas) grid = kSmoothMaxCtas;
    if (grid > M) grid = M;
    const T* xp = static_cast<const T*>(x);
    const T* gp = static_cast<const T*>(gamma);
    uint8_t* qp = static_cast<uint8_t*>(q);
    const float inv_n = 1.0f / float(n);
    if (maxs != nullptr) {
        smooth_rows_kernel<T, SILU, true><<<unsigned(grid), SNT, 0, stream>>>(xp, gp, smooth, M, int(n), eps, inv_n, qp, scale,
                                                                               rms, scratch, round_scale);
        if (int rc = check_launch("smooth_rows_kernel")) return rc;
        colmax_reduce_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(scratch, int(grid), int(n), maxs);
        return check_launch("colmax_reduce_kernel");
    }
    smooth_rows_kernel<T, SILU, false><<<unsigned(grid), SNT, 0, stream>>>(xp, gp, smooth, M, int(n), eps, inv_n, qp, scale, rms,
                                                                            nullptr, round_scale);
    return check_launch("smooth_rows_kernel");
}

template <typename T>
int launch_smooth_batch(const void* x, const void* w, int w_dtype, const float* smooth, const void* counts, int counts_i64,
                        int E, int64_t M, int64_t n, void* q, float* scale, float* emax, int round_scale, int reverse,
                        cudaStream_t stream) {
    // calibration merges per CTA and expert: fewer CTAs keep the atomic traffic small
    int64_t grid = int64_t(sm_count()) * (emax != nullptr ? 2 : 8);
    if (grid > M) grid = M;
    const size_t smem = size_t(E + 1) * sizeof(int64_t);
    const T* xp = static_cast<const T*>(x);
    uint8_t* qp = static_cast<uint8_t*>(q);
    if (emax != nullptr) {
        const cudaError_t e = cudaMemsetAsync(emax, 0, size_t(E) * size_t(n) * 4, stream);
        if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return int(e); }
        smooth_batch_kernel<T, true><<<unsigned(grid), SNT, smem, stream>>>(xp, w, w_dtype, smooth, counts, counts_i64, E, M, int(n),
                                                                             qp, scale, emax, round_scale, reverse);
    } else {
        smooth_batch_kernel<T, false><<<unsigned(grid), SNT, smem, stream>>>(xp, w, w_dtype, smooth, counts, counts_i64, E, M, int(n),
                                                                              qp, scale, nullptr, round_scale, reverse);
    }
    return check_launch("smooth_batch_kernel");
}

}  // namespace

// Per-expert SwiGLU + smooth quantisation; emax (optional) [E, n] receives the calibration maxima.
int smooth_quant_batch_fwd(const void* x, const void* w, int dtype, int w_dtype, const float* smooth, const void* counts,
                           int counts_type, int E, int64_t M, int64_t n, void* q, float* scale, float* emax,
                           int round_scale, int reverse, cudaStream_t stream) {
    const char* what = "batch_silu_smoothquant_fwd";
    if (dtype != LH_BF16 && dtype != LH_F16 && dtype != LH_F32) return fail_arg("%s: dtype must be bf16, f16 or f32", what);
    if (w_dtype != LH_BF16 && w_dtype != LH_F16 && w_dtype != LH_F32) return fail_arg("%s: weight dtype must be bf16, f16 or f32", what);
    if (counts_type != LH_I32 && counts_type != LH_I64) return fail_arg("%s: counts must be int32 or int64", what);
    if (M < 0 || n <= 0 || n > 8192 || (n % 8) != 0 || E <= 0 || E > 4096)
        return fail_arg("%s: need 0 < n <= 8192, n %% 8 == 0, 0 < E <= 4096 (M=%lld n=%lld E=%d)", what, (long long)M, (long long)n, E);
    if (M == 0) {
        if (emax != nullptr) {
            const cudaError_t e = cudaMemsetAsync(emax, 0, size_t(E) * size_t(n) * 4, stream);
            return e == cudaSuccess ? LH_OK : int(e);
        }
        return LH_OK;
    }
    if (!x || !w || !smooth || !counts || !q || !scale) return fail_arg("%s: NULL pointer", what);
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(smooth) | reinterpret_cast<uintptr_t>(q)) & 15)
        return fail_arg("%s: pointers must be 16-byte aligned", what);
    const int i64 = counts_type == LH_I64;
    if (dtype == LH_F16) return launch_smooth_batch<__half>(x, w, w_dtype, smooth, counts, i64, E, M, n, q, scale, emax, round_scale, reverse, stream);
    if (dtype == LH_F32) return launch_smooth_batch<float>(x, w, w_dtype, smooth, counts, i64, E, M, n, q, scale, emax, round_scale, reverse, stream);
    return launch_smooth_batch<__nv_bfloat16>(x, w, w_dtype, smooth, counts, i64, E, M, n, q, scale, emax, round_scale, reverse, stream);
}

int64_t smooth_bwd_scratch(int64_t n) { return int64_t(kSmoothMaxCtas) * 2 * n * 4; }

// dx codes [M,2n] + row scales [M]; transposed codes [2n,M] + column scales [2n].  n <= 4096 per half.
int smooth_quant_silu_bwd(const void* g, const void* x, const float* smooth, const float* tsmooth, int dtype, int64_t M,
                          int64_t n, void* q, float* scale, void* qt, float* tscale, void* scratch, int64_t scratch_bytes,
                          int round_scale, int reverse, cudaStream_t stream) {
    const char* what = "silu_smoothquant_bwd";
    if (dtype != LH_BF16 && dtype != LH_F16 && dtype != LH_F32) return fail_arg("%s: dtype must be bf16, f16 or f32", what);
    if (M < 0 || n <= 0 || n > 4096 || (n % 8) != 0) return fail_arg("%s: need 0 < n <= 4096, n %% 8 == 0 (M=%lld n=%lld)", what, (long long)M, (long long)n);
    if (!tscale) return fail_arg("%s: NULL pointer", what);
    if (M == 0) {   // no rows: every column maximum is zero, the scales sit on their floor
        colscale_reduce_kernel<<<unsigned((2 * n + 255) / 256), 256, 0, stream>>>(nullptr, 0, int(2 * n), tscale, round_scale);
        return check_launch("colscale_reduce_kernel");
    }
    if (!g || !x || !smooth || !tsmooth || !q || !scale || !qt || !scratch) return fail_arg("%s: NULL pointer", what);
    if ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(smooth) |
         reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(scratch)) & 15)
        return fail_arg("%s: pointers must be 16-byte aligned", what);
    if (scratch_bytes < smooth_bwd_scratch(n)) return fail_arg("%s: scratch too small (%lld < %lld)", what, (long long)scratch_bytes, (long long)smooth_bwd_scratch(n));
    int64_t grid = int64_t(sm_count()) * 8;
    if (grid > kSmoothMaxCtas) grid = kSmoothMaxCtas;
    if (grid > M) grid = M;
    float* sp = static_cast<float*>(scratch);
    const dim3 cgrid(unsigned((M + 127) / 128), unsigned(n / 8));
#define LH_SBWD(T)                                                                                                     \
    do {                                                                                                               \
        smooth_bwd_rows_kernel<T><<<unsigned(grid), SNT, 0, stream>>>(static_cast<const T*>(g), static_cast<const T*>(x), smooth, \
            tsmooth, M, int(n), static_cast<uint8_t*>(q), scale, sp, round_scale, reverse);                            \
        if (int rc = check_launch("smooth_bwd_rows_kernel")) return rc;                                                \
        colscale_reduce_kernel<<<unsigned((2 * n + 255) / 256), 256, 0, stream>>>(sp, int(grid), int(2 * n), tscale, round_scale); \
        if (int rc = check_launch("colscale_reduce_kernel")) return rc;                                                \
        smooth_bwd_cols_kernel<T><<<cgrid, 128, 0, stream>>>(static_cast<const T*>(g), static_cast<const T*>(x), tsmooth, tscale, M, \
            int(n), static_cast<uint8_t*>(qt), reverse);                                                               \
    } while (0)
    if (dtype == LH_F16) LH_SBWD(__half);
    else if (dtype == LH_F32) LH_SBWD(float);
    else LH_SBWD(__nv_bfloat16);
#undef LH_SBWD
    return check_launch("smooth_bwd_cols_kernel");
}

// padded_rows = sum_e pad32(counts[e]) (the caller sized dxt_q from its host copy of the counts).
// dxt_scale [E, 2n] doubles as the buffer of the column maxima.
int smooth_quant_batch_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype, const float* smooth,
                           const float* tsmooth, const void* counts, int counts_type, int E, int64_t M, int64_t n,
                           int64_t padded_rows, void* q, float* scale, void* dw, void* qt, float* tscale,
                           int round_scale, int reverse, cudaStream_t stream) {
    const char* what = "batch_silu_smoothquant_bwd";
    if (dtype != LH_BF16 && dtype != LH_F16 && dtype != LH_F32) return fail_arg("%s: dtype must be bf16, f16 or f32", what);
    if (w_dtype != LH_BF16 && w_dtype != LH_F16 && w_dtype != LH_F32) return fail_arg("%s: weight dtype must be bf16, f16 or f32", what);
    if (counts_type != LH_I32 && counts_type != LH_I64) return fail_arg("%s: counts must be int32 or int64", what);
    if (M < 0 || n <= 0 || n > 4096 || (n % 8) != 0 || E <= 0 || E > 2048 || padded_rows < M)
        return fail_arg("%s: need 0 < n <= 4096, n %% 8 == 0, 0 < E <= 2048, padded_rows >= M (M=%lld n=%lld E=%d)", what, (long long)M, (long long)n, E);
    if (!tscale) return fail_arg("%s: NULL pointer", what);
    {
        const cudaError_t e = cudaMemsetAsync(tscale, 0, size_t(E) * size_t(2 * n) * 4, stream);
        if (e != cudaSuccess) { set_error("cudaMemsetAsync: %s", cudaGetErrorString(e)); return int(e); }
    }
    if (M == 0) return LH_OK;     // upstream returns zero scales when there is no row at all
    if (!g || !x || !w || !smooth || !tsmooth || !counts || !q || !scale || !dw || !qt) return fail_arg("%s: NULL pointer", what);
    if ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(smooth) |
         reinterpret_cast<uintptr_t>(q)) & 15)
        return fail_arg("%s: pointers must be 16-byte aligned", what);
    const int i64 = counts_type == LH_I64;
    int64_t grid = int64_t(sm_count()) * 2;
    if (grid > M) grid = M;
    const dim3 cgrid(unsigned((padded_rows + 127) / 128), unsigned(n / 8));
    const size_t smem1 = size_t(E + 1) * 8, smem2 = 2 * smem1;
    const int64_t cnt = int64_t(E) * 2 * n;
#define LH_SBB(T)                                                                                                      \
    do {                                                                                                               \
        smooth_batch_bwd_rows_kernel<T><<<unsigned(grid), SNT, smem1, stream>>>(static_cast<const T*>(g), static_cast<const T*>(x), \
            w, w_dtype, smooth, tsmooth, counts, i64, E, M, int(n), static_cast<uint8_t*>(q), scale, dw, tscale, round_scale, reverse); \
        if (int rc = check_launch("smooth_batch_bwd_rows_kernel")) return rc;                                          \
        scale_from_max_kernel<<<unsigned((cnt + 255) / 256), 256, 0, stream>>>(tscale, cnt, round_scale);             \
        if (int rc = check_launch("scale_from_max_kernel")) return rc;                                                 \
        smooth_batch_bwd_cols_kernel<T><<<cgrid, 128, smem2, stream>>>(static_cast<const T*>(g), static_cast<const T*>(x), w, w_dtype, \
            tsmooth, tscale, counts, i64, E, int(n), static_cast<uint8_t*>(qt), reverse);                              \
    } while (0)
    if (dtype == LH_F16) LH_SBB(__half);
    else if (dtype == LH_F32) LH_SBB(float);
    else LH_SBB(__nv_bfloat16);
#undef LH_SBB
    return check_launch("smooth_batch_bwd_cols_kernel");
}

int64_t smooth_quant_scratch(int64_t n) { return int64_t(kSmoothMaxCtas) * n * 4; }

// silu = 0: RMSNorm (gamma required, rms optional output); silu = 1: SwiGLU on x [M, 2n].
// maxs != NULL: calibration, needs scratch of smooth_quant_scratch(n) bytes.
int smooth_quant_fwd(int silu, const void* x, const void* gamma, const float* smooth, int dtype, int64_t M, int64_t n,
                     float eps, void* q, float* scale, float* rms, float* maxs, void* scratch, int64_t scratch_bytes,
                     int round_scale, cudaStream_t stream) {
    const char* what = silu ? "silu_smoothquant_fwd" : "rmsnorm_smoothquant_fwd";
    if (dtype != LH_BF16 && dtype != LH_F16 && dtype != LH_F32) return fail_arg("%s: dtype must be bf16, f16 or f32", what);
    if (M < 0 || n <= 0 || n > 8192 || (n % 8) != 0) return fail_arg("%s: need 0 < n <= 8192, n %% 8 == 0 (M=%lld n=%lld)", what, (long long)M, (long long)n);
    if (M > 0 && (!x || !smooth || !q || !scale || (!silu && !gamma))) return fail_arg("%s: NULL pointer", what);
    const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(smooth) | reinterpret_cast<uintptr_t>(q) |
                         reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(scratch);
    if (al & 15) return fail_arg("%s: pointers must be 16-byte aligned", what);
    if (maxs != nullptr && (!scratch || scratch_bytes < smooth_quant_scratch(n)))
        return fail_arg("%s: calibration needs %lld bytes of scratch", what, (long long)smooth_quant_scratch(n));
    if (M == 0) {
        if (maxs != nullptr) {
            const cudaError_t e = cudaMemsetAsync(maxs, 0, size_t(n) * 4, stream);
            return e == cudaSuccess ? LH_OK : int(e);
        }
        return LH_OK;
    }
    float* sp = static_cast<float*>(scratch);
#define LH_SMOOTH(T)                                                                                               \
    (silu ? launch_smooth<T, true>(x, gamma, smooth, M, n, eps, q, scale, rms, maxs, sp, round_scale, stream)      \
          : launch_smooth<T, false>(x, gamma, smooth, M, n, eps, q, scale, rms, maxs, sp, round_scale, stream))
    if (dtype == LH_F16) return LH_SMOOTH(__half);
    if (dtype == LH_F32) return LH_SMOOTH(float);
    return LH_SMOOTH(__nv_bfloat16);
#undef LH_SMOOTH
}

}  // namespace lh
