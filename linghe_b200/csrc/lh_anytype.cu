// float16 and float32 inputs for the row-wise entry points.
//
// The tuned streaming kernels of lh_small.cu / lh_rows.cu are written for bfloat16, the type the
// fused path sees in training.  The upstream wrappers accept any floating type (their kernels
// up-cast whatever they load), so the same entry points also take float16 and float32 here,
// through the plain kernels of this file: one CTA of 256 threads walks rows, every thread owns
// the 8-element vectors t, t + 256, ... of a row (at most four: n <= 8192), the arithmetic is
// the float32 math of the bfloat16 kernels, and outputs are written in the input type.
#include "lh_common.cuh"

#include <type_traits>

namespace lh {

int dgamma_reduce(const float* partial, int parts, int64_t n, float* dgamma, cudaStream_t stream);

namespace {

constexpr int NT = 256;
constexpr int MAXV = 4;   // 8-element vectors per thread and row: 4 * 256 * 8 = 8192 columns

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* f) {
    if constexpr (sizeof(T) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        const float4 b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        Elem<T>::unpack8(*reinterpret_cast<const uint4*>(p), f);
    }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float* f) {
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
    } else if constexpr (std::is_same<T, __half>::value) {
        *reinterpret_cast<uint4*>(p) = make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]),
                                                  pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
    } else {
        *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                  pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    }
}

// sum of `a` (and `b`) over the CTA; every thread gets the totals
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, d);
        b += __shfl_xor_sync(0xffffffffu, b, d);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();   // red[] of the previous row has been read
    if (lane == 0) { red[warp] = a; red[8 + warp] = b; }
    __syncthreads();
    a = 0.f; b = 0.f;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) { a += red[w]; b += red[8 + w]; }
}

// RMSNorm forward.  Y: write y = (x * r) * gamma in the input type; otherwise only 1/rms.
template <typename T, bool Y>
__global__ void __launch_bounds__(NT)
any_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, int64_t M, int n, float eps, float inv_n,
                    T* __restrict__ y, float* __restrict__ rms, int reuse_rms) {
    __shared__ float red[16];
    const int t = threadIdx.x;
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
        float v[MAXV][8];
        float ss = 0.f, unused = 0.f;
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int col = (k * NT + t) * 8;
            if (col < n) {
                load8(x + row * n + col, v[k]);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = fmaf(v[k][j], v[k][j], ss);
            }
        }
        float r;
        if (Y && reuse_rms) {
            r = rms[row];
        } else {
            block_sum2(ss, unused, red);
            r = rsqrt_nr(fmaf(ss, inv_n, eps));
            if (t == 0 && rms != nullptr) rms[row] = r;
        }
        if constexpr (Y) {
#pragma unroll
            for (int k = 0; k < MAXV; ++k) {
                const int col = (k * NT + t) * 8;
                if (col < n) {
                    float g[8], o[8];
                    load8(gamma + col, g);
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = (v[k][j] * r) * g[j];
                    store8(y + row * n + col, o);
                }
            }
        }
    }
}

// RMSNorm backward: dx = r*g*gamma - r^3 * x * sum(x*g*gamma)/n (input type), per-CTA dgamma
// partial sums [gridDim.x, n] that a second kernel adds in a fixed order.
template <typename T>
__global__ void __launch_bounds__(NT)
any_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                    const float* __restrict__ rms, int64_t M, int n, float eps, float inv_n, T* __restrict__ dx,
                    float* __restrict__ partial) {
    __shared__ float red[16];
    const int t = threadIdx.x;
    float acc[MAXV][8];
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
        float ss = 0.f, sc = 0.f;
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int col = (k * NT + t) * 8;
            if (col < n) {
                float xv[8], gv[8], wv[8];
                load8(x + row * n + col, xv);
                load8(dy + row * n + col, gv);
                load8(gamma + col, wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    ss = fmaf(xv[j], xv[j], ss);
                    sc = fmaf(xv[j], gv[j] * wv[j], sc);
                }
            }
        }
        block_sum2(ss, sc, red);
        const float r = rms != nullptr ? rms[row] : rsqrt_nr(fmaf(ss, inv_n, eps));
        const float ncoef = -(r * r * r * sc * inv_n);
        // second pass: the row is re-read (it is in L1/L2), which keeps the registers for dgamma
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int col = (k * NT + t) * 8;
            if (col < n) {
                float xv[8], gv[8], wv[8], o[8];
                load8(x + row * n + col, xv);
                load8(dy + row * n + col, gv);
                load8(gamma + col, wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    o[j] = fmaf(ncoef, xv[j], r * (gv[j] * wv[j]));
                    acc[k][j] = fmaf(xv[j] * gv[j], r, acc[k][j]);
                }
                store8(dx + row * n + col, o);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int col = (k * NT + t) * 8;
        if (col < n) {
            float4* dst = reinterpret_cast<float4*>(partial + int64_t(blockIdx.x) * n + col);
            dst[0] = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
            dst[1] = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
        }
    }
}

__device__ __forceinline__ float load_w(const void* w, int w_dtype, int64_t row) {
    if (w_dtype == LH_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[row]);
    if (w_dtype == LH_F16) return __half2float(reinterpret_cast<const __half*>(w)[row]);
    return reinterpret_cast<const float*>(w)[row];
}
__device__ __forceinline__ void store_w(void* w, int w_dtype, int64_t row, float v) {
    if (w_dtype == LH_BF16) reinterpret_cast<__nv_bfloat16*>(w)[row] = __float2bfloat16_rn(v);
    else if (w_dtype == LH_F16) reinterpret_cast<__half*>(w)[row] = __float2half_rn(v);
    else reinterpret_cast<float*>(w)[row] = v;
}

__device__ __forceinline__ float sigmoid_fast(float x) {
    return rcp_approx(1.0f + ex2_approx(x * -1.4426950408889634f));
}

// one warp = one row: y = silu(x1) * x2 (* w), and for the backward dx1, dx2 and dw
template <typename T, bool BWD>
__global__ void __launch_bounds__(NT)
any_weighted_silu_kernel(const T* __restrict__ g, const T* __restrict__ x, const void* __restrict__ w, int w_dtype,
                         int64_t M, int64_t n, T* __restrict__ out, void* __restrict__ dw) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const bool has_w = w != nullptr;
    for (int64_t row = warp0; row < M; row += nwarps) {
        const float wr = has_w ? load_w(w, w_dtype, row) : 1.f;
        float acc = 0.f;
        for (int64_t col = int64_t(lane) * 8; col < n; col += 256) {
            float x1[8], x2[8];
            load8(x + row * 2 * n + col, x1);
            load8(x + row * 2 * n + n + col, x2);
            if constexpr (!BWD) {
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    o[j] = (sigmoid_fast(x1[j]) * x1[j]) * x2[j];
                    if (has_w) o[j] *= wr;
                }
                store8(out + row * n + col, o);
            } else {
                float gg[8], d1[8], d2[8];
                load8(g + row * n + col, gg);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float sg = sigmoid_fast(x1[j]);
                    const float sgg = sg * gg[j];
                    const float b2 = sgg * x1[j];                                  // d/dx2 (unweighted)
                    const float u = fmaf(x1[j], 1.0f - sg, 1.0f);
                    const float b1 = (sgg * x2[j]) * u;                            // d/dx1 (unweighted)
                    acc = fmaf(b2, x2[j], acc);
                    d1[j] = has_w ? b1 * wr : b1;
                    d2[j] = has_w ? b2 * wr : b2;
                }
                store8(out + row * 2 * n + col, d1);
                store8(out + row * 2 * n + n + col, d2);
            }
        }
        if constexpr (BWD) {
            if (has_w) {
#pragma unroll
                for (int d = 16; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
                if (lane == 0) store_w(dw, w_dtype, row, acc);
            }
        }
    }
}

unsigned row_grid(int64_t M, int per_sm) {
    int64_t g = int64_t(sm_count()) * per_sm;
    if (g > M) g = M;
    return unsigned(g < 1 ? 1 : g);
}


// Transposed-only (128x1) outputs for row widths that are not a multiple of 128.  The upstream
// column-only kernels tile the width by 32 (RMSNorm) or 64 (SwiGLU) columns, so they accept such
// widths; the 128x128 tile kernels here do not.  One CTA = the 128 rows of a band x 32 columns:
// thread t holds row t's 32 values, column maxima by a transposing butterfly inside each warp
// (31 shuffles for 32 columns) and a 4-way maximum through shared memory, then byte stores that
// are consecutive across the CTA for every column.  SILU: x is [M, 2n], value = silu(x1) * x2.
// The arithmetic is that of the tile kernel's fused variants (approximate reciprocal of the scale).
template <typename T, bool SILU>
__global__ void __launch_bounds__(128)
any_col_strip_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const float* __restrict__ r, int64_t M, int n,
                     uint8_t* __restrict__ qt, float* __restrict__ st, int round_scale) {
    __shared__ float cmax[4][32];
    __shared__ float cy[32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int64_t band = blockIdx.x;
    const int c0 = int(blockIdx.y) * 32;
    const int64_t row = band * 128 + t;
    float v[32];
    if (row < M) {
        if constexpr (SILU) {
            const T* x1 = x + row * (2 * int64_t(n)) + c0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float a[8], b[8];
                load8(x1 + 8 * k, a);
                load8(x1 + n + 8 * k, b);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 x1p = make_float2(a[j], a[j + 1]);
                    const float2 y = mul2(mul2(sigmoid_fast2(x1p), x1p), make_float2(b[j], b[j + 1]));
                    v[8 * k + j] = y.x; v[8 * k + j + 1] = y.y;
                }
            }
        } else {
            const float rr = r[row];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float a[8], g[8];
                load8(x + row * n + c0 + 8 * k, a);
                load8(gamma + c0 + 8 * k, g);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[8 * k + j] = (a[j] * rr) * g[j];
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
    }
    // after the butterfly lane L holds the maximum of column L over the warp's 32 rows
    float a[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) a[j] = fabsf(v[j]);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const bool up = (lane & d) != 0;
#pragma unroll
        for (int i = 0; i < d; ++i) {
            const float send = up ? a[i] : a[i + d];
            const float keep = up ? a[i + d] : a[i];
            a[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, d));
        }
    }
    cmax[warp][lane] = a[0];
    __syncthreads();
    if (t < 32) {
        const float m = fmaxf(fmaxf(cmax[0][t], cmax[1][t]), fmaxf(cmax[2][t], cmax[3][t]));
        const float sc = scale_from_amax(m, round_scale != 0);
        cy[t] = rcp_approx(sc);
        st[band * n + c0 + t] = sc;
    }
    __syncthreads();
    if (row < M) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const uint32_t c4 = cvt_e4m3x4(v[j] * cy[j], v[j + 1] * cy[j + 1], v[j + 2] * cy[j + 2], v[j + 3] * cy[j + 3]);
#pragma unroll
            for (int k = 0; k < 4; ++k) qt[int64_t(c0 + j + k) * M + row] = uint8_t(c4 >> (8 * k));
        }
    }
}

}  // namespace

// 1/rms per row (float32 [M]) of a float16 / float32 matrix
int any_rms(const void* x, int dtype, int64_t M, int64_t n, float eps, float* rms, cudaStream_t stream) {
    const unsigned grid = row_grid(M, 8);
    if (dtype == LH_F16)
        any_norm_fwd_kernel<__half, false><<<grid, NT, 0, stream>>>(static_cast<const __half*>(x), nullptr, M, int(n), eps,
                                                                    1.0f / float(n), nullptr, rms, 0);
    else
        any_norm_fwd_kernel<float, false><<<grid, NT, 0, stream>>>(static_cast<const float*>(x), nullptr, M, int(n), eps,
                                                                   1.0f / float(n), nullptr, rms, 0);
    return check_launch("any_norm_fwd_kernel");
}

int any_norm_fwd(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* y, float* rms,
                 int reuse_rms, cudaStream_t stream) {
    const unsigned grid = row_grid(M, 8);
    if (dtype == LH_F16)
        any_norm_fwd_kernel<__half, true><<<grid, NT, 0, stream>>>(static_cast<const __half*>(x),
                                                                   static_cast<const __half*>(gamma), M, int(n), eps,
                                                                   1.0f / float(n), static_cast<__half*>(y), rms, reuse_rms);
    else
        any_norm_fwd_kernel<float, true><<<grid, NT, 0, stream>>>(static_cast<const float*>(x),
                                                                  static_cast<const float*>(gamma), M, int(n), eps,
                                                                  1.0f / float(n), static_cast<float*>(y), rms, reuse_rms);
    return check_launch("any_norm_fwd_kernel");
}

// partial: [max_parts, n] float32 scratch
int any_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M, int64_t n,
                 float eps, void* dx, float* dgamma, float* partial, int max_parts, cudaStream_t stream) {
    unsigned grid = row_grid(M, 2);
    if (grid > unsigned(max_parts)) grid = unsigned(max_parts);
    if (dtype == LH_F16)
        any_norm_bwd_kernel<__half><<<grid, NT, 0, stream>>>(static_cast<const __half*>(dy), static_cast<const __half*>(x),
                                                             static_cast<const __half*>(gamma), rms, M, int(n), eps,
                                                             1.0f / float(n), static_cast<__half*>(dx), partial);
    else
        any_norm_bwd_kernel<float><<<grid, NT, 0, stream>>>(static_cast<const float*>(dy), static_cast<const float*>(x),
                                                            static_cast<const float*>(gamma), rms, M, int(n), eps,
                                                            1.0f / float(n), static_cast<float*>(dx), partial);
    if (int rc = check_launch("any_norm_bwd_kernel")) return rc;
    return dgamma_reduce(partial, int(grid), n, dgamma, stream);
}

int any_weighted_silu(const void* g, const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n,
                      void* out, void* dw, int backward, cudaStream_t stream) {
    int64_t blocks = (M + 7) / 8;
    const int64_t cap = int64_t(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const dim3 grid(unsigned(blocks < 1 ? 1 : blocks));
    if (dtype == LH_F16) {
        if (backward)
            any_weighted_silu_kernel<__half, true><<<grid, NT, 0, stream>>>(
                static_cast<const __half*>(g), static_cast<const __half*>(x), w, w_dtype, M, n, static_cast<__half*>(out), dw);
        else
            any_weighted_silu_kernel<__half, false><<<grid, NT, 0, stream>>>(
                nullptr, static_cast<const __half*>(x), w, w_dtype, M, n, static_cast<__half*>(out), nullptr);
    } else {
        if (backward)
            any_weighted_silu_kernel<float, true><<<grid, NT, 0, stream>>>(
                static_cast<const float*>(g), static_cast<const float*>(x), w, w_dtype, M, n, static_cast<float*>(out), dw);
        else
            any_weighted_silu_kernel<float, false><<<grid, NT, 0, stream>>>(
                nullptr, static_cast<const float*>(x), w, w_dtype, M, n, static_cast<float*>(out), nullptr);
    }
    return check_launch("any_weighted_silu_kernel");
}

// Transposed-only outputs for n % 32 == 0 (any n).  silu: x is [M, 2n]; otherwise RMSNorm with
// the given 1/rms per row.
int any_col_strip(int silu, const void* x, const void* gamma, const float* r, int dtype, int64_t M, int64_t n,
                  void* qt, float* st, int round_scale, cudaStream_t stream) {
    if (M == 0) return LH_OK;
    const dim3 grid(unsigned((M + 127) / 128), unsigned(n / 32));
    uint8_t* q8 = static_cast<uint8_t*>(qt);
#define LH_STRIP(T)                                                                                                   \
    do {                                                                                                              \
        if (silu) any_col_strip_kernel<T, true><<<grid, 128, 0, stream>>>(static_cast<const T*>(x), nullptr, nullptr, M, int(n), q8, st, round_scale); \
        else any_col_strip_kernel<T, false><<<grid, 128, 0, stream>>>(static_cast<const T*>(x), static_cast<const T*>(gamma), r, M, int(n), q8, st, round_scale); \
    } while (0)
    if (dtype == LH_F16) LH_STRIP(__half);
    else if (dtype == LH_F32) LH_STRIP(float);
    else LH_STRIP(__nv_bfloat16);
#undef LH_STRIP
    return check_launch("any_col_strip_kernel");
}

}  // namespace lh
