// Small helper kernels around the fused paths: the per-row reduction of the SwiGLU
// weight-gradient partials, and the plain (unquantised) weighted SwiGLU forward and
// backward that share the activation math.  Straight vectorised global loads at full
// occupancy; these are bandwidth-bound streaming kernels with no data reuse.
#include "lh_common.cuh"

namespace lh {

// dw[row] = sum_b dws[row, b]   (fixed order -> deterministic)
__global__ void dw_reduce_kernel(const float* __restrict__ dws, int64_t R, int nb, void* __restrict__ dw,
                                 int w_bf16) {
    const int64_t row = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (row >= R) return;
    float a = 0.f;
    for (int b = 0; b < nb; ++b) a += dws[row * nb + b];
    if (w_bf16) reinterpret_cast<__nv_bfloat16*>(dw)[row] = __float2bfloat16_rn(a);
    else reinterpret_cast<float*>(dw)[row] = a;
}

int dw_reduce(const float* dws, int64_t R, int64_t nb, void* dw, int w_dtype, cudaStream_t stream) {
    if (R == 0) return LH_OK;
    dw_reduce_kernel<<<dim3(unsigned((R + 255) / 256)), dim3(256), 0, stream>>>(dws, R, int(nb), dw,
                                                                                 w_dtype == LH_BF16);
    return check_launch("dw_reduce_kernel");
}

__device__ __forceinline__ float load_w(const void* w, int w_bf16, int64_t row) {
    return w_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[row])
                  : reinterpret_cast<const float*>(w)[row];
}

// one thread = 8 consecutive outputs per step; (row, column group) advance by a fixed step, so
// the only 64-bit division is the one that places the thread.  Same arithmetic as the fused
// kernels: packed float32x2, sigmoid = rcp.approx(1 + ex2.approx(-x log2 e)).
__global__ void __launch_bounds__(256)
weighted_silu_fwd_kernel(const uint8_t* __restrict__ x, const void* __restrict__ w, int w_bf16, int64_t M,
                         int64_t n, uint8_t* __restrict__ y) {
    const int64_t gpr = n >> 3;                                   // 8-element groups per row
    const int64_t step = int64_t(gridDim.x) * blockDim.x;
    const int64_t dq = step / gpr, dr = step - dq * gpr;
    const int64_t g0 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    int64_t row = g0 / gpr, cg = g0 - row * gpr;
    const bool has_w = w != nullptr;
    for (; row < M;) {
        const uint8_t* xr = x + (row * 2 * n + (cg << 3)) * 2;
        const uint4 r1 = *reinterpret_cast<const uint4*>(xr);
        const uint4 r2 = *reinterpret_cast<const uint4*>(xr + n * 2);
        const float2 w2 = splat2(has_w ? load_w(w, w_bf16, row) : 1.f);
        const uint32_t a1[4] = {r1.x, r1.y, r1.z, r1.w}, a2[4] = {r2.x, r2.y, r2.z, r2.w};
        uint32_t o[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float2 x1 = bf16x2_to_f2(a1[c]), x2 = bf16x2_to_f2(a2[c]);
            float2 v = mul2(mul2(sigmoid_fast2(x1), x1), x2);
            if (has_w) v = mul2(v, w2);
            o[c] = pack_bf16x2(v.x, v.y);
        }
        *reinterpret_cast<uint4*>(y + (row * n + (cg << 3)) * 2) = make_uint4(o[0], o[1], o[2], o[3]);
        row += dq;
        cg += dr;
        if (cg >= gpr) { cg -= gpr; ++row; }
    }
}

// one warp = one row; dw is the row sum of sigmoid*x1*x2*g
__global__ void __launch_bounds__(256)
weighted_silu_bwd_kernel(const uint8_t* __restrict__ g, const uint8_t* __restrict__ x, const void* __restrict__ w,
                         int w_bf16, int64_t M, int64_t n, uint8_t* __restrict__ dx, void* __restrict__ dw) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const bool has_w = w != nullptr;
    for (int64_t row = warp0; row < M; row += nwarps) {
        const float2 w2 = splat2(has_w ? load_w(w, w_bf16, row) : 1.f);
        float2 acc = make_float2(0.f, 0.f);
        for (int64_t col = int64_t(lane) * 8; col < n; col += 256) {
            const uint4 rg = *reinterpret_cast<const uint4*>(g + (row * n + col) * 2);
            const uint4 r1 = *reinterpret_cast<const uint4*>(x + (row * 2 * n + col) * 2);
            const uint4 r2 = *reinterpret_cast<const uint4*>(x + (row * 2 * n + n + col) * 2);
            const uint32_t ag[4] = {rg.x, rg.y, rg.z, rg.w}, a1[4] = {r1.x, r1.y, r1.z, r1.w}, a2[4] = {r2.x, r2.y, r2.z, r2.w};
            uint32_t o1[4], o2[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float2 gg = bf16x2_to_f2(ag[c]), x1 = bf16x2_to_f2(a1[c]), x2 = bf16x2_to_f2(a2[c]);
                const float2 sg = sigmoid_fast2(x1);
                const float2 sgg = mul2(sg, gg);                                   // sigmoid * g
                const float2 b2 = mul2(sgg, x1);                                   // d/dx2 (unweighted)
                const float2 oms = fma2(sg, splat2(-1.f), splat2(1.f));            // 1 - sigmoid
                const float2 u = fma2(x1, oms, splat2(1.f));
                const float2 b1 = mul2(mul2(sgg, x2), u);                          // d/dx1 (unweighted)
                acc = fma2(b2, x2, acc);
                const float2 d1 = has_w ? mul2(b1, w2) : b1, d2 = has_w ? mul2(b2, w2) : b2;
                o1[c] = pack_bf16x2(d1.x, d1.y);
                o2[c] = pack_bf16x2(d2.x, d2.y);
            }
            *reinterpret_cast<uint4*>(dx + (row * 2 * n + col) * 2) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
            *reinterpret_cast<uint4*>(dx + (row * 2 * n + n + col) * 2) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
        }
        if (has_w) {
            float a = acc.x + acc.y;
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
            if (lane == 0) {
                if (w_bf16) reinterpret_cast<__nv_bfloat16*>(dw)[row] = __float2bfloat16_rn(a);
                else reinterpret_cast<float*>(dw)[row] = a;
            }
        }
    }
}

int weighted_silu_fwd(const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n, void* y,
                      cudaStream_t stream) {
    if (dtype != LH_BF16) return fail_arg("weighted_silu_fwd: only bf16 inputs are supported");
    if (n <= 0 || (n % 128) != 0 || M < 0) return fail_arg("weighted_silu_fwd: need n %% 128 == 0");
    if (M == 0) return LH_OK;
    const int64_t total = M * (n >> 3);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = int64_t(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    weighted_silu_fwd_kernel<<<dim3(unsigned(blocks)), dim3(256), 0, stream>>>(
        static_cast<const uint8_t*>(x), w, w_dtype == LH_BF16, M, n, static_cast<uint8_t*>(y));
    return check_launch("weighted_silu_fwd_kernel");
}

int weighted_silu_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n,
                      void* dx, void* dw, cudaStream_t stream) {
    if (dtype != LH_BF16) return fail_arg("weighted_silu_bwd: only bf16 inputs are supported");
    if (n <= 0 || (n % 128) != 0 || M < 0) return fail_arg("weighted_silu_bwd: need n %% 128 == 0");
    if (w != nullptr && dw == nullptr) return fail_arg("weighted_silu_bwd: dw is NULL");
    if (M == 0) return LH_OK;
    int64_t blocks = (M + 7) / 8;
    const int64_t cap = int64_t(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    weighted_silu_bwd_kernel<<<dim3(unsigned(blocks)), dim3(256), 0, stream>>>(
        static_cast<const uint8_t*>(g), static_cast<const uint8_t*>(x), w, w_dtype == LH_BF16, M, n,
        static_cast<uint8_t*>(dx), dw);
    return check_launch("weighted_silu_bwd_kernel");
}

}  // namespace lh
