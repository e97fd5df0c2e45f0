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

// one thread = 8 consecutive outputs
__global__ void __launch_bounds__(256)
weighted_silu_fwd_kernel(const uint8_t* __restrict__ x, const void* __restrict__ w, int w_bf16, int64_t M,
                         int64_t n, uint8_t* __restrict__ y) {
    const int64_t groups_per_row = n >> 3;
    const int64_t total = M * groups_per_row;
    for (int64_t gidx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; gidx < total;
         gidx += int64_t(gridDim.x) * blockDim.x) {
        const int64_t row = gidx / groups_per_row;
        const int64_t col = (gidx - row * groups_per_row) << 3;
        const uint4 r1 = *reinterpret_cast<const uint4*>(x + (row * 2 * n + col) * 2);
        const uint4 r2 = *reinterpret_cast<const uint4*>(x + (row * 2 * n + n + col) * 2);
        float x1[8], x2[8], o[8];
        Elem<__nv_bfloat16>::unpack8(r1, x1);
        Elem<__nv_bfloat16>::unpack8(r2, x2);
        const bool has_w = w != nullptr;
        const float wv = has_w ? load_w(w, w_bf16, row) : 1.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float v = __fmul_rn(__fmul_rn(sigmoid_ref(x1[c]), x1[c]), x2[c]);
            o[c] = has_w ? __fmul_rn(v, wv) : v;
        }
        *reinterpret_cast<uint4*>(y + (row * n + col) * 2) =
            make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]),
                       pack_bf16x2(o[6], o[7]));
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
        const float wv = has_w ? load_w(w, w_bf16, row) : 1.f;
        float acc = 0.f;
        for (int64_t col = int64_t(lane) * 8; col < n; col += 256) {
            const uint4 rg = *reinterpret_cast<const uint4*>(g + (row * n + col) * 2);
            const uint4 r1 = *reinterpret_cast<const uint4*>(x + (row * 2 * n + col) * 2);
            const uint4 r2 = *reinterpret_cast<const uint4*>(x + (row * 2 * n + n + col) * 2);
            float gg[8], x1[8], x2[8], d1[8], d2[8];
            Elem<__nv_bfloat16>::unpack8(rg, gg);
            Elem<__nv_bfloat16>::unpack8(r1, x1);
            Elem<__nv_bfloat16>::unpack8(r2, x2);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float sg = sigmoid_ref(x1[c]);
                const float sgg = sg * gg[c];
                const float b2 = sgg * x1[c];
                const float u = fmaf(x1[c], 1.f - sg, 1.f);
                const float b1 = sgg * x2[c] * u;
                acc = fmaf(b2, x2[c], acc);
                d1[c] = has_w ? b1 * wv : b1;
                d2[c] = has_w ? b2 * wv : b2;
            }
            *reinterpret_cast<uint4*>(dx + (row * 2 * n + col) * 2) =
                make_uint4(pack_bf16x2(d1[0], d1[1]), pack_bf16x2(d1[2], d1[3]), pack_bf16x2(d1[4], d1[5]),
                           pack_bf16x2(d1[6], d1[7]));
            *reinterpret_cast<uint4*>(dx + (row * 2 * n + n + col) * 2) =
                make_uint4(pack_bf16x2(d2[0], d2[1]), pack_bf16x2(d2[2], d2[3]), pack_bf16x2(d2[4], d2[5]),
                           pack_bf16x2(d2[6], d2[7]));
        }
        if (has_w) {
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
            if (lane == 0) {
                if (w_bf16) reinterpret_cast<__nv_bfloat16*>(dw)[row] = __float2bfloat16_rn(acc);
                else reinterpret_cast<float*>(dw)[row] = acc;
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
