// C ABI of the library: argument validation, error reporting and dispatch to the kernel
// launchers.  Nothing here allocates device memory or synchronises (lh_device_status
// excepted, which reads a word back).
#include "lh_common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace lh {

constexpr int64_t kSmallRowElements = int64_t(24) << 20;   // output elements up to which the one-CTA-per-row kernels win (measured)

__device__ int g_device_status = 0;

extern int g_band_cluster;
// lh_tuning("rmsnorm_both_single_pass"): 0 = always the two-launch path for both-axes RMSNorm + quant,
// 1 = the single-pass kernel where it is ahead or level (rows narrower than 6144: 1.04-1.26x below 4096
// columns, 1.0-1.04x from 4096 to 6144; at 8192 the two launches win by 4-9 %), 2 = always
static int g_band_kernel = 1;
static int g_band_bwd = 0;
static int g_second_descends = 1;   // second launch of a two-launch path walks the row bands last to first
static int g_bwd_two_role_min_n = 1 << 30;
extern int g_bwd_stream_min_n;   // lh_rows.cu
static bool use_band_kernel(int64_t n) { return g_band_kernel == 2 || (g_band_kernel == 1 && n < 6144); }

__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, int code) {
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > 4000000000LL) {
            atomicCAS(&g_device_status, 0, code);
            return false;
        }
    }
}

// One warp waits on a barrier that never completes, with a short poll limit: exercises the
// give-up path (status word, normal return) without any production kernel having to fail.
__global__ void __launch_bounds__(32) selftest_wait_kernel(uint32_t polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncwarp();
    bool dead = false;
    if (!mbar_wait_polls(&bar, 0, DEVERR_FULL_WAIT, polls)) dead = true;
    mbar_wait_or_mark<true>(&bar, 0, DEVERR_EMPTY_WAIT, dead);   // a dead thread skips later waits
}

static thread_local char tl_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
    va_end(ap);
}

int fail_arg(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
    va_end(ap);
    return LH_ERR_ARG;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return LH_OK;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return int(e);
}

int sm_count(int* out_device) {
    static int cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (out_device) *out_device = dev;
    if (dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = n > 0 ? n : 148;
    }
    return cached[dev];
}

int make_tensor_map(CUtensorMap* out, const void* base, int dtype, uint64_t rows, uint64_t cols,
                    uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle128) {
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
            set_error("cuTensorMapEncodeTiled is not available from the driver (%s)", cudaGetErrorString(e));
            return e != cudaSuccess ? int(e) : int(cudaErrorNotSupported);
        }
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const CUtensorMapDataType dt = dtype == LH_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : dtype == LH_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : dtype == LH_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu pitch=%llu)", int(r),
                  (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch_bytes);
        return int(cudaErrorInvalidValue);
    }
    return LH_OK;
}

// launchers implemented in the kernel translation units
int rows_norm_yq(const void* x, const void* gamma, int64_t M, int n, float eps, void* y, void* q, float* s, float* rms,
                 int round_scale, cudaStream_t stream);
int64_t router_gemm_scratch(int64_t N, int64_t K);
int router_gemm(const void* x, const void* gamma, const void* w, const float* rms, float* logits, int64_t M, int64_t N,
                int64_t K, void* scratch, int64_t scratch_bytes, cudaStream_t stream);
int64_t route_scratch_bytes(int64_t E);
int make_row_id_map_and_index(const void* map, int map_is_i32, int64_t T, int64_t E, int multiple_of, int32_t* row_map,
                              int32_t* row_index, void* scratch, int64_t scratch_bytes, cudaStream_t stream);
int unpermute_with_mask_map(const void* grad, int dtype, const int32_t* row_map, const void* probs, int probs_dtype,
                            int64_t tokens, int64_t E, int64_t n, void* out, void* prob_out, cudaStream_t stream);
int small_group_quant(const void* x, int dtype, int64_t M, int64_t n, void* q, float* s, int scale_rowmajor,
                      int round_scale, cudaStream_t stream);
int small_silu_quant(const void* x, int64_t M, int64_t n, void* q, float* s, int round_scale, cudaStream_t stream);
int small_norm_quant(const void* x, const void* gamma, int64_t M, int64_t n, float eps, void* q, float* s, float* rms,
                     int round_scale, cudaStream_t stream, void* y = nullptr);
int small_norm_y(const void* x, const void* gamma, int64_t M, int64_t n, float eps, void* y, float* rms, int reuse_rms,
                 cudaStream_t stream);
int fp8_gemm(const void* a, const void* b, const float* a_s, const float* b_s, void* c, int64_t M, int64_t N, int64_t K,
             int block, int a_s_transposed, int b_s_transposed, int out_dtype, cudaStream_t stream, int group_2d = 0);
int tile_quant(const void* x, int dtype, const void* counts, int counts_type, int E, int64_t M, int64_t N,
               void* q, float* s, void* qt, float* st, int round_scale, int mode, int scale_rowmajor,
               cudaStream_t stream, int descending = 0);
int64_t smooth_quant_scratch(int64_t n);
int smooth_quant_fwd(int silu, const void* x, const void* gamma, const float* smooth, int dtype, int64_t M, int64_t n,
                     float eps, void* q, float* scale, float* rms, float* maxs, void* scratch, int64_t scratch_bytes,
                     int round_scale, cudaStream_t stream);
int smooth_quant_batch_fwd(const void* x, const void* w, int dtype, int w_dtype, const float* smooth, const void* counts,
                           int counts_type, int E, int64_t M, int64_t n, void* q, float* scale, float* emax,
                           int round_scale, int reverse, cudaStream_t stream);
int64_t smooth_bwd_scratch(int64_t n);
int smooth_quant_silu_bwd(const void* g, const void* x, const float* smooth, const float* tsmooth, int dtype, int64_t M,
                          int64_t n, void* q, float* scale, void* qt, float* tscale, void* scratch, int64_t scratch_bytes,
                          int round_scale, int reverse, cudaStream_t stream);
int smooth_quant_batch_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype, const float* smooth,
                           const float* tsmooth, const void* counts, int counts_type, int E, int64_t M, int64_t n,
                           int64_t padded_rows, void* q, float* scale, void* dw, void* qt, float* tscale,
                           int round_scale, int reverse, cudaStream_t stream);
int any_col_strip(int silu, const void* x, const void* gamma, const float* r, int dtype, int64_t M, int64_t n,
                  void* qt, float* st, int round_scale, cudaStream_t stream);
int tile_gather_quant(const void* x, int dtype, const void* probs, int probs_dtype, const void* indices,
                      int idx_type, const void* counts, int counts_type, int E, int64_t m, int64_t Mout, int64_t N,
                      void* q, float* s, void* qt, float* st, void* prob_out, int round_scale, cudaStream_t stream);
int tile_norm(const void* x, const void* gamma, const float* r, int dtype, int64_t M, int64_t n, void* q, float* s,
              void* qt, float* st, int round_scale, int mode, cudaStream_t stream, int descending = 0);
int tile_silu_fwd(const void* x, const void* w, int w_dtype, int dtype, const void* counts, int counts_type, int E,
                  int64_t M, int64_t n, void* q, float* s, void* qt, float* st, int round_scale, int mode,
                  cudaStream_t stream);
int tile_silu_bwd(const void* g, const void* x, const void* w, int w_dtype, int dtype, const void* counts,
                  int counts_type, int E, int64_t M, int64_t n, void* dx_q, float* dx_s, void* dx_qt, float* dx_st,
                  void* hp, float* dws, int round_scale, cudaStream_t stream);
int band_norm_fwd(const void* x, const void* gamma, int64_t M, int64_t n, float eps, void* q, float* s, float* rms,
                  void* qt, float* st, int round_scale, cudaStream_t stream);
int64_t band_norm_bwd_scratch(int64_t M, int64_t n);
int band_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int64_t M, int64_t n, float eps,
                  void* dx, float* dgamma, void* dy_q, float* dy_s, void* dy_qt, float* dy_st, int round_scale,
                  void* scratch, int64_t scratch_bytes, cudaStream_t stream);
int any_rms(const void* x, int dtype, int64_t M, int64_t n, float eps, float* rms, cudaStream_t stream);
int any_weighted_silu(const void* g, const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n,
                      void* out, void* dw, int backward, cudaStream_t stream);
int rows_norm_quant(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* q,
                    float* s, float* rms, int round_scale, cudaStream_t stream);
int rows_norm_y(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* y,
                float* rms, int reuse_rms, cudaStream_t stream);
int64_t rows_norm_bwd_scratch(int64_t n);
int rows_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M,
                  int64_t n, float eps, void* dx, float* dgamma, void* scratch, int64_t scratch_bytes,
                  cudaStream_t stream, void* dy_q = nullptr, float* dy_s = nullptr, int round_scale = 0,
                  int* dy_rows_done = nullptr, void* dy_qt = nullptr, float* dy_st = nullptr, int two_role_min_n = 1 << 30);
int64_t rows_norm_bwd_static_bytes();
int rows_norm_bwd_static(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M,
                         int64_t n, float eps, void* dx, float* dgamma, cudaStream_t stream);
int dw_reduce(const float* dws, int64_t R, int64_t nb, void* dw, int w_dtype, cudaStream_t stream);
int weighted_silu_fwd(const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n, void* y,
                      cudaStream_t stream);
int weighted_silu_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n,
                      void* dx, void* dw, cudaStream_t stream);

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// col_only_unit: column granularity the entry point accepts in output_mode 1 (transposed outputs
// only), where the row width need not be a whole number of 1x128 blocks; 128 = no such mode
static int check_fused(const char* what, int dtype, int64_t M, int64_t n, int mode, int col_only_unit = 128) {
    if (dtype != LH_BF16 && dtype != LH_F16 && dtype != LH_F32) return fail_arg("%s: dtype must be bf16, f16 or f32", what);
    const int unit = mode == 1 ? col_only_unit : 128;
    if (M < 0 || n <= 0 || (n % unit) != 0) return fail_arg("%s: need n %% %d == 0 (M=%lld n=%lld)", what, unit, (long long)M, (long long)n);
    if (mode < 0 || mode > 2) return fail_arg("%s: output_mode must be 0, 1 or 2", what);
    return LH_OK;
}

}  // namespace lh

using namespace lh;

extern "C" {

int lh_version(void) { return LH_VERSION; }

const char* lh_last_error(void) { return tl_error; }

int lh_device_check(int device) {
    cudaDeviceProp prop;
    const cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { set_error("cudaGetDeviceProperties(%d): %s", device, cudaGetErrorString(e)); return int(e); }
    if (prop.major != 10) return fail_arg("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    return LH_OK;
}

int lh_device_status(int* status) {
    if (!status) return fail_arg("status is NULL");
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int));
    if (e != cudaSuccess) { set_error("cudaMemcpyFromSymbol: %s", cudaGetErrorString(e)); return int(e); }
    *status = v;
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
        if (e != cudaSuccess) { set_error("cudaMemcpyToSymbol: %s", cudaGetErrorString(e)); return int(e); }
    }
    return LH_OK;
}

int lh_tuning(const char* key, int value) {
    if (key && !strcmp(key, "rmsnorm_both_single_pass")) { const int old = g_band_kernel; g_band_kernel = value; return old; }
    if (key && !strcmp(key, "rmsnorm_bwd_quant_single_pass")) { const int old = g_band_bwd; g_band_bwd = value; return old; }
    if (key && !strcmp(key, "rmsnorm_bwd_stream_min_n")) { const int old = g_bwd_stream_min_n; g_bwd_stream_min_n = value; return old; }
    if (key && !strcmp(key, "rmsnorm_bwd_quant_two_role_min_n")) { const int old = g_bwd_two_role_min_n; g_bwd_two_role_min_n = value; return old; }
    if (key && !strcmp(key, "second_launch_descends")) { const int old = g_second_descends; g_second_descends = value; return old; }
    if (key && !strcmp(key, "band_cluster")) { const int old = g_band_cluster; g_band_cluster = value; return old; }
    return fail_arg("tuning: unknown key");
}

int lh_selftest_wait_timeout(int polls, void* stream) {
    if (polls < 1 || polls > 65536) return fail_arg("selftest_wait_timeout: polls must be in 1..65536");
    selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(uint32_t(polls));
    return check_launch("selftest_wait_kernel");
}

// Row-only outputs of small and medium problems go to the one-CTA-per-row kernels, large ones to
// the persistent TMA-ring kernels.
// The one-CTA-per-row kernels give every thread 16 elements of each 2048-element span of the row:
// rows that are a whole number of spans keep every thread busy, and then the streaming kernels
// (SwiGLU+quant, plain norm, the pure 1x128 quantiser) are ahead of the ring and tile kernels at
// every size (measured up to 65536 x 8192).
static bool whole_spans(int64_t n) { return (n % 2048) == 0; }

static bool use_small_rows(int64_t elements) { return elements <= kSmallRowElements; }


int64_t lh_scratch_bytes(const char* what, int64_t rows, int64_t cols) {
    if (!what) return -1;
    if (!strcmp(what, "rmsnorm_bwd")) return rows_norm_bwd_scratch(cols);
    if (!strcmp(what, "rmsnorm_bwd_blockquant")) {   // the larger of the single-pass and the two-launch needs
        const int64_t a = rows_norm_bwd_scratch(cols), b = band_norm_bwd_scratch(rows, cols);
        return a > b ? a : b;
    }
    if (!strcmp(what, "batch_silu_bwd")) return rows * (cols / 128) * 4;
    if (!strcmp(what, "smooth_quant")) return smooth_quant_scratch(cols);       // calibration only
    if (!strcmp(what, "smooth_quant_bwd")) return smooth_bwd_scratch(cols);     // cols = n (half the row)
    if (!strcmp(what, "rmsnorm_bwd_static")) return 0;  // it carries its own
    if (!strcmp(what, "row_id_map")) return route_scratch_bytes(cols);          // cols = experts
    if (!strcmp(what, "rmsnorm_gemm")) return router_gemm_scratch(rows, cols);   // rows = N, cols = K
    return -1;
}

int lh_blockwise_quant(const void* x, int dtype, int64_t M, int64_t N, void* q, float* s, void* qt, float* st,
                       int round_scale, int output_mode, void* stream) {
    if (output_mode < 0 || output_mode > 2) return fail_arg("blockwise_quant: output_mode must be 0, 1 or 2");
    if (output_mode == 0 && (dtype == LH_BF16 || dtype == LH_F16) && M > 0 && N > 0 && (N % 128) == 0 && x && q && s && aligned16(x) &&
        aligned16(q) && use_small_rows(whole_spans(N) ? 0 : M * N))
        return small_group_quant(x, dtype, M, N, q, s, 0, round_scale, static_cast<cudaStream_t>(stream));
    return tile_quant(x, dtype, nullptr, 0, 1, M, N, q, s, qt, st, round_scale, output_mode, 0,
                      static_cast<cudaStream_t>(stream));
}

int lh_group_quant(const void* x, int dtype, int64_t M, int64_t N, void* q, float* s, int round_scale,
                   void* stream) {
    if ((dtype == LH_BF16 || dtype == LH_F16) && M > 0 && N > 0 && (N % 128) == 0 && x && q && s && aligned16(x) && aligned16(q) &&
        use_small_rows(whole_spans(N) ? 0 : M * N))
        return small_group_quant(x, dtype, M, N, q, s, 1, round_scale, static_cast<cudaStream_t>(stream));
    return tile_quant(x, dtype, nullptr, 0, 1, M, N, q, s, nullptr, nullptr, round_scale, 0, 1,
                      static_cast<cudaStream_t>(stream));
}

int lh_block_quant(const void* x, int dtype, int64_t M, int64_t N, void* q, float* s, int round_scale,
                   void* stream) {
    if ((M % 128) != 0) return fail_arg("block_quant: need M %% 128 == 0");
    return tile_quant(x, dtype, nullptr, 0, 1, M, N, q, s, nullptr, nullptr, round_scale, 3, 0,
                      static_cast<cudaStream_t>(stream));
}

int lh_batch_blockwise_quant(const void* x, int dtype, const void* counts, int counts_type, int E, int64_t R,
                             int64_t N, void* q, float* s, void* qt, float* st, int round_scale, void* stream) {
    if (!counts || E <= 0) return fail_arg("batch_blockwise_quant: counts is NULL or E <= 0");
    return tile_quant(x, dtype, counts, counts_type, E, R, N, q, s, qt, st, round_scale, 2, 0,
                      static_cast<cudaStream_t>(stream));
}

int lh_batch_block_pad_permute(const void* x, int dtype, const void* probs, int probs_dtype, const void* indices,
                               int indices_type, const void* counts, int counts_type, int E, int64_t m,
                               int64_t M_out, int64_t N, void* q, float* s, void* qt, float* st, void* prob_out,
                               int round_scale, void* stream) {
    return tile_gather_quant(x, dtype, probs, probs_dtype, indices, indices_type, counts, counts_type, E, m, M_out, N,
                             q, s, qt, st, prob_out, round_scale, static_cast<cudaStream_t>(stream));
}

int lh_rmsnorm_fwd(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* y,
                   float* rms, int reuse_rms, void* stream) {
    if (dtype == LH_BF16 && M > 0 && n > 0 && n <= 8192 && (n % 128) == 0 && x && gamma && y && (!reuse_rms || rms) &&
        aligned16(x) && aligned16(y) && aligned16(gamma) && use_small_rows(whole_spans(n) ? 0 : M * n))
        return small_norm_y(x, gamma, M, n, eps, y, rms, reuse_rms, static_cast<cudaStream_t>(stream));
    return rows_norm_y(x, gamma, dtype, M, n, eps, y, rms, reuse_rms, static_cast<cudaStream_t>(stream));
}

int lh_rmsnorm_blockquant_fwd(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps,
                              void* q, float* s, float* rms, void* qt, float* st, int round_scale,
                              int output_mode, void* stream) {
    if (int rc = check_fused("rmsnorm_blockquant_fwd", dtype, M, n, output_mode, 32)) return rc;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (!rms) return fail_arg("rmsnorm_blockquant_fwd: rms is NULL");
    if ((n % 128) != 0) {   // output_mode 1 on a width the 128 x 128 tiles do not cover
        if (!x || !gamma || !qt || !st || !aligned16(x) || !aligned16(gamma)) return fail_arg("rmsnorm_blockquant_fwd: NULL or unaligned pointer");
        return any_col_strip(0, x, gamma, rms, dtype, M, n, qt, st, round_scale, cs);
    }
    if (dtype != LH_BF16) {
        // float16 / float32: 1/rms per row from a plain row kernel, then the tile kernel in the
        // requested mode (one pass over x for every output)
        if (n > 8192) return fail_arg("rmsnorm_blockquant_fwd: need n <= 8192");
        if (!x || !gamma || !aligned16(x) || !aligned16(gamma)) return fail_arg("rmsnorm_blockquant_fwd: NULL or unaligned pointer");
        if ((output_mode != 1 && (!q || !s || !aligned16(q))) || (output_mode != 0 && (!qt || !st || !aligned16(qt))))
            return fail_arg("rmsnorm_blockquant_fwd: NULL or unaligned output pointer");
        if (M == 0) return LH_OK;
        if (output_mode != 1)
            if (int rc = any_rms(x, dtype, M, n, eps, rms, cs)) return rc;
        return tile_norm(x, gamma, rms, dtype, M, n, q, s, qt, st, round_scale, output_mode, cs);
    }
    if (output_mode == 2 && M > 0 && n <= 8192 && use_band_kernel(n)) {
        // both axes from one pass over x in HBM (lh_band.cu); where thread-block clusters cannot be
        // launched the two-launch path below runs instead
        if (!x || !gamma || !q || !s || !qt || !st) return fail_arg("rmsnorm_blockquant_fwd: NULL pointer");
        if (!aligned16(x) || !aligned16(gamma) || !aligned16(q) || !aligned16(qt))
            return fail_arg("rmsnorm_blockquant_fwd: pointers must be 16-byte aligned");
        const int rc = band_norm_fwd(x, gamma, M, n, eps, q, s, rms, qt, st, round_scale, cs);
        if (rc != -999) return rc;
    }
    if (output_mode == 0 || output_mode == 2) {
        // The ring kernel's slab holds whole rows of at most 8192 elements in all; rows that fill
        // less than three quarters of it (e.g. n = 5120: 135 vs 102 us at 32768 rows) and long runs of
        // rows wider than 4096 go to the register kernels, like every small problem.
        const bool poor_fill = (8192 / n) * n * 4 < 8192 * 3;
        const bool small = M > 0 && use_small_rows((poor_fill || n > 4096) ? 0 : M * n) && x && gamma && q && s &&
                           dtype == LH_BF16 && aligned16(x) && aligned16(q) && aligned16(gamma);
        if (small) {
            if (int rc = small_norm_quant(x, gamma, M, n, eps, q, s, rms, round_scale, cs)) return rc;
        } else if (int rc = rows_norm_quant(x, gamma, dtype, M, n, eps, q, s, rms, round_scale, cs)) {
            return rc;
        }
    }
    if (output_mode == 1 || output_mode == 2) {
        if (!qt || !st || !x || !gamma) return fail_arg("rmsnorm_blockquant_fwd: NULL pointer");
        if (!aligned16(x) || !aligned16(qt) || !aligned16(gamma)) return fail_arg("rmsnorm_blockquant_fwd: pointers must be 16-byte aligned");
        if (M == 0) return LH_OK;
        return tile_norm(x, gamma, rms, LH_BF16, M, n, nullptr, nullptr, qt, st, round_scale, 1, cs, output_mode == 2 ? g_second_descends : 0);
    }
    return LH_OK;
}

int lh_rmsnorm_gemm_blockquant_fwd(const void* x, const void* gamma, const void* route_w, int dtype, int64_t M,
                                   int64_t K, int64_t N, float eps, void* y, float* rms, float* logits, void* q,
                                   float* s, void* qt, float* st, int round_scale, int output_mode, void* scratch,
                                   int64_t scratch_bytes, void* stream) {
    if (output_mode != 0 && output_mode != 1) return fail_arg("rmsnorm_gemm_blockquant_fwd: output_mode must be 0 or 1");
    if (dtype != LH_BF16) return fail_arg("rmsnorm_gemm_blockquant_fwd: bf16 inputs only");
    if (M <= 0 || (M % 128) || (K % 128) || (N % 128) || K <= 0 || N <= 0 || K > 8192)
        return fail_arg("rmsnorm_gemm_blockquant_fwd: need M, K, N positive multiples of 128 and K <= 8192");
    if (!x || !gamma || !rms) return fail_arg("rmsnorm_gemm_blockquant_fwd: NULL pointer");
    if (!aligned16(x) || !aligned16(gamma)) return fail_arg("rmsnorm_gemm_blockquant_fwd: pointers must be 16-byte aligned");
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (output_mode == 1) {
        if (!qt || !st || !aligned16(qt)) return fail_arg("rmsnorm_gemm_blockquant_fwd: NULL or unaligned transposed output");
        return tile_norm(x, gamma, rms, LH_BF16, M, K, nullptr, nullptr, qt, st, round_scale, 1, cs);
    }
    if (!y || !q || !s || !logits || !route_w) return fail_arg("rmsnorm_gemm_blockquant_fwd: NULL pointer");
    if (!aligned16(y) || !aligned16(q)) return fail_arg("rmsnorm_gemm_blockquant_fwd: pointers must be 16-byte aligned");
    if (use_small_rows(M * K)) {
        if (int rc = small_norm_quant(x, gamma, M, K, eps, q, s, rms, round_scale, cs, y)) return rc;
    } else if (int rc = rows_norm_yq(x, gamma, M, int(K), eps, y, q, s, rms, round_scale, cs)) {
        return rc;
    }
    return router_gemm(x, gamma, route_w, rms, logits, M, N, K, scratch, scratch_bytes, cs);
}

int lh_make_row_id_map_and_index(const void* routing_map, int map_is_i32, int64_t tokens, int64_t experts,
                                 int multiple_of, int32_t* row_id_map, int32_t* row_index, void* scratch,
                                 int64_t scratch_bytes, void* stream) {
    return make_row_id_map_and_index(routing_map, map_is_i32, tokens, experts, multiple_of, row_id_map, row_index,
                                     scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

int lh_unpermute_with_mask_map(const void* grad, int dtype, const int32_t* row_id_map, const void* probs,
                               int probs_dtype, int64_t tokens, int64_t experts, int64_t n, void* out,
                               void* prob_out, void* stream) {
    return unpermute_with_mask_map(grad, dtype, row_id_map, probs, probs_dtype, tokens, experts, n, out, prob_out,
                                   static_cast<cudaStream_t>(stream));
}

int lh_fp8_gemm(const void* a, const void* b, const float* a_s, const float* b_s, void* c, int64_t M, int64_t N,
                int64_t K, int block_size, int a_s_transposed, int b_s_transposed, int out_dtype, void* stream) {
    return fp8_gemm(a, b, a_s, b_s, c, M, N, K, block_size, a_s_transposed, b_s_transposed, out_dtype,
                    static_cast<cudaStream_t>(stream));
}

int lh_rmsnorm_smoothquant_fwd(const void* x, const void* gamma, const float* smooth_scale, int dtype, int64_t M,
                               int64_t n, float eps, void* q, float* scale, float* rms, float* maxs, void* scratch,
                               int64_t scratch_bytes, int round_scale, void* stream) {
    return smooth_quant_fwd(0, x, gamma, smooth_scale, dtype, M, n, eps, q, scale, rms, maxs, scratch, scratch_bytes,
                            round_scale, static_cast<cudaStream_t>(stream));
}

int lh_silu_smoothquant_fwd(const void* x, const float* smooth_scale, int dtype, int64_t M, int64_t n, void* q,
                            float* scale, float* maxs, void* scratch, int64_t scratch_bytes, int round_scale,
                            void* stream) {
    return smooth_quant_fwd(1, x, nullptr, smooth_scale, dtype, M, n, 0.f, q, scale, nullptr, maxs, scratch, scratch_bytes,
                            round_scale, static_cast<cudaStream_t>(stream));
}

int lh_batch_silu_smoothquant_fwd(const void* x, const void* w, int dtype, int w_dtype, const float* smooth_scale,
                                  const void* counts, int counts_type, int E, int64_t R, int64_t n, void* q, float* scale,
                                  float* maxs, int round_scale, int reverse, void* stream) {
    return smooth_quant_batch_fwd(x, w, dtype, w_dtype, smooth_scale, counts, counts_type, E, R, n, q, scale, maxs,
                                  round_scale, reverse, static_cast<cudaStream_t>(stream));
}

int lh_silu_smoothquant_bwd(const void* g, const void* x, const float* smooth_scale, const float* transpose_smooth_scale,
                            int dtype, int64_t M, int64_t n, void* dx_q, float* dx_scale, void* dxt_q, float* dxt_scale,
                            void* scratch, int64_t scratch_bytes, int round_scale, int reverse, void* stream) {
    return smooth_quant_silu_bwd(g, x, smooth_scale, transpose_smooth_scale, dtype, M, n, dx_q, dx_scale, dxt_q, dxt_scale,
                                 scratch, scratch_bytes, round_scale, reverse, static_cast<cudaStream_t>(stream));
}

int lh_batch_silu_smoothquant_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype,
                                  const float* smooth_scale, const float* transpose_smooth_scale, const void* counts,
                                  int counts_type, int E, int64_t R, int64_t n, int64_t padded_rows, void* dx_q,
                                  float* dx_scale, void* dw, void* dxt_q, float* dxt_scale, int round_scale, int reverse,
                                  void* stream) {
    return smooth_quant_batch_bwd(g, x, w, dtype, w_dtype, smooth_scale, transpose_smooth_scale, counts, counts_type, E, R, n,
                                  padded_rows, dx_q, dx_scale, dw, dxt_q, dxt_scale, round_scale, reverse,
                                  static_cast<cudaStream_t>(stream));
}

int lh_fp8_gemm_bb(const void* a, const void* b, const float* a_s, const float* b_s, void* c, int64_t M, int64_t N,
                   int64_t K, int block_size, int out_dtype, void* stream) {
    return fp8_gemm(a, b, a_s, b_s, c, M, N, K, block_size, 0, 0, out_dtype, static_cast<cudaStream_t>(stream), 1);
}

int lh_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M,
                   int64_t n, float eps, void* dx, float* dgamma, void* scratch, int64_t scratch_bytes,
                   void* stream) {
    return rows_norm_bwd(dy, x, gamma, rms, dtype, M, n, eps, dx, dgamma, scratch, scratch_bytes,
                         static_cast<cudaStream_t>(stream));
}

int lh_rmsnorm_bwd_static(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M,
                          int64_t n, float eps, void* dx, float* dgamma, void* stream) {
    return rows_norm_bwd_static(dy, x, gamma, rms, dtype, M, n, eps, dx, dgamma, static_cast<cudaStream_t>(stream));
}

int lh_rmsnorm_bwd_blockquant(const void* dy, const void* x, const void* gamma, const float* rms, int dtype,
                              int64_t M, int64_t n, float eps, void* dx, float* dgamma, void* dy_q, float* dy_s,
                              void* dy_qt, float* dy_st, int round_scale, void* scratch, int64_t scratch_bytes,
                              void* stream) {
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (dtype == LH_BF16 && M > 0 && n > 0 && (n % 128) == 0 && n <= 8192 && g_band_bwd != 0 && dy && x && gamma && dx &&
        dgamma && dy_q && dy_s && dy_qt && dy_st && scratch && aligned16(dy) && aligned16(x) && aligned16(gamma) &&
        aligned16(dx) && aligned16(dy_q) && aligned16(dy_qt) && aligned16(scratch)) {
        // x and dy read from HBM once (lh_band.cu); otherwise, or where clusters cannot be launched, two launches
        const int rc = band_norm_bwd(dy, x, gamma, rms, M, n, eps, dx, dgamma, dy_q, dy_s, dy_qt, dy_st, round_scale,
                                     scratch, scratch_bytes, cs);
        if (rc != -999) return rc;
    }
    // Where the backward runs as the streaming kernel it also quantises dy row-wise from the registers
    // it already holds, and the tile kernel is left with the transposed copy only.
    // g_bwd_two_role_min_n: from this row width on the streaming kernel's CTAs carry a second role that writes
    // the transposed copy tile by tile beside the walk, and no second kernel runs
    int rows_done = 0;
    if (int rc = rows_norm_bwd(dy, x, gamma, rms, dtype, M, n, eps, dx, dgamma, scratch, scratch_bytes, cs, dy_q, dy_s,
                               round_scale, &rows_done, dy_qt, dy_st, g_bwd_two_role_min_n))
        return rc;
    if (rows_done == 2) return LH_OK;
    return tile_quant(dy, dtype, nullptr, 0, 1, M, n, dy_q, dy_s, dy_qt, dy_st, round_scale, rows_done ? 1 : 2, 0, cs,
                      rows_done ? g_second_descends : 0);
}

int lh_weighted_silu_fwd(const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n, void* y,
                         void* stream) {
    if (!x || !y || !aligned16(x) || !aligned16(y)) return fail_arg("weighted_silu_fwd: NULL or unaligned pointer");
    if (dtype == LH_F16 || dtype == LH_F32) {
        if (n <= 0 || (n % 128) != 0 || M < 0) return fail_arg("weighted_silu_fwd: need n %% 128 == 0");
        if (M == 0) return LH_OK;
        return any_weighted_silu(nullptr, x, w, dtype, w_dtype, M, n, y, nullptr, 0, static_cast<cudaStream_t>(stream));
    }
    return weighted_silu_fwd(x, w, dtype, w_dtype, M, n, y, static_cast<cudaStream_t>(stream));
}

int lh_weighted_silu_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype, int64_t M, int64_t n,
                         void* dx, void* dw, void* stream) {
    if (!g || !x || !dx || !aligned16(g) || !aligned16(x) || !aligned16(dx)) return fail_arg("weighted_silu_bwd: NULL or unaligned pointer");
    if (dtype == LH_F16 || dtype == LH_F32) {
        if (n <= 0 || (n % 128) != 0 || M < 0) return fail_arg("weighted_silu_bwd: need n %% 128 == 0");
        if (w != nullptr && dw == nullptr) return fail_arg("weighted_silu_bwd: dw is NULL");
        if (M == 0) return LH_OK;
        return any_weighted_silu(g, x, w, dtype, w_dtype, M, n, dx, dw, 1, static_cast<cudaStream_t>(stream));
    }
    return weighted_silu_bwd(g, x, w, dtype, w_dtype, M, n, dx, dw, static_cast<cudaStream_t>(stream));
}

int lh_silu_blockquant_fwd(const void* x, int dtype, int64_t M, int64_t n, void* q, float* s, void* qt, float* st,
                           int round_scale, int output_mode, void* stream) {
    if (int rc = check_fused("silu_blockquant_fwd", dtype, M, n, output_mode, 64)) return rc;
    if (!x || !aligned16(x) || !aligned16(q) || !aligned16(qt)) return fail_arg("silu_blockquant_fwd: NULL or unaligned pointer");
    if ((output_mode != 1 && (!q || !s)) || (output_mode != 0 && (!qt || !st))) return fail_arg("silu_blockquant_fwd: output pointer is NULL");
    if (M == 0) return LH_OK;
    if ((n % 128) != 0)     // output_mode 1 on a width the 128 x 128 tiles do not cover
        return any_col_strip(1, x, nullptr, nullptr, dtype, M, n, qt, st, round_scale, static_cast<cudaStream_t>(stream));
    if (output_mode == 0 && dtype == LH_BF16)   // the register kernels at every size and width
        return small_silu_quant(x, M, n, q, s, round_scale, static_cast<cudaStream_t>(stream));
    return tile_silu_fwd(x, nullptr, LH_F32, dtype, nullptr, 0, 1, M, n, q, s, qt, st, round_scale, output_mode,
                         static_cast<cudaStream_t>(stream));
}

int lh_silu_blockquant_bwd(const void* g, const void* x, int dtype, int64_t M, int64_t n, void* dx_q, float* dx_s,
                           void* dx_qt, float* dx_st, void* dx_hp, int round_scale, void* stream) {
    if (int rc = check_fused("silu_blockquant_bwd", dtype, M, n, 2)) return rc;
    if (!g || !x || !dx_q || !dx_s || !dx_qt || !dx_st) return fail_arg("silu_blockquant_bwd: NULL pointer");
    if (!aligned16(g) || !aligned16(x) || !aligned16(dx_q) || !aligned16(dx_qt) || !aligned16(dx_hp)) return fail_arg("silu_blockquant_bwd: pointers must be 16-byte aligned");
    if (M == 0) return LH_OK;
    return tile_silu_bwd(g, x, nullptr, LH_F32, dtype, nullptr, 0, 1, M, n, dx_q, dx_s, dx_qt, dx_st, dx_hp, nullptr,
                         round_scale, static_cast<cudaStream_t>(stream));
}

int lh_batch_silu_blockquant_fwd(const void* x, const void* w, int dtype, int w_dtype, const void* counts,
                                 int counts_type, int E, int64_t R, int64_t n, void* q, float* s, void* qt,
                                 float* st, int round_scale, int output_mode, void* stream) {
    if (int rc = check_fused("batch_silu_blockquant_fwd", dtype, R, n, output_mode)) return rc;
    if (!counts || E <= 0) return fail_arg("batch_silu_blockquant_fwd: counts is NULL or E <= 0");
    if (R == 0) return LH_OK;
    if (!x || !w || !aligned16(x) || !aligned16(q) || !aligned16(qt)) return fail_arg("batch_silu_blockquant_fwd: NULL or unaligned pointer");
    if ((output_mode != 1 && (!q || !s)) || (output_mode != 0 && (!qt || !st))) return fail_arg("batch_silu_blockquant_fwd: output pointer is NULL");
    return tile_silu_fwd(x, w, w_dtype, dtype, counts, counts_type, E, R, n, q, s, qt, st, round_scale, output_mode,
                         static_cast<cudaStream_t>(stream));
}

int lh_batch_silu_blockquant_bwd(const void* g, const void* x, const void* w, int dtype, int w_dtype,
                                 const void* counts, int counts_type, int E, int64_t R, int64_t n, void* dx_q,
                                 float* dx_s, void* dw, void* dx_qt, float* dx_st, int round_scale, void* scratch,
                                 int64_t scratch_bytes, void* stream) {
    if (int rc = check_fused("batch_silu_blockquant_bwd", dtype, R, n, 2)) return rc;
    if (!counts || E <= 0) return fail_arg("batch_silu_blockquant_bwd: counts is NULL or E <= 0");
    if (R == 0) return LH_OK;
    if (!g || !x || !w || !dx_q || !dx_s || !dw || !dx_qt || !dx_st) return fail_arg("batch_silu_blockquant_bwd: NULL pointer");
    if (!aligned16(g) || !aligned16(x) || !aligned16(dx_q) || !aligned16(dx_qt)) return fail_arg("batch_silu_blockquant_bwd: pointers must be 16-byte aligned");
    const int64_t need = R * (n / 128) * 4;
    if (!scratch || scratch_bytes < need) return fail_arg("batch_silu_blockquant_bwd: scratch too small (%lld < %lld)", (long long)scratch_bytes, (long long)need);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (int rc = tile_silu_bwd(g, x, w, w_dtype, dtype, counts, counts_type, E, R, n, dx_q, dx_s, dx_qt, dx_st, nullptr,
                               static_cast<float*>(scratch), round_scale, cs)) return rc;
    return dw_reduce(static_cast<const float*>(scratch), R, n / 128, dw, w_dtype, cs);
}

}  // extern "C"
