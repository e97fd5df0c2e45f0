// float16 and float32 instantiations of the fused 128x128-tile producers (lh_tile.cuh): RMSNorm
// with known 1/rms in every output mode, SwiGLU forward and backward.  Kept in a translation
// unit of their own so that they compile in parallel with the bfloat16 set.
#include "lh_tile.cuh"

namespace lh {

int tile_norm_any(const void* x, const void* gamma, const float* r, int dtype, int64_t M, int64_t n, void* q, float* s,
                  void* qt, float* st, int round_scale, int mode, cudaStream_t stream) {
    if (dtype == LH_F16) return tile_norm_t<__half, true>(x, gamma, r, dtype, M, n, q, s, qt, st, round_scale, mode, stream);
    if (dtype == LH_F32) return tile_norm_t<float, true>(x, gamma, r, dtype, M, n, q, s, qt, st, round_scale, mode, stream);
    return fail_arg("unsupported dtype %d", dtype);
}

int tile_silu_fwd_any(const void* x, const void* w, int w_dtype, int dtype, const void* counts, int counts_type, int E,
                      int64_t M, int64_t n, void* q, float* s, void* qt, float* st, int round_scale, int mode,
                      cudaStream_t stream) {
    if (dtype == LH_F16)
        return tile_silu_fwd_t<__half>(x, w, w_dtype, dtype, counts, counts_type, E, M, n, q, s, qt, st, round_scale, mode, stream);
    if (dtype == LH_F32)
        return tile_silu_fwd_t<float>(x, w, w_dtype, dtype, counts, counts_type, E, M, n, q, s, qt, st, round_scale, mode, stream);
    return fail_arg("unsupported dtype %d", dtype);
}

int tile_silu_bwd_any(const void* g, const void* x, const void* w, int w_dtype, int dtype, const void* counts,
                      int counts_type, int E, int64_t M, int64_t n, void* dx_q, float* dx_s, void* dx_qt, float* dx_st,
                      void* hp, float* dws, int round_scale, cudaStream_t stream) {
    if (dtype == LH_F16)
        return tile_silu_bwd_t<__half>(g, x, w, w_dtype, dtype, counts, counts_type, E, M, n, dx_q, dx_s, dx_qt, dx_st, hp,
                                       dws, round_scale, stream);
    if (dtype == LH_F32)
        return tile_silu_bwd_t<float>(g, x, w, w_dtype, dtype, counts, counts_type, E, M, n, dx_q, dx_s, dx_qt, dx_st, hp,
                                      dws, round_scale, stream);
    return fail_arg("unsupported dtype %d", dtype);
}

}  // namespace lh
