// Host-side dispatch of the 128x128-tile kernels (lh_tile.cuh): the pure quantisers for every
// input type and the fused producers for bfloat16; lh_tile_any.cu holds the float16 / float32
// instantiations of the fused producers.
#include "lh_tile.cuh"

namespace lh {

template <typename InT>
static int quant_dispatch(const TileParams& p, int mode, cudaStream_t st) {
    constexpr int S = sizeof(InT) == 2 ? 2 : 2;
    constexpr int CPS = sizeof(InT) == 2 ? 2 : 1;
    switch (mode) {
        case MODE_ROW: return launch_tile<OP_IDENT, InT, MODE_ROW, true, 8, S, CPS>(p, st);
        case MODE_COL: return launch_tile<OP_IDENT, InT, MODE_COL, true, 8, S, CPS>(p, st);
        case MODE_BOTH: return launch_tile<OP_IDENT, InT, MODE_BOTH, true, 8, S, CPS>(p, st);
        case MODE_BLOCK: return launch_tile<OP_IDENT, InT, MODE_BLOCK, true, 8, S, CPS>(p, st);
    }
    return fail_arg("output_mode must be 0, 1 or 2");
}

static int quant_any(const TileParams& p, int dtype, int mode, cudaStream_t st) {
    switch (dtype) {
        case LH_BF16: return quant_dispatch<__nv_bfloat16>(p, mode, st);
        case LH_F16: return quant_dispatch<__half>(p, mode, st);
        case LH_F32: return quant_dispatch<float>(p, mode, st);
    }
    return fail_arg("unsupported dtype %d", dtype);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int tile_quant(const void* x, int dtype, const void* counts, int counts_type, int E, int64_t M, int64_t N,
               void* q, float* s, void* qt, float* st, int round_scale, int mode, int scale_rowmajor,
               cudaStream_t stream, int descending) {
    if (M < 0 || N <= 0 || (N % 128) != 0) return fail_arg("quant: need N %% 128 == 0 (M=%lld N=%lld)", (long long)M, (long long)N);
    if (M == 0) return LH_OK;
    if (!aligned16(x) || !aligned16(q) || !aligned16(qt)) return fail_arg("quant: pointers must be 16-byte aligned");
    if (!x) return fail_arg("quant: x is NULL");
    if ((mode == MODE_ROW || mode == MODE_BOTH || mode == MODE_BLOCK) && (!q || !s)) return fail_arg("quant: q/s NULL");
    if ((mode == MODE_COL || mode == MODE_BOTH) && (!qt || !st)) return fail_arg("quant: qt/st NULL");
    TileParams p{};
    if (int rc = make_tensor_map(&p.tmap[0], x, dtype, uint64_t(M), uint64_t(N),
                                 uint64_t(N) * (dtype == LH_F32 ? 4 : 2), 128, 128)) return rc;
    p.counts = counts; p.counts_i64 = counts_type == LH_I64; p.E = counts ? E : 1;
    p.M = M; p.n = N;
    p.q = static_cast<uint8_t*>(q); p.s = s; p.qt = static_cast<uint8_t*>(qt); p.st = st;
    p.round_scale = round_scale; p.scale_rowmajor = scale_rowmajor; p.descending = descending;
    return quant_any(p, dtype, mode, stream);
}

static bool aligned16(const void* p);

template <typename InT>
static int gather_launch(const TileParams& p, cudaStream_t st) {
    return launch_tile<OP_GATHER, InT, MODE_BOTH, true, 8, 2, (sizeof(InT) == 2 ? 2 : 1)>(p, st);
}

int tile_gather_quant(const void* x, int dtype, const void* probs, int probs_dtype, const void* indices,
                      int idx_type, const void* counts, int counts_type, int E, int64_t m, int64_t Mout, int64_t N,
                      void* q, float* s, void* qt, float* st, void* prob_out, int round_scale, cudaStream_t stream) {
    if (N <= 0 || (N % 128) != 0 || m < 0 || Mout < 0) return fail_arg("pad_permute: need N %% 128 == 0");
    if (!counts || E <= 0) return fail_arg("pad_permute: counts is NULL or E <= 0");
    if (Mout == 0 || m == 0) return LH_OK;
    if (m >= (int64_t(1) << 31)) return fail_arg("pad_permute: more than 2^31 source rows");
    if (!x || !indices || !q || !s || !qt || !st) return fail_arg("pad_permute: NULL pointer");
    if ((probs == nullptr) != (prob_out == nullptr)) return fail_arg("pad_permute: probs and prob_out go together");
    if (!aligned16(x) || !aligned16(q) || !aligned16(qt)) return fail_arg("pad_permute: pointers must be 16-byte aligned");
    TileParams p{};
    p.counts = counts; p.counts_i64 = counts_type == LH_I64; p.E = E; p.pad16 = 1;
    p.M = Mout; p.n = N;
    p.gx = static_cast<const uint8_t*>(x); p.indices = indices; p.indices_i64 = idx_type == LH_I64;
    p.probs = probs; p.prob_out = prob_out; p.probs_dtype = probs_dtype;
    p.q = static_cast<uint8_t*>(q); p.s = s; p.qt = static_cast<uint8_t*>(qt); p.st = st;
    p.round_scale = round_scale;
    switch (dtype) {
        case LH_BF16: return gather_launch<__nv_bfloat16>(p, stream);
        case LH_F16: return gather_launch<__half>(p, stream);
        case LH_F32: return gather_launch<float>(p, stream);
    }
    return fail_arg("unsupported dtype %d", dtype);
}

// float16 / float32 instantiations (lh_tile_any.cu)
int tile_norm_any(const void* x, const void* gamma, const float* r, int dtype, int64_t M, int64_t n, void* q, float* s,
                  void* qt, float* st, int round_scale, int mode, cudaStream_t stream);
int tile_silu_fwd_any(const void* x, const void* w, int w_dtype, int dtype, const void* counts, int counts_type, int E,
                      int64_t M, int64_t n, void* q, float* s, void* qt, float* st, int round_scale, int mode,
                      cudaStream_t stream);
int tile_silu_bwd_any(const void* g, const void* x, const void* w, int w_dtype, int dtype, const void* counts,
                      int counts_type, int E, int64_t M, int64_t n, void* dx_q, float* dx_s, void* dx_qt, float* dx_st,
                      void* hp, float* dws, int round_scale, cudaStream_t stream);

// RMSNorm with known 1/rms + quantisation.  bfloat16: transposed outputs only (mode 1); the other
// input types: every mode.
int tile_norm(const void* x, const void* gamma, const float* r, int dtype, int64_t M, int64_t n, void* q, float* s,
              void* qt, float* st, int round_scale, int mode, cudaStream_t stream, int descending) {
    if (dtype != LH_BF16) return tile_norm_any(x, gamma, r, dtype, M, n, q, s, qt, st, round_scale, mode, stream);
    return tile_norm_t<__nv_bfloat16, false>(x, gamma, r, dtype, M, n, q, s, qt, st, round_scale, mode, stream, descending);
}

int tile_silu_fwd(const void* x, const void* w, int w_dtype, int dtype, const void* counts, int counts_type, int E,
                  int64_t M, int64_t n, void* q, float* s, void* qt, float* st, int round_scale, int mode,
                  cudaStream_t stream) {
    if (dtype != LH_BF16)
        return tile_silu_fwd_any(x, w, w_dtype, dtype, counts, counts_type, E, M, n, q, s, qt, st, round_scale, mode, stream);
    return tile_silu_fwd_t<__nv_bfloat16>(x, w, w_dtype, dtype, counts, counts_type, E, M, n, q, s, qt, st, round_scale,
                                          mode, stream);
}

int tile_silu_bwd(const void* g, const void* x, const void* w, int w_dtype, int dtype, const void* counts,
                  int counts_type, int E, int64_t M, int64_t n, void* dx_q, float* dx_s, void* dx_qt, float* dx_st,
                  void* hp, float* dws, int round_scale, cudaStream_t stream) {
    if (dtype != LH_BF16)
        return tile_silu_bwd_any(g, x, w, w_dtype, dtype, counts, counts_type, E, M, n, dx_q, dx_s, dx_qt, dx_st, hp, dws,
                                 round_scale, stream);
    return tile_silu_bwd_t<__nv_bfloat16>(g, x, w, w_dtype, dtype, counts, counts_type, E, M, n, dx_q, dx_s, dx_qt, dx_st,
                                          hp, dws, round_scale, stream);
}

}  // namespace lh
