// Row-slab kernels: operations that need a whole row before anything can be emitted
// (RMSNorm forward with 1x128 quantisation or plain output, RMSNorm backward).
//
// Execution model (sm_100a): persistent CTAs walk slabs of RB complete rows
// (RB * n <= 8192 elements).  A producer warp brings each slab in with ONE bulk
// asynchronous copy per operand (rows are contiguous in memory) into a shared-memory
// ring guarded by mbarriers; consumer threads each own EPT contiguous elements of the
// slab, pull them into registers (releasing the ring slot at once), reduce the per-row
// sums through shuffles + one named barrier, and stage the outputs in shared memory
// from where one bulk copy per slab writes them back.  No tensor cores: HBM-bound.
#include "lh_common.cuh"

#ifndef LH_ROWS_EXACT
#define LH_ROWS_EXACT true
#endif

namespace lh {

enum : int { ROP_NORM_Q = 0, ROP_NORM_Y = 1, ROP_NORM_BWD = 2 };

constexpr int kSlabElems = 8192;
constexpr int kMaxRowCtas = 296;

struct RowParams {
    const uint8_t* x;
    const uint8_t* dy;
    const void* gamma;
    float* rms;          // [M] 1/rms (written unless reuse_rms)
    int reuse_rms;
    float eps;
    int64_t M;
    int n;
    int RB;              // rows per slab
    uint8_t* q;          // ROP_NORM_Q: codes [M,n]
    float* s;            // ROP_NORM_Q: scales [n/128, M]
    uint8_t* hp;         // ROP_NORM_Y: y [M,n]; ROP_NORM_BWD: dx [M,n]
    float* partial;      // ROP_NORM_BWD: [gridDim.x, n] per-CTA dgamma partial sums
    int round_scale;
};

template <int ROP, int EPT, int STAGES>
struct RowCfg {
    static constexpr int NIN = ROP == ROP_NORM_BWD ? 2 : 1;
    static constexpr int NT = kSlabElems / EPT;       // consumer threads
    static constexpr int NW = NT / 32;
    static constexpr int NTHREADS = NT;
    static constexpr int SLABB = kSlabElems * 2;      // bytes of one operand slab (16-bit inputs)
    static constexpr int STAGEB = NIN * SLABB;
    static constexpr int OUTB = ROP == ROP_NORM_Q ? kSlabElems : kSlabElems * 2;
    static constexpr int OFF_STAGES = 0;
    static constexpr int OFF_OUT = STAGES * STAGEB;   // two output buffers
    static constexpr int OFF_RED = OFF_OUT + 2 * OUTB;            // [2][2][64] partial sums
    static constexpr int OFF_BAR = OFF_RED + 2 * 2 * 64 * 4;
    static constexpr int SMEM = OFF_BAR + 2 * STAGES * 8;
};

template <int ROP, int EPT, int STAGES, int MINB>
__global__ void __launch_bounds__(RowCfg<ROP, EPT, STAGES>::NTHREADS, MINB)
rows_kernel(const __grid_constant__ RowParams p) {
    using C = RowCfg<ROP, EPT, STAGES>;
    constexpr int NT = C::NT, NW = C::NW, NCH = EPT / 8;  // 16-byte chunks per thread and operand
    constexpr int LPB = 128 / EPT;                         // lanes per 128-element block
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem + C::OFF_STAGES;
    uint8_t* outb = smem + C::OFF_OUT;
    float* red = reinterpret_cast<float*>(smem + C::OFF_RED);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty = full + STAGES;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int n = p.n, RB = p.RB;
    const int64_t slabs = (p.M + RB - 1) / RB;

    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    // Thread 0 doubles as the producer: one bulk copy per operand and slab.
    auto issue = [&](int64_t slab, int stage) {
        const int64_t r0 = slab * RB;
        const int nrows = int(p.M - r0 < RB ? p.M - r0 : RB);
        const uint32_t bytes = uint32_t(nrows) * uint32_t(n) * 2u;
        uint8_t* dst = stages + size_t(stage) * C::STAGEB;
        mbar_expect_tx(&full[stage], bytes * C::NIN);
        bulk_g2s(dst, p.x + r0 * n * 2, bytes, &full[stage]);
        if constexpr (C::NIN == 2) bulk_g2s(dst + C::SLABB, p.dy + r0 * n * 2, bytes, &full[stage]);
    };
    if (tid == 0) {
        int64_t slab = blockIdx.x;
        for (int j = 0; j < STAGES && slab < slabs; ++j, slab += gridDim.x) issue(slab, j);
    }

    // ================================ consumers ===================================
    const int t = tid;
    const int e0 = t * EPT;                        // first element of this thread inside the slab
    const int my_row = e0 / n;                     // row inside the slab
    const int col0 = e0 - my_row * n;              // first column
    const bool in_slab = my_row < RB;              // threads beyond RB*n idle (n not dividing 8192)
    const int TPR = n / EPT;                       // threads per row
    const bool warp_rows = (TPR % 32) == 0;        // rows are made of whole warps
    const int nb = n >> 7;
    const int sw = NCH == 4 ? ((t >> 1) & 3) : ((t >> 2) & 1);  // bank-conflict-free chunk order
    const bool rs = p.round_scale != 0;

    // gamma for this thread's columns, in the (swizzled) chunk order used for x
    float gam[EPT];
    if (in_slab) {
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.gamma) +
                                                              (col0 + 8 * (k ^ sw)) * 2);
            Elem<__nv_bfloat16>::unpack8(raw, gam + 8 * k);
        }
    } else {
#pragma unroll
        for (int i = 0; i < EPT; ++i) gam[i] = 0.f;
    }
    float acc[ROP == ROP_NORM_BWD ? EPT : 1];
#pragma unroll
    for (int i = 0; i < (ROP == ROP_NORM_BWD ? EPT : 1); ++i) acc[i] = 0.f;

    int it = 0;
    for (int64_t slab = blockIdx.x; slab < slabs; slab += gridDim.x, ++it) {
        const int stage = it % STAGES;
        const int buf = it & 1;
        if (tid == 0 && it > 0) {
            // every warp released stage (it-1)%STAGES before the barriers of iteration it-1
            const int64_t nxt = slab + int64_t(STAGES - 1) * gridDim.x;
            if (nxt < slabs) {
                const int ps = (it - 1) % STAGES;
                if (mbar_wait(&empty[ps], ((it - 1) / STAGES) & 1, DEVERR_EMPTY_WAIT)) issue(nxt, ps);
            }
        }
        const int64_t row0 = slab * RB;
        const int rows = int(p.M - row0 < RB ? p.M - row0 : RB);
        const bool active = in_slab && my_row < rows;
        if (!mbar_wait(&full[stage], (it / STAGES) & 1, DEVERR_FULL_WAIT)) return;
        const uint8_t* sx = stages + size_t(stage) * C::STAGEB + size_t(e0) * 2;

        float x[EPT];
        float g[ROP == ROP_NORM_BWD ? EPT : 1];
        {
            uint4 raw[NCH];
#pragma unroll
            for (int k = 0; k < NCH; ++k) raw[k] = *reinterpret_cast<const uint4*>(sx + 16 * (k ^ sw));
            if constexpr (ROP == ROP_NORM_BWD) {
                uint4 rawg[NCH];
#pragma unroll
                for (int k = 0; k < NCH; ++k)
                    rawg[k] = *reinterpret_cast<const uint4*>(sx + C::SLABB + 16 * (k ^ sw));
#pragma unroll
                for (int k = 0; k < NCH; ++k) Elem<__nv_bfloat16>::unpack8(rawg[k], g + 8 * k);
            }
#pragma unroll
            for (int k = 0; k < NCH; ++k) Elem<__nv_bfloat16>::unpack8(raw[k], x + 8 * k);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);   // data is in registers: free the slot
        if (!active) {
#pragma unroll
            for (int i = 0; i < EPT; ++i) x[i] = 0.f;
            if constexpr (ROP == ROP_NORM_BWD) {
#pragma unroll
                for (int i = 0; i < EPT; ++i) g[i] = 0.f;
            }
        }

        // ---- per-row sums: sum x^2 (unless 1/rms is given) and, backward, sum x*g*gamma
        float ss = 0.f, sc = 0.f;
        if (!p.reuse_rms) {
#pragma unroll
            for (int i = 0; i < EPT; ++i) ss = fmaf(x[i], x[i], ss);
        }
        if constexpr (ROP == ROP_NORM_BWD) {
#pragma unroll
            for (int i = 0; i < EPT; ++i) sc = fmaf(x[i], g[i] * gam[i], sc);
        }
        float* red_ss = red + buf * 128;
        float* red_sc = red + buf * 128 + 64;
        if (warp_rows) {
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) {
                ss += __shfl_xor_sync(0xffffffffu, ss, d);
                if constexpr (ROP == ROP_NORM_BWD) sc += __shfl_xor_sync(0xffffffffu, sc, d);
            }
            if (lane == 0) { red_ss[warp] = ss; if constexpr (ROP == ROP_NORM_BWD) red_sc[warp] = sc; }
        } else {
#pragma unroll
            for (int d = LPB / 2; d >= 1; d >>= 1) {
                ss += __shfl_xor_sync(0xffffffffu, ss, d);
                if constexpr (ROP == ROP_NORM_BWD) sc += __shfl_xor_sync(0xffffffffu, sc, d);
            }
            if ((t % LPB) == 0) { red_ss[t / LPB] = ss; if constexpr (ROP == ROP_NORM_BWD) red_sc[t / LPB] = sc; }
        }
        if (t == 0) bulk_wait_read<1>();               // output buffer `buf` is free again
        named_bar<1, NT>();
        float tot_ss = 0.f, tot_sc = 0.f;
        if (in_slab) {
            const int cnt = warp_rows ? TPR / 32 : nb;
            const int first = my_row * cnt;
            for (int i = 0; i < cnt; ++i) {
                tot_ss += red_ss[first + i];
                if constexpr (ROP == ROP_NORM_BWD) tot_sc += red_sc[first + i];
            }
        }
        float r;
        if (p.reuse_rms) {
            r = active ? p.rms[row0 + my_row] : 0.f;
        } else {
            r = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(tot_ss, float(n)), p.eps)));
            if (active && col0 == 0 && p.rms != nullptr) p.rms[row0 + my_row] = r;
        }

        if constexpr (ROP == ROP_NORM_Q) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < EPT; ++i) {
                x[i] = __fmul_rn(__fmul_rn(x[i], r), gam[i]);
                a = fmaxf(a, fabsf(x[i]));
            }
#pragma unroll
            for (int d = LPB / 2; d >= 1; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
            const float scale = scale_from_amax(a, rs);
            const Divisor dv(scale);
            uint8_t* so = outb + buf * C::OUTB + e0;
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const float* v = x + 8 * k;
                const uint32_t lo = cvt_e4m3x4(dv.quot<LH_ROWS_EXACT>(v[0]), dv.quot<LH_ROWS_EXACT>(v[1]),
                                               dv.quot<LH_ROWS_EXACT>(v[2]), dv.quot<LH_ROWS_EXACT>(v[3]));
                const uint32_t hi = cvt_e4m3x4(dv.quot<LH_ROWS_EXACT>(v[4]), dv.quot<LH_ROWS_EXACT>(v[5]),
                                               dv.quot<LH_ROWS_EXACT>(v[6]), dv.quot<LH_ROWS_EXACT>(v[7]));
                *reinterpret_cast<uint2*>(so + 8 * (k ^ sw)) = make_uint2(lo, hi);
            }
            if (active && (t % LPB) == 0) p.s[int64_t(col0 >> 7) * p.M + row0 + my_row] = scale;
        } else if constexpr (ROP == ROP_NORM_Y) {
            uint8_t* so = outb + buf * C::OUTB + size_t(e0) * 2;
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                float y[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) y[c] = __fmul_rn(__fmul_rn(x[8 * k + c], r), gam[8 * k + c]);
                *reinterpret_cast<uint4*>(so + 16 * (k ^ sw)) =
                    make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]), pack_bf16x2(y[4], y[5]),
                               pack_bf16x2(y[6], y[7]));
            }
        } else {  // ROP_NORM_BWD: dx = r*g*gamma - r^3 * x * sum(x*g*gamma)/n ; dgamma += x*g*r
            const float coef = r * r * r * tot_sc / float(n);
            uint8_t* so = outb + buf * C::OUTB + size_t(e0) * 2;
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                float d[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int i = 8 * k + c;
                    d[c] = fmaf(-coef, x[i], r * (g[i] * gam[i]));
                    acc[i] = fmaf(x[i] * g[i], r, acc[i]);
                }
                *reinterpret_cast<uint4*>(so + 16 * (k ^ sw)) =
                    make_uint4(pack_bf16x2(d[0], d[1]), pack_bf16x2(d[2], d[3]), pack_bf16x2(d[4], d[5]),
                               pack_bf16x2(d[6], d[7]));
            }
        }
        fence_async_smem();
        named_bar<2, NT>();
        if (t == 0) {
            const uint32_t out_bytes = uint32_t(rows) * uint32_t(n) * (ROP == ROP_NORM_Q ? 1u : 2u);
            uint8_t* gdst = (ROP == ROP_NORM_Q ? p.q : p.hp) + row0 * n * (ROP == ROP_NORM_Q ? 1 : 2);
            bulk_s2g(gdst, outb + buf * C::OUTB, out_bytes);
            bulk_commit();
        }
    }
    if (t == 0) bulk_wait_all();

    if constexpr (ROP == ROP_NORM_BWD) {
        // Fold the per-thread dgamma sums of the RB rows of a slab into one row and
        // publish this CTA's partial; a second kernel adds the partials in a fixed order.
        float* fold = reinterpret_cast<float*>(stages);   // ring is idle: every slab was consumed
        named_bar<1, NT>();
#pragma unroll
        for (int i = 0; i < EPT; ++i) fold[(8 * ((i >> 3) ^ sw) + (i & 7)) * NT + t] = acc[i];
        named_bar<2, NT>();
        if (t < TPR) {
            for (int j = 0; j < EPT; ++j) {   // j: column offset inside this thread's span
                float a = 0.f;
                for (int rr = 0; rr < RB; ++rr) a += fold[j * NT + t + rr * TPR];
                p.partial[int64_t(blockIdx.x) * n + col0 + j] = a;
            }
        }
    }
}

__global__ void dgamma_reduce_kernel(const float* __restrict__ partial, int parts, int n, float* __restrict__ out) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    float a = 0.f;
    for (int b = 0; b < parts; ++b) a += partial[int64_t(b) * n + j];
    out[j] = a;
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
template <int ROP, int EPT, int STAGES, int CTAS_PER_SM>
static int launch_rows(RowParams p, int* grid_out, cudaStream_t stream) {
    using C = RowCfg<ROP, EPT, STAGES>;
    auto kern = rows_kernel<ROP, EPT, STAGES, CTAS_PER_SM>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(C::SMEM));
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return int(e); }
    p.RB = kSlabElems / p.n;
    const int64_t slabs = (p.M + p.RB - 1) / p.RB;
    int64_t grid = int64_t(sm_count()) * CTAS_PER_SM;
    if (grid > kMaxRowCtas) grid = kMaxRowCtas;
    if (slabs < grid) grid = slabs;
    if (grid_out) *grid_out = int(grid);
    kern<<<dim3(unsigned(grid)), dim3(C::NTHREADS), C::SMEM, stream>>>(p);
    return check_launch("rows_kernel");
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_rows(const char* what, int dtype, int64_t M, int64_t n) {
    if (dtype != LH_BF16) return fail_arg("%s: only bf16 inputs are supported", what);
    if (M < 0 || n <= 0 || (n % 128) != 0 || n > kSlabElems)
        return fail_arg("%s: need n %% 128 == 0 and n <= 8192 (M=%lld n=%lld)", what, (long long)M, (long long)n);
    return LH_OK;
}

int rows_norm_quant(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* q,
                    float* s, float* rms, int round_scale, cudaStream_t stream) {
    if (int rc = check_rows("rmsnorm_blockquant_fwd", dtype, M, n)) return rc;
    if (!x || !gamma || !q || !s || !rms) return fail_arg("rmsnorm_blockquant_fwd: NULL pointer");
    if (!aligned16(x) || !aligned16(q) || !aligned16(gamma)) return fail_arg("rmsnorm_blockquant_fwd: pointers must be 16-byte aligned");
    if (M == 0) return LH_OK;
    RowParams p{};
    p.x = static_cast<const uint8_t*>(x); p.gamma = gamma; p.rms = rms; p.eps = eps; p.M = M; p.n = int(n);
    p.q = static_cast<uint8_t*>(q); p.s = s; p.round_scale = round_scale;
    return launch_rows<ROP_NORM_Q, 32, 4, 2>(p, nullptr, stream);
}

int rows_norm_y(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* y,
                float* rms, int reuse_rms, cudaStream_t stream) {
    if (int rc = check_rows("rmsnorm_fwd", dtype, M, n)) return rc;
    if (!x || !gamma || !y || (reuse_rms && !rms)) return fail_arg("rmsnorm_fwd: NULL pointer");
    if (!aligned16(x) || !aligned16(y) || !aligned16(gamma)) return fail_arg("rmsnorm_fwd: pointers must be 16-byte aligned");
    if (M == 0) return LH_OK;
    RowParams p{};
    p.x = static_cast<const uint8_t*>(x); p.gamma = gamma; p.rms = rms; p.reuse_rms = reuse_rms; p.eps = eps;
    p.M = M; p.n = int(n); p.hp = static_cast<uint8_t*>(y);
    return launch_rows<ROP_NORM_Y, 32, 4, 2>(p, nullptr, stream);
}

int64_t rows_norm_bwd_scratch(int64_t n) { return int64_t(kMaxRowCtas) * n * 4; }

int rows_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M,
                  int64_t n, float eps, void* dx, float* dgamma, void* scratch, int64_t scratch_bytes,
                  cudaStream_t stream) {
    if (int rc = check_rows("rmsnorm_bwd", dtype, M, n)) return rc;
    if (!x || !dy || !gamma || !dx || !dgamma) return fail_arg("rmsnorm_bwd: NULL pointer");
    if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(gamma)) return fail_arg("rmsnorm_bwd: pointers must be 16-byte aligned");
    if (!scratch || scratch_bytes < rows_norm_bwd_scratch(n)) return fail_arg("rmsnorm_bwd: scratch too small (%lld < %lld)", (long long)scratch_bytes, (long long)rows_norm_bwd_scratch(n));
    if (M == 0) {
        cudaError_t e = cudaMemsetAsync(dgamma, 0, size_t(n) * 4, stream);
        return e == cudaSuccess ? LH_OK : int(e);
    }
    RowParams p{};
    p.x = static_cast<const uint8_t*>(x); p.dy = static_cast<const uint8_t*>(dy); p.gamma = gamma;
    p.rms = const_cast<float*>(rms); p.reuse_rms = rms != nullptr; p.eps = eps; p.M = M; p.n = int(n);
    p.hp = static_cast<uint8_t*>(dx); p.partial = static_cast<float*>(scratch);
    int grid = 0;
    if (int rc = launch_rows<ROP_NORM_BWD, 16, 3, 1>(p, &grid, stream)) return rc;
    dgamma_reduce_kernel<<<dim3(unsigned((n + 127) / 128)), dim3(128), 0, stream>>>(p.partial, grid, int(n), dgamma);
    return check_launch("dgamma_reduce_kernel");
}

}  // namespace lh
