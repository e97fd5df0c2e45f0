// Row-slab kernels: RMSNorm forward (+1x128 FP8 quantisation, or plain) and RMSNorm backward
// -- the operations whose outputs depend on a whole row, so they stream rows through the SM.
//
// Execution model (sm_100a): persistent CTAs walk slabs of at most 8192 elements (RB complete
// rows).  Thread 0 of warp 0 brings each slab into a shared-memory ring with bulk asynchronous
// copies (TMA; the rows of a slab are contiguous, so one copy per operand) that complete on an
// mbarrier.  Every thread owns EPT
// contiguous elements: it pulls them into registers (freeing the ring slot at once), does
// the arithmetic with packed float32x2 instructions, reduces per-row sums through
// shuffles and one named barrier, and stages the outputs in shared memory from where one
// bulk copy per warp writes them back.  No tensor cores: the path is HBM-bound.
#include "lh_common.cuh"

namespace lh {

int small_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int64_t M, int64_t n, float eps,
                   void* dx, float* partial, int max_parts, int* parts, void* dy_q, float* dy_s, int round_scale,
                   cudaStream_t stream, void* dy_qt = nullptr, float* dy_st = nullptr);
// float16 / float32 inputs (lh_anytype.cu)
int any_norm_fwd(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* y, float* rms,
                 int reuse_rms, cudaStream_t stream);
int any_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M, int64_t n,
                 float eps, void* dx, float* dgamma, float* partial, int max_parts, cudaStream_t stream);

enum : int { ROP_NORM_Q = 0, ROP_NORM_Y = 1, ROP_NORM_BWD = 2, ROP_NORM_YQ = 4 };

constexpr int kSlabElems = 8192;
constexpr int kMaxRowCtas = 592;   // four CTAs per SM at most

struct RowParams {
    const uint8_t* x;
    const uint8_t* dy;
    const void* gamma;
    float* rms;          // [M] 1/rms (written unless reuse_rms)
    int reuse_rms;
    float eps;
    float inv_n;         // 1 / n
    int64_t M;
    int n;               // output columns
    int RB;              // rows per slab
    uint8_t* q;          // *_Q: codes [M,n]
    float* s;            // *_Q: scales [n/128, M]
    uint8_t* hp;         // ROP_NORM_Y, ROP_NORM_YQ: y [M,n]; ROP_NORM_BWD: dx [M,n]
    float* partial;      // ROP_NORM_BWD: [gridDim.x, n] per-CTA dgamma partial sums
    int round_scale;
};

template <int ROP, int EPT, int STAGES>
struct RowCfg {
    static constexpr int NIN = ROP == ROP_NORM_BWD ? 2 : 1;
    static constexpr bool QUANT = ROP == ROP_NORM_Q || ROP == ROP_NORM_YQ;
    static constexpr int NT = kSlabElems / EPT;       // threads
    static constexpr int NW = NT / 32;
    static constexpr int SLABB = kSlabElems * 2;      // bytes of one operand slab (16-bit inputs)
    static constexpr int STAGEB = NIN * SLABB;
    static constexpr int OUTB = QUANT ? kSlabElems : kSlabElems * 2;
    static constexpr int OFF_STAGES = 0;
    static constexpr int OFF_OUT = STAGES * STAGEB;               // two output buffers
    static constexpr int OFF_RED = OFF_OUT + 2 * OUTB;            // [2][2][64] partial sums
    static constexpr int OFF_BAR = OFF_RED + 2 * 2 * 64 * 4;
    static constexpr int SMEM = OFF_BAR + 2 * STAGES * 8;
};

struct SlabLoc {
    int64_t row0;
    int rows;   // valid rows
};

template <int ROP, int EPT, int STAGES, int MINB>
__global__ void __launch_bounds__(RowCfg<ROP, EPT, STAGES>::NT, MINB)
rows_kernel(const __grid_constant__ RowParams p) {
    using C = RowCfg<ROP, EPT, STAGES>;
    constexpr int NT = C::NT, NW = C::NW;
    constexpr int NCH = EPT / 8;     // 16-byte chunks per thread and operand
    constexpr int NP = EPT / 2;      // float2 pairs per thread
    constexpr int LPB = 128 / EPT;   // lanes per 128-element block
    constexpr int OB = C::QUANT ? 1 : 2;          // bytes per output element
    constexpr int WSPAN = 32 * EPT;               // elements owned by one warp in a slab
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem + C::OFF_STAGES;
    uint8_t* outb = smem + C::OFF_OUT;
    float* red = reinterpret_cast<float*>(smem + C::OFF_RED);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty = full + STAGES;

    const int t = threadIdx.x;
    const int warp = t >> 5, lane = t & 31;
    const int n = p.n;
    const int RB = p.RB;
    const int64_t slabs = (p.M + RB - 1) / RB;

    if (t == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    auto locate = [&](int64_t slab) {
        SlabLoc L;
        L.row0 = slab * RB;
        const int64_t left = p.M - L.row0;
        L.rows = left < RB ? int(left) : RB;
        return L;
    };

    // Lane 0 of warp 0 doubles as the producer.
    auto issue = [&](int64_t slab, int stage) {
        const SlabLoc L = locate(slab);
        uint8_t* dst = stages + size_t(stage) * C::STAGEB;
        if (lane == 0) {
            const uint32_t bytes = uint32_t(L.rows) * uint32_t(n) * 2u;
            mbar_expect_tx(&full[stage], bytes * C::NIN);
            bulk_g2s(dst, p.x + L.row0 * n * 2, bytes, &full[stage]);
            if constexpr (ROP == ROP_NORM_BWD) bulk_g2s(dst + C::SLABB, p.dy + L.row0 * n * 2, bytes, &full[stage]);
        }
    };
    if (warp == 0) {
        int64_t slab = blockIdx.x;
        for (int j = 0; j < STAGES && slab < slabs; ++j, slab += gridDim.x) issue(slab, j);
    }

    const int e0 = t * EPT;                        // first element of this thread inside the slab
    const int sw = NCH == 4 ? ((t >> 1) & 3) : ((t >> 2) & 1);  // bank-conflict-free chunk order
    const bool rs = p.round_scale != 0;
    const bool reuse = ROP != ROP_NORM_Q && ROP != ROP_NORM_YQ && p.reuse_rms != 0;

    // A slab is RB full rows, so a thread's columns never change: keep gamma for them in
    // registers, in the (swizzled) chunk order used for x.
    float2 gam[NP];
    const int my_row = e0 / n;
    const int col0 = e0 - my_row * n;
    const bool in_slab = my_row < RB;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (in_slab)
            raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.gamma) + (col0 + 8 * (k ^ sw)) * 2);
        gam[4 * k + 0] = bf16x2_to_f2(raw.x);
        gam[4 * k + 1] = bf16x2_to_f2(raw.y);
        gam[4 * k + 2] = bf16x2_to_f2(raw.z);
        gam[4 * k + 3] = bf16x2_to_f2(raw.w);
    }
    const int TPR = n / EPT;                       // threads per row (norm kernels)
    const bool warp_rows = (TPR % 32) == 0;        // rows are made of whole warps
    const int red_cnt = warp_rows ? TPR / 32 : (n >> 7);
    const int red_first = my_row * red_cnt;
    const bool row_bar = warp_rows && RB <= 8 && RB * TPR == NT;   // the same for every thread
    float2 acc[ROP == ROP_NORM_BWD ? NP : 1];
#pragma unroll
    for (int i = 0; i < (ROP == ROP_NORM_BWD ? NP : 1); ++i) acc[i] = make_float2(0.f, 0.f);

    int stage = 0, prev_stage = 0;
    uint32_t phase = 0, prev_phase = 0;
    int buf = 0;
    bool first_it = true;
    bool dead = false;   // a bounded wait of this thread gave up (see mbar_wait_or_mark)
    for (int64_t slab = blockIdx.x; slab < slabs; slab += gridDim.x) {
        if (warp == 0 && !first_it) {
            // every warp released the previous stage early in the previous iteration
            const int64_t nxt = slab + int64_t(STAGES - 1) * gridDim.x;
            if (nxt < slabs) {
                mbar_wait_or_mark<true>(&empty[prev_stage], prev_phase, DEVERR_EMPTY_WAIT, dead);
                if (!dead) issue(nxt, prev_stage);
            }
        }
        const SlabLoc L = locate(slab);
        const int slab_elems = L.rows * n;                 // valid elements in this slab
        const bool active = in_slab && my_row < L.rows;
        mbar_wait_or_mark<true>(&full[stage], phase, DEVERR_FULL_WAIT, dead);
        const uint8_t* sx = stages + size_t(stage) * C::STAGEB + size_t(e0) * 2;

        float2 x[NP];
        float2 g[C::NIN == 2 ? NP : 1];
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const uint4 raw = *reinterpret_cast<const uint4*>(sx + 16 * (k ^ sw));
            x[4 * k + 0] = bf16x2_to_f2(raw.x);
            x[4 * k + 1] = bf16x2_to_f2(raw.y);
            x[4 * k + 2] = bf16x2_to_f2(raw.z);
            x[4 * k + 3] = bf16x2_to_f2(raw.w);
        }
        if constexpr (C::NIN == 2) {
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const uint4 raw = *reinterpret_cast<const uint4*>(sx + C::SLABB + 16 * (k ^ sw));
                g[4 * k + 0] = bf16x2_to_f2(raw.x);
                g[4 * k + 1] = bf16x2_to_f2(raw.y);
                g[4 * k + 2] = bf16x2_to_f2(raw.z);
                g[4 * k + 3] = bf16x2_to_f2(raw.w);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);   // data is in registers: free the slot
        if (__any_sync(0xffffffffu, !active)) {      // only ragged slabs get here
            if (!active) {
#pragma unroll
                for (int i = 0; i < NP; ++i) x[i] = make_float2(0.f, 0.f);
                if constexpr (C::NIN == 2) {
#pragma unroll
                    for (int i = 0; i < NP; ++i) g[i] = make_float2(0.f, 0.f);
                }
            }
        }
        // this warp's output span of the previous use of `buf` must have been read out
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();

        float r = 0.f, tot_sc = 0.f;
        {
            // ---- per-row sums: sum x^2 (unless 1/rms is given) and, backward, sum x*g*gamma
            float2 ss2 = make_float2(0.f, 0.f), ss3 = ss2, sc2 = ss2, sc3 = ss2;
            if (!reuse) {
#pragma unroll
                for (int i = 0; i < NP; i += 2) {
                    ss2 = fma2(x[i], x[i], ss2);
                    ss3 = fma2(x[i + 1], x[i + 1], ss3);
                }
            }
            if constexpr (ROP == ROP_NORM_BWD) {
#pragma unroll
                for (int i = 0; i < NP; i += 2) {
                    sc2 = fma2(x[i], mul2(g[i], gam[i]), sc2);
                    sc3 = fma2(x[i + 1], mul2(g[i + 1], gam[i + 1]), sc3);
                }
            }
            ss2 = add2(ss2, ss3);
            sc2 = add2(sc2, sc3);
            float ss = ss2.x + ss2.y, sc = sc2.x + sc2.y;
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
            // rows are independent: when a row is made of whole warps only its own warps meet
            // (barrier 1 + row), so the row groups of a slab drift apart and overlap their phases
            if (row_bar) asm volatile("bar.sync %0, %1;" ::"r"(1 + my_row), "r"(TPR) : "memory");
            else named_bar<1, NT>();
            float tot_ss = 0.f;
            if (red_cnt == 8) {   // one row per slab: two vector loads
                const float4 a = *reinterpret_cast<const float4*>(red_ss + red_first);
                const float4 b = *reinterpret_cast<const float4*>(red_ss + red_first + 4);
                tot_ss = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
                if constexpr (ROP == ROP_NORM_BWD) {
                    const float4 c = *reinterpret_cast<const float4*>(red_sc + red_first);
                    const float4 d = *reinterpret_cast<const float4*>(red_sc + red_first + 4);
                    tot_sc = ((c.x + c.y) + (c.z + c.w)) + ((d.x + d.y) + (d.z + d.w));
                }
            } else if (in_slab) {
#pragma unroll 4
                for (int i = 0; i < red_cnt; ++i) {
                    tot_ss += red_ss[red_first + i];
                    if constexpr (ROP == ROP_NORM_BWD) tot_sc += red_sc[red_first + i];
                }
            }
            if (reuse) {
                r = active ? p.rms[L.row0 + my_row] : 0.f;
            } else {
                r = rsqrt_nr(fmaf(tot_ss, p.inv_n, p.eps));
                if (active && col0 == 0 && p.rms != nullptr) p.rms[L.row0 + my_row] = r;
            }
        }

        uint8_t* so = outb + buf * C::OUTB + size_t(e0) * OB;
        if constexpr (C::QUANT) {
            {
                const float2 r2 = splat2(r);
#pragma unroll
                for (int i = 0; i < NP; ++i) x[i] = mul2(mul2(x[i], r2), gam[i]);
                if constexpr (ROP == ROP_NORM_YQ) {
                    // the 16-bit y goes straight from registers to global memory
                    if (active) {
                        uint8_t* yo = p.hp + ((L.row0 + my_row) * n + col0) * 2;
#pragma unroll
                        for (int k = 0; k < NCH; ++k)
                            *reinterpret_cast<uint4*>(yo + 16 * (k ^ sw)) =
                                make_uint4(pack_bf16x2(x[4 * k + 0].x, x[4 * k + 0].y), pack_bf16x2(x[4 * k + 1].x, x[4 * k + 1].y),
                                           pack_bf16x2(x[4 * k + 2].x, x[4 * k + 2].y), pack_bf16x2(x[4 * k + 3].x, x[4 * k + 3].y));
                    }
                }
            }
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int i = 0; i < NP; i += 2) {
                a0 = max3abs(x[i].x, x[i].y, a0);
                a1 = max3abs(x[i + 1].x, x[i + 1].y, a1);
            }
            float a = fmaxf(a0, a1);
#pragma unroll
            for (int d = LPB / 2; d >= 1; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
            const float scale = scale_from_amax(a, rs);
            const float2 inv = splat2(rcp_approx(scale));
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const float2 q0 = mul2(x[4 * k + 0], inv), q1 = mul2(x[4 * k + 1], inv);
                const float2 q2 = mul2(x[4 * k + 2], inv), q3 = mul2(x[4 * k + 3], inv);
                const uint32_t lo = cvt_e4m3x4(q0.x, q0.y, q1.x, q1.y);
                const uint32_t hi = cvt_e4m3x4(q2.x, q2.y, q3.x, q3.y);
                *reinterpret_cast<uint2*>(so + 8 * (k ^ sw)) = make_uint2(lo, hi);
            }
            if (active && (t % LPB) == 0) p.s[int64_t(col0 >> 7) * p.M + L.row0 + my_row] = scale;
        } else if constexpr (ROP == ROP_NORM_Y) {
            const float2 r2 = splat2(r);
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 y = mul2(mul2(x[4 * k + j], r2), gam[4 * k + j]);
                    w[j] = pack_bf16x2(y.x, y.y);
                }
                *reinterpret_cast<uint4*>(so + 16 * (k ^ sw)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {  // ROP_NORM_BWD: dx = r*g*gamma - r^3 * x * sum(x*g*gamma)/n ; dgamma += x*g*r
            const float2 ncoef = splat2(-(r * r * r * tot_sc * p.inv_n));
            const float2 r2 = splat2(r);
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = 4 * k + j;
                    const float2 d = fma2(ncoef, x[i], mul2(r2, mul2(g[i], gam[i])));
                    acc[i] = fma2(mul2(x[i], g[i]), r2, acc[i]);
                    w[j] = pack_bf16x2(d.x, d.y);
                }
                *reinterpret_cast<uint4*>(so + 16 * (k ^ sw)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        // Each warp writes back its own contiguous span of the slab with one bulk copy.
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            int cnt = slab_elems - warp * WSPAN;
            cnt = cnt > WSPAN ? WSPAN : cnt;
            if (cnt > 0) {
                uint8_t* gbase = C::QUANT ? p.q : p.hp;
                const int64_t gofs = L.row0 * n;
                bulk_s2g(gbase + (gofs + warp * WSPAN) * OB,
                         outb + buf * C::OUTB + size_t(warp) * WSPAN * OB, uint32_t(cnt) * OB);
            }
            bulk_commit();
        }
        first_it = false;
        prev_stage = stage; prev_phase = phase;
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        buf ^= 1;
    }
    if (lane == 0) bulk_wait_all();

    if constexpr (ROP == ROP_NORM_BWD) {
        // Fold the per-thread dgamma sums of the RB rows of a slab into one row and
        // publish this CTA's partial; a second kernel adds the partials in a fixed order.
        float* fold = reinterpret_cast<float*>(stages);   // ring is idle: every slab was consumed
        named_bar<10, NT>();
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const int j = 8 * ((i >> 2) ^ sw) + 2 * (i & 3);   // column offset inside this thread's span
            fold[j * NT + t] = acc[i].x;
            fold[(j + 1) * NT + t] = acc[i].y;
        }
        named_bar<11, NT>();
        if (t < TPR) {
            for (int j = 0; j < EPT; ++j) {
                float a = 0.f;
                for (int rr = 0; rr < RB; ++rr) a += fold[j * NT + t + rr * TPR];
                p.partial[int64_t(blockIdx.x) * n + col0 + j] = a;
            }
        }
    }
}

// ------------------------------------------------------------------------------------
// RMSNorm + 1x128 quantisation, U slabs per iteration.
//
// Same data flow as rows_kernel<ROP_NORM_Q>, but one iteration covers U consecutive slabs
// (U * RB rows): the per-iteration control work (barrier waits, the CTA barrier of the
// row-sum reduction, address set-up, the producer's refill) is paid once per U slabs, and
// the two independent rows give the schedulers more to overlap.  To keep the register
// budget of one slab, each slab is read from shared memory twice: once for sum x^2, and
// again after the barrier for normalise + quantise.
// ------------------------------------------------------------------------------------
template <int U, int STAGES>
struct NormQCfg {
    static constexpr int NT = 256, NW = 8, EPT = 32;
    static constexpr int STAGEB = U * kSlabElems * 2;
    static constexpr int OUTB = U * kSlabElems;
    static constexpr int OFF_OUT = STAGES * STAGEB;
    static constexpr int OFF_RED = OFF_OUT + 2 * OUTB;            // [2][U][64]
    static constexpr int OFF_BAR = OFF_RED + 2 * U * 64 * 4;
    static constexpr int SMEM = OFF_BAR + 2 * STAGES * 8;
};

template <int U, int STAGES, int MINB>
__global__ void __launch_bounds__(256, MINB)
normq_kernel(const __grid_constant__ RowParams p) {
    using C = NormQCfg<U, STAGES>;
    constexpr int NT = C::NT, NW = C::NW, EPT = C::EPT, NCH = 4, NP = 16, LPB = 4, WSPAN = 1024;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem;
    uint8_t* outb = smem + C::OFF_OUT;
    float* red = reinterpret_cast<float*>(smem + C::OFF_RED);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty = full + STAGES;

    const int t = threadIdx.x;
    const int warp = t >> 5, lane = t & 31;
    const int n = p.n;
    const int RB = p.RB;                       // rows per slab
    const int GR = U * RB;                     // rows per iteration
    const int64_t groups = (p.M + GR - 1) / GR;

    if (t == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    auto issue = [&](int64_t grp, int stage) {   // thread 0 only
        const int64_t r0 = grp * GR;
        const int64_t left = p.M - r0;
        const uint32_t rows = uint32_t(left < GR ? left : GR);
        const uint32_t bytes = rows * uint32_t(n) * 2u;
        uint8_t* dst = stages + size_t(stage) * C::STAGEB;
        mbar_expect_tx(&full[stage], bytes);
        if (RB * n == kSlabElems) {            // slabs are dense: one copy for the whole group
            bulk_g2s(dst, p.x + r0 * n * 2, bytes, &full[stage]);
        } else {                               // n does not divide 8192: slabs have a tail gap
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int rws = int(rows) - u * RB;
                if (rws > 0)
                    bulk_g2s(dst + u * kSlabElems * 2, p.x + (r0 + u * RB) * n * 2,
                             uint32_t(rws < RB ? rws : RB) * uint32_t(n) * 2u, &full[stage]);
            }
        }
    };
    if (t == 0) {
        int64_t grp = blockIdx.x;
        for (int j = 0; j < STAGES && grp < groups; ++j, grp += gridDim.x) issue(grp, j);
    }

    const int e0 = t * EPT;
    const int sw = (t >> 1) & 3;
    const bool rs = p.round_scale != 0;
    const int my_row = e0 / n;
    const int col0 = e0 - my_row * n;
    const bool in_slab = my_row < RB;
    float2 gam[NP];
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (in_slab)
            raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.gamma) + (col0 + 8 * (k ^ sw)) * 2);
        gam[4 * k + 0] = bf16x2_to_f2(raw.x);
        gam[4 * k + 1] = bf16x2_to_f2(raw.y);
        gam[4 * k + 2] = bf16x2_to_f2(raw.z);
        gam[4 * k + 3] = bf16x2_to_f2(raw.w);
    }
    const int TPR = n / EPT;
    const bool warp_rows = (TPR % 32) == 0;
    const int red_cnt = warp_rows ? TPR / 32 : (n >> 7);
    const int red_first = my_row * red_cnt;
    float* const s_col = p.s + int64_t(col0 >> 7) * p.M + my_row;   // + global row of the slab

    int stage = 0, prev_stage = 0, buf = 0;
    uint32_t phase = 0, prev_phase = 0;
    bool first_it = true;
    bool dead = false;   // a bounded wait of this thread gave up (see mbar_wait_or_mark)
    for (int64_t grp = blockIdx.x; grp < groups; grp += gridDim.x) {
        if (t == 0 && !first_it) {
            const int64_t nxt = grp + int64_t(STAGES - 1) * gridDim.x;
            if (nxt < groups) {
                mbar_wait_or_mark<false>(&empty[prev_stage], prev_phase, DEVERR_EMPTY_WAIT, dead);
                if (!dead) issue(nxt, prev_stage);
            }
        }
        const int64_t r0 = grp * GR;
        const int64_t left = p.M - r0;
        const int rows = int(left < GR ? left : GR);        // valid rows in this group
        mbar_wait_or_mark<false>(&full[stage], phase, DEVERR_FULL_WAIT, dead);
        const uint8_t* sx = stages + size_t(stage) * C::STAGEB + size_t(e0) * 2;
        float* red_b = red + buf * (U * 64);

        // ---- pass 1: sum of squares of every slab -------------------------------------
        float ss[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float2 a0 = make_float2(0.f, 0.f), a1 = a0;
            const bool act = in_slab && (u * RB + my_row) < rows;
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const uint4 raw = *reinterpret_cast<const uint4*>(sx + u * kSlabElems * 2 + 16 * (k ^ sw));
                const float2 v0 = bf16x2_to_f2(raw.x), v1 = bf16x2_to_f2(raw.y);
                const float2 v2 = bf16x2_to_f2(raw.z), v3 = bf16x2_to_f2(raw.w);
                a0 = fma2(v0, v0, a0); a1 = fma2(v1, v1, a1);
                a0 = fma2(v2, v2, a0); a1 = fma2(v3, v3, a1);
            }
            a0 = add2(a0, a1);
            ss[u] = act ? a0.x + a0.y : 0.f;
        }
        if (warp_rows) {
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) {
#pragma unroll
                for (int u = 0; u < U; ++u) ss[u] += __shfl_xor_sync(0xffffffffu, ss[u], d);
            }
            if (lane == 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) red_b[u * 64 + warp] = ss[u];
            }
        } else {
#pragma unroll
            for (int d = LPB / 2; d >= 1; d >>= 1) {
#pragma unroll
                for (int u = 0; u < U; ++u) ss[u] += __shfl_xor_sync(0xffffffffu, ss[u], d);
            }
            if ((t % LPB) == 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) red_b[u * 64 + t / LPB] = ss[u];
            }
        }
        if (lane == 0) bulk_wait_read<U>();      // this warp's spans of out[buf] have been read out
        named_bar<1, NT>();

        // ---- pass 2: normalise, quantise, stage the codes ----------------------------
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float tot = 0.f;
            if (red_cnt == 8) {
                const float4 a = *reinterpret_cast<const float4*>(red_b + u * 64 + red_first);
                const float4 b = *reinterpret_cast<const float4*>(red_b + u * 64 + red_first + 4);
                tot = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
            } else if (in_slab) {
#pragma unroll 4
                for (int i = 0; i < red_cnt; ++i) tot += red_b[u * 64 + red_first + i];
            }
            const float r = rsqrt_nr(fmaf(tot, p.inv_n, p.eps));
            const bool act = in_slab && (u * RB + my_row) < rows;
            const float2 r2 = splat2(act ? r : 0.f);
            float2 x[NP];
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const uint4 raw = *reinterpret_cast<const uint4*>(sx + u * kSlabElems * 2 + 16 * (k ^ sw));
                x[4 * k + 0] = mul2(mul2(bf16x2_to_f2(raw.x), r2), gam[4 * k + 0]);
                x[4 * k + 1] = mul2(mul2(bf16x2_to_f2(raw.y), r2), gam[4 * k + 1]);
                x[4 * k + 2] = mul2(mul2(bf16x2_to_f2(raw.z), r2), gam[4 * k + 2]);
                x[4 * k + 3] = mul2(mul2(bf16x2_to_f2(raw.w), r2), gam[4 * k + 3]);
            }
            if (u == U - 1) {                    // last read of the stage: hand it back
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[stage]);
            }
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int i = 0; i < NP; i += 2) {
                a0 = max3abs(x[i].x, x[i].y, a0);
                a1 = max3abs(x[i + 1].x, x[i + 1].y, a1);
            }
            float a = fmaxf(a0, a1);
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
            const float scale = scale_from_amax(a, rs);
            const float2 inv = splat2(rcp_approx(scale));
            uint8_t* so = outb + buf * C::OUTB + u * kSlabElems + e0;
#pragma unroll
            for (int k = 0; k < NCH; ++k) {
                const float2 q0 = mul2(x[4 * k + 0], inv), q1 = mul2(x[4 * k + 1], inv);
                const float2 q2 = mul2(x[4 * k + 2], inv), q3 = mul2(x[4 * k + 3], inv);
                *reinterpret_cast<uint2*>(so + 8 * (k ^ sw)) =
                    make_uint2(cvt_e4m3x4(q0.x, q0.y, q1.x, q1.y), cvt_e4m3x4(q2.x, q2.y, q3.x, q3.y));
            }
            if (act) {
                const int64_t grow = r0 + u * RB;
                if ((t % LPB) == 0) s_col[grow] = scale;
                if (col0 == 0) p.rms[grow + my_row] = r;
            }
        }
        // ---- each warp writes back its own contiguous span of every slab -------------
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                int rws = rows - u * RB;
                rws = rws < RB ? rws : RB;
                int cnt = rws * n - warp * WSPAN;                 // valid elements left for this warp
                cnt = cnt > WSPAN ? WSPAN : cnt;
                if (cnt > 0)
                    bulk_s2g(p.q + (r0 + u * RB) * n + warp * WSPAN,
                             outb + buf * C::OUTB + u * kSlabElems + warp * WSPAN, uint32_t(cnt));
                bulk_commit();
            }
        }
        first_it = false;
        prev_stage = stage; prev_phase = phase;
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        buf ^= 1;
    }
    if (lane == 0) bulk_wait_all();
}

// dgamma[j] = sum over the per-CTA partial rows, added in a fixed order (deterministic).  One CTA
// covers 128 columns: lane = 4 columns (one 16-byte load per partial row), the 32 warps split the
// partial rows among themselves so that every thread has only a handful of independent loads,
// and warp 0 then adds the 32 sub-sums.  A single thread walking all the rows would pay the
// L2 latency dozens of times in a row.  n is a multiple of 128 and the scratch rows are
// 16-byte aligned.
__global__ void __launch_bounds__(1024)
dgamma_reduce_kernel(const float* __restrict__ partial, int parts, int n, float* __restrict__ out) {
    __shared__ float4 red[32][32];
    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int col = blockIdx.x * 128 + lane * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < n) {
#pragma unroll 4
        for (int b = grp; b < parts; b += 32) {
            const float4 v = *reinterpret_cast<const float4*>(partial + int64_t(b) * n + col);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
    }
    red[grp][lane] = a;
    __syncthreads();
    if (grp == 0 && col < n) {
        float4 s = red[0][lane];
#pragma unroll
        for (int g = 1; g < 32; ++g) {
            const float4 v = red[g][lane];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        out[col] = s.x; out[col + 1] = s.y; out[col + 2] = s.z; out[col + 3] = s.w;
    }
}

int dgamma_reduce(const float* partial, int parts, int64_t n, float* dgamma, cudaStream_t stream) {
    dgamma_reduce_kernel<<<dim3(unsigned((n + 127) / 128)), dim3(1024), 0, stream>>>(partial, parts, int(n), dgamma);
    return check_launch("dgamma_reduce_kernel");
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
template <int ROP, int EPT, int STAGES, int CTAS_PER_SM>
static int launch_rows(RowParams p, int* grid_out, cudaStream_t stream, int grid_cap = kMaxRowCtas) {
    using C = RowCfg<ROP, EPT, STAGES>;
    int64_t slabs;
    p.inv_n = 1.0f / float(p.n);
    p.RB = kSlabElems / p.n;
    slabs = (p.M + p.RB - 1) / p.RB;
    int64_t grid = int64_t(sm_count()) * CTAS_PER_SM;
    if (grid > grid_cap) grid = grid_cap;
    if (slabs < grid) grid = slabs;
    if (grid_out) *grid_out = int(grid);
    auto go = [&](auto kern) -> int {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(C::SMEM));
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return int(e); }
        kern<<<dim3(unsigned(grid)), dim3(C::NT), C::SMEM, stream>>>(p);
        return check_launch("rows_kernel");
    };
    return go(rows_kernel<ROP, EPT, STAGES, CTAS_PER_SM>);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_rows(const char* what, int dtype, int64_t M, int64_t n) {
    if (dtype != LH_BF16 && dtype != LH_F16 && dtype != LH_F32) return fail_arg("%s: dtype must be bf16, f16 or f32", what);
    if (M < 0 || n <= 0 || (n % 128) != 0 || n > kSlabElems)
        return fail_arg("%s: need n %% 128 == 0 and n <= 8192 (M=%lld n=%lld)", what, (long long)M, (long long)n);
    return LH_OK;
}

int rows_norm_quant(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* q,
                    float* s, float* rms, int round_scale, cudaStream_t stream) {
    if (int rc = check_rows("rmsnorm_blockquant_fwd", dtype, M, n)) return rc;
    if (dtype != LH_BF16) return fail_arg("rmsnorm_blockquant_fwd: the ring kernel takes bf16 only");
    if (!x || !gamma || !q || !s || !rms) return fail_arg("rmsnorm_blockquant_fwd: NULL pointer");
    if (!aligned16(x) || !aligned16(q) || !aligned16(gamma)) return fail_arg("rmsnorm_blockquant_fwd: pointers must be 16-byte aligned");
    if (M == 0) return LH_OK;
    RowParams p{};
    p.x = static_cast<const uint8_t*>(x); p.gamma = gamma; p.rms = rms; p.eps = eps; p.M = M; p.n = int(n);
    p.q = static_cast<uint8_t*>(q); p.s = s; p.round_scale = round_scale;
    // two slabs per iteration once there is enough work to fill the machine that way
    constexpr int U = 2, STAGES = 2;
    p.inv_n = 1.0f / float(p.n);
    p.RB = kSlabElems / p.n;
    const int64_t groups = (M + int64_t(U) * p.RB - 1) / (int64_t(U) * p.RB);
    int64_t grid = int64_t(sm_count()) * 2;
    if (grid > kMaxRowCtas) grid = kMaxRowCtas;
    if (groups < 2 * grid) return launch_rows<ROP_NORM_Q, 32, 4, 2>(p, nullptr, stream);
    using C = NormQCfg<U, STAGES>;
    auto kern = normq_kernel<U, STAGES, 2>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(C::SMEM));
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return int(e); }
    kern<<<dim3(unsigned(grid)), dim3(C::NT), C::SMEM, stream>>>(p);
    return check_launch("normq_kernel");
}

int rows_norm_yq(const void* x, const void* gamma, int64_t M, int n, float eps, void* y, void* q, float* s, float* rms,
                 int round_scale, cudaStream_t stream) {
    RowParams p{};
    p.x = static_cast<const uint8_t*>(x);
    p.gamma = gamma;
    p.M = M;
    p.n = n;
    p.eps = eps;
    p.hp = static_cast<uint8_t*>(y);
    p.q = static_cast<uint8_t*>(q);
    p.s = s;
    p.rms = rms;
    p.round_scale = round_scale;
    return launch_rows<ROP_NORM_YQ, 32, 4, 2>(p, nullptr, stream);
}

int rows_norm_y(const void* x, const void* gamma, int dtype, int64_t M, int64_t n, float eps, void* y,
                float* rms, int reuse_rms, cudaStream_t stream) {
    if (int rc = check_rows("rmsnorm_fwd", dtype, M, n)) return rc;
    if (!x || !gamma || !y || (reuse_rms && !rms)) return fail_arg("rmsnorm_fwd: NULL pointer");
    if (!aligned16(x) || !aligned16(y) || !aligned16(gamma)) return fail_arg("rmsnorm_fwd: pointers must be 16-byte aligned");
    if (M == 0) return LH_OK;
    if (dtype != LH_BF16) return any_norm_fwd(x, gamma, dtype, M, n, eps, y, rms, reuse_rms, stream);
    RowParams p{};
    p.x = static_cast<const uint8_t*>(x); p.gamma = gamma; p.rms = rms; p.reuse_rms = reuse_rms; p.eps = eps;
    p.M = M; p.n = int(n); p.hp = static_cast<uint8_t*>(y);
    return launch_rows<ROP_NORM_Y, 32, 4, 2>(p, nullptr, stream);
}

int64_t rows_norm_bwd_scratch(int64_t n) { return int64_t(kMaxRowCtas) * n * 4; }

// narrowest row that takes the streaming register kernel instead of the TMA ring (lh_tuning "rmsnorm_bwd_stream_min_n"):
// streaming / ring at 65536 rows: 1024 columns 107.5 / 83.3 us, 1536 119.5 / 133.3, 2048 135.1 / 160.3
int g_bwd_stream_min_n = 1536;

// dy_q / dy_s (optional): where the streaming kernel runs it also writes the row-wise 1x128 codes
// and scales ([n/128, M]) of dy and sets *dy_rows_done = 1; with dy_qt / dy_st as well (and M a
// multiple of 16) also the transposed 128x1 copy, *dy_rows_done = 2.  Otherwise they are left
// untouched.  two_role_min_n: narrowest row for which the fused call prefers the streaming kernel.
int rows_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M,
                  int64_t n, float eps, void* dx, float* dgamma, void* scratch, int64_t scratch_bytes,
                  cudaStream_t stream, void* dy_q, float* dy_s, int round_scale, int* dy_rows_done, void* dy_qt,
                  float* dy_st, int two_role_min_n) {
    if (dy_rows_done) *dy_rows_done = 0;
    if (int rc = check_rows("rmsnorm_bwd", dtype, M, n)) return rc;
    if (!x || !dy || !gamma || !dx || !dgamma) return fail_arg("rmsnorm_bwd: NULL pointer");
    if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(gamma)) return fail_arg("rmsnorm_bwd: pointers must be 16-byte aligned");
    if (!scratch || scratch_bytes < rows_norm_bwd_scratch(n)) return fail_arg("rmsnorm_bwd: scratch too small (%lld < %lld)", (long long)scratch_bytes, (long long)rows_norm_bwd_scratch(n));
    if (M == 0) {
        cudaError_t e = cudaMemsetAsync(dgamma, 0, size_t(n) * 4, stream);
        return e == cudaSuccess ? LH_OK : int(e);
    }
    if (dtype != LH_BF16)
        return any_norm_bwd(dy, x, gamma, rms, dtype, M, n, eps, dx, dgamma, static_cast<float*>(scratch), kMaxRowCtas, stream);
    RowParams p{};
    p.x = static_cast<const uint8_t*>(x); p.dy = static_cast<const uint8_t*>(dy); p.gamma = gamma;
    p.rms = const_cast<float*>(rms); p.reuse_rms = rms != nullptr; p.eps = eps; p.M = M; p.n = int(n);
    p.hp = static_cast<uint8_t*>(dx); p.partial = static_cast<float*>(scratch);
    int grid = 0;
    // Rows of 1536 columns and more take the streaming register kernel (67.7 vs 83 us at 16384 x 4096,
    // 268.8 vs 301 us at 65536 x 4096, 254.6 vs 370 us at 32768 x 8192), narrower ones the TMA ring.
    const bool qdy = dy_q != nullptr && dy_s != nullptr && aligned16(dy_q) && dy_rows_done != nullptr;
    const bool colq = qdy && dy_qt != nullptr && dy_st != nullptr && aligned16(dy_qt) && (M % 16) == 0 && n >= two_role_min_n;
    // the fused call (row codes of dy wanted) keeps the ring up to 2048 columns: there the streaming kernel runs
    // without the prefetch and the two paths measure level (65536 x 1536: 237.7 vs 218.2 us for the ring)
    if ((qdy ? n > 2048 : n >= g_bwd_stream_min_n) || colq) {
        int rc = small_norm_bwd(dy, x, gamma, rms, M, n, eps, dx, p.partial, kMaxRowCtas, &grid, qdy ? dy_q : nullptr,
                                dy_s, round_scale, stream, colq ? dy_qt : nullptr, dy_st);
        bool cols_done = colq;
        if (rc == LH_ERR_ARG - 1000 && colq) {   // the two-role kernel cannot launch here: rows only, the caller adds the columns
            cols_done = false;
            rc = small_norm_bwd(dy, x, gamma, rms, M, n, eps, dx, p.partial, kMaxRowCtas, &grid, dy_q, dy_s, round_scale,
                                stream, nullptr, nullptr);
        }
        if (rc) return rc;
        if (qdy) *dy_rows_done = cols_done ? 2 : 1;
    } else if (int rc = launch_rows<ROP_NORM_BWD, 16, 3, 1>(p, &grid, stream)) {
        return rc;
    }
    dgamma_reduce_kernel<<<dim3(unsigned((n + 127) / 128)), dim3(1024), 0, stream>>>(p.partial, grid, int(n), dgamma);
    return check_launch("dgamma_reduce_kernel");
}

// ------------------------------------------------------------------------------------
// RMSNorm backward without any allocation: the per-CTA dgamma partials live in a
// file-scope device array instead of caller-provided scratch.
// ------------------------------------------------------------------------------------
constexpr int kStaticCtas = 148;                       // partial rows held by the array
constexpr int kStaticMaxCols = kSlabElems;             // widest row supported (8192)
static __device__ __align__(256) float g_static_dgamma_partials[kStaticCtas * kStaticMaxCols];

int64_t rows_norm_bwd_static_bytes() { return int64_t(sizeof(float)) * kStaticCtas * kStaticMaxCols; }

// Device address of the array for the current device.  The symbol name is only a host-side
// handle; the address a kernel can use comes from cudaGetSymbolAddress, once per device.
static int static_partials_ptr(float** out) {
    static float* cached[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_error("cudaGetDevice: %s", cudaGetErrorString(e)); return int(e); }
    if (dev < 0 || dev >= 64) return fail_arg("rmsnorm_bwd_static: device index %d out of range", dev);
    if (cached[dev] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_dgamma_partials);
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("cudaGetSymbolAddress(static dgamma partials): %s", cudaGetErrorString(e));
            return e != cudaSuccess ? int(e) : int(cudaErrorInvalidSymbol);
        }
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return LH_OK;
}

int rows_norm_bwd_static(const void* dy, const void* x, const void* gamma, const float* rms, int dtype, int64_t M,
                         int64_t n, float eps, void* dx, float* dgamma, cudaStream_t stream) {
    if (int rc = check_rows("rmsnorm_bwd_static", dtype, M, n)) return rc;
    if (n > kStaticMaxCols)
        return fail_arg("rmsnorm_bwd_static: n=%lld exceeds the built-in scratch (at most %d columns)", (long long)n, kStaticMaxCols);
    if (!x || !dy || !gamma || !dx || !dgamma) return fail_arg("rmsnorm_bwd_static: NULL pointer");
    if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(gamma)) return fail_arg("rmsnorm_bwd_static: pointers must be 16-byte aligned");
    float* partial = nullptr;
    if (int rc = static_partials_ptr(&partial)) return rc;
    if (M == 0) {
        cudaError_t e = cudaMemsetAsync(dgamma, 0, size_t(n) * 4, stream);
        return e == cudaSuccess ? LH_OK : int(e);
    }
    if (dtype != LH_BF16)
        return any_norm_bwd(dy, x, gamma, rms, dtype, M, n, eps, dx, dgamma, partial, kStaticCtas, stream);
    RowParams p{};
    p.x = static_cast<const uint8_t*>(x); p.dy = static_cast<const uint8_t*>(dy); p.gamma = gamma;
    p.rms = const_cast<float*>(rms); p.reuse_rms = rms != nullptr; p.eps = eps; p.M = M; p.n = int(n);
    p.hp = static_cast<uint8_t*>(dx); p.partial = partial;
    int grid = 0;
    // Every launched CTA overwrites its whole partial row [0, n) and the reduction reads only
    // the `grid` rows written by this call, so nothing in the array has to start at zero.
    if (int rc = launch_rows<ROP_NORM_BWD, 16, 3, 1>(p, &grid, stream, kStaticCtas)) return rc;
    dgamma_reduce_kernel<<<dim3(unsigned((n + 127) / 128)), dim3(1024), 0, stream>>>(partial, grid, int(n), dgamma);
    return check_launch("dgamma_reduce_kernel");
}

}  // namespace lh
