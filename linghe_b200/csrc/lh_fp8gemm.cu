// Blockwise-scaled FP8 GEMM: the consumer of the quantisers' wire format
// (replaces triton_tt_fp8_gemm / fp8_gemm_tt_kernel, linghe/gemm/blockwise_fp8_gemm.py:106-183).
//
//   C[m,n] = sum_i ( sum_{k in block i} a[m,k] * b[n,k] ) * a_s[m,i] * b_s[n,i]
//
// a [M,K], b [N,K] e4m3 codes, one float32 scale per 1 x BLOCK run of k (BLOCK = 128 or 64).
// Each k-block's partial product is an exact e4m3 x e4m3 contraction on the tensor cores
// (tcgen05.mma kind::f8f6f4, float32 accumulator in tensor memory, started from zero per
// block); the CUDA cores then fold it into float32 register accumulators with the two
// scales.  Four partial buffers in tensor memory let the tensor cores run ahead of the fold.
//
// One CTA = one 128 x 128 tile of C.  warp 0: TMA producer; warp 1: MMA issuer and owner
// of the tensor-memory allocation; warps 2-17: fold + store, thread = (row, 32-column group).
#include "lh_common.cuh"

namespace lh {

namespace {

constexpr int FM = 128, FN = 128, FKB = 128;   // tile; FKB = bytes (= e4m3 elements) of k per stage
constexpr int FSTAGES = 5;
constexpr int F_TILE = FM * FKB;               // 16 KB
constexpr int F_STAGE = 2 * F_TILE;
constexpr int F_BAR_OFF = FSTAGES * F_STAGE;
constexpr int F_SB_OFF = F_BAR_OFF + 256;      // b scales of this tile, [k-block][128] float32
constexpr int F_SB_MAX = 128;                  // scale blocks along k that fit
constexpr int F_SMEM = 1024 + F_SB_OFF + F_SB_MAX * FN * 4;
constexpr int FBUFS = 4;                        // partial-product buffers in tensor memory
constexpr int F_TMEM_COLS = FBUFS * FN;
constexpr int F_FOLD_WARPS = 16;                // each folds 32 accumulator rows x 32 columns
constexpr int F_THREADS = 64 + 32 * F_FOLD_WARPS;

enum : int { DEVERR_PART_WAIT = 5 };

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand, rows of 128 bytes, 128-byte swizzle, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
           (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// D f32, A and B e4m3 (format 0), both K-major, N = 128, M = 128
constexpr uint32_t kIdescF8 = (1u << 4) | (uint32_t(FN >> 3) << 17) | (uint32_t(FM >> 4) << 24);

__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kIdescF8), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
// One lane polls; the others then observe the completed phase with one try_wait of their own.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int code, int lane) {
    bool ok = true;
    if (lane == 0) ok = mbar_wait_inline(bar, parity, code);
    ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
    if (ok && lane != 0) ok = mbar_try_wait(bar, parity);
    return __all_sync(0xffffffffu, ok);
}

struct Fp8GemmParams {
    const float* a_s;
    const float* b_s;
    void* c;
    int64_t M;
    int N, K;
    int nsb;             // scale blocks along k
    int a_s_transposed;  // 0: a_s [M, nsb]   1: a_s [nsb, M]
    int b_s_transposed;  // 0: b_s [N, nsb]   1: b_s [nsb, N]
    int group;           // rows of a (of b) that share a scale: 1 = one scale per row and k-block, otherwise
                         // the block size (2-D block scales: a_s [ceil(M/group), nsb], b_s [ceil(N/group), nsb])
    int out_dtype;
};

// SUB = scale blocks per 128-byte k-stage (1: blocks of 128, 2: blocks of 64)
template <int SUB>
__global__ void __launch_bounds__(F_THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ Fp8GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t* tiles = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + F_BAR_OFF);   // TMA landed
    uint64_t* empty = full + FSTAGES;                                   // MMAs have read the stage
    uint64_t* part_full = empty + FSTAGES;                              // partial product complete
    uint64_t* part_empty = part_full + FBUFS;                           // partial product read out
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + FBUFS);
    float* sb = reinterpret_cast<float*>(tiles + F_SB_OFF);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int m0 = blockIdx.y * FM, n0 = blockIdx.x * FN;
    const int kstages = p.K / FKB;
    const int nsb = p.nsb;

    if (t == 0) {
        for (int i = 0; i < FSTAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < FBUFS; ++i) {
            mbar_init(&part_full[i], 1);
            mbar_init(&part_empty[i], F_FOLD_WARPS);
        }
        mbar_fence_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(uint32_t(F_TMEM_COLS))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == 0) {
        if (lane == 0) {
            for (int ks = 0; ks < kstages; ++ks) {
                const int s = ks % FSTAGES;
                const uint32_t use = uint32_t(ks / FSTAGES);
                if (ks >= FSTAGES && !mbar_wait(&empty[s], (use & 1u) ^ 1u, DEVERR_EMPTY_WAIT)) break;
                uint8_t* st = tiles + size_t(s) * F_STAGE;
                mbar_expect_tx(&full[s], F_STAGE);
                tma_load_2d(st, &map_a, ks * FKB, m0, &full[s]);
                tma_load_2d(st + F_TILE, &map_b, ks * FKB, n0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int ks = 0; ks < kstages && ok; ++ks) {
                const int s = ks % FSTAGES;
                ok = mbar_wait(&full[s], uint32_t(ks / FSTAGES) & 1u, DEVERR_FULL_WAIT);
                if (!ok) break;
                const uint32_t a = smem_u32(tiles + size_t(s) * F_STAGE);
                const uint64_t da = umma_desc(a), db = umma_desc(a + F_TILE);
#pragma unroll
                for (int h = 0; h < SUB; ++h) {
                    const int blk = ks * SUB + h;                  // scale block = partial product
                    const int buf = blk % FBUFS;
                    if (blk >= FBUFS) {
                        ok = mbar_wait(&part_empty[buf], (uint32_t(blk / FBUFS) & 1u) ^ 1u, DEVERR_PART_WAIT);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    constexpr int STEPS = (FKB / 32) / SUB;         // MMAs (k = 32) per scale block
#pragma unroll
                    for (int k4 = 0; k4 < STEPS; ++k4) {
                        const int kk = h * STEPS + k4;              // 32 bytes = 2 descriptor units per step
                        umma_f8(tmem + uint32_t(buf * FN), da + 2 * kk, db + 2 * kk, k4 != 0);
                    }
                    if (h == SUB - 1) umma_commit(&empty[s]);
                    umma_commit(&part_full[buf]);
                }
            }
        }
    } else {
        // ---- fold the partial products into register accumulators, then store
        // b scales of this tile's 128 columns -> shared memory, [scale block][column]; only these
        // warps need them, so the loads and the MMAs start meanwhile
        for (int i = t - 64; i < nsb * FN; i += F_THREADS - 64) {
            const int blk = i / FN, col = i - blk * FN;
            const int n = n0 + col;
            float v = 0.f;
            if (n < p.N) v = p.b_s_transposed ? p.b_s[int64_t(blk) * p.N + n] : p.b_s[int64_t(n / p.group) * nsb + blk];
            sb[i] = v;
        }
        named_bar<1, F_THREADS - 64>();
        const int quarter = warp & 3, cgrp = (warp - 2) >> 2;       // tensor-memory lane quarter, 32-column group
        const int64_t row = int64_t(m0) + quarter * 32 + lane;
        const bool row_ok = row < p.M;
        const float* as_ptr = p.a_s + (p.a_s_transposed ? row : (row / p.group) * nsb);
        const int64_t as_step = p.a_s_transposed ? p.M : 1;
        float2 acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = make_float2(0.f, 0.f);
        // Four fold warps per scheduler: their tensor-memory loads, shared-memory reads and FMAs
        // overlap across warps, so each warp simply loads a block's 32 columns and folds them.
        bool ok = true;
        const uint32_t tbase = tmem + (uint32_t(quarter * 32) << 16) + uint32_t(cgrp * 32);
        float sa_next = row_ok ? as_ptr[0] : 0.f;
        for (int blk = 0; blk < nsb && ok; ++blk) {
            const int buf = blk % FBUFS;
            const float sa = sa_next;
            if (blk + 1 < nsb && row_ok) sa_next = as_ptr[int64_t(blk + 1) * as_step];
            ok = mbar_wait_warp(&part_full[buf], uint32_t(blk / FBUFS) & 1u, DEVERR_PART_WAIT, lane);
            if (!ok) break;
            tc_fence_after();
            uint32_t v[32];
            tmem_ld32(tbase + uint32_t(buf * FN), v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&part_empty[buf]);        // the tensor cores may overwrite this buffer
            const float2 sa2 = splat2(sa);
            const float2* sbp = reinterpret_cast<const float2*>(sb + blk * FN + cgrp * 32);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float2 pr = make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                acc[j] = fma2(mul2(pr, sbp[j]), sa2, acc[j]);
            }
        }
        if (ok && row_ok) {
            const int c0 = n0 + cgrp * 32;
            if (p.out_dtype == LH_F32) {
                float* out = static_cast<float*>(p.c) + row * p.N + c0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (c0 + 2 * j < p.N) out[2 * j] = acc[j].x;
                    if (c0 + 2 * j + 1 < p.N) out[2 * j + 1] = acc[j].y;
                }
            } else {
                uint16_t* out = static_cast<uint16_t*>(p.c) + row * p.N + c0;
                const bool vec = (p.N % 8) == 0;
#pragma unroll
                for (int j8 = 0; j8 < 4; ++j8) {                 // 8 columns per step
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 a = acc[4 * j8 + j];
                        if (p.out_dtype == LH_BF16) {
                            w[j] = pack_bf16x2(a.x, a.y);
                        } else {
                            const __half2 h = __floats2half2_rn(a.x, a.y);
                            w[j] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    }
                    const int c = c0 + 8 * j8;
                    if (vec && c + 8 <= p.N) {
                        *reinterpret_cast<uint4*>(out + 8 * j8) = make_uint4(w[0], w[1], w[2], w[3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (c + j < p.N) out[8 * j8 + j] = uint16_t(w[j >> 1] >> (16 * (j & 1)));
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(F_TMEM_COLS))
                     : "memory");
    }
}

}  // namespace

// c [M,N] = blockwise-scaled a [M,K] . b [N,K]^T ; block = 128 or 64 along k, K a multiple of 128.
// group_2d != 0: 2-D block scales (one per block x block sub-matrix of a and of b), never transposed.
int fp8_gemm(const void* a, const void* b, const float* a_s, const float* b_s, void* c, int64_t M, int64_t N, int64_t K,
             int block, int a_s_transposed, int b_s_transposed, int out_dtype, cudaStream_t stream, int group_2d) {
    if (!a || !b || !a_s || !b_s || !c) return fail_arg("fp8_gemm: NULL pointer");
    if (block != 128 && block != 64) return fail_arg("fp8_gemm: block_size must be 128 or 64");
    if (M < 0 || N <= 0 || K <= 0 || (K % FKB)) return fail_arg("fp8_gemm: need K a positive multiple of 128 and N > 0");
    if (out_dtype != LH_BF16 && out_dtype != LH_F16 && out_dtype != LH_F32) return fail_arg("fp8_gemm: bad out dtype");
    const int64_t nsb = K / block;
    if (nsb > F_SB_MAX) return fail_arg("fp8_gemm: at most %d scale blocks along k", F_SB_MAX);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15)
        return fail_arg("fp8_gemm: pointers must be 16-byte aligned");
    if (M > 0x7fffffff - FM || N > 0x7fffffff - FN) return fail_arg("fp8_gemm: size out of range");
    if (M == 0) return LH_OK;
    CUtensorMap ma, mb;
    if (int rc = make_tensor_map(&ma, a, LH_U8, uint64_t(M), uint64_t(K), uint64_t(K), FM, FKB, 1)) return rc;
    if (int rc = make_tensor_map(&mb, b, LH_U8, uint64_t(N), uint64_t(K), uint64_t(K), FN, FKB, 1)) return rc;
    Fp8GemmParams p{};
    p.a_s = a_s; p.b_s = b_s; p.c = c;
    p.M = M; p.N = int(N); p.K = int(K); p.nsb = int(nsb);
    p.a_s_transposed = group_2d ? 0 : a_s_transposed; p.b_s_transposed = group_2d ? 0 : b_s_transposed; p.out_dtype = out_dtype;
    p.group = group_2d ? block : 1;
    const dim3 grid(unsigned((N + FN - 1) / FN), unsigned((M + FM - 1) / FM));
    auto go = [&](auto kern) -> int {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return int(e); }
        kern<<<grid, F_THREADS, F_SMEM, stream>>>(ma, mb, p);
        return check_launch("fp8_gemm_kernel");
    };
    return block == 128 ? go(fp8_gemm_kernel<1>) : go(fp8_gemm_kernel<2>);
}

}  // namespace lh
