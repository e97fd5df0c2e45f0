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
// One persistent CTA per SM walks 128 x 128 tiles of C.  warp 0: TMA producer; warp 1: MMA issuer and owner
// of the tensor-memory allocation; warps 2-17: fold + store, thread = (row, 32-column group).
#include "lh_common.cuh"

#include <type_traits>

namespace lh {

namespace {

constexpr int FM = 128, FN = 256, FKB = 128;   // tile; FKB = bytes (= e4m3 elements) of k per stage
constexpr int FSTAGES = 4;
constexpr int F_TILE = FM * FKB;               // a: 16 KB, then b: 32 KB
constexpr int F_STAGE = F_TILE + FN * FKB;
constexpr int F_BAR_OFF = FSTAGES * F_STAGE;
constexpr int F_SC_OFF = F_BAR_OFF + 256;      // scales, two chunk buffers
constexpr int F_CH = 8;                        // scale blocks per staged chunk
constexpr int F_SA_LD = F_CH + 1;              // a scales [row][block], odd stride: one bank per row
constexpr int F_SC_FLOATS = FM * F_SA_LD + F_CH * FN;   // + b scales [block][column]
constexpr int F_SMEM = 1024 + F_SC_OFF + 2 * F_SC_FLOATS * 4;
constexpr int FBUFS = 512 / FN;                       // partial-product buffers in tensor memory
constexpr int F_TMEM_COLS = FBUFS * FN;
constexpr int F_FOLD_WARPS = 16;                // each folds 32 accumulator rows x FN/4 columns
constexpr int F_CW = FN / 4;                    // columns per fold warp
static_assert(F_SMEM <= 232448, "shared memory");
constexpr int F_SCALE_WARP = 2 + F_FOLD_WARPS;  // warp that stages the scales
constexpr int F_THREADS = 32 * (F_SCALE_WARP + 1);

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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
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

// true in one lane of the (converged) warp, the same lane every time
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
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
    int group_shift;     // log2 of the rows of a (of b) that share a scale: 0 = one scale per row and k-block,
                         // otherwise log2 of the block size (2-D block scales: a_s [ceil(M/block), nsb], b_s likewise)
    int out_dtype;
};

// SUB = scale blocks per 128-byte k-stage (1: blocks of 128, 2: blocks of 64)
template <int SUB>
__global__ void __launch_bounds__(F_THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ Fp8GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t* tile_smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(tile_smem + F_BAR_OFF);   // TMA landed
    uint64_t* empty = full + FSTAGES;                                   // MMAs have read the stage
    uint64_t* part_full = empty + FSTAGES;                              // partial product complete
    uint64_t* part_empty = part_full + FBUFS;                           // partial product read out
    uint64_t* sc_full = part_empty + FBUFS;                             // a chunk of scales is in shared memory
    uint64_t* sc_empty = sc_full + 2;                                   // the fold warps are done with it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sc_empty + 2);
    float* sc_all = reinterpret_cast<float*>(tile_smem + F_SC_OFF);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int kstages = p.K / FKB;
    const int nsb = p.nsb;
    // Persistent: a CTA takes tiles blockIdx.x, + gridDim.x, ... (column tile fastest, so the tiles in
    // flight share a few row blocks of a and all of b in L2).  Barriers, the tensor-memory allocation
    // and the three roles live across tiles; the stage and partial-buffer counters simply keep
    // counting, so the loads and MMAs of the next tile start while the fold warps still store this one.
    const int tiles_n = (p.N + FN - 1) / FN;
    const int64_t tiles = int64_t((p.M + FM - 1) / FM) * tiles_n;

    if (t == 0) {
        for (int i = 0; i < FSTAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < FBUFS; ++i) {
            mbar_init(&part_full[i], 1);
            mbar_init(&part_empty[i], F_FOLD_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sc_full[i], 1);
            mbar_init(&sc_empty[i], F_FOLD_WARPS);
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

    // Warps 0 and 1 run their loops with all 32 lanes and elect one lane only for the instructions that
    // issue work: the loop counters, shared-memory addresses and descriptors are then warp-uniform
    // values, which is what the TMA and tcgen05 instructions take as operands.
    if (warp == 0) {
        int s = 0;
        uint32_t ph = 0;                                            // stage and its phase, over all tiles
        bool first_pass = true, ok = true;
        for (int64_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const int m0 = int(tile / tiles_n) * FM, n0 = int(tile % tiles_n) * FN;
            for (int ks = 0; ks < kstages; ++ks) {
                if (!first_pass) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, DEVERR_EMPTY_WAIT));
                    if (!ok) break;
                }
                if (elect_one()) {
                    uint8_t* st = tile_smem + size_t(s) * F_STAGE;
                    mbar_expect_tx(&full[s], F_STAGE);
                    tma_load_2d(st, &map_a, ks * FKB, m0, &full[s]);
                    tma_load_2d(st + F_TILE, &map_b, ks * FKB, n0, &full[s]);
                }
                if (++s == FSTAGES) { s = 0; ph ^= 1u; first_pass = false; }
            }
        }
    } else if (warp == 1) {
        int s = 0, buf = 0;
        uint32_t ph = 0, bph = 0;                                   // stage / partial buffer and their phases
        bool first_bufs = true, ok = true;
        for (int64_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            for (int ks = 0; ks < kstages && ok; ++ks) {
                ok = __all_sync(0xffffffffu, mbar_wait(&full[s], ph, DEVERR_FULL_WAIT));
                if (!ok) break;
                const uint32_t a = smem_u32(tile_smem + size_t(s) * F_STAGE);
                const uint64_t da = umma_desc(a), db = umma_desc(a + F_TILE);
#pragma unroll
                for (int h = 0; h < SUB; ++h) {                     // scale block = partial product
                    if (!first_bufs) {
                        ok = __all_sync(0xffffffffu, mbar_wait(&part_empty[buf], bph ^ 1u, DEVERR_PART_WAIT));
                        if (!ok) break;
                    }
                    tc_fence_after();
                    if (elect_one()) {
                        constexpr int STEPS = (FKB / 32) / SUB;     // MMAs (k = 32) per scale block
#pragma unroll
                        for (int k4 = 0; k4 < STEPS; ++k4) {
                            const int kk = h * STEPS + k4;          // 32 bytes = 2 descriptor units per step
                            umma_f8(tmem + uint32_t(buf * FN), da + 2 * kk, db + 2 * kk, k4 != 0);
                        }
                        umma_commit(&part_full[buf]);       // the one commit per block: issuing costs this thread ~100 cycles
                    }
                    if (++buf == FBUFS) { buf = 0; bph ^= 1u; first_bufs = false; }
                }
                if (++s == FSTAGES) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == F_SCALE_WARP) {
        // ---- the scales reach shared memory in chunks of F_CH k-blocks, one chunk ahead of the fold
        // warps (the next chunk may be the next tile's first): a scale read straight from global
        // memory inside the fold loop would put the load's latency into every block.
        const int chunks = (nsb + F_CH - 1) / F_CH;
        uint32_t q = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const int m0 = int(tile / tiles_n) * FM, n0 = int(tile % tiles_n) * FN;
            for (int chunk = 0; chunk < chunks; ++chunk, ++q) {
                if (q >= 2) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&sc_empty[q & 1u], ((q >> 1) & 1u) ^ 1u, DEVERR_PART_WAIT));
                    if (!ok) break;
                }
                float* sa_s = sc_all + (q & 1u) * F_SC_FLOATS;
                float* sb_s = sa_s + FM * F_SA_LD;
                const int blk0 = chunk * F_CH;
                // 32 loads in flight per lane; consecutive lanes take consecutive global addresses in either
                // layout.  Element i = lane + 32 k + 1024 j of a chunk is (r, bl) = (i / F_CH, i % F_CH) in the
                // row-major layout and (i % EXT, i / EXT) in the transposed one; with lane < 32 both split into
                // a per-lane part and compile-time steps.
                auto copy = [&](auto is_a_tag, auto tr_tag) {
                    constexpr bool IS_A = decltype(is_a_tag)::value, TR = decltype(tr_tag)::value;
                    constexpr int EXT = IS_A ? FM : FN, BATCH = 32;
                    static_assert(F_CH == 8 && (EXT * F_CH) % (32 * BATCH) == 0, "index split below");
                    const float* src = IS_A ? p.a_s : p.b_s;
                    const int rows = IS_A ? int(p.M) : p.N;
                    const int base = IS_A ? m0 : n0;
#pragma unroll
                    for (int j = 0; j < EXT * F_CH / (32 * BATCH); ++j) {
                        float v[BATCH];
#pragma unroll
                        for (int k = 0; k < BATCH; ++k) {
                            const int r = TR ? lane + 32 * (k % (EXT / 32)) : (lane >> 3) + 4 * k + 128 * j;
                            const int bl = TR ? k / (EXT / 32) + (1024 / EXT) * j : (lane & 7);
                            const int row = base + r, blk = blk0 + bl;
                            v[k] = 0.f;
                            if (row < rows && blk < nsb)
                                v[k] = src[TR ? int64_t(blk) * rows + row : int64_t(row >> p.group_shift) * nsb + blk];
                        }
#pragma unroll
                        for (int k = 0; k < BATCH; ++k) {
                            const int r = TR ? lane + 32 * (k % (EXT / 32)) : (lane >> 3) + 4 * k + 128 * j;
                            const int bl = TR ? k / (EXT / 32) + (1024 / EXT) * j : (lane & 7);
                            if (IS_A) sa_s[r * F_SA_LD + bl] = v[k];
                            else sb_s[bl * FN + r] = v[k];
                        }
                    }
                };
                if (p.a_s_transposed) copy(std::true_type{}, std::true_type{}); else copy(std::true_type{}, std::false_type{});
                if (p.b_s_transposed) copy(std::false_type{}, std::true_type{}); else copy(std::false_type{}, std::false_type{});
                __syncwarp();
                if (lane == 0) mbar_arrive(&sc_full[q & 1u]);
            }
        }
    } else {
        // ---- fold the partial products into register accumulators, then store
        const int quarter = warp & 3, cgrp = (warp - 2) >> 2;       // tensor-memory lane quarter, column group
        const uint32_t tbase = tmem + (uint32_t(quarter * 32) << 16) + uint32_t(cgrp * F_CW);
        const int chunks = (nsb + F_CH - 1) / F_CH;
        bool ok = true;                                             // a failed wait skips the work, not the barriers
        uint32_t gb = 0, q = 0;                                     // scale blocks and chunks so far
        for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            const int m0 = int(tile / tiles_n) * FM, n0 = int(tile % tiles_n) * FN;
            const int64_t row = int64_t(m0) + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            float2 acc[F_CW / 2];
#pragma unroll
            for (int j = 0; j < F_CW / 2; ++j) acc[j] = make_float2(0.f, 0.f);
            // Four fold warps per scheduler: their tensor-memory loads, shared-memory reads and FMAs
            // overlap across warps, so each warp simply loads a block's 32 columns and folds them.
            for (int chunk = 0; chunk < chunks; ++chunk, ++q) {
                if (ok) ok = mbar_wait_warp(&sc_full[q & 1u], (q >> 1) & 1u, DEVERR_PART_WAIT, lane);
                const float* sc = sc_all + (q & 1u) * F_SC_FLOATS;
                const float* sa_s = sc + (quarter * 32 + lane) * F_SA_LD;
                const float* sb_s = sc + FM * F_SA_LD + cgrp * F_CW;
                const int nblk = min(F_CH, nsb - chunk * F_CH);
                for (int bl = 0; bl < nblk && ok; ++bl, ++gb) {
                    const int buf = int(gb % FBUFS);
                    const float sa = sa_s[bl];
                    ok = mbar_wait_warp(&part_full[buf], (gb / FBUFS) & 1u, DEVERR_PART_WAIT, lane);
                    if (!ok) break;
                    // the block's MMAs are complete, so its k-stage may be refilled: one fold lane tells the producer
                    // (a second tcgen05.commit by the MMA thread would say the same, at a higher price)
                    if (t == 64 && (gb % SUB) == SUB - 1) mbar_arrive(&empty[(gb / SUB) % FSTAGES]);
                    tc_fence_after();
                    const float2 sa2 = splat2(sa);
                    const float4* sbp = reinterpret_cast<const float4*>(sb_s + bl * FN);   // 128-bit broadcast reads
#pragma unroll
                    for (int piece = 0; piece < F_CW / 16; ++piece) {       // 16 columns at a time
                        uint32_t v[16];
                        tmem_ld16(tbase + uint32_t(buf * FN + piece * 16), v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (piece == F_CW / 16 - 1) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&part_empty[buf]);   // the tensor cores may overwrite this buffer
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 sb4 = sbp[piece * 4 + j];
                            const float2 p0 = make_float2(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]));
                            const float2 p1 = make_float2(__uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                            acc[piece * 8 + 2 * j] = fma2(mul2(p0, make_float2(sb4.x, sb4.y)), sa2, acc[piece * 8 + 2 * j]);
                            acc[piece * 8 + 2 * j + 1] = fma2(mul2(p1, make_float2(sb4.z, sb4.w)), sa2, acc[piece * 8 + 2 * j + 1]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sc_empty[q & 1u]);      // the scale warp may refill this buffer
            }
            if (ok && row_ok) {
                const int c0 = n0 + cgrp * F_CW;
                if (p.out_dtype == LH_F32) {
                    float* out = static_cast<float*>(p.c) + row * p.N + c0;
                    const bool vec = (p.N % 8) == 0 && (reinterpret_cast<uintptr_t>(p.c) & 31) == 0;
#pragma unroll
                    for (int j4 = 0; j4 < F_CW / 8; ++j4) {          // 8 columns per step
                        const int c = c0 + 8 * j4;
                        if (vec && c + 8 <= p.N) {
                            const float2 a0 = acc[4 * j4], a1 = acc[4 * j4 + 1], a2 = acc[4 * j4 + 2], a3 = acc[4 * j4 + 3];
                            st_global_256(out + 8 * j4,
                                          make_uint4(__float_as_uint(a0.x), __float_as_uint(a0.y), __float_as_uint(a1.x), __float_as_uint(a1.y)),
                                          make_uint4(__float_as_uint(a2.x), __float_as_uint(a2.y), __float_as_uint(a3.x), __float_as_uint(a3.y)));
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (c + 2 * j < p.N) out[8 * j4 + 2 * j] = acc[4 * j4 + j].x;
                                if (c + 2 * j + 1 < p.N) out[8 * j4 + 2 * j + 1] = acc[4 * j4 + j].y;
                            }
                        }
                    }
                } else {
                    uint16_t* out = static_cast<uint16_t*>(p.c) + row * p.N + c0;
                    // a thread owns F_CW consecutive columns of its row: 32-byte stores fill whole sectors
                    const bool vec = (p.N % 16) == 0 && (reinterpret_cast<uintptr_t>(p.c) & 31) == 0;
#pragma unroll
                    for (int j16 = 0; j16 < F_CW / 16; ++j16) {      // 16 columns per step
                        uint32_t w[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float2 a = acc[8 * j16 + j];
                            if (p.out_dtype == LH_BF16) {
                                w[j] = pack_bf16x2(a.x, a.y);
                            } else {
                                const __half2 h = __floats2half2_rn(a.x, a.y);
                                w[j] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                        }
                        const int c = c0 + 16 * j16;
                        if (vec && c + 16 <= p.N) {
                            st_global_256(out + 16 * j16, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c + j < p.N) out[16 * j16 + j] = uint16_t(w[j >> 1] >> (16 * (j & 1)));
                        }
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
    p.group_shift = group_2d ? (block == 128 ? 7 : 6) : 0;
    const int64_t tiles = ((N + FN - 1) / FN) * ((M + FM - 1) / FM);
    const dim3 grid(unsigned(std::min<int64_t>(tiles, sm_count())));
    auto go = [&](auto kern) -> int {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return int(e); }
        kern<<<grid, F_THREADS, F_SMEM, stream>>>(ma, mb, p);
        return check_launch("fp8_gemm_kernel");
    };
    return block == 128 ? go(fp8_gemm_kernel<1>) : go(fp8_gemm_kernel<2>);
}

}  // namespace lh
