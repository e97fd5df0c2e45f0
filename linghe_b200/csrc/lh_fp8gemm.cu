// Blockwise-scaled FP8 GEMM: the consumer of the quantisers' wire format
// (replaces triton_tt_fp8_gemm / fp8_gemm_tt_kernel, linghe/gemm/blockwise_fp8_gemm.py:106-183).
//
//   C[m,n] = sum_i ( sum_{k in block i} a[m,k] * b[n,k] ) * a_s[m,i] * b_s[n,i]
//
// a [M,K], b [N,K] e4m3 codes, one float32 scale per 1 x BLOCK run of k (BLOCK = 128 or 64).
// Each k-block's partial product is an exact e4m3 x e4m3 contraction on the tensor cores
// (tcgen05.mma kind::f8f6f4, float32 accumulator in tensor memory, started from zero per
// block); the CUDA cores then fold it into float32 register accumulators with the two
// scales.  Four 128 x 128 partial buffers fill the 512 tensor-memory columns, so the tensor
// cores run up to four blocks ahead of the fold.
//
// One persistent CTA per SM walks 128 x 128 tiles of C (column tile fastest).  Roles:
//   warp 0      TMA producer (a and b: 128 rows x 128 bytes each per k-stage, 6 stages)
//   warp 1      MMA issuer and owner of the tensor-memory allocation: four MMAs (k = 32 each) and ONE
//               tcgen05.commit per block -- each tcgen05 instruction costs the issuing thread about a
//               hundred cycles; the k-stage is handed back to the producer by a fold lane instead
//   warps 2-17  fold + store, a warp = 32 accumulator rows x 32 columns, read in the 16x256b fragment
//               layout (4 row scales + 8 column scales per thread and block instead of 1 + 32)
//   warp 18     stages the scales of the next chunk of 8 k-blocks in shared memory
// Waits are inline mbarrier polls by every lane of a role (a shuffle-and-vote around one polling lane,
// or a call into a shared wait routine, adds its latency to every hand-over of a buffer).
// The tile width is a compile-time constant (FN): 256 halves the MMA instructions per flop and cuts the
// L2 -> shared-memory traffic by a quarter, but leaves two partial buffers and 64 accumulator registers
// per fold thread; measured level with 128 at 8192^3 and behind it at 4096^3, where 512 tiles on 148 SMs
// quantise badly.  At 128 the kernel moves 32 KB per block and SM through L2, about 9.5 TB/s in all.
#include "lh_common.cuh"

#include <type_traits>

namespace lh {

namespace {

constexpr int FM = 128, FN = 128, FKB = 128;   // tile; FKB = bytes (= e4m3 elements) of k per stage
constexpr int FSTAGES = 6;
constexpr int F_TILE = FM * FKB;               // a: 16 KB, then b: FN x 128 bytes
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
// 16 lanes x 32 columns in the accumulator-fragment layout: register 4 i + 2 hi + lo of thread t holds
// lane (t / 4) + 8 hi, column 8 i + 2 (t % 4) + lo, counted from the address.  A thread then owns two
// rows and eight columns instead of one row and 32 columns, so it needs far fewer column scales.
__device__ __forceinline__ void tmem_ld_frag(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
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
                    ok = __all_sync(0xffffffffu, mbar_wait_inline(&empty[s], ph ^ 1u, DEVERR_EMPTY_WAIT));
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
                ok = __all_sync(0xffffffffu, mbar_wait_inline(&full[s], ph, DEVERR_FULL_WAIT));
                if (!ok) break;
                const uint32_t a = smem_u32(tile_smem + size_t(s) * F_STAGE);
                const uint64_t da = umma_desc(a), db = umma_desc(a + F_TILE);
#pragma unroll
                for (int h = 0; h < SUB; ++h) {                     // scale block = partial product
                    if (!first_bufs) {
                        ok = __all_sync(0xffffffffu, mbar_wait_inline(&part_empty[buf], bph ^ 1u, DEVERR_PART_WAIT));
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
                    ok = __all_sync(0xffffffffu, mbar_wait_inline(&sc_empty[q & 1u], ((q >> 1) & 1u) ^ 1u, DEVERR_PART_WAIT));
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
        const int tq = lane >> 2, tc = lane & 3;                    // fragment coordinates of this thread
        const uint32_t tbase = tmem + (uint32_t(quarter * 32) << 16) + uint32_t(cgrp * F_CW);
        const int chunks = (nsb + F_CH - 1) / F_CH;
        constexpr int CH = F_CW / 32;                               // 32-column pieces per warp
        bool ok = true;                                             // a failed wait skips the work, not the barriers
        uint32_t gb = 0, q = 0;                                     // scale blocks and chunks so far
        for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            const int m0 = int(tile / tiles_n) * FM, n0 = int(tile % tiles_n) * FN;
            // The warp folds 32 accumulator rows x F_CW columns.  A thread owns rows tq + 16 half + 8 hi and,
            // per 8-column group i of each 32-column piece, the column pair 2 tc: 4 row scales and
            // F_CW / 4 column scales per block instead of 1 and F_CW, a third of the shared-memory loads
            // (the same data pipe feeds the tensor cores' operand reads and takes the TMA writes).
            float2 acc[2 * CH * 4 * 2];                             // [half][piece][i][hi]
#pragma unroll
            for (int j = 0; j < 2 * CH * 4 * 2; ++j) acc[j] = make_float2(0.f, 0.f);
            for (int chunk = 0; chunk < chunks; ++chunk, ++q) {
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait_inline(&sc_full[q & 1u], (q >> 1) & 1u, DEVERR_PART_WAIT));
                const float* sc = sc_all + (q & 1u) * F_SC_FLOATS;
                const float* sa_s = sc + (quarter * 32 + tq) * F_SA_LD;
                const float* sb_s = sc + FM * F_SA_LD + cgrp * F_CW + 2 * tc;
                const int nblk = min(F_CH, nsb - chunk * F_CH);
                for (int bl = 0; bl < nblk && ok; ++bl, ++gb) {
                    const int buf = int(gb % FBUFS);
                    ok = __all_sync(0xffffffffu, mbar_wait_inline(&part_full[buf], (gb / FBUFS) & 1u, DEVERR_PART_WAIT));
                    if (!ok) break;
                    // the block's MMAs are complete, so its k-stage may be refilled: one fold lane tells the producer
                    // (a second tcgen05.commit by the MMA thread would say the same, at a higher price)
                    if (t == 64 && (gb % SUB) == SUB - 1) mbar_arrive(&empty[(gb / SUB) % FSTAGES]);
                    tc_fence_after();
                    const float* sbp = sb_s + bl * FN;
                    // all of the warp's 32 x F_CW partial in flight at once, one wait: the hand-over of the buffer
                    // back to the tensor cores is on the critical path, the registers are there (acc is F_CW floats)
                    uint32_t v[2 * CH][16];
#pragma unroll
                    for (int half = 0; half < 2; ++half)
#pragma unroll
                        for (int ch = 0; ch < CH; ++ch)
                            tmem_ld_frag(tbase + (uint32_t(16 * half) << 16) + uint32_t(buf * FN + 32 * ch), v[half * CH + ch]);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&part_empty[buf]);   // the tensor cores may overwrite this buffer
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const float2 sa2[2] = {splat2(sa_s[(16 * half) * F_SA_LD + bl]), splat2(sa_s[(16 * half + 8) * F_SA_LD + bl])};
#pragma unroll
                        for (int ch = 0; ch < CH; ++ch) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 sb2 = *reinterpret_cast<const float2*>(sbp + 32 * ch + 8 * i);
#pragma unroll
                                for (int hi = 0; hi < 2; ++hi) {
                                    const uint32_t* vv = v[half * CH + ch];
                                    const float2 pr = make_float2(__uint_as_float(vv[4 * i + 2 * hi]), __uint_as_float(vv[4 * i + 2 * hi + 1]));
                                    float2& a = acc[((half * CH + ch) * 4 + i) * 2 + hi];
                                    a = fma2(mul2(pr, sb2), sa2[hi], a);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sc_empty[q & 1u]);      // the scale warp may refill this buffer
            }
            if (ok) {
                const int col0 = n0 + cgrp * F_CW;                  // first column of the warp
                const int64_t row0 = int64_t(m0) + quarter * 32 + tq;
                if (p.out_dtype == LH_F32) {
                    // four lanes hold 8 consecutive columns of a row: 32 contiguous bytes
                    const bool vec = (p.N % 2) == 0;
#pragma unroll
                    for (int half = 0; half < 2; ++half)
#pragma unroll
                        for (int hi = 0; hi < 2; ++hi) {
                            const int64_t row = row0 + 16 * half + 8 * hi;
                            if (row >= p.M) continue;
                            float* out = static_cast<float*>(p.c) + row * p.N;
#pragma unroll
                            for (int ch = 0; ch < CH; ++ch)
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float2 a = acc[((half * CH + ch) * 4 + i) * 2 + hi];
                                    const int c = col0 + 32 * ch + 8 * i + 2 * tc;
                                    if (vec && c + 2 <= p.N) {
                                        *reinterpret_cast<float2*>(out + c) = a;
                                    } else {
                                        if (c < p.N) out[c] = a.x;
                                        if (c + 1 < p.N) out[c + 1] = a.y;
                                    }
                                }
                        }
                } else {
                    // 16-bit output: the four lanes of a row exchange their words (a 4 x 4 transpose over the
                    // 8-column groups) so that each lane stores 16 contiguous bytes, four lanes 64
                    const bool vec = (p.N % 8) == 0;
#pragma unroll
                    for (int half = 0; half < 2; ++half)
#pragma unroll
                        for (int hi = 0; hi < 2; ++hi) {
                            const int64_t row = row0 + 16 * half + 8 * hi;
                            uint16_t* out = static_cast<uint16_t*>(p.c) + row * p.N;
#pragma unroll
                            for (int ch = 0; ch < CH; ++ch) {
                                uint32_t w[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float2 a = acc[((half * CH + ch) * 4 + i) * 2 + hi];
                                    if (p.out_dtype == LH_BF16) {
                                        w[i] = pack_bf16x2(a.x, a.y);
                                    } else {
                                        const __half2 h = __floats2half2_rn(a.x, a.y);
                                        w[i] = *reinterpret_cast<const uint32_t*>(&h);
                                    }
                                }
                                const int cbase = col0 + 32 * ch;
                                if (vec && cbase + 32 <= p.N) {      // warp-uniform: every lane takes part in the shuffles
                                    // w[i] of lane tc  ->  w[tc'] of lane i
                                    {
                                        const bool odd = (tc & 1) != 0;
                                        const uint32_t x0 = odd ? w[0] : w[1], x1 = odd ? w[2] : w[3];
                                        const uint32_t y0 = __shfl_xor_sync(0xffffffffu, x0, 1), y1 = __shfl_xor_sync(0xffffffffu, x1, 1);
                                        if (odd) { w[0] = y0; w[2] = y1; } else { w[1] = y0; w[3] = y1; }
                                    }
                                    {
                                        const bool up = (tc & 2) != 0;
                                        const uint32_t x0 = up ? w[0] : w[2], x1 = up ? w[1] : w[3];
                                        const uint32_t y0 = __shfl_xor_sync(0xffffffffu, x0, 2), y1 = __shfl_xor_sync(0xffffffffu, x1, 2);
                                        if (up) { w[0] = y0; w[1] = y1; } else { w[2] = y0; w[3] = y1; }
                                    }
                                    if (row < p.M) *reinterpret_cast<uint4*>(out + cbase + 8 * tc) = make_uint4(w[0], w[1], w[2], w[3]);
                                } else if (row < p.M) {
#pragma unroll
                                    for (int i = 0; i < 4; ++i) {
                                        const int c = cbase + 8 * i + 2 * tc;
                                        if (c < p.N) out[c] = uint16_t(w[i]);
                                        if (c + 1 < p.N) out[c + 1] = uint16_t(w[i] >> 16);
                                    }
                                }
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
