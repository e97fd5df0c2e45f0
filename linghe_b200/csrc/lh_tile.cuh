// 128x128-tile kernels: produce a tile of float32 values (identity / RMSNorm with known
// 1/rms / SwiGLU forward / SwiGLU backward), quantise it along rows (1x128) and/or
// columns (128x1, written transposed) to FP8 e4m3 and store codes and scales in the
// dense or per-expert packed layouts.
//
// Execution model (sm_100a): persistent CTAs walk a static round-robin list of tiles.
// Thread 0 feeds a multi-stage shared-memory ring with tensor-map TMA copies (one
// cp.async.bulk.tensor.2d per operand tile, completion counted on an mbarrier); all
// warps hold a 128x128 tile in registers (RPT rows x 8 columns per thread, as float2
// pairs for the packed float32x2 pipe), reduce row maxima by shuffles and column maxima
// through shared memory, and write the transposed codes through an XOR-swizzled
// shared-memory tile so that every global store is a full 128-byte row.
// No tensor cores: the path is HBM-bound.
#pragma once

#include "lh_common.cuh"

#include <type_traits>

namespace lh {

enum : int { OP_IDENT = 0, OP_NORM = 1, OP_SILU_F = 2, OP_SILU_B = 3, OP_GATHER = 4 };
enum : int { MODE_ROW = 0, MODE_COL = 1, MODE_BOTH = 2, MODE_BLOCK = 3 };

struct TileParams {
    CUtensorMap tmap[2];   // [0]: x (or g for the backward), [1]: x for the backward
    const void* w;         // optional per-row weight
    int w_dtype;           // LH_F32 / LH_BF16 / LH_F16
    const float* r;        // OP_NORM: 1/rms per row
    const void* gamma;     // OP_NORM: weight per column
    const void* counts;    // per-expert row counts (NULL = dense)
    int rt_cap;            // entries of the row-tile -> expert table that fit in shared memory (0: none)
    int pad16;             // segments are padded to multiples of 16 rows (OP_GATHER)
    const uint8_t* gx;     // OP_GATHER: source matrix [m, n]
    const void* indices;   // OP_GATHER: source row of every padded output row
    int indices_i64;
    const void* probs;     // OP_GATHER: optional routing weights [m, E]
    void* prob_out;        // OP_GATHER: optional [sum of padded counts]
    int probs_dtype;
    int counts_i64;
    int E;
    int64_t M;             // rows (dense) / total rows (batched)
    int64_t n;             // output columns per half
    uint8_t* q;
    float* s;
    uint8_t* qt;
    float* st;
    void* hp;              // OP_SILU_B: optional dx in the input dtype
    float* dws;            // OP_SILU_B: optional per-(row, column block) partial dw
    int round_scale;
    int scale_rowmajor;    // MODE_ROW only: s[i*nb + b] instead of s[b*M + i]
    int descending;        // walk the tiles from the last row band to the first: for a launch that re-reads
                           // a tensor the previous launch has just streamed in ascending order, so that it
                           // starts with the part of it that is still in L2
};

template <int OP> struct OpTraits;
template <> struct OpTraits<OP_IDENT> { static constexpr int K = 1, NHALF = 1; };
template <> struct OpTraits<OP_NORM> { static constexpr int K = 1, NHALF = 1; };
template <> struct OpTraits<OP_SILU_F> { static constexpr int K = 2, NHALF = 1; };
template <> struct OpTraits<OP_SILU_B> { static constexpr int K = 3, NHALF = 2; };
template <> struct OpTraits<OP_GATHER> { static constexpr int K = 1, NHALF = 1; };

template <int OP, typename InT, int RPT, int STAGES>
struct TileCfg {
    static constexpr int K = OpTraits<OP>::K;
    static constexpr int NHALF = OpTraits<OP>::NHALF;
    static constexpr int NMAP = OP == OP_SILU_B ? 2 : (OP == OP_GATHER ? 0 : 1);   // tensor maps (x1 and x2 share one)
    static constexpr int EB = Elem<InT>::BYTES;
    static constexpr int ROWB = 128 * EB;            // bytes of one tile row of one operand
    static constexpr int TILEB = 128 * ROWB;         // one operand tile
    static constexpr int STAGEB = K * TILEB;
    static constexpr int NW = 128 / (2 * RPT);       // consumer warps
    static constexpr int NCONS = NW * 32;
    static constexpr int NTHREADS = NCONS;
    // shared memory carve-up (bytes)
    static constexpr int OFF_STAGES = 0;
    static constexpr int OFF_QT = OFF_STAGES + STAGES * STAGEB;  // 128 x 128 transposed codes
    static constexpr int OFF_PART = OFF_QT + 128 * 128;          // [NW][128] column maxima
    static constexpr int OFF_CS = OFF_PART + NW * 128 * 4;       // [128] column scale
    static constexpr int OFF_CY = OFF_CS + 512;                  // [128] 1/scale
    static constexpr int OFF_BAR = OFF_CY + 512;                 // full[STAGES], empty[STAGES]
    static constexpr int OFF_SEG = OFF_BAR + 2 * STAGES * 8;     // segS[E+1] int64, segB[E+1] int32
    static constexpr size_t smem_bytes(int E) { return size_t(OFF_SEG) + size_t(E + 1) * 16 + 16; }
};

struct TileLoc {
    int64_t S;   // first row of the segment
    int64_t c;   // rows in the segment
    int64_t B;   // 128-row blocks before the segment
    int T;       // 128-row block index inside the segment
    int ct;      // column tile
    int valid;   // valid rows in this tile (1..128)
    int e;       // segment (expert) index
};

__device__ __forceinline__ int find_expert(int rt, const int* segB, int E) {
    int lo = 0, hi = E - 1;
    while (lo < hi) {  // smallest e with segB[e+1] > rt
        const int mid = (lo + hi) >> 1;
        if (segB[mid + 1] > rt) hi = mid; else lo = mid + 1;
    }
    return lo;
}

// `tab` (optional): expert of every 128-row tile, filled once per CTA, so that the per-tile
// lookup is one shared-memory read instead of a binary search
__device__ __forceinline__ TileLoc locate(int tile, int col_tiles, const int64_t* segS, const int* segB,
                                          int E, const uint16_t* tab = nullptr) {
    TileLoc t;
    const int rt = tile / col_tiles;
    t.ct = tile - rt * col_tiles;
    const int lo = tab != nullptr ? int(tab[rt]) : find_expert(rt, segB, E);
    t.e = lo;
    t.S = segS[lo];
    t.c = segS[lo + 1] - t.S;
    t.B = segB[lo];
    t.T = rt - int(t.B);
    const int64_t left = t.c - int64_t(t.T) * 128;
    t.valid = left < 128 ? int(left) : 128;
    return t;
}

// 8 consecutive elements of a tile row -> 4 float2 pairs (NEG: the negated values)
template <typename InT, bool NEG = false>
__device__ __forceinline__ void load8p(const uint8_t* row_base, int l16, float2* f) {
    if constexpr (sizeof(InT) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(row_base + l16 * 32);
        const float4 b = *reinterpret_cast<const float4*>(row_base + l16 * 32 + 16);
        f[0] = make_float2(a.x, a.y); f[1] = make_float2(a.z, a.w);
        f[2] = make_float2(b.x, b.y); f[3] = make_float2(b.z, b.w);
        if constexpr (NEG) {
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = mul2(f[i], splat2(-1.f));
        }
    } else {
        const uint4 raw = *reinterpret_cast<const uint4*>(row_base + l16 * 16);
        if constexpr (std::is_same<InT, __half>::value) {
            const uint32_t w[4] = {raw.x ^ (NEG ? 0x80008000u : 0u), raw.y ^ (NEG ? 0x80008000u : 0u),
                                   raw.z ^ (NEG ? 0x80008000u : 0u), raw.w ^ (NEG ? 0x80008000u : 0u)};
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        } else if constexpr (NEG) {
            f[0] = bf16x2_to_neg_f2(raw.x); f[1] = bf16x2_to_neg_f2(raw.y);
            f[2] = bf16x2_to_neg_f2(raw.z); f[3] = bf16x2_to_neg_f2(raw.w);
        } else {
            f[0] = bf16x2_to_f2(raw.x); f[1] = bf16x2_to_f2(raw.y);
            f[2] = bf16x2_to_f2(raw.z); f[3] = bf16x2_to_f2(raw.w);
        }
    }
}

template <typename InT>
__device__ __forceinline__ void store8_hp(void* dst, const float2* f) {
    if constexpr (sizeof(InT) == 4) {
        float4* d = reinterpret_cast<float4*>(dst);
        d[0] = make_float4(f[0].x, f[0].y, f[1].x, f[1].y);
        d[1] = make_float4(f[2].x, f[2].y, f[3].x, f[3].y);
    } else if constexpr (std::is_same<InT, __half>::value) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(pack_f16x2(f[0].x, f[0].y), pack_f16x2(f[1].x, f[1].y),
                                                    pack_f16x2(f[2].x, f[2].y), pack_f16x2(f[3].x, f[3].y));
    } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(f[0].x, f[0].y), pack_bf16x2(f[1].x, f[1].y),
                                                    pack_bf16x2(f[2].x, f[2].y), pack_bf16x2(f[3].x, f[3].y));
    }
}

__device__ __forceinline__ float max16(float a) {
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 8));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    return a;
}
__device__ __forceinline__ float sum16(float a) {
    a += __shfl_xor_sync(0xffffffffu, a, 8);
    a += __shfl_xor_sync(0xffffffffu, a, 4);
    a += __shfl_xor_sync(0xffffffffu, a, 2);
    a += __shfl_xor_sync(0xffffffffu, a, 1);
    return a;
}

// the same quotient for one value that is held as x itself (ny = -RN(1/s)); operand negations
// are instruction modifiers
__device__ __forceinline__ float quot_exact(float x, float s, float ny) {
    const float q0 = x * -ny;
    const float r = fmaf(s, q0, -x);
    return fmaf(r, ny, q0);
}
constexpr float kTinyScale = 8.0e-28f;   // ~2^-90: below this take IEEE division

// 8 values of one row, one scale -> 8 codes.
//   EXACT: `y` is -RN(1/s) and v holds the negated values (NEGV) or the values; a positive
//          `y` marks a block whose scale is so small that the residual of the exact quotient
//          could underflow (0 < amax < ~3.6e-25): those take IEEE division.  All-zero blocks
//          do not need it.
//   else:  v holds the values and `y` an approximate 1/s.
template <bool EXACT, bool NEGV, bool CHECK = true>
__device__ __forceinline__ uint2 quant_row8(const float2* v, float sc, float y) {
    float2 q[4];
    if constexpr (EXACT) {
        if constexpr (NEGV) {
            const float2 s2 = splat2(sc), ny2 = splat2(y);
#pragma unroll
            for (int j = 0; j < 4; ++j) q[j] = quot_exact2(v[j], s2, ny2);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) q[j] = make_float2(quot_exact(v[j].x, sc, y), quot_exact(v[j].y, sc, y));
        }
        if (CHECK && y > 0.f) {   // rare; CHECK = false: the caller knows no block of the warp needs it
            const float sg = NEGV ? -1.f : 1.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) q[j] = make_float2(__fdiv_rn(sg * v[j].x, sc), __fdiv_rn(sg * v[j].y, sc));
        }
    } else {
        const float2 y2 = splat2(y);
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = mul2(v[j], y2);
    }
    return make_uint2(cvt_e4m3x4(q[0].x, q[0].y, q[1].x, q[1].y), cvt_e4m3x4(q[2].x, q[2].y, q[3].x, q[3].y));
}

// the multiplier quant_row8 takes: the negated correctly rounded reciprocal where exact
// quotients are required (+1 as the "use IEEE division" marker for non-zero blocks with a
// denormal-range scale), else an approximate reciprocal
template <bool EXACT>
__device__ __forceinline__ float scale_rcp(float sc, float amax) {
    if constexpr (EXACT) return (sc < kTinyScale && amax > 0.f) ? 1.f : -__frcp_rn(sc);
    return rcp_approx(sc);
}

// Row maxima across the 16 lanes that share a tile row, for RPT rows at once: a
// transposing butterfly halves the number of live values at each step, so RPT rows cost
// RPT + log2(16/RPT) shuffles instead of 4*RPT.  On return a[0] holds the maximum of row
// (l16 * RPT / 16), replicated over 16/RPT neighbouring lanes.
template <int RPT>
__device__ __forceinline__ float row_max_transposed(float* a, int l16) {
    static_assert(RPT == 8 || RPT == 4, "RPT");
    if constexpr (RPT == 8) {
        const bool up = (l16 & 8) != 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float recv = __shfl_xor_sync(0xffffffffu, up ? a[i] : a[i + 4], 8);
            a[i] = fmaxf(up ? a[i + 4] : a[i], recv);
        }
    }
    {
        const bool up = (l16 & (RPT == 8 ? 4 : 8)) != 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float recv = __shfl_xor_sync(0xffffffffu, up ? a[i] : a[i + 2], RPT == 8 ? 4 : 8);
            a[i] = fmaxf(up ? a[i + 2] : a[i], recv);
        }
    }
    {
        const bool up = (l16 & (RPT == 8 ? 2 : 4)) != 0;
        const float recv = __shfl_xor_sync(0xffffffffu, up ? a[0] : a[1], RPT == 8 ? 2 : 4);
        a[0] = fmaxf(up ? a[1] : a[0], recv);
    }
    if constexpr (RPT == 4) a[0] = fmaxf(a[0], __shfl_xor_sync(0xffffffffu, a[0], 2));
    a[0] = fmaxf(a[0], __shfl_xor_sync(0xffffffffu, a[0], 1));
    return a[0];
}

template <int OP, typename InT, int MODE, bool EXACT, int RPT, int STAGES, int MINB, bool WEIGHTED>
__global__ void __launch_bounds__(TileCfg<OP, InT, RPT, STAGES>::NTHREADS, MINB)
tile_kernel(const __grid_constant__ TileParams p) {
    static_assert(!EXACT || OP == OP_IDENT || OP == OP_GATHER, "exact quotients: pure quantisers only");
    // The plain quantiser keeps negated values so that its exact quotients are packed; the
    // gathering one has no registers to spare for the register pairs that packed math needs.
    constexpr bool NEGV = EXACT && OP == OP_IDENT;
    using C = TileCfg<OP, InT, RPT, STAGES>;
    constexpr int K = C::K, NHALF = C::NHALF, NW = C::NW, NCONS = C::NCONS;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stages = smem + C::OFF_STAGES;
    uint8_t* qts = smem + C::OFF_QT;
    float* part = reinterpret_cast<float*>(smem + C::OFF_PART);
    float* cs = reinterpret_cast<float*>(smem + C::OFF_CS);
    float* cy = reinterpret_cast<float*>(smem + C::OFF_CY);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty = full + STAGES;
    int64_t* segS = reinterpret_cast<int64_t*>(smem + ((C::OFF_SEG + 15) & ~15));
    int* segB = reinterpret_cast<int*>(segS + (p.E + 1));
    int* segC = segB + (p.E + 1);   // true (unpadded) row counts

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int E = p.E;

    // ---- prologue: barriers + segment table (exclusive scans of counts) ------------
    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], NW);
        }
        mbar_fence_init();
#pragma unroll
        for (int k = 0; k < C::NMAP; ++k) tma_prefetch_desc(&p.tmap[k]);
    }
    // counts -> shared memory with one load per thread (a single round trip to L2), then
    // warp 0 scans them from there
    if (p.counts != nullptr) {
        for (int e = tid; e < E; e += C::NTHREADS)
            segC[e] = p.counts_i64 ? int(reinterpret_cast<const int64_t*>(p.counts)[e])
                                   : reinterpret_cast<const int32_t*>(p.counts)[e];
    }
    __syncthreads();
    if (warp == 0) {
        if (p.counts == nullptr) {
            if (lane == 0) {
                segS[0] = 0; segS[1] = p.M;
                segB[0] = 0; segB[1] = int((p.M + 127) >> 7);
                segC[0] = int(p.M);
            }
        } else {
            const int per = (E + 31) / 32;
            const int e0 = lane * per;
            int64_t sumS = 0, sumB = 0;
            for (int e = e0; e < e0 + per && e < E; ++e) {
                const int64_t c = segC[e];
                sumS += p.pad16 ? ((c + 15) >> 4) << 4 : c;
                sumB += (c + 127) >> 7;
            }
            int64_t preS = sumS, preB = sumB;  // inclusive warp scan
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int64_t a = __shfl_up_sync(0xffffffffu, preS, d);
                const int64_t b = __shfl_up_sync(0xffffffffu, preB, d);
                if (lane >= d) { preS += a; preB += b; }
            }
            int64_t accS = preS - sumS, accB = preB - sumB;
            for (int e = e0; e < e0 + per && e < E; ++e) {
                const int64_t c = segC[e];
                segS[e] = accS; segB[e] = int(accB);
                accS += p.pad16 ? ((c + 15) >> 4) << 4 : c; accB += (c + 127) >> 7;
            }
            if (lane == 31) { segS[E] = preS; segB[E] = int(preB); }
        }
    }
    __syncthreads();

    // The table's presence is a predicate and its address is recomputed per tile, so that the
    // dense instantiations do not carry a pointer through the main loop.
    const bool has_tab = E > 1 && segB[E] <= p.rt_cap;
    auto tab_ptr = [&]() -> const uint16_t* {
        return has_tab ? reinterpret_cast<const uint16_t*>(smem + ((C::OFF_SEG + 15) & ~15) + size_t(E + 1) * 16)
                       : nullptr;
    };
    if (has_tab) {
        uint16_t* tw = const_cast<uint16_t*>(tab_ptr());
        for (int rt = tid; rt < segB[E]; rt += C::NTHREADS) tw[rt] = uint16_t(find_expert(rt, segB, E));
        __syncthreads();
    }
    const int col_tiles = int(p.n >> 7);
    const int64_t total_tiles = int64_t(segB[E]) * col_tiles;
    const int64_t nb = p.n >> 7;

    // Thread 0 doubles as the producer: it fills the ring before the loop and, at the top
    // of every iteration, refills the stage that all warps released one iteration ago.
    // One tensor-map copy per operand brings a whole 128x128 tile; rows past the end of
    // the matrix read as zero, rows of a following expert segment are masked by `valid`.
    auto issue = [&](int tile, int stage) {
        if constexpr (OP == OP_GATHER) return;   // gathered rows are loaded straight into registers
        const TileLoc t = locate(p.descending ? int(total_tiles) - 1 - tile : tile, col_tiles, segS, segB, E, tab_ptr());
        uint8_t* dst = stages + size_t(stage) * C::STAGEB;
        const int r0 = int(t.S + int64_t(t.T) * 128);
        const int c0 = t.ct * 128;
        mbar_expect_tx(&full[stage], uint32_t(C::STAGEB));
        if constexpr (OP == OP_SILU_F) {
            tma_load_2d(dst, &p.tmap[0], c0, r0, &full[stage]);
            tma_load_2d(dst + C::TILEB, &p.tmap[0], int(p.n) + c0, r0, &full[stage]);
        } else if constexpr (OP == OP_SILU_B) {
            tma_load_2d(dst, &p.tmap[0], c0, r0, &full[stage]);
            tma_load_2d(dst + C::TILEB, &p.tmap[1], c0, r0, &full[stage]);
            tma_load_2d(dst + 2 * C::TILEB, &p.tmap[1], int(p.n) + c0, r0, &full[stage]);
        } else {
            tma_load_2d(dst, &p.tmap[0], c0, r0, &full[stage]);
        }
    };
    const int n_tiles = int(total_tiles);   // fits 32 bits (checked on the host)
    if (tid == 0) {
        int tile = int(blockIdx.x);
        for (int j = 0; j < STAGES && tile < n_tiles; ++j, tile += int(gridDim.x)) issue(tile, j);
    }

    const int cw = warp;                 // warp index
    const int hw = lane >> 4;            // half-warp
    const int l16 = lane & 15;           // 8-column group inside the tile
    const int row0 = cw * (2 * RPT) + hw * RPT;
    const bool rs = p.round_scale != 0;

    // ---- OP_GATHER: per-thread index registers and cp.async row fetches ----------------------
    int gidx_next[OP == OP_GATHER ? RPT : 1];   // source rows fit 31 bits
    auto gather_indices = [&](int tile, int* idx) {      // source rows of this thread's rows of `tile`
#pragma unroll
        for (int s = 0; s < RPT; ++s) idx[s] = -1;           // -1: padding row (zeros) or no tile
        if (tile < 0) return;
        const TileLoc tl = locate(p.descending ? int(total_tiles) - 1 - tile : tile, col_tiles, segS, segB, E, tab_ptr());
        const int cnt = segC[tl.e] - tl.T * 128 - row0;      // real (unpadded) rows left for this thread
        const int64_t g0 = tl.S + int64_t(tl.T) * 128 + row0;
#pragma unroll
        for (int s = 0; s < RPT; ++s) {
            if (s < cnt)
                idx[s] = p.indices_i64 ? int(reinterpret_cast<const int64_t*>(p.indices)[g0 + s])
                                       : reinterpret_cast<const int32_t*>(p.indices)[g0 + s];
        }
    };
    // Also writes the gathered routing probabilities of the tile's rows (first column tile only),
    // so that the indices need not stay in registers until the tile is processed.
    auto gather_issue = [&](int tile, const int* idx, int stg) {
        if (tile >= 0) {
            const int ct = tile % col_tiles;
            if (p.prob_out != nullptr && ct == 0 && l16 == 0) {
                const TileLoc tl = locate(p.descending ? int(total_tiles) - 1 - tile : tile, col_tiles, segS, segB, E, tab_ptr());
                const int64_t g0 = tl.S + int64_t(tl.T) * 128 + row0;
                const int nr = tl.valid - row0;
#pragma unroll
                for (int s = 0; s < RPT; ++s) {
                    if (s < nr) {
                        float pv = 0.f;
                        if (idx[s] >= 0)
                            pv = p.probs_dtype == LH_BF16
                                     ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.probs)[int64_t(idx[s]) * E + tl.e])
                                     : reinterpret_cast<const float*>(p.probs)[int64_t(idx[s]) * E + tl.e];
                        if (p.probs_dtype == LH_BF16)
                            reinterpret_cast<__nv_bfloat16*>(p.prob_out)[g0 + s] = __float2bfloat16_rn(pv);
                        else
                            reinterpret_cast<float*>(p.prob_out)[g0 + s] = pv;
                    }
                }
            }
            uint8_t* dst = stages + size_t(stg) * C::STAGEB + row0 * C::ROWB + l16 * (8 * C::EB);
#pragma unroll
            for (int s = 0; s < RPT; ++s) {
                const bool real = idx[s] >= 0;
                const uint8_t* src = p.gx + (int64_t(real ? idx[s] : 0) * p.n + int64_t(ct) * 128 + l16 * 8) * C::EB;
#pragma unroll
                for (int b = 0; b < (8 * C::EB) / 16; ++b)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst + s * C::ROWB + 16 * b)),
                                 "l"(src + 16 * b), "r"(real ? 16 : 0)
                                 : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if constexpr (OP == OP_GATHER) {
        const int t0 = int(blockIdx.x);
        gather_indices(t0 < n_tiles ? t0 : -1, gidx_next);
        gather_issue(t0 < n_tiles ? t0 : -1, gidx_next, 0);
        const int64_t t1 = int64_t(t0) + gridDim.x;
        gather_indices(t1 < n_tiles ? int(t1) : -1, gidx_next);
    }

    int stage = 0, prev_stage = 0;
    uint32_t phase = 0, prev_phase = 0;
    bool first_it = true;
    bool dead = false;   // a bounded wait of this thread gave up (see mbar_wait_or_mark)
    for (int tile = int(blockIdx.x); tile < n_tiles; tile += int(gridDim.x)) {
        if (OP != OP_GATHER && tid == 0 && !first_it) {
            // the previous tile's stage is free once every warp has released it: refill it with
            // the tile STAGES-1 steps ahead.  Copies issued here are consumed by this CTA, so
            // none is in flight when the loop ends.
            const int64_t nxt = int64_t(tile) + int64_t(STAGES - 1) * gridDim.x;
            if (nxt < n_tiles) {
                mbar_wait_or_mark<true>(&empty[prev_stage], prev_phase, DEVERR_EMPTY_WAIT, dead);
                if (!dead) issue(int(nxt), prev_stage);
            }
        }
        const TileLoc t = locate(p.descending ? int(total_tiles) - 1 - tile : tile, col_tiles, segS, segB, E, tab_ptr());
        const int64_t grow0 = t.S + int64_t(t.T) * 128;   // global row of tile row 0
        const int64_t gcol0 = int64_t(t.ct) * 128;        // column inside a half
        // Per-row and per-column side inputs come straight from global memory: fetch them
        // before blocking on the tile so that their latency hides behind the TMA copy.
        const int nrows = t.valid - row0;   // rows of this thread that exist (may exceed RPT or be <= 0)
        constexpr bool HAS_AUX = OP == OP_NORM || ((OP == OP_SILU_F || OP == OP_SILU_B) && WEIGHTED);
        float aux[HAS_AUX ? RPT : 1];
        if constexpr (OP == OP_NORM) {
#pragma unroll
            for (int s = 0; s < RPT; ++s) aux[s] = s < nrows ? p.r[grow0 + row0 + s] : 0.f;
        } else if constexpr (HAS_AUX) {
#pragma unroll
            for (int s = 0; s < RPT; ++s) {
                aux[s] = 1.f;
                if (s < nrows)
                    aux[s] = p.w_dtype == LH_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.w)[grow0 + row0 + s])
                             : p.w_dtype == LH_F16 ? __half2float(reinterpret_cast<const __half*>(p.w)[grow0 + row0 + s])
                                                   : reinterpret_cast<const float*>(p.w)[grow0 + row0 + s];
            }
        }
        float2 gam[OP == OP_NORM ? 4 : 1];
        if constexpr (OP == OP_NORM)   // gamma has the input's element type
            load8p<InT>(reinterpret_cast<const uint8_t*>(p.gamma) + gcol0 * C::EB, l16, gam);
        if constexpr (OP != OP_GATHER) {
            // Inline wait where a call would spill live registers around it; the transposed-only
            // norm instantiation has none to spill and measures 2 % faster with the call.
            mbar_wait_or_mark<!(OP == OP_NORM && MODE == 1)>(&full[stage], phase, DEVERR_FULL_WAIT, dead);
        }
        const uint8_t* sbase = stages + size_t(stage) * C::STAGEB;

        const int cur_stage = stage;
        first_it = false;
        prev_stage = stage; prev_phase = phase;
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }

        float2 v[NHALF][RPT][4];
        float dwp[OP == OP_SILU_B ? RPT : 1];
        if constexpr (OP == OP_GATHER) {
            // Software pipeline over three tiles: the rows of this tile were fetched with
            // cp.async during the previous iteration; now fetch the next tile with the indices
            // read one iteration ago, and read the indices of the tile after that.  Every
            // thread copies exactly the 16-byte chunks it later reads, so no barrier is needed.
            const int64_t t1 = int64_t(tile) + gridDim.x, t2 = t1 + gridDim.x;
            gather_issue(t1 < n_tiles ? int(t1) : -1, gidx_next, stage);            // `stage` already points at the next slot
            gather_indices(t2 < n_tiles ? int(t2) : -1, gidx_next);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        }
#pragma unroll
        for (int s = 0; s < RPT; ++s) {
            const uint8_t* srow = sbase + (row0 + s) * C::ROWB;
            if constexpr (OP == OP_IDENT || OP == OP_GATHER) {
                load8p<InT, NEGV>(srow, l16, v[0][s]);
            } else if constexpr (OP == OP_NORM) {
                float2 x[4];
                load8p<InT>(srow, l16, x);
                const float2 r2 = splat2(aux[s]);
#pragma unroll
                for (int j = 0; j < 4; ++j) v[0][s][j] = mul2(mul2(x[j], r2), gam[j]);
            } else if constexpr (OP == OP_SILU_F) {
                float2 x1[4], x2[4];
                load8p<InT>(srow, l16, x1);
                load8p<InT>(srow + C::TILEB, l16, x2);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 sg = EXACT ? make_float2(sigmoid_ref(x1[j].x), sigmoid_ref(x1[j].y))
                                            : sigmoid_fast2(x1[j]);
                    float2 y = mul2(mul2(sg, x1[j]), x2[j]);
                    if constexpr (WEIGHTED) y = mul2(y, splat2(aux[s]));
                    v[0][s][j] = y;
                }
            } else {  // OP_SILU_B
                float2 g[4], x1[4], x2[4];
                load8p<InT>(srow, l16, g);
                load8p<InT>(srow + C::TILEB, l16, x1);
                load8p<InT>(srow + 2 * C::TILEB, l16, x2);
                float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 sg = EXACT ? make_float2(sigmoid_ref(x1[j].x), sigmoid_ref(x1[j].y))
                                            : sigmoid_fast2(x1[j]);
                    const float2 sgg = mul2(sg, g[j]);                                // sigmoid * g
                    const float2 d2 = mul2(sgg, x1[j]);                               // d/dx2 (unweighted)
                    const float2 oms = fma2(sg, splat2(-1.f), splat2(1.f));           // 1 - sigmoid
                    const float2 u = fma2(x1[j], oms, splat2(1.f));
                    const float2 d1 = mul2(mul2(sgg, x2[j]), u);                      // d/dx1 (unweighted)
                    acc = fma2(d2, x2[j], acc);                                       // sigmoid*x1*x2*g
                    v[0][s][j] = WEIGHTED ? mul2(d1, splat2(aux[s])) : d1;
                    v[1][s][j] = WEIGHTED ? mul2(d2, splat2(aux[s])) : d2;
                }
                dwp[s] = acc.x + acc.y;
            }
        }
        if (t.valid < 128) {   // ragged last tile of a segment: rows past its end count as zeros
#pragma unroll
            for (int s = 0; s < RPT; ++s) {
                if (s >= nrows) {
#pragma unroll
                    for (int h = 0; h < NHALF; ++h)
#pragma unroll
                        for (int j = 0; j < 4; ++j) v[h][s][j] = NEGV ? make_float2(-0.f, -0.f) : make_float2(0.f, 0.f);
                    if constexpr (OP == OP_SILU_B) dwp[s] = 0.f;
                }
            }
        }
        // all shared-memory reads of this stage are done: hand it back to the producer
        if constexpr (OP != OP_GATHER) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[cur_stage]);
        }

        if constexpr (OP == OP_SILU_B) {
            if (p.dws != nullptr) {
#pragma unroll
                for (int s = 0; s < RPT; ++s) {
                    const float tot = sum16(dwp[s]);
                    const int rr = row0 + s;
                    if (l16 == 0 && rr < t.valid) p.dws[(grow0 + rr) * nb + t.ct] = tot;
                }
            }
            if (p.hp != nullptr) {
#pragma unroll
                for (int h = 0; h < NHALF; ++h) {
                    uint8_t* dst = reinterpret_cast<uint8_t*>(p.hp) +
                                   ((grow0 + row0) * (2 * p.n) + h * p.n + gcol0 + l16 * 8) * C::EB;
#pragma unroll
                    for (int s = 0; s < RPT; ++s) {
                        if (row0 + s < t.valid) store8_hp<InT>(dst, v[h][s]);
                        dst += 2 * p.n * C::EB;
                    }
                }
            }
        }

#pragma unroll
        for (int h = 0; h < NHALF; ++h) {
            // -------------------------- 128x128 single-scale blocks -----------------
            if constexpr (MODE == MODE_BLOCK) {
                float m = 0.f;
#pragma unroll
                for (int s = 0; s < RPT; ++s)
#pragma unroll
                    for (int j = 0; j < 4; ++j) m = max3abs(v[h][s][j].x, v[h][s][j].y, m);
                m = max16(m);
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
                if (lane == 0) part[cw] = m;
                named_bar<1, NCONS>();
                float bm = part[0];
#pragma unroll
                for (int w2 = 1; w2 < NW; ++w2) bm = fmaxf(bm, part[w2]);
                const float sc = scale_from_amax(bm, rs);
                const float y = scale_rcp<EXACT>(sc, bm);
#pragma unroll
                for (int s = 0; s < RPT; ++s) {
                    const int rr = row0 + s;
                    const uint2 codes = quant_row8<EXACT, NEGV>(v[h][s], sc, y);
                    if (rr < t.valid) st_global_v2(p.q + (grow0 + rr) * p.n + gcol0 + l16 * 8, codes.x, codes.y);
                }
                if (tid == 0) p.s[(t.B + t.T) * nb + t.ct] = sc;
                named_bar<1, NCONS>();  // part[] is rewritten by the next tile
            }
            // ------------------------------ row-wise 1x128 --------------------------
            if constexpr (MODE == MODE_ROW || MODE == MODE_BOTH) {
                constexpr int G = 16 / RPT;   // lanes that end up holding the same row maximum
                float a[RPT];
#pragma unroll
                for (int s = 0; s < RPT; ++s) {
                    float m = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) m = max3abs(v[h][s][j].x, v[h][s][j].y, m);
                    a[s] = m;
                }
                const float mymax = row_max_transposed<RPT>(a, l16);
                const float mysc = scale_from_amax(mymax, rs);
                const float myy = scale_rcp<EXACT>(mysc, mymax);
                {
                    const int rr = row0 + l16 / G;   // the row this lane holds the scale of
                    if ((l16 % G) == 0 && rr < t.valid) {
                        if (p.scale_rowmajor)
                            p.s[(grow0 + rr) * nb + t.ct] = mysc;
                        else
                            p.s[t.S * (NHALF * nb) + (h * nb + t.ct) * t.c + int64_t(t.T) * 128 + rr] = mysc;
                    }
                }
                const int64_t ldq = NHALF * p.n;
                uint8_t* qrow = p.q + (grow0 + row0) * ldq + h * p.n + gcol0 + l16 * 8;
                // one warp-uniform test for the IEEE-division fallback instead of one per row
                auto row_pass = [&](auto check) {
#pragma unroll
                    for (int s = 0; s < RPT; ++s) {
                        const float sc = __shfl_sync(0xffffffffu, mysc, s * G, 16);
                        const float y = __shfl_sync(0xffffffffu, myy, s * G, 16);
                        const uint2 codes = quant_row8<EXACT, NEGV, decltype(check)::value>(v[h][s], sc, y);
                        st_global_v2_if(s < nrows, qrow, codes.x, codes.y);
                        qrow += ldq;
                    }
                };
                if (EXACT && __any_sync(0xffffffffu, myy > 0.f)) row_pass(std::true_type{});
                else row_pass(std::false_type{});
            }
            // ------------------------ column-wise 128x1, transposed -----------------
            if constexpr (MODE == MODE_COL || MODE == MODE_BOTH) {
                float2 cm[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float mx = 0.f, my = 0.f;
#pragma unroll
                    for (int s = 0; s < RPT; s += 2) {
                        mx = max3abs(v[h][s][j].x, v[h][s + 1][j].x, mx);
                        my = max3abs(v[h][s][j].y, v[h][s + 1][j].y, my);
                    }
                    cm[j].x = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    cm[j].y = fmaxf(my, __shfl_xor_sync(0xffffffffu, my, 16));
                }
                if (hw == 0) {
                    float4* dst = reinterpret_cast<float4*>(part + cw * 128 + l16 * 8);
                    dst[0] = make_float4(cm[0].x, cm[0].y, cm[1].x, cm[1].y);
                    dst[1] = make_float4(cm[2].x, cm[2].y, cm[3].x, cm[3].y);
                }
                named_bar<1, NCONS>();
                if (tid < 128) {
                    float m = part[tid];
#pragma unroll
                    for (int w2 = 1; w2 < NW; ++w2) m = fmaxf(m, part[w2 * 128 + tid]);
                    const float sc = scale_from_amax(m, rs);
                    cs[tid] = sc;
                    cy[tid] = scale_rcp<EXACT>(sc, m);
                    p.st[(t.B + t.T) * (NHALF * p.n) + h * p.n + gcol0 + tid] = sc;
                }
                named_bar<1, NCONS>();
                float2 sc2[4], y2[4];
                {
                    const float4 a = *reinterpret_cast<const float4*>(cs + l16 * 8);
                    const float4 b = *reinterpret_cast<const float4*>(cs + l16 * 8 + 4);
                    const float4 c = *reinterpret_cast<const float4*>(cy + l16 * 8);
                    const float4 e = *reinterpret_cast<const float4*>(cy + l16 * 8 + 4);
                    sc2[0] = make_float2(a.x, a.y); sc2[1] = make_float2(a.z, a.w);
                    sc2[2] = make_float2(b.x, b.y); sc2[3] = make_float2(b.z, b.w);
                    y2[0] = make_float2(c.x, c.y); y2[1] = make_float2(c.z, c.w);
                    y2[2] = make_float2(e.x, e.y); y2[3] = make_float2(e.z, e.w);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 q[RPT];
                    if constexpr (EXACT) {
#pragma unroll
                        for (int s = 0; s < RPT; ++s)
                            q[s] = NEGV ? quot_exact2(v[h][s][j], sc2[j], y2[j])
                                        : make_float2(quot_exact(v[h][s][j].x, sc2[j].x, y2[j].x),
                                                      quot_exact(v[h][s][j].y, sc2[j].y, y2[j].y));
                        if (y2[j].x > 0.f || y2[j].y > 0.f) {   // rare: denormal-range scale, IEEE division
                            const float sg = NEGV ? -1.f : 1.f;
#pragma unroll
                            for (int s = 0; s < RPT; ++s)
                                q[s] = make_float2(__fdiv_rn(sg * v[h][s][j].x, sc2[j].x), __fdiv_rn(sg * v[h][s][j].y, sc2[j].y));
                        }
                    } else {
#pragma unroll
                        for (int s = 0; s < RPT; ++s) q[s] = mul2(v[h][s][j], y2[j]);
                    }
                    const int colx = l16 * 8 + 2 * j;
                    if constexpr (RPT == 8) {
                        const int rc = cw * 2 + hw;
                        const uint32_t off = uint32_t((rc ^ l16) << 3);
                        *reinterpret_cast<uint2*>(qts + colx * 128 + off) = make_uint2(
                            cvt_e4m3x4(q[0].x, q[1].x, q[2].x, q[3].x), cvt_e4m3x4(q[4].x, q[5].x, q[6].x, q[7].x));
                        *reinterpret_cast<uint2*>(qts + (colx + 1) * 128 + off) = make_uint2(
                            cvt_e4m3x4(q[0].y, q[1].y, q[2].y, q[3].y), cvt_e4m3x4(q[4].y, q[5].y, q[6].y, q[7].y));
                    } else {
                        static_assert(RPT == 8 || RPT == 4, "RPT");
                        const uint32_t off = uint32_t(((cw ^ l16) << 3) + hw * 4);
                        *reinterpret_cast<uint32_t*>(qts + colx * 128 + off) =
                            cvt_e4m3x4(q[0].x, q[1].x, q[2].x, q[3].x);
                        *reinterpret_cast<uint32_t*>(qts + (colx + 1) * 128 + off) =
                            cvt_e4m3x4(q[0].y, q[1].y, q[2].y, q[3].y);
                    }
                }
                named_bar<1, NCONS>();
                // copy-out: 128 columns x 16 chunks of 8 rows; thread u handles chunk (u & 15)
                // of columns (u >> 4) + k * NCONS / 16
                {
                    const int rc = tid & 15, colb = tid >> 4;
                    uint8_t* dst = p.qt + t.S * (NHALF * p.n) + (h * p.n + gcol0 + colb) * t.c + int64_t(t.T) * 128 + rc * 8;
                    const int64_t dstep = int64_t(NCONS / 16) * t.c;
                    const uint8_t* src = qts + colb * 128;
                    const int nvalid = t.valid - rc * 8;
                    if ((t.c & 7) == 0 && t.valid == 128) {
#pragma unroll
                        for (int k = 0; k < 2048 / NCONS; ++k) {
                            const int col = colb + k * (NCONS / 16);
                            *reinterpret_cast<uint2*>(dst) =
                                *reinterpret_cast<const uint2*>(src + k * (NCONS / 16) * 128 + ((rc ^ ((col >> 3) & 15)) << 3));
                            dst += dstep;
                        }
                    } else {
                        const bool vec = (t.c & 7) == 0 && nvalid >= 8;
                        for (int k = 0; k < 2048 / NCONS; ++k) {
                            const int col = colb + k * (NCONS / 16);
                            const uint2 val =
                                *reinterpret_cast<const uint2*>(src + k * (NCONS / 16) * 128 + ((rc ^ ((col >> 3) & 15)) << 3));
                            if (vec) {
                                *reinterpret_cast<uint2*>(dst) = val;
                            } else if (nvalid > 0) {
                                const uint64_t bits = (uint64_t(val.y) << 32) | val.x;
                                for (int b2 = 0; b2 < 8 && b2 < nvalid; ++b2) dst[b2] = uint8_t(bits >> (8 * b2));
                            }
                            dst += dstep;
                        }
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
template <int OP, typename InT, int MODE, bool EXACT, int RPT, int STAGES, int CTAS_PER_SM, bool WEIGHTED = false>
static int launch_tile(const TileParams& p, cudaStream_t stream) {
    using C = TileCfg<OP, InT, RPT, STAGES>;
    auto kern = tile_kernel<OP, InT, MODE, EXACT, RPT, STAGES, CTAS_PER_SM, WEIGHTED>;
    size_t smem = C::smem_bytes(p.E);
    if (smem > 227 * 1024) return fail_arg("too many experts for the shared-memory segment table (E=%d)", p.E);
    TileParams pp = p;
    pp.rt_cap = 0;
    if (p.counts != nullptr && p.E > 1 && p.E < 65536) {   // room for the row-tile -> expert table?
        const size_t budget = size_t(CTAS_PER_SM == 2 ? 113 : 227) * 1024;
        int64_t want = (p.M + 127) / 128 + p.E;
        if (smem + 16 < budget) {
            const int64_t fit = int64_t((budget - smem - 16) / 2);
            if (want > fit) want = 0;                       // does not fit: binary search per tile
            pp.rt_cap = int(want);
            smem += size_t(want) * 2 + 16;
        }
    }
    if (((p.M + 127) / 128 + p.E) * (p.n / 128) >= (int64_t(1) << 31)) return fail_arg("tensor too large: tile count exceeds 2^31");
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return int(e); }
    const int sms = sm_count();
    int64_t grid = int64_t(sms) * CTAS_PER_SM;
    if (p.counts == nullptr) {
        const int64_t tiles = ((p.M + 127) / 128) * (p.n / 128);
        if (tiles < grid) grid = tiles;
    }
    if (grid <= 0) return LH_OK;
    kern<<<dim3(unsigned(grid)), dim3(C::NTHREADS), smem, stream>>>(pp);
    return check_launch("tile_kernel");
}

// Fused variants (norm / SwiGLU producers) use the reciprocal-multiply quotient and the
// hardware ex2 / rcp approximations; the pure quantisers always use exact quotients.
#ifndef LH_FUSED_EXACT
#define LH_FUSED_EXACT false
#endif

// ---- fused producers, one instantiation set per input type -------------------------------------
// 16-bit inputs: two (norm) / one (SwiGLU) CTAs per SM with 2-3 stages; float32 tiles are twice as
// large, so the SwiGLU variants run with a single stage (correct, not tuned: float32 activations
// are not what the fused path sees in training).
template <typename InT>
struct FusedCfg {
    static constexpr bool WIDE = sizeof(InT) == 4;
    static constexpr int NORM_CPS = WIDE ? 1 : 2;
    static constexpr int SILU_F_STAGES = WIDE ? 1 : 3;
    static constexpr int SILU_B_STAGES = WIDE ? 1 : 2;
};

// y = (x * r) * gamma with known 1/rms per row; ALL_MODES = false instantiates only the
// transposed-output kernel (the bfloat16 row-wise outputs come from the streaming kernels)
template <typename InT, bool ALL_MODES>
static int tile_norm_t(const void* x, const void* gamma, const float* r, int dtype, int64_t M, int64_t n, void* q,
                       float* s, void* qt, float* st, int round_scale, int mode, cudaStream_t stream, int descending = 0) {
    TileParams p{};
    if (int rc = make_tensor_map(&p.tmap[0], x, dtype, uint64_t(M), uint64_t(n), uint64_t(n) * sizeof(InT), 128, 128)) return rc;
    p.r = r; p.gamma = gamma; p.E = 1; p.M = M; p.n = n; p.descending = descending;
    p.q = static_cast<uint8_t*>(q); p.s = s; p.qt = static_cast<uint8_t*>(qt); p.st = st; p.round_scale = round_scale;
    constexpr int CPS = FusedCfg<InT>::NORM_CPS;
    if (mode == MODE_COL) return launch_tile<OP_NORM, InT, MODE_COL, LH_FUSED_EXACT, 8, 2, CPS>(p, stream);
    if constexpr (ALL_MODES) {
        if (mode == MODE_ROW) return launch_tile<OP_NORM, InT, MODE_ROW, LH_FUSED_EXACT, 8, 2, CPS>(p, stream);
        if (mode == MODE_BOTH) return launch_tile<OP_NORM, InT, MODE_BOTH, LH_FUSED_EXACT, 8, 2, CPS>(p, stream);
    }
    return fail_arg("rmsnorm_blockquant_fwd: output_mode %d not available for this input type", mode);
}

template <typename InT>
static int tile_silu_fwd_t(const void* x, const void* w, int w_dtype, int dtype, const void* counts, int counts_type,
                           int E, int64_t M, int64_t n, void* q, float* s, void* qt, float* st, int round_scale,
                           int mode, cudaStream_t stream) {
    TileParams p{};
    if (int rc = make_tensor_map(&p.tmap[0], x, dtype, uint64_t(M), uint64_t(2 * n), uint64_t(2 * n) * sizeof(InT), 128, 128)) return rc;
    p.w = w; p.w_dtype = w_dtype;
    p.counts = counts; p.counts_i64 = counts_type == LH_I64; p.E = counts ? E : 1;
    p.M = M; p.n = n;
    p.q = static_cast<uint8_t*>(q); p.s = s; p.qt = static_cast<uint8_t*>(qt); p.st = st;
    p.round_scale = round_scale;
    constexpr int ST = FusedCfg<InT>::SILU_F_STAGES;
    if (w != nullptr) {
        switch (mode) {
            case MODE_ROW: return launch_tile<OP_SILU_F, InT, MODE_ROW, LH_FUSED_EXACT, 4, ST, 1, true>(p, stream);
            case MODE_COL: return launch_tile<OP_SILU_F, InT, MODE_COL, LH_FUSED_EXACT, 4, ST, 1, true>(p, stream);
            case MODE_BOTH: return launch_tile<OP_SILU_F, InT, MODE_BOTH, LH_FUSED_EXACT, 4, ST, 1, true>(p, stream);
        }
    } else {
        switch (mode) {
            case MODE_ROW: return launch_tile<OP_SILU_F, InT, MODE_ROW, LH_FUSED_EXACT, 4, ST, 1, false>(p, stream);
            case MODE_COL: return launch_tile<OP_SILU_F, InT, MODE_COL, LH_FUSED_EXACT, 4, ST, 1, false>(p, stream);
            case MODE_BOTH: return launch_tile<OP_SILU_F, InT, MODE_BOTH, LH_FUSED_EXACT, 4, ST, 1, false>(p, stream);
        }
    }
    return fail_arg("output_mode must be 0, 1 or 2");
}

template <typename InT>
static int tile_silu_bwd_t(const void* g, const void* x, const void* w, int w_dtype, int dtype, const void* counts,
                           int counts_type, int E, int64_t M, int64_t n, void* dx_q, float* dx_s, void* dx_qt,
                           float* dx_st, void* hp, float* dws, int round_scale, cudaStream_t stream) {
    TileParams p{};
    if (int rc = make_tensor_map(&p.tmap[0], g, dtype, uint64_t(M), uint64_t(n), uint64_t(n) * sizeof(InT), 128, 128)) return rc;
    if (int rc = make_tensor_map(&p.tmap[1], x, dtype, uint64_t(M), uint64_t(2 * n), uint64_t(2 * n) * sizeof(InT), 128, 128)) return rc;
    p.w = w; p.w_dtype = w_dtype;
    p.counts = counts; p.counts_i64 = counts_type == LH_I64; p.E = counts ? E : 1;
    p.M = M; p.n = n;
    p.q = static_cast<uint8_t*>(dx_q); p.s = dx_s; p.qt = static_cast<uint8_t*>(dx_qt); p.st = dx_st;
    p.hp = hp; p.dws = dws; p.round_scale = round_scale;
    constexpr int ST = FusedCfg<InT>::SILU_B_STAGES;
    if (w != nullptr) return launch_tile<OP_SILU_B, InT, MODE_BOTH, LH_FUSED_EXACT, 4, ST, 1, true>(p, stream);
    return launch_tile<OP_SILU_B, InT, MODE_BOTH, LH_FUSED_EXACT, 4, ST, 1, false>(p, stream);
}

}  // namespace lh
