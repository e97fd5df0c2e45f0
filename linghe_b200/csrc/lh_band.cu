// Single-pass both-axes kernel: RMSNorm forward + row-wise AND column-wise FP8 quantisation with
// x read from HBM exactly once.
//
// Every output of a row needs the row's sum of squares, while a column block needs 128 rows.  The
// unit of work is a 128-row band of x.  A band (128 * n * 2 bytes, 2 MB at n = 8192) is shared by
// the C CTAs of a thread-block cluster, CTA r taking the 128 x 128 tiles r, r + C, ... of the band,
// and is processed in two passes:
//   pass A  the CTA streams its tiles through shared memory (TMA tensor copies) and adds up, per
//           row, the squares of its columns; the 128 partial sums go to every CTA of the cluster
//           through distributed shared memory, one cluster barrier makes them visible, and every
//           CTA adds the C partials in rank order (deterministic) to get 1/rms of the 128 rows;
//   pass B  the CTA streams the same tiles again and produces all four outputs of each (row codes /
//           scales, transposed codes / scales).  The second read is served by L2: the clusters in
//           flight hold (clusters x band) bytes, and C is chosen so that this stays a fraction of
//           the 126 MB L2, so HBM sees x once.
// The exchange costs one cluster barrier per band and CTA (under a microsecond against tens of
// microseconds of work), no scratch memory and no inter-CTA polling.
//
// A CTA is 16 warps in two groups of eight (8 rows x 8 columns per thread, as in the tile kernels).
// The groups take alternate tiles and synchronise only within themselves, so one group computes
// while the other waits at a barrier.  Each group owns three of the six tile buffers; its first
// thread refills the buffer the group has just left with the tile three of its own operations
// ahead -- across the A/B boundary and into the next band, so the rings never drain.  The
// transposed codes are staged in the tile's own buffer once the tile is in registers.
// Every mbarrier wait is bounded and reports through the device status word; the cluster barrier
// is reached by every thread of the cluster unconditionally.
// No tensor cores: the path is bound by HBM and by instruction issue, not by arithmetic.
#include "lh_tile.cuh"

namespace lh {

namespace {

constexpr int kComputeWarps = 16;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kBandThreads = kComputeThreads;
constexpr int kGroupThreads = 256;
constexpr int kTileBytes = 128 * 128 * 2;
constexpr int kSlots = 6;
constexpr int kMaxCluster = 8;

struct BandParams {
    CUtensorMap tmap_x;     // x [M, n] bf16, box 128 x 128
    const uint8_t* gamma;   // [n] bf16
    float eps, inv_n;
    int64_t M;
    int n;
    int S;                  // tiles per band = n / 128
    int bands;
    uint8_t* q;             // [M, n]
    float* s;               // [n/128, M]
    float* rms;             // [M]
    uint8_t* qt;            // [n, M]
    float* st;              // [ceil(M/128), n]
    int round_scale;
};

struct BandCfg {
    static constexpr int OFF_PART = kSlots * kTileBytes;          // [2 groups][8][128] column maxima
    static constexpr int OFF_CS = OFF_PART + 2 * 8 * 128 * 4;     // [2][128] column scale
    static constexpr int OFF_CY = OFF_CS + 2 * 512;               // [2][128] 1/scale
    static constexpr int OFF_RSUM = OFF_CY + 2 * 512;             // [2 groups][128] row sums of this CTA's tiles
    static constexpr int OFF_RINV = OFF_RSUM + 2 * 512;           // [128] 1/rms of the band's rows
    static constexpr int OFF_PEER = OFF_RINV + 512;               // [2 parities][kMaxCluster][128] partials of every rank
    static constexpr int OFF_BAR = OFF_PEER + 2 * kMaxCluster * 512;   // full[6], empty[6]
    static constexpr int SMEM = OFF_BAR + 2 * kSlots * 8 + 16;
};

// sum over the 16 lanes that share a tile row, for eight rows at once (transposing butterfly);
// on return lane l16 holds the sum of row (l16 >> 1)
__device__ __forceinline__ float row_sum_transposed8(float* a, int l16) {
    {
        const bool up = (l16 & 8) != 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float recv = __shfl_xor_sync(0xffffffffu, up ? a[i] : a[i + 4], 8);
            a[i] = (up ? a[i + 4] : a[i]) + recv;
        }
    }
    {
        const bool up = (l16 & 4) != 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float recv = __shfl_xor_sync(0xffffffffu, up ? a[i] : a[i + 2], 4);
            a[i] = (up ? a[i + 2] : a[i]) + recv;
        }
    }
    {
        const bool up = (l16 & 2) != 0;
        const float recv = __shfl_xor_sync(0xffffffffu, up ? a[0] : a[1], 2);
        a[0] = (up ? a[1] : a[0]) + recv;
    }
    a[0] += __shfl_xor_sync(0xffffffffu, a[0], 1);
    return a[0];
}

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_nctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// store a float into the shared memory of CTA `rank` of the cluster, at the address `local` has in this CTA
__device__ __forceinline__ void st_cluster_f32(const float* local, uint32_t rank, float v) {
    uint32_t raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(raddr), "f"(v) : "memory");
}

__global__ void __launch_bounds__(kBandThreads, 1)
band_norm_fwd_kernel(const __grid_constant__ BandParams p) {
    using C = BandCfg;
    constexpr int RPT = 8, GW = 8, NG = kGroupThreads;
    extern __shared__ __align__(128) uint8_t smem[];
    float* rsum = reinterpret_cast<float*>(smem + C::OFF_RSUM);
    float* rinv = reinterpret_cast<float*>(smem + C::OFF_RINV);
    float* peer = reinterpret_cast<float*>(smem + C::OFF_PEER);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty = full + kSlots;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int CS = int(cluster_nctarank()), rank = int(cluster_ctarank());
    const int S = p.S;
    const int cluster_id = int(blockIdx.x) / CS, nclusters = int(gridDim.x) / CS;
    const int Tc = (S - rank + CS - 1) / CS;          // tiles of this CTA in every band: rank, rank + CS, ...
    // bands of this cluster: cluster_id, cluster_id + nclusters, ...
    const int nbands = cluster_id < p.bands ? (p.bands - cluster_id + nclusters - 1) / nclusters : 0;

    if (tid == 0) {
        for (int i = 0; i < kSlots; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], GW); }
        mbar_fence_init();
        tma_prefetch_desc(&p.tmap_x);
    }
    __syncthreads();
    // every CTA of the cluster has its barriers and buffers before any peer writes into them
    cluster_arrive();
    cluster_wait();

    bool dead = false;   // a bounded wait of this thread gave up: later waits are skipped (see mbar_wait_or_mark)

    // Operation n of this CTA (counted over all its bands): band index n / (2 Tc), then pass A over the
    // Tc tiles, then pass B over them; consumed by group n & 1 from buffer n % 6 (so group g cycles
    // through the buffers g, g + 2, g + 4).
    const int g = warp >> 3, gw = warp & 7, gtid = tid & (NG - 1);
    const int hw = lane >> 4, l16 = lane & 15;
    const int row0 = gw * (2 * RPT) + hw * RPT;
    const bool rs = p.round_scale != 0;
    float* part = reinterpret_cast<float*>(smem + C::OFF_PART) + g * GW * 128;
    float* cs = reinterpret_cast<float*>(smem + C::OFF_CS) + g * 128;
    float* cy = reinterpret_cast<float*>(smem + C::OFF_CY) + g * 128;
    auto group_bar = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + g), "n"(NG) : "memory"); };
    auto compute_bar = [&]() { asm volatile("bar.sync 3, %0;" ::"n"(kComputeThreads) : "memory"); };

    // The operations of this CTA, band after band: pass A over its Tc tiles, then pass B over them.  The
    // groups take alternate operations (2 Tc is even, so group g has the tiles o = g, g + 2, ... of pass A
    // and o = g ^ (Tc & 1), ... of pass B) and each group runs through its own three buffers g, g + 2, g + 4.
    struct Cursor {
        int bi, pass, o;
    };
    auto settle = [&](Cursor& c) {   // skip passes in which the group has no tile
        while (c.o >= Tc && c.bi < nbands) {
            if (c.pass == 0) { c.pass = 1; c.o = g ^ (Tc & 1); }
            else { c.pass = 0; ++c.bi; c.o = g; }
        }
    };
    auto advance = [&](Cursor& c) { c.o += 2; settle(c); };
    auto issue = [&](const Cursor& c, int slot) {   // first thread of the group: one tile into a buffer
        const int b = cluster_id + c.bi * nclusters;
        const int ct = rank + c.o * CS;
        mbar_expect_tx(&full[slot], uint32_t(kTileBytes));
        tma_load_2d(smem + size_t(slot) * kTileBytes, &p.tmap_x, ct * 128, b * 128, &full[slot]);
    };
    Cursor pc{0, 0, g};          // the next operation to load
    settle(pc);
    if (gtid == 0) {
        for (int k = 0; k < 3 && pc.bi < nbands; ++k) { issue(pc, 2 * k + g); advance(pc); }
    } else {
        for (int k = 0; k < 3 && pc.bi < nbands; ++k) advance(pc);
    }
    int js = 0;                  // buffer index of the current operation inside the group's ring (0..2)
    uint32_t jph = 0;            // phase parity of that buffer
    bool first_op = true;
    // start of an operation: the group's first thread refills the buffer of the group's previous operation
    // (released by every warp of the group, or about to be) with the operation three ahead
    auto begin_op = [&]() -> int {
        if (!first_op && pc.bi < nbands) {
            if (gtid == 0) {
                const int prev = js == 0 ? 2 : js - 1;
                mbar_wait_or_mark<false>(&empty[2 * prev + g], js == 0 ? (jph ^ 1u) : jph, DEVERR_EMPTY_WAIT, dead);
                if (!dead) issue(pc, 2 * prev + g);
            }
            advance(pc);
        }
        first_op = false;
        const int slot = 2 * js + g;
        mbar_wait_or_mark<true>(&full[slot], jph, DEVERR_FULL_WAIT, dead);
        return slot;
    };
    auto end_op = [&](int slot) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
        if (++js == 3) { js = 0; jph ^= 1u; }
    };

    Cursor c{0, 0, g};
    settle(c);
    for (int bi = 0; bi < nbands; ++bi) {
        const int b = cluster_id + bi * nclusters;
        const int par = bi & 1;
        // ---------------- pass A: row sums of squares over this group's tiles ----------------
        float a[RPT];
#pragma unroll
        for (int s = 0; s < RPT; ++s) a[s] = 0.f;
        while (c.bi == bi && c.pass == 0) {
            const int slot = begin_op();
            const uint8_t* base = smem + size_t(slot) * kTileBytes + row0 * 256 + l16 * 16;
#pragma unroll
            for (int s = 0; s < RPT; ++s) {
                const uint4 raw = *reinterpret_cast<const uint4*>(base + s * 256);
                const float2 v0 = bf16x2_to_f2(raw.x), v1 = bf16x2_to_f2(raw.y);
                const float2 v2 = bf16x2_to_f2(raw.z), v3 = bf16x2_to_f2(raw.w);
                float2 acc = mul2(v0, v0);
                acc = fma2(v1, v1, acc); acc = fma2(v2, v2, acc); acc = fma2(v3, v3, acc);
                a[s] += acc.x + acc.y;
            }
            end_op(slot);
            advance(c);
        }
        {
            const float tot = row_sum_transposed8(a, l16);
            if ((l16 & 1) == 0) rsum[g * 128 + row0 + (l16 >> 1)] = tot;
        }
        // gamma of the group's first pass-B tile: in flight across the exchange (each later tile's gamma is
        // fetched one tile ahead), so that no tile waits for a global load
        uint4 gnext = make_uint4(0, 0, 0, 0);
        if (c.bi == bi && c.pass == 1)
            gnext = __ldg(reinterpret_cast<const uint4*>(p.gamma + (rank + c.o * CS) * 256 + l16 * 16));
        __syncthreads();
        if (tid < 128) {
            const float mine = rsum[tid] + rsum[128 + tid];
            for (int r = 0; r < CS; ++r) st_cluster_f32(peer + (par * kMaxCluster + rank) * 128 + tid, uint32_t(r), mine);
        }
        cluster_arrive();
        cluster_wait();
        if (tid < 128) {
            float tot = 0.f;
            for (int r = 0; r < CS; ++r) tot += peer[(par * kMaxCluster + r) * 128 + tid];
            const float r1 = rsqrt_nr(fmaf(tot, p.inv_n, p.eps));
            const int64_t grow = int64_t(b) * 128 + tid;
            const bool in = grow < p.M;
            rinv[tid] = in ? r1 : 0.f;           // rows past the end of the matrix count as zeros
            if (rank == 0 && in) p.rms[grow] = r1;
        }
        __syncthreads();
        // ---------------- pass B: all four outputs of this group's tiles ----------------
        const int64_t grow0 = int64_t(b) * 128;
        const int64_t left = p.M - grow0;
        const int valid = left < 128 ? int(left) : 128;
        const int nrows = valid - row0;
        // per-band bases of this thread's outputs; a tile adds its column offset
        uint8_t* const q_band = p.q + (grow0 + row0) * p.n + l16 * 8;
        float* const s_band = p.s + grow0 + row0 + (l16 >> 1);
        uint8_t* const qt_band = p.qt + int64_t(gtid >> 4) * p.M + grow0 + (gtid & 15) * 8;
        float* const st_band = p.st + int64_t(b) * p.n + gtid;
        float ri[RPT];
        {
            const float4 ra = *reinterpret_cast<const float4*>(rinv + row0);
            const float4 rb = *reinterpret_cast<const float4*>(rinv + row0 + 4);
            ri[0] = ra.x; ri[1] = ra.y; ri[2] = ra.z; ri[3] = ra.w; ri[4] = rb.x; ri[5] = rb.y; ri[6] = rb.z; ri[7] = rb.w;
        }
        while (c.bi == bi && c.pass == 1) {
            const int slot = begin_op();
            const int ct = rank + c.o * CS;
            uint8_t* tile = smem + size_t(slot) * kTileBytes;
            uint8_t* qts = tile;                 // reused once the tile is in registers
            const int gcol0 = ct * 128;
            float2 v[RPT][4];
            {
                const float2 gam[4] = {bf16x2_to_f2(gnext.x), bf16x2_to_f2(gnext.y), bf16x2_to_f2(gnext.z), bf16x2_to_f2(gnext.w)};
                if (c.o + 2 < Tc) gnext = __ldg(reinterpret_cast<const uint4*>(p.gamma + (ct + 2 * CS) * 256 + l16 * 16));
#pragma unroll
                for (int s = 0; s < RPT; ++s) {
                    float2 x[4];
                    load8p<__nv_bfloat16>(tile + (row0 + s) * 256, l16, x);
                    const float2 r2 = splat2(ri[s]);   // 0 for rows past the end of the matrix
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[s][j] = mul2(mul2(x[j], r2), gam[j]);
                }
            }
            // ---- row-wise 1x128 ----
            {
                constexpr int G = 16 / RPT;
                float am[RPT];
#pragma unroll
                for (int s = 0; s < RPT; ++s) {
                    float m = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) m = max3abs(v[s][j].x, v[s][j].y, m);
                    am[s] = m;
                }
                const float mymax = row_max_transposed<RPT>(am, l16);
                const float mysc = scale_from_amax(mymax, rs);
                const float myy = rcp_approx(mysc);
                if ((l16 % G) == 0 && row0 + l16 / G < valid) s_band[int64_t(ct) * p.M] = mysc;
                uint8_t* qrow = q_band + gcol0;
                if (nrows >= RPT) {   // every row of this thread exists (always, except in a ragged last band)
#pragma unroll
                    for (int s = 0; s < RPT; ++s) {
                        const float y = __shfl_sync(0xffffffffu, myy, s * G, 16);
                        const uint2 codes = quant_row8<false, false>(v[s], 0.f, y);
                        *reinterpret_cast<uint2*>(qrow) = codes;
                        qrow += p.n;
                    }
                } else {
#pragma unroll
                    for (int s = 0; s < RPT; ++s) {
                        const float y = __shfl_sync(0xffffffffu, myy, s * G, 16);
                        const uint2 codes = quant_row8<false, false>(v[s], 0.f, y);
                        if (s < nrows) *reinterpret_cast<uint2*>(qrow) = codes;
                        qrow += p.n;
                    }
                }
            }
            // ---- column-wise 128x1, transposed ----
            float2 cm[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float mx = 0.f, my = 0.f;
#pragma unroll
                for (int s = 0; s < RPT; s += 2) {
                    mx = max3abs(v[s][j].x, v[s + 1][j].x, mx);
                    my = max3abs(v[s][j].y, v[s + 1][j].y, my);
                }
                cm[j].x = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                cm[j].y = fmaxf(my, __shfl_xor_sync(0xffffffffu, my, 16));
            }
            if (hw == 0) {
                float4* dst = reinterpret_cast<float4*>(part + gw * 128 + l16 * 8);
                dst[0] = make_float4(cm[0].x, cm[0].y, cm[1].x, cm[1].y);
                dst[1] = make_float4(cm[2].x, cm[2].y, cm[3].x, cm[3].y);
            }
            group_bar();   // every thread of the group has its tile values in registers: the tile buffer is free
            if (gtid < 128) {
                float m = part[gtid];
#pragma unroll
                for (int w2 = 1; w2 < GW; ++w2) m = fmaxf(m, part[w2 * 128 + gtid]);
                const float sc = scale_from_amax(m, rs);
                cs[gtid] = sc;
                cy[gtid] = rcp_approx(sc);
                st_band[gcol0] = sc;
            }
            group_bar();
            float2 y2[4];
            {
                const float4 c0 = *reinterpret_cast<const float4*>(cy + l16 * 8);
                const float4 c1 = *reinterpret_cast<const float4*>(cy + l16 * 8 + 4);
                y2[0] = make_float2(c0.x, c0.y); y2[1] = make_float2(c0.z, c0.w);
                y2[2] = make_float2(c1.x, c1.y); y2[3] = make_float2(c1.z, c1.w);
            }
            {
                uint8_t* qw = qts + (l16 * 8) * 128 + (((gw * 2 + hw) ^ l16) << 3);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 qv[RPT];
#pragma unroll
                    for (int s = 0; s < RPT; ++s) qv[s] = mul2(v[s][j], y2[j]);
                    *reinterpret_cast<uint2*>(qw + (2 * j) * 128) = make_uint2(
                        cvt_e4m3x4(qv[0].x, qv[1].x, qv[2].x, qv[3].x), cvt_e4m3x4(qv[4].x, qv[5].x, qv[6].x, qv[7].x));
                    *reinterpret_cast<uint2*>(qw + (2 * j + 1) * 128) = make_uint2(
                        cvt_e4m3x4(qv[0].y, qv[1].y, qv[2].y, qv[3].y), cvt_e4m3x4(qv[4].y, qv[5].y, qv[6].y, qv[7].y));
                }
            }
            group_bar();
            // copy-out: 128 columns x 16 chunks of 8 rows; thread u handles chunk (u & 15) of columns (u >> 4) + 16 k
            {
                const int rc = gtid & 15, colb = gtid >> 4;
                uint8_t* dst = qt_band + int64_t(gcol0) * p.M;
                const int64_t dstep = int64_t(NG / 16) * p.M;
                const uint8_t* src = qts + colb * 128;
                const int nvalid = valid - rc * 8;
                if ((p.M & 7) == 0 && valid == 128) {   // the common case, free of per-store tests
                    uint2 val[2048 / NG];
#pragma unroll
                    for (int kk = 0; kk < 2048 / NG; ++kk) {
                        const int col = colb + kk * (NG / 16);
                        val[kk] = *reinterpret_cast<const uint2*>(src + kk * (NG / 16) * 128 + ((rc ^ ((col >> 3) & 15)) << 3));
                    }
#pragma unroll
                    for (int kk = 0; kk < 2048 / NG; ++kk) {
                        *reinterpret_cast<uint2*>(dst) = val[kk];
                        dst += dstep;
                    }
                } else {
                    const bool vec = (p.M & 7) == 0 && nvalid >= 8;
                    for (int kk = 0; kk < 2048 / NG; ++kk) {
                        const int col = colb + kk * (NG / 16);
                        const uint2 val = *reinterpret_cast<const uint2*>(src + kk * (NG / 16) * 128 + ((rc ^ ((col >> 3) & 15)) << 3));
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
            fence_async_smem();   // the buffer's next writer is a TMA copy
            end_op(slot);
            advance(c);
        }
        // No barrier here: rsum and rinv are rewritten only behind the next band's barriers, which no
        // thread passes before every compute thread has finished this pass.
    }
}

// ------------------------------------------------------------------------------------------------
// RMSNorm backward + dual-axis quantisation of dy, x and dy read from HBM exactly once.
//
// Same band / cluster / two-pass scheme as the forward kernel, with a pair of tiles (x, dy) per
// operation:
//   pass A  per row, sum x * dy * gamma and (unless 1/rms is given) sum x^2 over the CTA's columns;
//           exchanged through distributed shared memory, one cluster barrier per band;
//   pass B  dx = r * dy * gamma - r^3 * x * sum(x dy gamma) / n (input type), this band's dgamma
//           contribution of the tile's 128 columns (to a scratch row per band, added over the bands
//           in a fixed order by the reduction kernel that follows), and the row-wise and transposed
//           FP8 copies of dy -- bit-exact against the plain quantiser: exact quotients on negated
//           values, as in the tile kernels.
// A tile pair is 64 KB, so the ring holds three of them and the CTA works as one group of 16
// warps (4 rows x 8 columns per thread and operand); its first thread refills the buffer the CTA
// has just left.
// ------------------------------------------------------------------------------------------------
constexpr int kPairBytes = 2 * kTileBytes;
constexpr int kBwdSlots = 3;

struct BandBwdParams {
    CUtensorMap tmap_x, tmap_dy;   // [M, n] bf16, box 128 x 128
    const uint8_t* gamma;          // [n] bf16
    const float* rms;              // [M] 1/rms or NULL (recomputed)
    float eps, inv_n;
    int64_t M;
    int n;
    int S;                         // tiles per band
    int bands;
    uint8_t* dx;                   // [M, n] bf16
    float* dgamma_partial;         // [bands][n]
    uint8_t* q;                    // dy codes [M, n]
    float* s;                      // [n/128, M]
    uint8_t* qt;                   // [n, M]
    float* st;                     // [ceil(M/128), n]
    int round_scale;
};

struct BandBwdCfg {
    static constexpr int OFF_PART = kBwdSlots * kPairBytes;       // [16][128] column maxima of dy
    static constexpr int OFF_DPART = OFF_PART + 16 * 128 * 4;     // [16][128] dgamma sub-sums
    static constexpr int OFF_CS = OFF_DPART + 16 * 128 * 4;       // [128] column scale
    static constexpr int OFF_CY = OFF_CS + 512;                   // [128] -1/scale (or the IEEE-division marker)
    static constexpr int OFF_RSUM = OFF_PART;                     // [2][128] this CTA's row sums: x dy gamma, x^2 (pass A only, shares `part`)
    static constexpr int OFF_RINV = OFF_CY + 512;                 // [128] -1/rms
    static constexpr int OFF_NCOEF = OFF_RINV + 512;              // [128] -r^3 c / n
    static constexpr int OFF_PEER = OFF_NCOEF + 512;              // [2 parities][kMaxCluster][2][128]
    static constexpr int OFF_BAR = OFF_PEER + 2 * kMaxCluster * 2 * 512;   // full[3], empty[3]
    static constexpr int SMEM = OFF_BAR + 2 * kBwdSlots * 8 + 16;
    static_assert(SMEM <= 227 * 1024, "shared memory of the backward band kernel");
};

__device__ __forceinline__ float row_sum_transposed4(float* a, int l16) {
    {
        const bool up = (l16 & 8) != 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float recv = __shfl_xor_sync(0xffffffffu, up ? a[i] : a[i + 2], 8);
            a[i] = (up ? a[i + 2] : a[i]) + recv;
        }
    }
    {
        const bool up = (l16 & 4) != 0;
        const float recv = __shfl_xor_sync(0xffffffffu, up ? a[0] : a[1], 4);
        a[0] = (up ? a[1] : a[0]) + recv;
    }
    a[0] += __shfl_xor_sync(0xffffffffu, a[0], 2);
    a[0] += __shfl_xor_sync(0xffffffffu, a[0], 1);
    return a[0];
}

__global__ void __launch_bounds__(kBandThreads, 1)
band_norm_bwd_kernel(const __grid_constant__ BandBwdParams p) {
    using C = BandBwdCfg;
    constexpr int RPT = 4, NW = kComputeWarps, NT = kBandThreads;
    extern __shared__ __align__(128) uint8_t smem[];
    float* part = reinterpret_cast<float*>(smem + C::OFF_PART);
    float* dpart = reinterpret_cast<float*>(smem + C::OFF_DPART);
    float* cs = reinterpret_cast<float*>(smem + C::OFF_CS);
    float* cy = reinterpret_cast<float*>(smem + C::OFF_CY);
    float* rsum = reinterpret_cast<float*>(smem + C::OFF_RSUM);
    float* nrinv = reinterpret_cast<float*>(smem + C::OFF_RINV);
    float* ncoef = reinterpret_cast<float*>(smem + C::OFF_NCOEF);
    float* peer = reinterpret_cast<float*>(smem + C::OFF_PEER);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty = full + kBwdSlots;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hw = lane >> 4, l16 = lane & 15;
    const int row0 = warp * (2 * RPT) + hw * RPT;
    const int CS = int(cluster_nctarank()), rank = int(cluster_ctarank());
    const int S = p.S;
    const int cluster_id = int(blockIdx.x) / CS, nclusters = int(gridDim.x) / CS;
    const int Tc = (S - rank + CS - 1) / CS;
    const int nbands = cluster_id < p.bands ? (p.bands - cluster_id + nclusters - 1) / nclusters : 0;
    const bool rs = p.round_scale != 0;
    const bool have_rms = p.rms != nullptr;

    if (tid == 0) {
        for (int i = 0; i < kBwdSlots; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], NW); }
        mbar_fence_init();
        tma_prefetch_desc(&p.tmap_x);
        tma_prefetch_desc(&p.tmap_dy);
    }
    __syncthreads();
    cluster_arrive();
    cluster_wait();

    bool dead = false;   // a bounded wait of this thread gave up: later waits are skipped (see mbar_wait_or_mark)
    const int64_t total_ops = int64_t(nbands) * 2 * Tc;
    auto issue = [&](int64_t n) {   // thread 0: the tile pair of operation n into its buffer
        if (n >= total_ops) return;
        const int64_t bi = n / (2 * Tc);
        const int o = int(n - bi * 2 * Tc);
        const int b = cluster_id + int(bi) * nclusters;
        const int ct = rank + (o % Tc) * CS;
        const int slot = int(n % kBwdSlots);
        uint8_t* dst = smem + size_t(slot) * kPairBytes;
        mbar_expect_tx(&full[slot], uint32_t(kPairBytes));
        tma_load_2d(dst, &p.tmap_x, ct * 128, b * 128, &full[slot]);
        tma_load_2d(dst + kTileBytes, &p.tmap_dy, ct * 128, b * 128, &full[slot]);
    };
    // at the start of operation n thread 0 refills the buffer of operation n - 1 with operation n + 2
    auto refill = [&](int64_t n) {
        if (tid == 0 && n >= 1 && n + 2 < total_ops) {
            const int64_t prev = n - 1;
            mbar_wait_or_mark<false>(&empty[prev % kBwdSlots], uint32_t((prev / kBwdSlots) & 1), DEVERR_EMPTY_WAIT, dead);
            if (!dead) issue(n + 2);
        }
    };
    if (tid == 0) { issue(0); issue(1); issue(2); }

    int64_t n = 0;
    for (int bi = 0; bi < nbands; ++bi) {
        const int b = cluster_id + bi * nclusters;
        const int par = bi & 1;
        const int64_t grow0 = int64_t(b) * 128;
        const int64_t left = p.M - grow0;
        const int valid = left < 128 ? int(left) : 128;
        const int nrows = valid - row0;
        // ---------------- pass A: per-row sums over this CTA's tiles ----------------
        float ac[RPT], as[RPT];
#pragma unroll
        for (int s = 0; s < RPT; ++s) { ac[s] = 0.f; as[s] = 0.f; }
        for (int o = 0; o < Tc; ++o, ++n) {
            refill(n);
            const int slot = int(n % kBwdSlots);
            const int ct = rank + o * CS;
            mbar_wait_or_mark<true>(&full[slot], uint32_t((n / kBwdSlots) & 1), DEVERR_FULL_WAIT, dead);
            const uint8_t* tx = smem + size_t(slot) * kPairBytes + row0 * 256;
            float2 gam[4];
            load8p<__nv_bfloat16>(p.gamma + int64_t(ct) * 256, l16, gam);
#pragma unroll
            for (int s = 0; s < RPT; ++s) {
                float2 x[4], d[4];
                load8p<__nv_bfloat16>(tx + s * 256, l16, x);
                load8p<__nv_bfloat16>(tx + kTileBytes + s * 256, l16, d);
                float2 c2 = mul2(x[0], mul2(d[0], gam[0]));
                float2 s2 = mul2(x[0], x[0]);
#pragma unroll
                for (int j = 1; j < 4; ++j) {
                    c2 = fma2(x[j], mul2(d[j], gam[j]), c2);
                    s2 = fma2(x[j], x[j], s2);
                }
                ac[s] += c2.x + c2.y;
                as[s] += s2.x + s2.y;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
        }
        {
            const float tc = row_sum_transposed4(ac, l16);
            const float ts = row_sum_transposed4(as, l16);
            if ((l16 & 3) == 0) { rsum[row0 + (l16 >> 2)] = tc; rsum[128 + row0 + (l16 >> 2)] = ts; }
        }
        __syncthreads();
        if (tid < 256) {   // 0..127: sum x dy gamma, 128..255: sum x^2
            const float mine = rsum[tid];
            for (int r = 0; r < CS; ++r) st_cluster_f32(peer + ((par * kMaxCluster + rank) * 2) * 128 + tid, uint32_t(r), mine);
        }
        cluster_arrive();
        cluster_wait();
        if (tid < 128) {
            float tc = 0.f, ts = 0.f;
            for (int r = 0; r < CS; ++r) {
                tc += peer[((par * kMaxCluster + r) * 2) * 128 + tid];
                ts += peer[((par * kMaxCluster + r) * 2 + 1) * 128 + tid];
            }
            const int64_t grow = grow0 + tid;
            float r1 = 0.f;
            if (grow < p.M) r1 = have_rms ? p.rms[grow] : rsqrt_nr(fmaf(ts, p.inv_n, p.eps));
            nrinv[tid] = -r1;
            ncoef[tid] = -(r1 * r1 * r1 * tc * p.inv_n);
        }
        __syncthreads();
        // ---------------- pass B: dx, dgamma contribution, dy codes on both axes ----------------
        for (int o = 0; o < Tc; ++o, ++n) {
            refill(n);
            const int slot = int(n % kBwdSlots);
            const int ct = rank + o * CS;
            const int64_t gcol0 = int64_t(ct) * 128;
            mbar_wait_or_mark<true>(&full[slot], uint32_t((n / kBwdSlots) & 1), DEVERR_FULL_WAIT, dead);
            uint8_t* tile = smem + size_t(slot) * kPairBytes;
            uint8_t* qts = tile;                 // reused once both tiles are in registers
            float2 x[RPT][4], nd[RPT][4];        // x and the NEGATED dy
            float2 gam[4];
            load8p<__nv_bfloat16>(p.gamma + gcol0 * 2, l16, gam);
#pragma unroll
            for (int s = 0; s < RPT; ++s) {
                load8p<__nv_bfloat16>(tile + (row0 + s) * 256, l16, x[s]);
                load8p<__nv_bfloat16, true>(tile + kTileBytes + (row0 + s) * 256, l16, nd[s]);
            }
            // dx and the dgamma sub-sums of this thread's rows
            float2 dg[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) dg[j] = make_float2(0.f, 0.f);
            {
                const float4 nr4 = *reinterpret_cast<const float4*>(nrinv + row0);
                const float4 nc4 = *reinterpret_cast<const float4*>(ncoef + row0);
                const float nr[4] = {nr4.x, nr4.y, nr4.z, nr4.w}, nc[4] = {nc4.x, nc4.y, nc4.z, nc4.w};
                uint8_t* dxrow = p.dx + ((grow0 + row0) * p.n + gcol0 + l16 * 8) * 2;
#pragma unroll
                for (int s = 0; s < RPT; ++s) {
                    const float2 nr2 = splat2(nr[s]), nc2 = splat2(nc[s]);
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // dx = r g gamma - r^3 c/n x = (-r)(-g) gamma + ncoef x ; dgamma += x g r = x (-g) (-r)
                        const float2 d = fma2(nc2, x[s][j], mul2(nr2, mul2(nd[s][j], gam[j])));
                        dg[j] = fma2(mul2(x[s][j], nd[s][j]), nr2, dg[j]);
                        w[j] = pack_bf16x2(d.x, d.y);
                    }
                    if (s < nrows) *reinterpret_cast<uint4*>(dxrow) = make_uint4(w[0], w[1], w[2], w[3]);
                    dxrow += int64_t(p.n) * 2;
                }
            }
            // ---- row-wise 1x128 codes of dy (exact) ----
            {
                constexpr int G = 16 / RPT;
                float a[RPT];
#pragma unroll
                for (int s = 0; s < RPT; ++s) {
                    float m = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) m = max3abs(nd[s][j].x, nd[s][j].y, m);
                    a[s] = m;
                }
                const float mymax = row_max_transposed<RPT>(a, l16);
                const float mysc = scale_from_amax(mymax, rs);
                const float myy = scale_rcp<true>(mysc, mymax);
                const int rr = row0 + l16 / G;
                if ((l16 % G) == 0 && rr < valid) p.s[int64_t(ct) * p.M + grow0 + rr] = mysc;
                uint8_t* qrow = p.q + (grow0 + row0) * p.n + gcol0 + l16 * 8;
                auto row_pass = [&](auto check) {
#pragma unroll
                    for (int s = 0; s < RPT; ++s) {
                        const float sc = __shfl_sync(0xffffffffu, mysc, s * G, 16);
                        const float y = __shfl_sync(0xffffffffu, myy, s * G, 16);
                        const uint2 codes = quant_row8<true, true, decltype(check)::value>(nd[s], sc, y);
                        st_global_v2_if(s < nrows, qrow, codes.x, codes.y);
                        qrow += p.n;
                    }
                };
                if (__any_sync(0xffffffffu, myy > 0.f)) row_pass(std::true_type{});
                else row_pass(std::false_type{});
            }
            // ---- column maxima of dy and dgamma sub-sums through shared memory ----
            {
                float2 cm[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float mx = 0.f, my = 0.f;
#pragma unroll
                    for (int s = 0; s < RPT; s += 2) {
                        mx = max3abs(nd[s][j].x, nd[s + 1][j].x, mx);
                        my = max3abs(nd[s][j].y, nd[s + 1][j].y, my);
                    }
                    cm[j].x = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    cm[j].y = fmaxf(my, __shfl_xor_sync(0xffffffffu, my, 16));
                    dg[j].x += __shfl_xor_sync(0xffffffffu, dg[j].x, 16);
                    dg[j].y += __shfl_xor_sync(0xffffffffu, dg[j].y, 16);
                }
                if (hw == 0) {
                    float4* dst = reinterpret_cast<float4*>(part + warp * 128 + l16 * 8);
                    dst[0] = make_float4(cm[0].x, cm[0].y, cm[1].x, cm[1].y);
                    dst[1] = make_float4(cm[2].x, cm[2].y, cm[3].x, cm[3].y);
                    float4* dd = reinterpret_cast<float4*>(dpart + warp * 128 + l16 * 8);
                    dd[0] = make_float4(dg[0].x, dg[0].y, dg[1].x, dg[1].y);
                    dd[1] = make_float4(dg[2].x, dg[2].y, dg[3].x, dg[3].y);
                }
            }
            named_bar<1, NT>();   // every thread has both tiles in registers: the buffer is free for staging
            if (tid < 128) {
                float m = part[tid];
#pragma unroll
                for (int w2 = 1; w2 < NW; ++w2) m = fmaxf(m, part[w2 * 128 + tid]);
                const float sc = scale_from_amax(m, rs);
                cs[tid] = sc;
                cy[tid] = scale_rcp<true>(sc, m);
                p.st[int64_t(b) * p.n + gcol0 + tid] = sc;
            } else if (tid < 256) {
                const int c = tid - 128;
                float t = dpart[c];
#pragma unroll
                for (int w2 = 1; w2 < NW; ++w2) t += dpart[w2 * 128 + c];
                p.dgamma_partial[int64_t(b) * p.n + gcol0 + c] = t;
            }
            named_bar<1, NT>();
            {
                float2 sc2[4], y2[4];
                const float4 a0 = *reinterpret_cast<const float4*>(cs + l16 * 8);
                const float4 a1 = *reinterpret_cast<const float4*>(cs + l16 * 8 + 4);
                const float4 c0 = *reinterpret_cast<const float4*>(cy + l16 * 8);
                const float4 c1 = *reinterpret_cast<const float4*>(cy + l16 * 8 + 4);
                sc2[0] = make_float2(a0.x, a0.y); sc2[1] = make_float2(a0.z, a0.w);
                sc2[2] = make_float2(a1.x, a1.y); sc2[3] = make_float2(a1.z, a1.w);
                y2[0] = make_float2(c0.x, c0.y); y2[1] = make_float2(c0.z, c0.w);
                y2[2] = make_float2(c1.x, c1.y); y2[3] = make_float2(c1.z, c1.w);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 qv[RPT];
#pragma unroll
                    for (int s = 0; s < RPT; ++s) qv[s] = quot_exact2(nd[s][j], sc2[j], y2[j]);
                    if (y2[j].x > 0.f || y2[j].y > 0.f) {   // rare: denormal-range scale, IEEE division
#pragma unroll
                        for (int s = 0; s < RPT; ++s)
                            qv[s] = make_float2(__fdiv_rn(-nd[s][j].x, sc2[j].x), __fdiv_rn(-nd[s][j].y, sc2[j].y));
                    }
                    const int colx = l16 * 8 + 2 * j;
                    const uint32_t off = uint32_t(((warp ^ l16) << 3) + hw * 4);
                    *reinterpret_cast<uint32_t*>(qts + colx * 128 + off) = cvt_e4m3x4(qv[0].x, qv[1].x, qv[2].x, qv[3].x);
                    *reinterpret_cast<uint32_t*>(qts + (colx + 1) * 128 + off) = cvt_e4m3x4(qv[0].y, qv[1].y, qv[2].y, qv[3].y);
                }
            }
            named_bar<1, NT>();
            // copy-out: 128 columns x 16 chunks of 8 rows; thread u handles chunk (u & 15) of columns (u >> 4) + 32 k
            {
                const int rc = tid & 15, colb = tid >> 4;
                uint8_t* dst = p.qt + (gcol0 + colb) * p.M + grow0 + rc * 8;
                const int64_t dstep = int64_t(NT / 16) * p.M;
                const uint8_t* src = qts + colb * 128;
                const int nvalid = valid - rc * 8;
                if ((p.M & 7) == 0 && valid == 128) {
                    uint2 val[2048 / NT];
#pragma unroll
                    for (int kk = 0; kk < 2048 / NT; ++kk) {
                        const int col = colb + kk * (NT / 16);
                        val[kk] = *reinterpret_cast<const uint2*>(src + kk * (NT / 16) * 128 + ((rc ^ ((col >> 3) & 15)) << 3));
                    }
#pragma unroll
                    for (int kk = 0; kk < 2048 / NT; ++kk) {
                        *reinterpret_cast<uint2*>(dst) = val[kk];
                        dst += dstep;
                    }
                } else {
                    const bool vec = (p.M & 7) == 0 && nvalid >= 8;
                    for (int kk = 0; kk < 2048 / NT; ++kk) {
                        const int col = colb + kk * (NT / 16);
                        const uint2 val = *reinterpret_cast<const uint2*>(src + kk * (NT / 16) * 128 + ((rc ^ ((col >> 3) & 15)) << 3));
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
            fence_async_smem();   // the buffer's next writer is a TMA copy
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
        }
    }
}

}  // namespace

int g_band_cluster = 0;         // lh_tuning("band_cluster"): 0 = choose, else force 1 / 2 / 4 / 8

// Cluster size for bands of `tiles` 128-column tiles.  A cluster of C CTAs walks a band in
// ceil(tiles / C) tile steps plus one exchange, and min(bands, active clusters) bands are in flight,
// so a launch costs about  ceil(bands / in flight) x (ceil(tiles / C) + 1/4)  tile steps.  The
// measured times follow this count (active CTAs are 148 / 148 / 132 / 120 for C = 1 / 2 / 4 / 8 at
// this shared-memory footprint, so few bands want C = 4 and many bands want C = 2); the bytes of
// the bands in flight, which decide whether the second pass hits L2, moved the measured order only
// between candidates that this count puts within a few percent of one another, so among those the
// largest cluster (the smallest footprint in L2) is taken.
static int pick_cluster(int64_t tiles, const int* active /* [4]: sizes 1, 2, 4, 8 */, int64_t bands) {
    if (g_band_cluster == 1 || g_band_cluster == 2 || g_band_cluster == 4 || g_band_cluster == 8) {
        int i = 0;
        while ((1 << i) < g_band_cluster) ++i;
        if (active[i] > 0 && tiles >= g_band_cluster) return g_band_cluster;
    }
    int64_t cost[4];
    int64_t least = 0;
    int cands = 0;
    for (int i = 0; i < 4; ++i) {
        const int c = 1 << i;
        if (active[i] <= 0 || tiles < c) break;
        const int64_t ncl = bands < active[i] ? bands : active[i];
        const int64_t waves = (bands + ncl - 1) / ncl;
        cost[i] = waves * (4 * ((tiles + c - 1) / c) + 1);   // in quarter tile steps
        if (cands == 0 || cost[i] < least) least = cost[i];
        ++cands;
    }
    int best = 1;
    for (int i = 0; i < cands; ++i)
        if (cost[i] * 100 <= least * 105) best = 1 << i;
    return best;
}

// x bf16 [M, n], n % 128 == 0; all five outputs.  Returns LH_ERR_ARG + 1000 (-999) when clusters
// cannot be launched on this device, in which case nothing was enqueued.
int band_norm_fwd(const void* x, const void* gamma, int64_t M, int64_t n, float eps, void* q, float* s, float* rms,
                  void* qt, float* st, int round_scale, cudaStream_t stream) {
    const int64_t bands = (M + 127) / 128;
    const int64_t S = n / 128;
    BandParams p{};
    if (int rc = make_tensor_map(&p.tmap_x, x, LH_BF16, uint64_t(M), uint64_t(n), uint64_t(n) * 2, 128, 128)) return rc;
    p.gamma = static_cast<const uint8_t*>(gamma); p.eps = eps; p.inv_n = 1.0f / float(n);
    p.M = M; p.n = int(n); p.S = int(S); p.bands = int(bands);
    p.q = static_cast<uint8_t*>(q); p.s = s; p.rms = rms; p.qt = static_cast<uint8_t*>(qt); p.st = st;
    p.round_scale = round_scale;
    // active clusters per cluster size, once per device
    static int active_cache[64][4];
    static bool have[64];
    int dev = 0;
    sm_count(&dev);
    if (dev < 0 || dev >= 64) return -999;
    if (!have[dev]) {
        cudaError_t e = cudaFuncSetAttribute(band_norm_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(BandCfg::SMEM));
        if (e != cudaSuccess) { cudaGetLastError(); return -999; }
        for (int i = 0; i < 4; ++i) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(unsigned(8 << i)); cfg.blockDim = dim3(kBandThreads); cfg.dynamicSmemBytes = BandCfg::SMEM;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = unsigned(1 << i); at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at; cfg.numAttrs = 1;
            int ncl = 0;
            if (cudaOccupancyMaxActiveClusters(&ncl, band_norm_fwd_kernel, &cfg) != cudaSuccess) { cudaGetLastError(); ncl = 0; }
            active_cache[dev][i] = ncl;
        }
        have[dev] = true;
    }
    const int* active = active_cache[dev];
    if (active[0] <= 0) return -999;
    const int CSZ = pick_cluster(n / 128, active, bands);
    int idx = 0;
    while ((1 << idx) < CSZ) ++idx;
    int64_t nclusters = active[idx];
    if (bands < nclusters) nclusters = bands;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(nclusters * CSZ)); cfg.blockDim = dim3(kBandThreads); cfg.dynamicSmemBytes = BandCfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = unsigned(CSZ); at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, band_norm_fwd_kernel, p);
    if (e != cudaSuccess) { set_error("band_norm_fwd_kernel: %s", cudaGetErrorString(e)); cudaGetLastError(); return int(e); }
    return LH_OK;
}

int64_t band_norm_bwd_scratch(int64_t M, int64_t n) { return ((M + 127) / 128) * n * 4; }

int dgamma_reduce(const float* partial, int parts, int64_t n, float* dgamma, cudaStream_t stream);

// RMSNorm backward + dy dual-axis quantisation in one pass over x and dy; bf16, n % 128 == 0, M > 0.
// scratch: band_norm_bwd_scratch(M, n) bytes.  Returns -999 (nothing enqueued) where clusters cannot be launched.
int band_norm_bwd(const void* dy, const void* x, const void* gamma, const float* rms, int64_t M, int64_t n, float eps,
                  void* dx, float* dgamma, void* dy_q, float* dy_s, void* dy_qt, float* dy_st, int round_scale,
                  void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    const int64_t bands = (M + 127) / 128;
    if (scratch_bytes < band_norm_bwd_scratch(M, n)) return -999;
    BandBwdParams p{};
    if (int rc = make_tensor_map(&p.tmap_x, x, LH_BF16, uint64_t(M), uint64_t(n), uint64_t(n) * 2, 128, 128)) return rc;
    if (int rc = make_tensor_map(&p.tmap_dy, dy, LH_BF16, uint64_t(M), uint64_t(n), uint64_t(n) * 2, 128, 128)) return rc;
    p.gamma = static_cast<const uint8_t*>(gamma); p.rms = rms; p.eps = eps; p.inv_n = 1.0f / float(n);
    p.M = M; p.n = int(n); p.S = int(n / 128); p.bands = int(bands);
    p.dx = static_cast<uint8_t*>(dx); p.dgamma_partial = static_cast<float*>(scratch);
    p.q = static_cast<uint8_t*>(dy_q); p.s = dy_s; p.qt = static_cast<uint8_t*>(dy_qt); p.st = dy_st;
    p.round_scale = round_scale;
    static int active_cache[64][4];
    static bool have[64];
    int dev = 0;
    sm_count(&dev);
    if (dev < 0 || dev >= 64) return -999;
    if (!have[dev]) {
        cudaError_t e = cudaFuncSetAttribute(band_norm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(BandBwdCfg::SMEM));
        if (e != cudaSuccess) { cudaGetLastError(); return -999; }
        for (int i = 0; i < 4; ++i) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(unsigned(8 << i)); cfg.blockDim = dim3(kBandThreads); cfg.dynamicSmemBytes = BandBwdCfg::SMEM;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = unsigned(1 << i); at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at; cfg.numAttrs = 1;
            int ncl = 0;
            if (cudaOccupancyMaxActiveClusters(&ncl, band_norm_bwd_kernel, &cfg) != cudaSuccess) { cudaGetLastError(); ncl = 0; }
            active_cache[dev][i] = ncl;
        }
        have[dev] = true;
    }
    const int* active = active_cache[dev];
    if (active[0] <= 0) return -999;
    const int CSZ = pick_cluster(n / 128, active, bands);
    int idx = 0;
    while ((1 << idx) < CSZ) ++idx;
    int64_t nclusters = active[idx];
    if (bands < nclusters) nclusters = bands;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(nclusters * CSZ)); cfg.blockDim = dim3(kBandThreads); cfg.dynamicSmemBytes = BandBwdCfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = unsigned(CSZ); at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, band_norm_bwd_kernel, p);
    if (e != cudaSuccess) { set_error("band_norm_bwd_kernel: %s", cudaGetErrorString(e)); cudaGetLastError(); return int(e); }
    return dgamma_reduce(p.dgamma_partial, int(bands), n, dgamma, stream);
}

}  // namespace lh
