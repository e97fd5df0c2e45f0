// RMSNorm backward + row-wise and transposed FP8 copies of dy in one launch, as two roles per CTA.
//
// This file is compiled WITHOUT relocatable device code: ptxas ignores setmaxnreg in relocatable
// objects, and the register split between the roles is what lets both fit an SM.  It therefore
// references no device symbol of another translation unit.
#include "lh_small.cuh"

namespace lh {

namespace {

// The backward walk and the transposed 128x1 quantisation of dy as two roles of one CTA: the
// first NT threads walk rows (dx, the dgamma sums, the row-wise codes of dy), the last 128 threads
// take 128 x 128 tiles of dy (tile blockIdx.x, + gridDim.x, ... in band-major order) and write
// the transposed codes and scales.  Nothing depends on the order of the two, so there is no
// inter-role wait for correctness; the tile role only paces itself to stay within LEAD (8) bands of
// its own CTA's walk, so that whichever role touches a band second finds it in L2 and dy crosses
// the HBM interface once.  The roles hide each other's latencies on the SM's schedulers.  The
// register file is split by setmaxnreg: RREG per walking thread, CREG per tile thread; the host
// checks NT * RREG + 128 * CREG against the CTA's allocation before it launches.
template <int SPANS, int NT, int MINB, bool WIDE, int RREG, int CREG>
__global__ void __launch_bounds__(NT + 128, MINB)
small_norm_bwd_duo_kernel(const __grid_constant__ SmallParams p, const uint8_t* __restrict__ dy, float* __restrict__ partial) {
    constexpr int LEAD = 8;
    __shared__ __align__(16) float2 wsum[2][NT / 32];
    __shared__ float4 gam_s[4 * SPANS * NT];
    __shared__ __align__(16) float cq_cmax[8 * 128];
    __shared__ __align__(16) float cq_cs[128], cq_cy[128];
    __shared__ int walk_band;
    if (threadIdx.x == 0) walk_band = 0;
    __syncthreads();
    if (threadIdx.x < NT) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(RREG));
        norm_bwd_walk<SPANS, NT, WIDE, true, 1>(p, dy, partial, wsum, &walk_band, gam_s);
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(CREG));
        const int t = threadIdx.x - NT;
        const int nct = p.n >> 7;
        const int64_t col_tiles = ((p.M + 127) >> 7) * nct;
        bool pace = true;   // used by the role's first thread only
        for (int64_t tile = blockIdx.x; tile < col_tiles; tile += gridDim.x) {
            const int band = int(tile / nct);
            // One thread watches the walk, the others wait at the role's barrier (a hardware wait that
            // takes no issue slots from the walking warps; 128 polling threads did).  Bounded: it is a
            // pacing hint only, giving it up costs a second read of dy from HBM, not correctness.
            if (t == 0 && pace) {
                uint32_t polls = 0;
                while (*static_cast<volatile int*>(&walk_band) < band - LEAD) {   // walk_band ends at INT_MAX: no sum on that side
                    __nanosleep(500);
                    if (++polls > (1u << 20)) { pace = false; break; }
                }
            }
            role_sync<2, 128>();
            col_quant_tile<128, 2>(p, dy, band, int(tile - int64_t(band) * nct), t, cq_cmax, cq_cs, cq_cy);
        }
    }
}

}  // namespace

int small_norm_bwd_duo(const SmallParams& p, const uint8_t* dy, float* partial, unsigned grid, bool wide, cudaStream_t stream) {
    const int n = p.n;
#define LH_DUO_LAUNCH(S, NT_, MB, W, RR, CR)                                                            \
    do {                                                                                                \
        auto* k = small_norm_bwd_duo_kernel<S, NT_, MB, W, RR, CR>;                                     \
        cudaFuncAttributes fa;                                                                          \
        if (cudaFuncGetAttributes(&fa, k) != cudaSuccess || (NT_ + 128) * fa.numRegs < NT_ * RR + 128 * CR) { \
            cudaGetLastError();                                                                         \
            return LH_ERR_ARG - 1000;                                                                   \
        }                                                                                               \
        k<<<grid, NT_ + 128, 0, stream>>>(p, dy, partial);                                              \
    } while (0)
#define LH_DUO_PICK(W)                                                 \
    do {                                                               \
        if (n <= 2048) LH_DUO_LAUNCH(1, 128, 2, W, 168, 88);           \
        else if (n <= 4096) LH_DUO_LAUNCH(2, 128, 2, W, 184, 72);      \
        else LH_DUO_LAUNCH(2, 256, 1, W, 208, 88);                     \
    } while (0)
    if (wide) LH_DUO_PICK(true);
    else LH_DUO_PICK(false);
#undef LH_DUO_PICK
#undef LH_DUO_LAUNCH
    return check_launch("small_norm_bwd_duo_kernel");
}

}  // namespace lh
