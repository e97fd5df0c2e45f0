// Router logits for the fused RMSNorm + router GEMM + quantisation entry point
// (replaces the tl.dot of rms_norm_fp32_gemm_block_quant_forward_n_kernel,
// linghe/utils/norm.py:617-686).
//
//   logits[m, j] = sum_k y[m,k] * w[j,k],   y = (x * r_m) * gamma          (float32 y, never rounded)
//                = r_m * sum_k x[m,k] * (gamma[k] * w[j,k])
//
// x is 16-bit, so it feeds the tensor cores unchanged; gamma*w is a product of two 8-bit
// significands (16 bits) and splits exactly into two bf16 terms hi + lo.  The contraction
// is therefore two bf16 tcgen05 MMAs per k-step with float32 accumulation in tensor memory,
// and 1/rms is applied to the accumulator rows on the way out.  No operand is rounded.
//
// Layout of one CTA (128 threads, one per accumulator row): tile 128 rows x 128 logits,
// k-step 64 (one 128-byte swizzle row); a ring of stages, each holding the x tile and the
// hi and lo weight tiles, all loaded by TMA with the 128-byte swizzle the MMA descriptors
// name.  Thread 0 produces, thread 32 issues the MMAs, every warp drains its 32 lanes of
// the accumulator.
#include "lh_common.cuh"

namespace lh {

namespace {

constexpr int GM = 128, GN = 128, GK = 64;
constexpr int GSTAGES = 4;
constexpr int G_TILE = GM * GK * 2;            // 16 KB: one operand tile
constexpr int G_STAGE = 3 * G_TILE;            // x, w_hi, w_lo
constexpr int G_BAR_OFF = GSTAGES * G_STAGE;
constexpr int G_SMEM = 1024 + G_BAR_OFF + 128; // slack for the 1024-byte alignment + barriers
constexpr int G_TMEM_COLS = 128;

enum : int { DEVERR_ACCUM_WAIT = 4 };

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// shared-memory matrix descriptor: K-major operand, rows of 128 bytes, 128-byte swizzle,
// groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
           (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// instruction descriptor: D f32, A and B bf16, both K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(GN >> 3) << 17) | (uint32_t(GM >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
// arrive on `bar` once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// W'[j,k] = gamma[k] * w[j,k] as hi + lo bf16: rows [0,N) hold hi, rows [N,2N) hold lo.
__global__ void __launch_bounds__(256)
router_weight_split_kernel(const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ gamma,
                           __nv_bfloat16* __restrict__ out, int N, int K) {
    const int64_t total = int64_t(N) * K / 8;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t e = i * 8;
        const int k = int(e % K);
        const uint4 wv = *reinterpret_cast<const uint4*>(w + e);
        const uint4 gv = *reinterpret_cast<const uint4*>(gamma + k);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        const uint32_t gg[4] = {gv.x, gv.y, gv.z, gv.w};
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 a = bf16x2_to_f2(ww[j]), g = bf16x2_to_f2(gg[j]);
            const float p0 = a.x * g.x, p1 = a.y * g.y;          // exact: 16 significant bits
            hi[j] = pack_bf16x2(p0, p1);
            const float2 h = bf16x2_to_f2(hi[j]);
            lo[j] = pack_bf16x2(p0 - h.x, p1 - h.y);             // exact remainder, fits bf16
        }
        *reinterpret_cast<uint4*>(out + e) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(out + int64_t(N) * K + e) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

__global__ void __launch_bounds__(128, 1)
router_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   const float* __restrict__ rms, float* __restrict__ logits, int N, int K) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    uint8_t* tiles = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + G_BAR_OFF);
    uint64_t* empty = full + GSTAGES;
    uint64_t* accum = empty + GSTAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int m0 = blockIdx.x * GM, n0 = blockIdx.y * GN;
    const int ktiles = K / GK;

    if (t == 0) {
        for (int i = 0; i < GSTAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(accum, 1);
        mbar_fence_init();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {   // one warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(uint32_t(G_TMEM_COLS))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (t == 0) {
        // ---- producer: TMA loads into the ring
        for (int kt = 0; kt < ktiles; ++kt) {
            const int s = kt % GSTAGES;
            const uint32_t use = uint32_t(kt / GSTAGES);
            if (kt >= GSTAGES && !mbar_wait(&empty[s], (use & 1u) ^ 1u, DEVERR_EMPTY_WAIT)) break;
            uint8_t* st = tiles + size_t(s) * G_STAGE;
            mbar_expect_tx(&full[s], G_STAGE);
            tma_load_2d(st, &map_x, kt * GK, m0, &full[s]);
            tma_load_2d(st + G_TILE, &map_w, kt * GK, n0, &full[s]);
            tma_load_2d(st + 2 * G_TILE, &map_w, kt * GK, N + n0, &full[s]);
        }
    } else if (t == 32) {
        // ---- MMA issuer
        // The issue of an MMA blocks while the tensor pipe's queue is full, so after the last
        // MMA of a stage only little work is queued: the wait for the next stage's data sits
        // in the middle of the current stage's MMAs, not after them.
        bool ok = mbar_wait(&full[0], 0, DEVERR_FULL_WAIT);
        const uint64_t d0 = umma_desc(smem_u32(tiles));
        for (int kt = 0; kt < ktiles && ok; ++kt) {
            const int s = kt % GSTAGES;
            tc_fence_after();
            const uint64_t da = d0 + uint64_t(s) * (G_STAGE >> 4), dh = da + (G_TILE >> 4), dl = dh + (G_TILE >> 4);
#pragma unroll
            for (int k4 = 0; k4 < GK / 16; ++k4) {          // 16 elements = 32 bytes = 2 descriptor units per step
                if (k4 == GK / 32 && kt + 1 < ktiles)
                    ok = mbar_wait(&full[(kt + 1) % GSTAGES], uint32_t((kt + 1) / GSTAGES) & 1u, DEVERR_FULL_WAIT);
                umma_bf16(tmem, da + 2 * k4, dh + 2 * k4, (kt | k4) != 0);
                umma_bf16(tmem, da + 2 * k4, dl + 2 * k4, 1u);
            }
            umma_commit(&empty[s]);                          // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(accum);
    }
    __syncwarp();

    // ---- epilogue: thread = accumulator row; 1/rms applied here
    const bool done = __all_sync(0xffffffffu, mbar_wait(accum, 0, DEVERR_ACCUM_WAIT));
    tc_fence_after();
    if (done) {
        const int64_t row = int64_t(m0) + t;
        const float r = rms[row];
        float* out = logits + row * N + n0;
#pragma unroll 1
        for (int c = 0; c < GN / 32; ++c) {
            uint32_t v[32];
            const uint32_t taddr = tmem + (uint32_t(warp * 32) << 16) + uint32_t(c * 32);
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
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(out + c * 32 + 4 * j) =
                    make_float4(__uint_as_float(v[4 * j]) * r, __uint_as_float(v[4 * j + 1]) * r,
                                __uint_as_float(v[4 * j + 2]) * r, __uint_as_float(v[4 * j + 3]) * r);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(G_TMEM_COLS))
                     : "memory");
    }
}

}  // namespace

int64_t router_gemm_scratch(int64_t N, int64_t K) { return 2 * N * K * 2; }

// logits [M,N] f32 = rms[m] * (x [M,K] bf16) . (gamma ⊙ w [N,K])^T ; M, N, K multiples of 128.
int router_gemm(const void* x, const void* gamma, const void* w, const float* rms, float* logits, int64_t M, int64_t N,
                int64_t K, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    if (!x || !gamma || !w || !rms || !logits || !scratch) return fail_arg("router_gemm: NULL pointer");
    if ((M % GM) || (N % GN) || (K % 128) || M <= 0) return fail_arg("router_gemm: need M, N, K multiples of 128");
    if (scratch_bytes < router_gemm_scratch(N, K)) return fail_arg("router_gemm: scratch too small");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(gamma) |
         reinterpret_cast<uintptr_t>(scratch) | reinterpret_cast<uintptr_t>(logits)) & 15)
        return fail_arg("router_gemm: pointers must be 16-byte aligned");
    if (M / GM > 0x7fffffff / GM || 2 * N > 0x7fffffff) return fail_arg("router_gemm: size out of range");
    const int64_t vecs = N * K / 8;
    int64_t sgrid = (vecs + 255) / 256;
    if (sgrid > 4 * int64_t(sm_count())) sgrid = 4 * int64_t(sm_count());
    router_weight_split_kernel<<<dim3(unsigned(sgrid)), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(gamma),
        static_cast<__nv_bfloat16*>(scratch), int(N), int(K));
    if (int rc = check_launch("router_weight_split_kernel")) return rc;
    CUtensorMap mx, mw;
    if (int rc = make_tensor_map(&mx, x, LH_BF16, uint64_t(M), uint64_t(K), uint64_t(K) * 2, GM, GK, 1)) return rc;
    if (int rc = make_tensor_map(&mw, scratch, LH_BF16, uint64_t(2 * N), uint64_t(K), uint64_t(K) * 2, GN, GK, 1)) return rc;
    cudaError_t e = cudaFuncSetAttribute(router_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM);
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return int(e); }
    router_gemm_kernel<<<dim3(unsigned(M / GM), unsigned(N / GN)), 128, G_SMEM, stream>>>(mx, mw, rms, logits, int(N), int(K));
    return check_launch("router_gemm_kernel");
}

}  // namespace lh
