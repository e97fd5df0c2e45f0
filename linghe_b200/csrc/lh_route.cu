// Routing helpers around the permute + quantise step: the destination row of every routed
// (token, expert) pair with per-expert padding, the inverse list of source tokens, and the
// gradient gather that undoes the permutation.
// (replace triton_make_row_id_map_and_index, linghe/utils/gather.py:116-210, and
//  triton_unpermute_with_mask_map, linghe/utils/scatter.py:152-242)
//
// These move little data (the routing map is tokens x experts bytes); they are plain
// coalesced streaming kernels, one thread per expert column or per 16-byte chunk of a row.
#include "lh_common.cuh"

namespace lh {

namespace {

constexpr int kRouteBlocks = 128;   // token blocks: the map is scanned in two passes over them

__device__ __forceinline__ int load_route(const void* map, int is_i32, int64_t i) {
    return is_i32 ? (reinterpret_cast<const int32_t*>(map)[i] != 0) : (reinterpret_cast<const uint8_t*>(map)[i] != 0);
}

// counts[b, e] = routed tokens of expert e inside token block b
__global__ void __launch_bounds__(1024)
route_block_count_kernel(const void* __restrict__ map, int is_i32, int64_t T, int E, int64_t rows_per_block,
                         int32_t* __restrict__ counts) {
    const int64_t t0 = int64_t(blockIdx.x) * rows_per_block;
    int64_t t1 = t0 + rows_per_block;
    if (t1 > T) t1 = T;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int64_t t = t0; t < t1; ++t) c += load_route(map, is_i32, t * E + e);
        counts[int64_t(blockIdx.x) * E + e] = c;
    }
}

// row_map[t, e] = first padded row of expert e + rank of token t among e's tokens (or -1);
// row_index[that row] = t.  Padding rows of row_index keep what the caller put there.
__global__ void __launch_bounds__(1024)
route_row_map_kernel(const void* __restrict__ map, int is_i32, int64_t T, int E, int64_t rows_per_block, int pad,
                     const int32_t* __restrict__ counts, int32_t* __restrict__ row_map,
                     int32_t* __restrict__ row_index) {
    extern __shared__ int32_t sh[];          // [E] padded totals -> exclusive offsets
    __shared__ int32_t warp_sum[32];
    __shared__ int32_t carry;
    const int nb = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // totals per expert (padded) into shared memory
    for (int e = tid; e < E; e += blockDim.x) {
        int tot = 0;
        for (int b = 0; b < nb; ++b) tot += counts[int64_t(b) * E + e];
        sh[e] = (tot + pad - 1) / pad * pad;
    }
    if (tid == 0) carry = 0;
    __syncthreads();
    // exclusive scan over experts, blockDim.x experts per round
    for (int base = 0; base < E; base += blockDim.x) {
        const int e = base + tid;
        const int v = e < E ? sh[e] : 0;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += o;
        }
        if (lane == 31) warp_sum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = lane < int(blockDim.x >> 5) ? warp_sum[lane] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, w, d);
                if (lane >= d) w += o;
            }
            warp_sum[lane] = w;               // inclusive over warps
        }
        __syncthreads();
        const int before = carry + (warp ? warp_sum[warp - 1] : 0) + incl - v;
        __syncthreads();
        if (e < E) sh[e] = before;
        if (tid == blockDim.x - 1) carry = before + v;
        __syncthreads();
    }
    const int64_t t0 = int64_t(blockIdx.x) * rows_per_block;
    int64_t t1 = t0 + rows_per_block;
    if (t1 > T) t1 = T;
    for (int e = tid; e < E; e += blockDim.x) {
        int off = sh[e];
        for (int b = 0; b < int(blockIdx.x); ++b) off += counts[int64_t(b) * E + e];
        for (int64_t t = t0; t < t1; ++t) {
            const int v = load_route(map, is_i32, t * E + e);
            row_map[t * E + e] = v ? off : -1;
            if (v) { row_index[off] = int32_t(t); ++off; }
        }
    }
}

template <typename T> struct Chunk;   // one 16-byte chunk of a row as floats
template <> struct Chunk<__nv_bfloat16> {
    static constexpr int VEC = 8, EB = 2;
    static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 v = bf16x2_to_f2(w[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    }
};
template <> struct Chunk<__half> {
    static constexpr int VEC = 8, EB = 2;
    static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = v.x; f[2 * i + 1] = v.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        return make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]), pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
    }
};
template <> struct Chunk<float> {
    static constexpr int VEC = 4, EB = 4;
    static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};

// out[t, :] = sum over the experts of token t (in expert order) of grad[row_map[t, e], :],
// accumulated in float32; prob_out[t, e] = probs[row_map[t, e]] or 0.
// One warp per token: the lanes compact the token's valid rows into a shared list (ballot),
// then walk the rows with 16 independent 16-byte loads per lane in flight.
template <typename T>
__global__ void __launch_bounds__(256)
unpermute_kernel(const uint8_t* __restrict__ grad, const int32_t* __restrict__ row_map, const void* __restrict__ probs,
                 int probs_dtype, int64_t tokens, int E, int64_t n, uint8_t* __restrict__ out,
                 void* __restrict__ prob_out) {
    extern __shared__ int32_t lists[];       // [warps][E] valid destination rows, in expert order
    constexpr int EB = Chunk<T>::EB, VEC = Chunk<T>::VEC;
    constexpr int CPL = 4, RU = 4;           // 16-byte chunks per lane and pass; rows fetched together
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    int32_t* rows = lists + warp * E;
    const int64_t chunks = n / VEC;
    for (int64_t t = int64_t(blockIdx.x) * warps + warp; t < tokens; t += int64_t(gridDim.x) * warps) {
        int nv = 0;
        for (int base = 0; base < E; base += 32 * 8) {           // 8 independent map loads per lane, then the ballots
            int r[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int e = base + 32 * k + lane;
                r[k] = e < E ? row_map[t * E + e] : -1;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int e = base + 32 * k + lane;
                const unsigned m = __ballot_sync(0xffffffffu, r[k] >= 0);
                if (r[k] >= 0) rows[nv + __popc(m & ((1u << lane) - 1u))] = r[k];
                nv += __popc(m);
                if (prob_out != nullptr && e < E) {
                    if (probs_dtype == LH_BF16) {
                        reinterpret_cast<__nv_bfloat16*>(prob_out)[t * E + e] =
                            r[k] >= 0 ? reinterpret_cast<const __nv_bfloat16*>(probs)[r[k]] : __float2bfloat16_rn(0.f);
                    } else {
                        reinterpret_cast<float*>(prob_out)[t * E + e] =
                            r[k] >= 0 ? reinterpret_cast<const float*>(probs)[r[k]] : 0.f;
                    }
                }
            }
        }
        __syncwarp();
        for (int64_t c0 = 0; c0 < chunks; c0 += 32 * CPL) {      // 128 chunks (2 KB) of the row per pass
            float acc[CPL][VEC];
#pragma unroll
            for (int k = 0; k < CPL; ++k)
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc[k][j] = 0.f;
            for (int i0 = 0; i0 < nv; i0 += RU) {                // RU rows' loads in flight together
                uint4 raw[RU][CPL];
#pragma unroll
                for (int u = 0; u < RU; ++u) {
                    const bool on = i0 + u < nv;
                    const uint8_t* src = grad + (int64_t(on ? rows[i0 + u] : 0) * n + c0 * VEC) * EB;
#pragma unroll
                    for (int k = 0; k < CPL; ++k) {
                        const int64_t c = c0 + k * 32 + lane;
                        raw[u][k] = (on && c < chunks) ? *reinterpret_cast<const uint4*>(src + (k * 32 + lane) * 16)
                                                       : make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (int u = 0; u < RU; ++u) {                   // rows are added in list order
#pragma unroll
                    for (int k = 0; k < CPL; ++k) {
                        float v[VEC];
                        Chunk<T>::unpack(raw[u][k], v);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) acc[k][j] += v[j];
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < CPL; ++k) {
                const int64_t c = c0 + k * 32 + lane;
                if (c < chunks) *reinterpret_cast<uint4*>(out + (t * n + c * VEC) * EB) = Chunk<T>::pack(acc[k]);
            }
        }
        __syncwarp();
    }
}

}  // namespace

int64_t route_scratch_bytes(int64_t E) { return int64_t(kRouteBlocks) * E * 4; }

int make_row_id_map_and_index(const void* map, int map_is_i32, int64_t T, int64_t E, int multiple_of, int32_t* row_map,
                              int32_t* row_index, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    if (T < 0 || E <= 0 || multiple_of <= 0) return fail_arg("make_row_id_map_and_index: bad sizes");
    if (T == 0) return LH_OK;
    if (!map || !row_map || !row_index || !scratch) return fail_arg("make_row_id_map_and_index: NULL pointer");
    if (scratch_bytes < route_scratch_bytes(E)) return fail_arg("make_row_id_map_and_index: scratch too small");
    if (E > 0x7fffffff / 4 || T * E > (int64_t(1) << 40)) return fail_arg("make_row_id_map_and_index: size out of range");
    const int64_t rpb = (T + kRouteBlocks - 1) / kRouteBlocks;
    const int nb = int((T + rpb - 1) / rpb);
    int threads = int(E < 1024 ? ((E + 31) / 32) * 32 : 1024);
    route_block_count_kernel<<<nb, threads, 0, stream>>>(map, map_is_i32, T, int(E), rpb, static_cast<int32_t*>(scratch));
    if (int rc = check_launch("route_block_count_kernel")) return rc;
    const size_t smem = size_t(E) * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(route_row_map_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail_arg("make_row_id_map_and_index: too many experts (%lld)", (long long)E);
    }
    route_row_map_kernel<<<nb, threads, smem, stream>>>(map, map_is_i32, T, int(E), rpb, multiple_of,
                                                       static_cast<const int32_t*>(scratch), row_map, row_index);
    return check_launch("route_row_map_kernel");
}

int unpermute_with_mask_map(const void* grad, int dtype, const int32_t* row_map, const void* probs, int probs_dtype,
                            int64_t tokens, int64_t E, int64_t n, void* out, void* prob_out, cudaStream_t stream) {
    if (tokens < 0 || E <= 0 || n <= 0) return fail_arg("unpermute_with_mask_map: bad sizes");
    if (tokens == 0) return LH_OK;
    if (!grad || !row_map || !out) return fail_arg("unpermute_with_mask_map: NULL pointer");
    if ((probs == nullptr) != (prob_out == nullptr)) return fail_arg("unpermute_with_mask_map: probs and prob_out go together");
    const int eb = dtype == LH_F32 ? 4 : 2;
    if ((n * eb) % 16 != 0) return fail_arg("unpermute_with_mask_map: row length must be a multiple of 16 bytes");
    if ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail_arg("unpermute_with_mask_map: pointers must be 16-byte aligned");
    int warps = 8;
    while (warps > 1 && size_t(warps) * size_t(E) * 4 > 48 * 1024) warps >>= 1;
    const size_t smem = size_t(warps) * size_t(E) * 4;
    if (smem > 48 * 1024) return fail_arg("unpermute_with_mask_map: too many experts (%lld)", (long long)E);
    int64_t grid = (tokens + warps - 1) / warps;
    if (grid > int64_t(sm_count()) * 16) grid = int64_t(sm_count()) * 16;
    const uint8_t* g = static_cast<const uint8_t*>(grad);
    uint8_t* o = static_cast<uint8_t*>(out);
    const dim3 blk(unsigned(warps * 32));
    switch (dtype) {
        case LH_BF16:
            unpermute_kernel<__nv_bfloat16><<<unsigned(grid), blk, smem, stream>>>(g, row_map, probs, probs_dtype, tokens, int(E), n, o, prob_out);
            break;
        case LH_F16:
            unpermute_kernel<__half><<<unsigned(grid), blk, smem, stream>>>(g, row_map, probs, probs_dtype, tokens, int(E), n, o, prob_out);
            break;
        case LH_F32:
            unpermute_kernel<float><<<unsigned(grid), blk, smem, stream>>>(g, row_map, probs, probs_dtype, tokens, int(E), n, o, prob_out);
            break;
        default:
            return fail_arg("unpermute_with_mask_map: unsupported dtype %d", dtype);
    }
    return check_launch("unpermute_kernel");
}

}  // namespace lh
