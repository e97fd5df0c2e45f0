// Shared device helpers for the sm_100a fused norm / SwiGLU + FP8 e4m3 blockwise
// quantisation kernels: quantisation arithmetic that reproduces the PyTorch reference
// math bit for bit, mbarrier / bulk-copy (TMA) PTX wrappers with bounded waits, and
// the host-side error plumbing of the C ABI.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/linghe_b200.h"

namespace lh {

// ----------------------------------------------------------------------------------
// host-side error plumbing
// ----------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail_arg(const char* fmt, ...);      // records message, returns LH_ERR_ARG
int check_launch(const char* what);      // cudaGetLastError -> status code
int sm_count(int* out_device = nullptr); // SM count of the current device (cached)
// Tiled 2-D tensor map over a row-major [rows, cols] matrix with `pitch_bytes` between
// rows; the box is box_rows x box_cols elements, out-of-range reads give 0.  swizzle128:
// lay the box out with the 128-byte swizzle (box rows must then be 128 bytes long).
int make_tensor_map(CUtensorMap* out, const void* base, int dtype, uint64_t rows, uint64_t cols,
                    uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle128 = 0);

// Device status word: 0 = fine; otherwise the code of the first bounded wait that
// gave up.  Read back with lh_device_status().
extern __device__ int g_device_status;

enum : int {
    DEVERR_FULL_WAIT = 1,   // consumer gave up waiting for a tile to land
    DEVERR_EMPTY_WAIT = 2,  // producer gave up waiting for a free stage
    DEVERR_DRAIN_WAIT = 3,  // exit path gave up waiting for copies in flight
};

// ----------------------------------------------------------------------------------
// element types
// ----------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
    static constexpr int BYTES = 2;
    // 8 consecutive elements held in a uint4 -> 8 floats
    static __device__ __forceinline__ void unpack8(const uint4& r, float* f) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <> struct Elem<__half> {
    static constexpr int BYTES = 2;
    static __device__ __forceinline__ void unpack8(const uint4& r, float* f) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
};
template <> struct Elem<float> {
    static constexpr int BYTES = 4;
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// ----------------------------------------------------------------------------------
// quantisation arithmetic
// ----------------------------------------------------------------------------------
constexpr float kE4M3Max = 448.0f;
constexpr float kScaleFloor = 1e-30f;

// exp2(ceil(log2(s))) as the float32 reference computes it.  Away from powers of two
// the result is 2^(k+1) for s = 2^k * (1+f); within 64 ulps above a power of two a
// correctly rounded float log2 rounds back to k for some f, which is reproduced by
// rounding a double-precision log2 to float.
__device__ __forceinline__ float pow2_ceil(float s) {
    const uint32_t b = __float_as_uint(s);
    const int k = int(b >> 23) - 127;
    const uint32_t m = b & 0x7fffffu;
    int K;
    if (m == 0u) {
        K = k;
    } else if (m >= 64u) {
        K = k + 1;
    } else {
        K = int(ceilf(float(log2(double(s)))));
    }
    return __uint_as_float(uint32_t(K + 127) << 23);
}

// RN(a / 448) in three instructions: q = a*c with c = RN(1/448), residual r = a - 448*q
// (exact in an FMA), result q + r*c.  Correctly rounded (Markstein) whenever the residual
// cannot underflow, which holds for every a whose quotient is above the 1e-30 scale
// floor; below it the floor wins anyway.
__device__ __forceinline__ float div448(float a) {
    constexpr float c = 1.0f / 448.0f;
    const float q = a * c;
    const float r = fmaf(-448.0f, q, a);
    return fmaf(r, c, q);
}

// scale = max(amax / 448, 1e-30) (bit-identical to IEEE division), optionally rounded
// up to a power of two.
__device__ __forceinline__ float scale_from_amax(float amax, bool round_scale) {
    float s = fmaxf(div448(amax), kScaleFloor);
    if (round_scale) s = pow2_ceil(s);
    return s;
}

// 1/sqrt(a) to about 1 ulp: hardware approximation plus one Newton step.
__device__ __forceinline__ float rsqrt_nr(float a) {
    float y;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(a));
    const float t = a * y;
    const float e = fmaf(-t, y, 1.0f);
    return fmaf(0.5f * y, e, y);
}

// Per-block divisor.  `exact` quotients equal IEEE x / s bit for bit: q0 = x*y with
// y = RN(1/s), residual r' = s*q0 - x (exact in an FMA), q = q0 - r'*y.  The form with
// the negated residual keeps the sign of a zero quotient.  Blocks whose scale is so
// small that the residual could underflow take IEEE division instead.
struct Divisor {
    float s;      // scale
    float y;      // RN(1/s)
    float ny;     // -y
    bool tiny;    // residual may underflow: use __fdiv_rn
    __device__ __forceinline__ explicit Divisor(float scale) {
        s = scale;
        y = __frcp_rn(scale);
        ny = -y;
        tiny = scale < 8.0e-28f;  // ~2^-90
    }
    template <bool EXACT>
    __device__ __forceinline__ float quot(float x) const {
        if (EXACT) {
            if (tiny) return __fdiv_rn(x, s);
            const float q0 = x * y;
            const float r = fmaf(s, q0, -x);
            return fmaf(r, ny, q0);
        } else {
            return x * y;
        }
    }
};

// two floats -> two e4m3 codes (round to nearest even, saturating); lo in bits 0..7.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return uint32_t(r);
}
// four floats -> four e4m3 codes packed in a word (a in bits 0..7)
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
    uint32_t r;
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r)
        : "f"(a), "f"(b), "f"(c), "f"(d));
    return r;
}

__device__ __forceinline__ float amax8(const float* v) {
    float m = fmaxf(fabsf(v[0]), fabsf(v[1]));
#pragma unroll
    for (int i = 2; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
    return m;
}

// sigmoid as the reference computes it: 1 / (1 + exp(-x)), full-precision expf and a
// correctly rounded reciprocal.
__device__ __forceinline__ float sigmoid_ref(float x) {
    return __frcp_rn(1.0f + expf(-x));
}

// ---- packed float32x2 arithmetic (one FP32 pipe instruction per two lanes' worth) ----
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }

// two bf16 packed in a 32-bit word -> float2 (low element first)
__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// two bf16 packed in a word -> the NEGATED pair as float2.  Flipping the sign bit rides on the
// widening itself: adding 2^31 to (w << 16) and xor-ing it into the masked high half are the
// same integer instructions as the plain conversion, with one more constant operand.
// (Written as inline PTX: from C++ the compiler recognises the sign flip as a float negation and
// spends a separate FADD on it.)
__device__ __forceinline__ float2 bf16x2_to_neg_f2(uint32_t w) {
    uint32_t lo, hi;
    asm("mad.lo.u32 %0, %1, 65536, 0x80000000;" : "=r"(lo) : "r"(w));
    asm("lop3.b32 %0, %1, 0xffff0000, 0x80000000, 0x6a;" : "=r"(hi) : "r"(w));   // (w & 0xffff0000) ^ 0x80000000
    return make_float2(__uint_as_float(lo), __uint_as_float(hi));
}

// Exact quotients, two at a time.  The pure quantisers keep the NEGATED inputs nv = -x in
// registers (the negation is free in the load), so that the whole Markstein sequence runs on
// packed instructions without a separate negation: with ny = -RN(1/s),
//   q0 = nv * ny = x * y,   r' = s * q0 + nv = s*q0 - x (exact in an FMA),   q = r' * ny + q0.
// This equals IEEE x / s bit for bit unless the residual underflows, which needs a scale below
// ~2^-90, and the negated-residual form keeps the sign of a zero quotient (x = -0 gives -0).
__device__ __forceinline__ float2 quot_exact2(float2 nv, float2 s, float2 ny) {
    const float2 q0 = mul2(nv, ny);
    const float2 r = fma2(s, q0, nv);
    return fma2(r, ny, q0);
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// max(|a|, |b|, |c|) with the three-input max of sm_100 (absolute values are operand
// modifiers of the instruction, not separate operations)
__device__ __forceinline__ float max3abs(float a, float b, float c) {
    float r;
    asm("max.abs.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Fast sigmoid for a pair: 1 / (1 + 2^(-x*log2(e))) with the hardware ex2 / rcp
// approximations (each within 2 ulp).  Relative error of the result stays below ~4e-7
// wherever sigmoid(x) is not itself tiny, which is what bounds the error of block maxima.
__device__ __forceinline__ float2 sigmoid_fast2(float2 x) {
    const float2 t = mul2(x, splat2(-1.4426950408889634f));
    const float2 e = make_float2(ex2_approx(t.x), ex2_approx(t.y));
    const float2 d = add2(e, splat2(1.0f));
    return make_float2(rcp_approx(d.x), rcp_approx(d.y));
}

// ----------------------------------------------------------------------------------
// mbarrier + bulk copy (TMA) wrappers.  Every wait is bounded.
// ----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait (about two seconds of SM clock).  On give-up records `code` in the
// device status word and returns false; callers then stop issuing work.  The spin lives
// out of line so that the common case (data already there) costs two instructions.
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, int code);
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, code);
}

// Bounded wait without a function call: a call makes the compiler save every live register
// around it, which costs spills where many values are live across the wait.
__device__ __forceinline__ bool mbar_wait_inline(uint64_t* bar, uint32_t parity, int code) {
#pragma unroll 1
    for (uint32_t i = 0; i < (1u << 22); ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicCAS(&g_device_status, 0, code);
    return false;
}

// Wait used by the persistent kernels.  A wait that gives up does NOT make its thread leave the
// kernel: the thread records the code, marks itself `dead` and carries on with whatever the
// buffer holds, so every thread of the CTA still reaches every barrier, drains its stores and
// writes its partial results.  A dead thread skips all later waits, so a kernel spends at most
// one time limit per thread (they run out in parallel) before it finishes with the status word
// set; outputs of such a launch are undefined and the host learns of it from lh_device_status().
template <bool INLINE>
__device__ __forceinline__ void mbar_wait_or_mark(uint64_t* bar, uint32_t parity, int code, bool& dead) {
    if (dead) return;
    const bool ok = INLINE ? mbar_wait_inline(bar, parity, code) : mbar_wait(bar, parity, code);
    if (!ok) dead = true;
}

// The same bounded wait with a caller-chosen number of polls (self-test of the give-up path).
__device__ __forceinline__ bool mbar_wait_polls(uint64_t* bar, uint32_t parity, int code, uint32_t polls) {
#pragma unroll 1
    for (uint32_t i = 0; i < polls; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicCAS(&g_device_status, 0, code);
    return false;
}

// global -> shared bulk copy, completion counted in bytes on `bar`.
// src, dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// 2-D tiled tensor copy global -> shared through a tensor map (one instruction per tile).
// x = element column (x * element size must be a multiple of 16 bytes), y = row.
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst_smem)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// shared -> global bulk copy tracked by the thread's bulk async-group.
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// make generic-proxy shared-memory writes visible to the async proxy (bulk stores)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int ID, int N>
__device__ __forceinline__ void named_bar() {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(N) : "memory");
}

// 32 contiguous bytes per thread in one instruction (sm_100: 256-bit global accesses); the address
// must be 32-byte aligned.  A thread that owns 16 consecutive 16-bit elements then touches whole
// 32-byte sectors with every request instead of half of one.
__device__ __forceinline__ void ld_global_256(const void* p, uint4& a, uint4& b) {
    asm("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
        : "l"(p));
}
__device__ __forceinline__ void st_global_256(void* p, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z),
                 "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

__device__ __forceinline__ void st_global_v2(void* p, uint32_t a, uint32_t b) {
    *reinterpret_cast<uint2*>(p) = make_uint2(a, b);
}
// the same store under a predicate (one predicated instruction instead of a branch around it)
__device__ __forceinline__ void st_global_v2_if(bool pred, void* p, uint32_t a, uint32_t b) {
    asm volatile("{\n\t.reg .pred q;\n\t"
                 "setp.ne.u32 q, %3, 0;\n\t"
                 "@q st.global.v2.b32 [%0], {%1, %2};\n\t}"
                 ::"l"(p), "r"(a), "r"(b), "r"(uint32_t(pred))
                 : "memory");
}

}  // namespace lh
