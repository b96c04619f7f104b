// Shared device/host helpers for the sm_100a paged-KV kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ivab.h"

namespace ivab {

// Bits of the device-side status word (mirrored in include/ivab.h).
constexpr int kStatusWaitTimeout = IVAB_STATUS_WAIT_TIMEOUT;
constexpr int kStatusBadPage     = IVAB_STATUS_BAD_PAGE;
constexpr int kStatusBadCtxLen   = IVAB_STATUS_BAD_CTX_LEN;
constexpr int kStatusBadSlot     = IVAB_STATUS_BAD_SLOT;
constexpr int kStatusOverflow    = IVAB_STATUS_WORKSPACE_OVERFLOW;

// Host-side error plumbing (defined in abi.cu).
int  set_error(int code, const char* fmt, ...);
int  check_cuda(cudaError_t e, const char* what);
int  sm_count();                      // SMs of the current device (cached per device)
size_t dtype_size(int dtype);

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier -------------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization
// attribute may start while its predecessor in the stream still runs; grid_dependency_wait() then
// blocks until the predecessor has completed and its writes are visible (a no-op for a kernel
// launched the ordinary way).  grid_launch_dependents() lets the successor's CTAs be scheduled as
// soon as every CTA of this grid has called it or exited.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void fence_mbar_init() {
    // Makes the initialised barriers visible to the async (TMA) proxy.
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Every wait in these kernels is bounded: after `limit_ns` without the phase completing the
// waiter raises the CTA-wide abort flag and returns false; a waiter that sees the flag raised
// by someone else also returns false.  The caller then unwinds instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (((++spins) & 63u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// ---- TMA bulk copy (global -> shared, this CTA only) --------------------------------------------

__device__ __forceinline__ void tma_bulk_g2s(uint32_t dst_smem, const void* src_global, uint32_t bytes,
                                             uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_smem), "l"(src_global), "r"(bytes), "r"(bar)
        : "memory");
}

// L2 policy for data that is read exactly once (the K/V stream): evict first, so that the pages do
// not push the block tables, partials and q out of the cache.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ void tma_bulk_g2s_hint(uint32_t dst_smem, const void* src_global, uint32_t bytes,
                                                  uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst_smem), "l"(src_global), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_tile4d_g2s_hint(uint32_t dst_smem, const void* tensor_map, int c0, int c1, int c2,
                                                    int c3, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;"
        ::"r"(dst_smem), "l"(tensor_map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "l"(policy)
        : "memory");
}

// Tiled TMA copy (4-D tensor map, this CTA only): one box lands in shared memory with the swizzle
// recorded in the map.  The innermost coordinate times the element size must be a multiple of 16.
__device__ __forceinline__ void tma_tile4d_g2s(uint32_t dst_smem, const void* tensor_map, int c0, int c1, int c2,
                                               int c3, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst_smem), "l"(tensor_map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}

// Orders this thread's earlier generic-proxy accesses (ordinary loads and stores, global memory included)
// before later accesses of the async proxy (TMA copies) -- needed when a TMA copy must see what ordinary
// stores of the same CTA have just written to global memory.
__device__ __forceinline__ void fence_proxy_async_all() {
    asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Brings a tensor map (the 128-byte descriptor a tiled TMA copy reads) into the descriptor cache ahead of
// its first use.
__device__ __forceinline__ void prefetch_tensormap(const void* tensor_map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensor_map)) : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- warp-level matrix helpers (16-bit operands, fp32 accumulate) ---------------------------------

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// D(16x8) += A(16x16) * B(16x8) where rows 8..15 of A are zero: only the two accumulators of
// rows 0..7 (c0, c1) are live; the other two stay zero and are discarded.
template <typename T>
__device__ __forceinline__ void mma_m16n8k16_top(float (&c)[2], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma_m16n8k16_top<__nv_bfloat16>(float (&c)[2], uint32_t a0, uint32_t a2, uint32_t b0,
                                                                uint32_t b1) {
    float z2 = 0.f, z3 = 0.f;   // rows 8..15 of the tile: zero in, zero out
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(z2), "+f"(z3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

template <>
__device__ __forceinline__ void mma_m16n8k16_top<__half>(float (&c)[2], uint32_t a0, uint32_t a2, uint32_t b0,
                                                         uint32_t b1) {
    float z2 = 0.f, z3 = 0.f;   // rows 8..15 of the tile: zero in, zero out
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(z2), "+f"(z3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// Two e4m3 bytes (low byte first) to two fp16 values in one register; exact.
__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return r;
}

// Bytes of {a, b} picked by the four selector nibbles (0..3 = bytes of a, 4..7 = bytes of b).
__device__ __forceinline__ uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Full tile: rows 0..7 take a0/a2, rows 8..15 take a1/a3; all four accumulators are live.
template <typename T>
__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_m16n8k16<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                            uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_m16n8k16<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                     uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
}

// ---- small numeric helpers -------------------------------------------------------------------

__device__ __forceinline__ float warp_max_f32(float v) {
    // redux.sync on f32 exists on sm_100a; one instruction instead of five shuffles.
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ float warp_sum_f32(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T> struct Elt;
template <> struct Elt<float> {
    static constexpr int kPerVec = 4;
    __device__ __forceinline__ static void unpack(const uint4& u, float* f) {
        f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
    }
    __device__ __forceinline__ static float load(const float* p) { return *p; }
    __device__ __forceinline__ static void store(float* p, float v) { *p = v; }
};
template <> struct Elt<__nv_bfloat16> {
    static constexpr int kPerVec = 8;
    __device__ __forceinline__ static void unpack(const uint4& u, float* f) {
        // bf16 is the high half of an fp32: a shift or a mask per element.
        f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
        f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
        f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
        f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
    }
    __device__ __forceinline__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ __forceinline__ static void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Elt<__half> {
    static constexpr int kPerVec = 8;
    __device__ __forceinline__ static void unpack(const uint4& u, float* f) {
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(h[i]);
            f[2 * i] = t.x; f[2 * i + 1] = t.y;
        }
    }
    __device__ __forceinline__ static float load(const __half* p) { return __half2float(*p); }
    __device__ __forceinline__ static void store(__half* p, float v) { *p = __float2half_rn(v); }
};

template <> struct Elt<__nv_fp8_e4m3> {
    static constexpr int kPerVec = 16;
    // e4m3 -> fp32 is exact: two values per conversion to half2, then widened
    __device__ __forceinline__ static void unpack(const uint4& u, float* f) {
        const __nv_fp8x2_storage_t* p2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(p2[i], __NV_E4M3);
            const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&h));
            f[2 * i] = t.x; f[2 * i + 1] = t.y;
        }
    }
};

// fp32 -> e4m3 with saturation (round to nearest even), two at a time
__device__ __forceinline__ uint16_t pack_fp8x2(float lo, float hi) {
    return __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}

#endif  // __CUDACC__

}  // namespace ivab
