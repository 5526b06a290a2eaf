// Shared host/device helpers of librq_b200: status handling, dtype loads,
// small PTX wrappers.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/rq_b200.h"

namespace rq {

constexpr int kHeadDim = 128;       // the only head size the kernels are built for
constexpr int kHalfDim = 64;        // packed index bytes per (token, head)
constexpr int kSlotPerHead = 256;   // next_pow2(2 * (64 + 4)) bytes per head in a slot

// Thread-local message buffer behind rq_last_error().
char* error_buffer();
constexpr size_t kErrorBufferBytes = 512;

template <typename... Args>
inline int fail(int code, const char* fmt, Args... args) {
    snprintf(error_buffer(), kErrorBufferBytes, fmt, args...);
    return code;
}
inline int fail(int code, const char* msg) {
    snprintf(error_buffer(), kErrorBufferBytes, "%s", msg);
    return code;
}

inline int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return RQ_OK;
    return fail(RQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// Raise a kernel's dynamic shared-memory limit; remembered per (kernel, device) so that later
// launches skip the driver call.  Safe to call before every launch and from several threads.
int ensure_smem_impl(const void* kernel, size_t bytes);
template <typename Kernel>
inline int ensure_smem(Kernel k, size_t bytes) {
    return ensure_smem_impl(reinterpret_cast<const void*>(k), bytes);
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int dtype_bytes(int dt) { return dt == RQ_DTYPE_F32 ? 4 : 2; }

// Region offsets of one cache slot for H heads on this GPU.
struct SlotLayout {
    int k_idx, k_norm, v_idx, v_norm, payload_end, total;
};
__host__ __device__ inline SlotLayout slot_layout(int H) {
    SlotLayout l;
    l.k_idx = 0;
    l.k_norm = H * kHalfDim;
    l.v_idx = l.k_norm + H * 4;
    l.v_norm = l.v_idx + H * kHalfDim;
    l.payload_end = l.v_norm + H * 4;
    l.total = H * kSlotPerHead;
    return l;
}

// ---- device helpers --------------------------------------------------------

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// fp32 value of element i of a 16-byte chunk holding `T` elements.
template <typename T>
struct Chunk16;
template <>
struct Chunk16<float> {
    static constexpr int kElems = 4;
    __device__ static void unpack(const uint4& c, float* out) {
        out[0] = __uint_as_float(c.x); out[1] = __uint_as_float(c.y);
        out[2] = __uint_as_float(c.z); out[3] = __uint_as_float(c.w);
    }
};
template <>
struct Chunk16<__half> {
    static constexpr int kElems = 8;
    __device__ static void unpack(const uint4& c, float* out) {
        const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            float2 f = __half22float2(h);
            out[2 * i] = f.x; out[2 * i + 1] = f.y;
        }
    }
};
template <>
struct Chunk16<__nv_bfloat16> {
    static constexpr int kElems = 8;
    __device__ static void unpack(const uint4& c, float* out) {
        const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}


// ---- mbarrier (shared-memory barrier objects) -----------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
// Wait until the phase with the given parity has completed.  Every wait in this library is
// bounded (about one second of SM clocks); false means the bound expired.
// One non-blocking look: has the phase with the given parity completed?
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
constexpr long long kWaitCycles = 2000000000LL;
__device__ __forceinline__ bool mbar_wait_for(uint64_t* bar, uint32_t parity, long long limit_cycles) {
    const uint32_t addr = smem_u32(bar);
    long long start = 0;
    for (int spin = 0;; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (spin == 0) start = clock64();
        else if (clock64() - start > limit_cycles) return false;
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    return mbar_wait_for(bar, parity, kWaitCycles);
}

}  // namespace rq
