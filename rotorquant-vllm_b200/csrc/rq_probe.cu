// Measurement and self-test helpers of librq_b200 (no counterpart in the reference).
//
// rq_probe_mma_peak        how fast this GPU's tcgen05 tensor pipe runs back-to-back MMAs of one kind
//                          (INT8 or bf16) from shared-memory operands into tensor memory, with nothing
//                          else going on: the ceiling the INT8 prefill kernel is judged against.
// rq_selftest_bounded_wait lets one bounded mbarrier wait run out on purpose (a barrier nobody arrives
//                          on, a short limit) and reports what the wait returned: the same primitive
//                          every kernel of the library uses for its waits.
#include "rq_common.cuh"
#include "rq_tcgen05.cuh"

namespace rq {

constexpr int kProbeN = 256;                 // MMA N
constexpr int kProbeKSteps = 4;              // 32-byte K steps held in shared memory
constexpr uint32_t kProbeTmemCols = 512;     // two 128 x 256 accumulators

struct __align__(1024) ProbeSmem {
    uint8_t a[128 * 32 * kProbeKSteps];      // K-major core matrices: core (row/8)*8 + byte/16
    uint8_t b[kProbeN * 32 * kProbeKSteps];
    uint64_t bar;
    uint32_t tmem_base;
};

// KIND 0: kind::i8 (s8 x s8 -> s32), KIND 1: kind::f16 with bf16 operands (-> f32).
// One CTA per SM; thread 0 issues `iters` rounds of kProbeKSteps MMAs of 128 x 256 x 32 bytes,
// alternating between two accumulators, then commits and waits (bounded).
template <int KIND>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int iters, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    ProbeSmem& sm = *reinterpret_cast<ProbeSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const int tid = threadIdx.x;
    // finite, non-constant operand bytes (0x30..0x3F: small positive int8 / bf16 values); a and b are adjacent
    for (int i = tid; i < static_cast<int>(sizeof(sm.a) + sizeof(sm.b)) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(sm.a)[i] = 0x30303030u | ((static_cast<uint32_t>(i) * 0x01030507u) & 0x0F0F0F0Fu);
    if (tid == 0) {
        mbar_init(&sm.bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_async_proxy();
    if (tid < 32) tmem_alloc(&sm.tmem_base, kProbeTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    bool ok = true;
    if (tid == 0) {
        const uint32_t a_addr = smem_u32(sm.a), b_addr = smem_u32(sm.b);
        const uint32_t idesc = KIND == 0
            ? ((2u << 4) | (1u << 7) | (1u << 10) | ((kProbeN >> 3) << 17) | ((128u >> 4) << 24))
            : ((1u << 4) | (1u << 7) | (1u << 10) | ((kProbeN >> 3) << 17) | ((128u >> 4) << 24));
#pragma unroll 1
        for (int it = 0; it < iters; ++it) {
            const uint32_t d = tmem + (it & 1) * kProbeN;
#pragma unroll
            for (int s = 0; s < kProbeKSteps; ++s) {
                if constexpr (KIND == 0)
                    tc_mma_i8(d, smem_desc(a_addr + 256 * s, 128, 1024), smem_desc(b_addr + 256 * s, 128, 1024), idesc,
                              (it > 1 || s > 0) ? 1u : 0u);
                else
                    tc_mma_f16(d, smem_desc(a_addr + 256 * s, 128, 1024), smem_desc(b_addr + 256 * s, 128, 1024), idesc,
                               (it > 1 || s > 0) ? 1u : 0u);
            }
        }
        tc_commit(&sm.bar);
        ok = mbar_wait(&sm.bar, 0);
        if (!ok && status != nullptr) atomicExch(status, 1);
    }
    tc_fence_before();
    __syncthreads();
    if (tid < 32) tmem_dealloc(tmem, kProbeTmemCols);
}

// One thread waits on a barrier that nobody arrives on; the wait must return false after about
// `limit_cycles` SM clocks.  status[0] = 1 when it did (0 if the wait claimed success),
// status[1] = clocks the wait took, in units of 1024.
__global__ void bounded_wait_kernel(long long limit_cycles, int* __restrict__ status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const long long t0 = clock64();
        const bool done = mbar_wait_for(&bar, 0, limit_cycles);
        const long long t1 = clock64();
        status[0] = done ? 0 : 1;
        status[1] = static_cast<int>((t1 - t0) >> 10);
    }
}

}  // namespace rq

using namespace rq;

extern "C" int rq_probe_mma_peak(int kind, int iters, double* ops_out, int* status_dev, void* stream) {
    if ((kind != 0 && kind != 1) || iters <= 0 || iters > (1 << 20))
        return fail(RQ_ERR_INVALID_ARG, "rq_probe_mma_peak: kind must be 0 (int8) or 1 (bf16), iters in [1, 2^20]");
    int dev = 0, sms = 0;
    if (int e = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return e;
    if (int e = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute"))
        return e;
    const size_t smem = sizeof(ProbeSmem) + 1024;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (kind == 0) {
        if (int e = ensure_smem(mma_peak_kernel<0>, smem)) return e;
        mma_peak_kernel<0><<<sms, 128, smem, st>>>(iters, status_dev);
    } else {
        if (int e = ensure_smem(mma_peak_kernel<1>, smem)) return e;
        mma_peak_kernel<1><<<sms, 128, smem, st>>>(iters, status_dev);
    }
    // multiply-adds x 2 of one launch: K is 32 elements per step for int8, 16 for bf16
    if (ops_out != nullptr)
        *ops_out = 2.0 * 128.0 * kProbeN * (kind == 0 ? 32.0 : 16.0) * kProbeKSteps * static_cast<double>(iters) * sms;
    return check_cuda(cudaGetLastError(), "rq_probe_mma_peak launch");
}

extern "C" int rq_selftest_bounded_wait(long long limit_cycles, int* status_dev, void* stream) {
    if (limit_cycles <= 0 || limit_cycles > kWaitCycles || status_dev == nullptr)
        return fail(RQ_ERR_INVALID_ARG, "rq_selftest_bounded_wait: limit must be in (0, 2e9] cycles and status non-null");
    bounded_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, status_dev);
    return check_cuda(cudaGetLastError(), "rq_selftest_bounded_wait launch");
}
