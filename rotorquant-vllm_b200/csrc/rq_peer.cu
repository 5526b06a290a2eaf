// Arrive-and-wait between the GPUs of a head-sharded decode, sm_100a.
//
// After rq_decode_sharded every GPU has written its head outputs into all GPUs' gathered buffers with
// plain stores into peer memory.  What is left of the all-gather is to learn that every peer's stores
// have landed here: rq_peer_barrier launches one warp that writes this GPU's step number into a slot of
// every peer's flag array (symmetric memory mapped into this process) and then waits until all of its
// own slots have reached that number.  Step numbers only grow, so nothing is ever reset, and they live
// in device memory, so the launch can be replayed from a CUDA graph.  The wait is bounded: when it
// runs out the kernel records that in `state[1]` and returns; nothing traps.
//
// There is no counterpart in the reference (it has no multi-GPU path of its own); the collective this
// replaces is the all-gather of attention outputs that tensor parallelism runs after the layer.
#include "rq_common.cuh"

namespace rq {

constexpr int kBarrierPeers = 8;

struct PeerFlags {
    unsigned long long* flags[kBarrierPeers];     // flag array [world] of every GPU, as mapped here
};

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// state[0] = steps completed on this GPU, state[1] = 1 once a wait has run out.
__global__ void __launch_bounds__(32)
peer_barrier_kernel(const PeerFlags peers, int world, int rank, unsigned long long* __restrict__ state,
                    long long limit_cycles) {
    const int lane = threadIdx.x;
    const unsigned long long step = state[0] + 1;
    __syncwarp();
    bool expired = false;
    if (lane < world) {
        st_release_sys(peers.flags[lane] + rank, step);            // "my stores of this step are out"
        const unsigned long long* mine = peers.flags[rank] + lane;  // written by GPU `lane`
        const long long t0 = clock64();
        while (ld_acquire_sys(mine) < step) {
            if (clock64() - t0 > limit_cycles) { expired = true; break; }
            __nanosleep(100);
        }
    }
    expired = __any_sync(0xffffffffu, expired);
    if (lane == 0) {
        state[0] = step;
        if (expired) state[1] = 1;
    }
}

}  // namespace rq

using namespace rq;

extern "C" int rq_peer_barrier(void* const* peer_flags, int world, int rank, void* state,
                               long long limit_cycles, void* stream) {
    if (world <= 0 || world > kBarrierPeers || rank < 0 || rank >= world)
        return fail(RQ_ERR_INVALID_ARG, "rq_peer_barrier: rank %d of %d (at most %d GPUs)", rank, world, kBarrierPeers);
    if (!peer_flags || !state) return fail(RQ_ERR_INVALID_ARG, "rq_peer_barrier: null pointer");
    if (limit_cycles <= 0) limit_cycles = 2000000000LL;             // about one second of SM clocks
    PeerFlags pf{};
    for (int g = 0; g < world; ++g) {
        if (!peer_flags[g] || !aligned(peer_flags[g], 8))
            return fail(RQ_ERR_ALIGNMENT, "rq_peer_barrier: flag array %d must be a non-null 8-byte aligned pointer", g);
        pf.flags[g] = static_cast<unsigned long long*>(peer_flags[g]);
    }
    if (!aligned(state, 8)) return fail(RQ_ERR_ALIGNMENT, "rq_peer_barrier: state must be 8-byte aligned");
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        pf, world, rank, static_cast<unsigned long long*>(state), limit_cycles);
    return check_cuda(cudaGetLastError(), "rq_peer_barrier launch");
}
