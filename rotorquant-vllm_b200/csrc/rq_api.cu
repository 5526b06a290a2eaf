// Library identification and per-thread error text of librq_b200.
#include <map>
#include <mutex>
#include <utility>

#include "rq_common.cuh"

namespace rq {

int ensure_smem_impl(const void* kernel, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, size_t> granted;
    int dev = 0;
    if (int e = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return e;
    std::lock_guard<std::mutex> lock(mu);
    auto it = granted.find({kernel, dev});
    if (it != granted.end() && it->second >= bytes) return RQ_OK;
    if (int e = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(bytes)),
                           "cudaFuncSetAttribute"))
        return e;
    granted[{kernel, dev}] = bytes;
    return RQ_OK;
}

char* error_buffer() {
    static thread_local char buf[kErrorBufferBytes] = {0};
    return buf;
}
}  // namespace rq

extern "C" const char* rq_version(void) { return "rq_b200 0.1 (sm_100a)"; }

extern "C" const char* rq_last_error(void) { return rq::error_buffer(); }
