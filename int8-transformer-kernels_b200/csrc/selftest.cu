// Bounded-wait plumbing: reading a workspace status word back, and a probe
// kernel that waits on a barrier nothing ever signals so the give-up path can
// be exercised without faulting, trapping or hanging the GPU.
#include "common.cuh"

namespace i8tk {
namespace {

__global__ void bounded_wait_probe_kernel(uint32_t* status, uint32_t polls) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
    }
    __syncthreads();
    bool ok = true;
    for (uint32_t i = 0; i < polls; ++i) {          // nobody arrives on this barrier
        ok = mbar_try_wait(b, 0, 1000u);            // each poll parks for at most ~1 us
        if (ok) break;
    }
    if (!ok && threadIdx.x == 0) note_timeout(status);
}

}  // namespace
}  // namespace i8tk

using namespace i8tk;

extern "C" int i8tk_selftest_bounded_wait(void* status_word, int polls, i8tk_stream_t stream) {
    I8TK_REQUIRE(status_word != nullptr && polls > 0 && polls <= (1 << 20), I8TK_ERR_INVALID_ARGUMENT,
                 "status_word must be a device pointer and 0 < polls <= 2^20");
    bounded_wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint32_t*>(status_word), (uint32_t)polls);
    I8TK_CUDA(cudaGetLastError());
    return I8TK_OK;
}

extern "C" int i8tk_check_status_word(const void* status_word, i8tk_stream_t stream) {
    I8TK_REQUIRE(status_word != nullptr, I8TK_ERR_INVALID_ARGUMENT, "null status word");
    uint32_t host = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    I8TK_CUDA(cudaMemcpyAsync(&host, status_word, sizeof(host), cudaMemcpyDeviceToHost, st));
    I8TK_CUDA(cudaStreamSynchronize(st));
    I8TK_REQUIRE(host != kDeviceTimeoutMagic, I8TK_ERR_DEVICE_TIMEOUT,
                 "a kernel gave up a bounded wait (status word 0x%x)", host);
    I8TK_REQUIRE(host != kDeviceBadIndexMagic, I8TK_ERR_INVALID_ARGUMENT,
                 "a page id outside [0, num_pages) was met on the device (page 0 was read in its place)");
    return I8TK_OK;
}
