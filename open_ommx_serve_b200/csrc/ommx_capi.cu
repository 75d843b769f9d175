// Library-wide pieces of the C ABI: error text, launch counter, ABI version, and the host-side
// twins of the quantizer's two table-driven decisions.
#include "ommx_common.cuh"

namespace ommx {

std::atomic<long long> g_launches{0};

char *last_error_buf() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buf(), 512, fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace ommx

extern "C" int ommx_b200_abi_version(void) { return OMMX_B200_ABI_VERSION; }
extern "C" const char *ommx_b200_last_error(void) { return ommx::last_error_buf(); }
extern "C" int64_t ommx_b200_launch_count(void) { return (int64_t)ommx::g_launches.load(); }
extern "C" void ommx_b200_reset_launch_count(void) { ommx::g_launches.store(0); }

extern "C" int ommx_b200_host_pow2_exponent(float x) {
    return ommx::pow2_exponent_tbl(x, ommx::kPow2CutHost);
}
extern "C" int ommx_b200_host_fp4_encode(float m) {
    return ommx::fp4_encode_tbl(m, ommx::kFp4ThreshHost);
}

// ---- device memory other processes of the node can map (for the head-output exchange) ----------
extern "C" int ommx_b200_peer_alloc(size_t bytes, void **ptr, void *handle64) {
    using namespace ommx;
    if (!ptr || !handle64 || bytes == 0) return fail(OMMX_E_ARG, "peer_alloc: ptr, handle64 and a size are needed");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed as 64 bytes");
    void *p = nullptr;
    OMMX_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(OMMX_E_CUDA, "peer_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(handle64, &h, 64);
    *ptr = p;
    return 0;
}
extern "C" int ommx_b200_peer_open(const void *handle64, void **ptr) {
    using namespace ommx;
    if (!ptr || !handle64) return fail(OMMX_E_ARG, "peer_open: handle64 and ptr are needed");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    OMMX_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}
extern "C" int ommx_b200_peer_close(void *ptr) {
    using namespace ommx;
    if (!ptr) return 0;
    OMMX_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return 0;
}
extern "C" int ommx_b200_peer_free(void *ptr) {
    using namespace ommx;
    if (!ptr) return 0;
    OMMX_CUDA_TRY(cudaFree(ptr));
    return 0;
}
