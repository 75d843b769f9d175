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
