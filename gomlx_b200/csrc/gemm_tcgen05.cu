// Prefill GEMM (m > 16): placeholder until the tcgen05 kernel lands.
#include "common.cuh"
namespace b200q {
int launch_gemm(const Weight &, const void *, int, int64_t, const float *, int, float *, int64_t, cudaStream_t) {
    return fail(B200Q_ENOTIMPL, "dense: m > 16 is not implemented yet");
}
}  // namespace b200q
