#include "fba_common.cuh"
using namespace fba;
extern "C" int fba_bwd_scratch_bytes(int B, int Hq, int Sq, uint64_t* lse_delta_bytes, uint64_t* dq_accum_bytes) {
    if (B <= 0 || Hq <= 0 || Sq <= 0 || !lse_delta_bytes || !dq_accum_bytes)
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd_scratch_bytes: bad argument");
    const uint64_t rows = static_cast<uint64_t>(B) * Hq * ((Sq + 127) / 128) * 128;
    *lse_delta_bytes = rows * 2 * sizeof(float);
    *dq_accum_bytes = rows * 128 * sizeof(float);
    return FBA_OK;
}
extern "C" int fba_bwd(const void*, const void*, const void*, const void*, const float*, const void*, void*, void*, void*, int, int, int, int, int, const fba_list_t*, float*, float*, uint32_t*, void*) {
    return set_error(FBA_ERR_BAD_ARG, "fba_bwd: not built yet");
}
