// Error reporting, version query and TMA tensor-map construction for libfba_b200.so.
#include <stdio.h>
#include <string.h>

#include <nvtx3/nvToolsExt.h>

#include "fba_internal.cuh"

namespace fba {

static thread_local char g_err[512] = "";

int set_error(int code, const char* msg) {
    snprintf(g_err, sizeof(g_err), "%s", msg ? msg : "");
    return code;
}

static unsigned long long g_launches = 0;
static thread_local cudaEvent_t g_ev_start = nullptr, g_ev_stop = nullptr;
static thread_local int g_ev_which = 0;

void timing_mark(int which, bool start, cudaStream_t stream) {
    if (which != g_ev_which) return;
    cudaEvent_t ev = start ? g_ev_start : g_ev_stop;
    if (ev) cudaEventRecord(ev, stream);
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) {
        __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED);
        return FBA_OK;
    }
    snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return FBA_ERR_LAUNCH;
}

// Driver entry points are resolved through the runtime so the library has no link-time dependency
// on libcuda (it is built on machines without a driver).
static void* driver_entry(const char* name) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

typedef CUresult (*CtxGetFn)(CUcontext*);
typedef CUresult (*CtxSetFn)(CUcontext);
static CtxGetFn ctx_get_fn() {
    static CtxGetFn fn = reinterpret_cast<CtxGetFn>(driver_entry("cuCtxGetCurrent"));
    return fn;
}
static CtxSetFn ctx_set_fn() {
    static CtxSetFn fn = reinterpret_cast<CtxSetFn>(driver_entry("cuCtxSetCurrent"));
    return fn;
}

int DeviceGuard::bind(const void* ptr) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, ptr) != cudaSuccess || a.type != cudaMemoryTypeDevice) {
        cudaGetLastError();
        return set_error(FBA_ERR_BAD_ARG, "pointer is not device memory");
    }
    CtxGetFn get = ctx_get_fn();
    if (get && ctx_set_fn() && get(&prev_) == CUDA_SUCCESS) armed_ = true;
    if (cudaSetDevice(a.device) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "cudaSetDevice failed for the device that owns the buffers");
    }
    return FBA_OK;
}

int DeviceGuard::bind_current() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "cudaGetDevice failed");
    }
    CtxGetFn get = ctx_get_fn();
    if (get && ctx_set_fn() && get(&prev_) == CUDA_SUCCESS) armed_ = true;
    if (cudaSetDevice(dev) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "cudaSetDevice failed");
    }
    return FBA_OK;
}

DeviceGuard::~DeviceGuard() {
    if (!armed_) return;
    CUcontext now = nullptr;
    if (ctx_get_fn()(&now) == CUDA_SUCCESS && now != prev_) ctx_set_fn()(prev_);
}

ProfRange::ProfRange(const char* name) { nvtxRangePushA(name); }
ProfRange::~ProfRange() { nvtxRangePop(); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) fn = reinterpret_cast<EncodeTiledFn>(driver_entry("cuTensorMapEncodeTiled"));
    return fn;
}

int make_tmap_bf16(CUtensorMap* out, const void* base, int seq, long long n_bh, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(FBA_ERR_DRIVER, "cuTensorMapEncodeTiled is not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
        return set_error(FBA_ERR_BAD_ARG, "tensor base address must be 16-byte aligned");
    cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(n_bh)};
    cuuint64_t strides[2] = {128 * 2, static_cast<cuuint64_t>(seq) * 128 * 2};
    cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[128];
        snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return set_error(FBA_ERR_DRIVER, buf);
    }
    return FBA_OK;
}

int make_tmap_u8(CUtensorMap* out, const void* base, long long inner, long long rows, long long n_bh) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(FBA_ERR_DRIVER, "cuTensorMapEncodeTiled is not available");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || inner % 16 != 0)
        return set_error(FBA_ERR_BAD_ARG, "8-bit tensor base address and row length must be multiples of 16 bytes");
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(n_bh)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(inner) * static_cast<cuuint64_t>(rows)};
    cuuint32_t box[3] = {128, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[128];
        snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled (8-bit) failed with CUresult %d", (int)r);
        return set_error(FBA_ERR_DRIVER, buf);
    }
    return FBA_OK;
}

}  // namespace fba

extern "C" int fba_abi_version(void) { return FBA_ABI_VERSION; }
extern "C" uint64_t fba_launch_count(void) { return __atomic_load_n(&fba::g_launches, __ATOMIC_RELAXED); }
extern "C" int fba_set_timing_events(int which, void* start_event, void* stop_event) {
    if (which < 0 || which > 3) return fba::set_error(FBA_ERR_BAD_ARG, "fba_set_timing_events: which must be 0, 1, 2 or 3");
    if (which != 0 && (!start_event || !stop_event))
        return fba::set_error(FBA_ERR_BAD_ARG, "fba_set_timing_events: null event");
    fba::g_ev_which = which;
    fba::g_ev_start = static_cast<cudaEvent_t>(start_event);
    fba::g_ev_stop = static_cast<cudaEvent_t>(stop_event);
    return FBA_OK;
}
extern "C" const char* fba_last_error(void) { return fba::g_err; }

extern "C" int fba_check_status(uint32_t* status, void* stream_) {
    using namespace fba;
    if (!status) return set_error(FBA_ERR_BAD_ARG, "fba_check_status: null status buffer");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DeviceGuard guard;
    int rc = guard.bind(status);
    if (rc != FBA_OK) return rc;
    uint32_t w[StatusWords::kCount] = {0};
    if (cudaMemcpyAsync(w, status, sizeof(w), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {
        cudaError_t e = cudaGetLastError();
        char buf[256];
        snprintf(buf, sizeof(buf), "fba_check_status: reading the status words failed: %s", cudaGetErrorString(e));
        return set_error(FBA_ERR_LAUNCH, buf);
    }
    if (w[StatusWords::kFlag] == 0) return FBA_OK;
    cudaMemsetAsync(status, 0, sizeof(w), stream);
    char buf[256];
    snprintf(buf, sizeof(buf),
             "a device-side wait timed out (kernel=%u role=%u block=(%u,%u) iter=%u tag=%u); the outputs of that "
             "call are undefined",
             w[StatusWords::kKernel], w[StatusWords::kRole], w[StatusWords::kBx], w[StatusWords::kBy],
             w[StatusWords::kIter], w[StatusWords::kTag]);
    return set_error(FBA_ERR_TIMEOUT, buf);
}
