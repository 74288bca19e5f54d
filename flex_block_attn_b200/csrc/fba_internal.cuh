// Host-side helpers shared by the translation units of libfba_b200.so: error reporting,
// launch checking, device binding and TMA tensor-map construction.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fba.h"

namespace fba {

// Record `msg` as the calling thread's last error and return `code`.
int set_error(int code, const char* msg);
// cudaGetLastError() after a launch; returns FBA_OK or FBA_ERR_LAUNCH (with text recorded).
int check_launch(const char* what);

// Makes the device that owns a buffer current for the lifetime of the guard and puts the calling
// thread's previous CUDA context back when the guard goes out of scope, so an entry point leaves no
// trace in the caller's device selection.  Callers may arrive on threads that never touched CUDA
// (e.g. an autograd worker), where no context is current yet and the driver-level tensor-map
// encoder would fail; such a thread is left without a current context again afterwards.
class DeviceGuard {
  public:
    DeviceGuard() = default;
    ~DeviceGuard();
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
    // Switch to the device that owns `ptr` (must be device memory).  FBA_OK or an error code.
    int bind(const void* ptr);
    // Switch to the device that is current in the runtime (for calls that take no buffer).
    int bind_current();

  private:
    bool armed_ = false;
    CUcontext prev_ = nullptr;
};

// Named range on the profiler timeline (NVTX) covering one entry point; a no-op without a tool.
class ProfRange {
  public:
    explicit ProfRange(const char* name);
    ~ProfRange();
};

// Record the caller-supplied timing event (fba_set_timing_events) around main kernel `which`
// (1 = forward, 2 = backward main kernel, 3 = query-major dQ kernel); no-op unless that kernel was
// selected on this thread.
void timing_mark(int which, bool start, cudaStream_t stream);

// 3-D bf16 tensor map over a [n_bh, seq, 128] tensor viewed as (col, row, bh), box = 64 columns x
// `box_rows` rows x 1, 128-byte swizzle, out-of-range rows read as zero and are dropped on store.
int make_tmap_bf16(CUtensorMap* out, const void* base, int seq, long long n_bh, int box_rows);

// 3-D 8-bit tensor map over a [n_bh, rows, inner] byte tensor viewed as (inner, row, bh), box = 128 bytes x
// 128 rows x 1, 128-byte swizzle: one box is one [128][128] e4m3 operand tile.
int make_tmap_u8(CUtensorMap* out, const void* base, long long inner, long long rows, long long n_bh);

// Status-word layout written by the attention kernels when a bounded wait gives up.
//   [0] non-zero flag   [1] kernel id (1 fwd, 2 bwd, 3 dQ, 9 self-test)   [2] role id
//   [3] blockIdx.x      [4] blockIdx.y      [5] iteration                [6] barrier tag
struct StatusWords {
    enum { kFlag = 0, kKernel = 1, kRole = 2, kBx = 3, kBy = 4, kIter = 5, kTag = 6, kCount = 8 };
};

}  // namespace fba
