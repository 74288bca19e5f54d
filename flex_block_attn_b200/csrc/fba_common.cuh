// Device-side definitions shared by the forward and backward attention kernels.
#pragma once
#include "fba_internal.cuh"
#include "ptx.cuh"

namespace fba {

constexpr uint32_t kPanelBytes = 16384;  // [128 rows][64 bf16], 128-byte pitch, swizzled
constexpr uint32_t kTileBytes = 32768;   // two panels = one 128 x 128 bf16 tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kSoftmaxScale = 0.08838834764831845f;  // 1/sqrt(128), fixed like the reference

// UMMA instruction descriptors, M = 128, N = 128, bf16 -> fp32.
constexpr uint32_t kIdescKK = umma_idesc(128, 128, 0, 0);   // A K-major,  B K-major
constexpr uint32_t kIdescKM = umma_idesc(128, 128, 0, 1);   // A K-major (or TMEM), B MN-major
constexpr uint32_t kIdescMM = umma_idesc(128, 128, 1, 1);   // A MN-major, B MN-major

// Device view of fba_list_t.
struct ListDev {
    const int32_t* idx;
    const int32_t* cnt;
    const uint16_t* msk;
    const int32_t* order;   // optional work-item order (see fba_fwd_order / fba_bwd_order), or null
    int stride, rows_per_bh, bh_stride, rows_div, sub;
};

inline ListDev to_dev(const fba_list_t& l) {
    return ListDev{l.idx, l.cnt, l.msk, l.order, l.stride, l.rows_per_bh, l.bh_stride, l.rows_div, l.sub};
}

// Optional timeline probe for tuning (compiled out unless -DFBA_TRACE): CTA (0,0) stores SM clock
// stamps as 64-bit words after the 8 status words, so the status buffer must then be large.
#ifdef FBA_TRACE
#define FBA_TRACE_REC(status, idx)                                                              \
    do {                                                                                        \
        if (blockIdx.x == 0 && blockIdx.y == 0)                                                 \
            reinterpret_cast<unsigned long long*>(status)[8 + (idx)] = clock64();               \
    } while (0)
#else
#define FBA_TRACE_REC(status, idx) \
    do {                           \
    } while (0)
#endif

// Record the first place a bounded wait gave up.
__device__ __forceinline__ void report_timeout(uint32_t* status, uint32_t kernel, uint32_t role,
                                               uint32_t iter, uint32_t tag) {
    if (atomicCAS(status + StatusWords::kFlag, 0u, 1u) == 0u) {
        status[StatusWords::kKernel] = kernel;
        status[StatusWords::kRole] = role;
        status[StatusWords::kBx] = blockIdx.x;
        status[StatusWords::kBy] = blockIdx.y;
        status[StatusWords::kIter] = iter;
        status[StatusWords::kTag] = tag;
    }
}

// D[128 x 128] (+)= A * B^T, both operands K-major 128 x 128 bf16 tiles in shared memory
// (contraction over the 128 columns).
__device__ __forceinline__ void mma_tile_kk(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem,
                                            bool accumulate) {
    const uint32_t a = desc_lo_kmajor(a_smem), b = desc_lo_kmajor(b_smem);
#pragma unroll
    for (int k = 0; k < 8; ++k)
        umma_ss(d_tmem, a + kstep_kmajor(k), b + kstep_kmajor(k), kIdescKK, (accumulate || k > 0) ? 1u : 0u);
}
// D[128 x 128] (+)= A * B with A[128 x 128] bf16 in TMEM (row = lane, 8 columns per 16 k) and
// B[k = 128 rows][n = 128 columns] MN-major in shared memory.  `a_tmem_hi` is the TMEM address of
// k-steps 4..7 (A need not be column-contiguous across its two halves).
__device__ __forceinline__ void mma_tile_tm(uint32_t d_tmem, uint32_t a_tmem_lo, uint32_t a_tmem_hi,
                                            uint32_t b_smem, bool accumulate) {
    const uint32_t b = desc_lo_mnmajor(b_smem);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint32_t a = (k < 4 ? a_tmem_lo : a_tmem_hi) + static_cast<uint32_t>(k & 3) * 8u;
        umma_ts(d_tmem, a, b + kstep_mnmajor(k), kIdescKM, (accumulate || k > 0) ? 1u : 0u);
    }
}
// D[128 x 128] (+)= A * B, A K-major in smem ([m][k]), B MN-major in smem ([k][n]).
__device__ __forceinline__ void mma_tile_km(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem,
                                            bool accumulate) {
    const uint32_t a = desc_lo_kmajor(a_smem), b = desc_lo_mnmajor(b_smem);
#pragma unroll
    for (int k = 0; k < 8; ++k)
        umma_ss(d_tmem, a + kstep_kmajor(k), b + kstep_mnmajor(k), kIdescKM, (accumulate || k > 0) ? 1u : 0u);
}
// D[128 x 128] (+)= A^T-stored * B, both MN-major in smem: A stored [k][m], B stored [k][n].
__device__ __forceinline__ void mma_tile_mm(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem,
                                            bool accumulate) {
    const uint32_t a = desc_lo_mnmajor(a_smem), b = desc_lo_mnmajor(b_smem);
#pragma unroll
    for (int k = 0; k < 8; ++k)
        umma_ss(d_tmem, a + kstep_mnmajor(k), b + kstep_mnmajor(k), kIdescMM, (accumulate || k > 0) ? 1u : 0u);
}

}  // namespace fba
