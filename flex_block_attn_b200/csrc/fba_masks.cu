// Mask builders that emit index lists on the device, for the two mask families the reference
// advertises without shipping code for them (reference flex_block_attn/__init__.py:7-12 is
// commented out, README.md:54-55): the 3-D sliding-tile window (STA) and the hybrid of that window
// with a MoBA-style top-k of pooled query.key scores (SSTA).  They replace the torch expressions
// in flex_block_attn_b200/masks.py on the hot path: no [nQ, nK] score matrix round trip through
// topk / scatter / logical-or, and for STA no bool mask at all.
//
// Integer outputs follow the list format of fba_build_index (ascending, -1 padded) and are
// bit-identical to compacting the corresponding bool mask.
#include "fba_internal.cuh"

#include <cuda_bf16.h>

namespace fba {

// ---------------------------------------------------------------------------------------------
// STA: tile i attends tile j iff |dt| <= wt, |dh| <= wh, |dw| <= ww in tile coordinates; tile id =
// (t * Gh + h) * Gw + w.  The relation is symmetric, so one list serves both directions.
// One thread per tile; neighbours are visited in ascending id order.
__global__ void sta_lists_kernel(int Gt, int Gh, int Gw, int wt, int wh, int ww, int32_t* __restrict__ idx,
                                 int32_t* __restrict__ cnt) {
    const int n = Gt * Gh * Gw;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int w0 = i % Gw, h0 = (i / Gw) % Gh, t0 = i / (Gw * Gh);
    int32_t* out = idx + static_cast<long long>(i) * n;
    int c = 0;
    for (int t = max(t0 - wt, 0); t <= min(t0 + wt, Gt - 1); ++t)
        for (int h = max(h0 - wh, 0); h <= min(h0 + wh, Gh - 1); ++h)
            for (int w = max(w0 - ww, 0); w <= min(w0 + ww, Gw - 1); ++w) out[c++] = (t * Gh + h) * Gw + w;
    cnt[i] = c;
    for (; c < n; ++c) out[c] = -1;
}

// ---------------------------------------------------------------------------------------------
// Mean over each block of `block` consecutive rows of a bf16 [n_bh, S, 128] tensor -> fp32
// [n_bh, S / block, 128].  One CTA of 128 threads per (bh, block): thread t reads 16 bytes (columns
// 8 (t % 16) ..) of rows t / 16, t / 16 + 8, ... and the eight row groups are then added in a fixed
// order, so results do not depend on scheduling.  HBM-bound: one pass over the tensor.
__global__ void __launch_bounds__(128) block_mean_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out,
                                                        int S, int block) {
    __shared__ float part[8][128];
    const long long bh = blockIdx.y;
    const int blk = blockIdx.x;
    const int c8 = threadIdx.x & 15, rg = threadIdx.x >> 4;
    const uint4* src = reinterpret_cast<const uint4*>(x + (bh * S + static_cast<long long>(blk) * block) * 128) + c8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 4
    for (int r = rg; r < block; r += 8) {
        const uint4 v = src[static_cast<long long>(r) * 16];
        const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(v2[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) part[rg][8 * c8 + j] = acc[j];
    __syncthreads();
    const int d = threadIdx.x;
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) s += part[g][d];
    out[(bh * (S / block) + blk) * 128 + d] = s / static_cast<float>(block);
}

// ---------------------------------------------------------------------------------------------
// SSTA row selection.  One warp per (batch, head, query block): scores of the pooled query block
// against every pooled key block, top-k by repeated arg-max (ties -> lower index), union with the
// STA window of the tile that contains the query block, then the bool mask row and the ascending
// q-major list are written.  nK <= 32 * kMaxPerLane.
constexpr int kMaxPerLane = 32;

__global__ void __launch_bounds__(256)
ssta_select_kernel(const float* __restrict__ qp, const float* __restrict__ kp, int Hq, int Hkv, int nQ, int nK,
                   int q_per_tile, int Gt, int Gh, int Gw, int wt, int wh, int ww, int topk,
                   uint8_t* __restrict__ mask, int32_t* __restrict__ q2k_idx, int32_t* __restrict__ q2k_cnt,
                   long long total_rows) {
    const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= total_rows) return;
    const int lane = threadIdx.x & 31;
    const long long bh = row / nQ;
    const int qi = static_cast<int>(row % nQ);
    const long long bhk = (bh / Hq) * Hkv + (bh % Hq) / (Hq / Hkv);
    const float* qv = qp + row * 128;
    // each lane keeps 4 of the 128 query means
    float q0 = qv[lane], q1 = qv[32 + lane], q2 = qv[64 + lane], q3 = qv[96 + lane];

    float sc[kMaxPerLane];
    const int per_lane = (nK + 31) / 32;
#pragma unroll 1
    for (int u = 0; u < per_lane; ++u) {
#pragma unroll 1
        for (int src_lane = 0; src_lane < 32; ++src_lane) {
            // key block j = u * 32 + src_lane; the whole warp cooperates on one dot product
            const int j = u * 32 + src_lane;
            float partial = 0.f;
            if (j < nK) {
                const float* kv = kp + (bhk * nK + j) * 128;
                partial = q0 * kv[lane] + q1 * kv[32 + lane] + q2 * kv[64 + lane] + q3 * kv[96 + lane];
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, m);
            if (lane == src_lane) sc[u] = j < nK ? partial : -INFINITY;
        }
    }
    // selection bits: lane owns key blocks u * 32 + lane, bit u
    uint32_t sel = 0;
    const int k_eff = topk < nK ? topk : nK;
    for (int r = 0; r < k_eff; ++r) {
        float best = -INFINITY;
        int best_j = 0x7fffffff;
        for (int u = 0; u < per_lane; ++u) {
            const int j = u * 32 + lane;
            if (j < nK && !((sel >> u) & 1u) && (sc[u] > best || (sc[u] == best && j < best_j))) {
                best = sc[u];
                best_j = j;
            }
        }
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, m);
            const int oj = __shfl_xor_sync(0xffffffffu, best_j, m);
            if (ob > best || (ob == best && oj < best_j)) {
                best = ob;
                best_j = oj;
            }
        }
        if (best_j != 0x7fffffff && (best_j & 31) == lane) sel |= 1u << (best_j >> 5);
    }
    // window of the tile that contains this query block
    const int tile = qi / q_per_tile;
    const int w0 = tile % Gw, h0 = (tile / Gw) % Gh, t0 = tile / (Gw * Gh);
    for (int u = 0; u < per_lane; ++u) {
        const int j = u * 32 + lane;
        if (j < nK) {
            const int wj = j % Gw, hj = (j / Gw) % Gh, tj = j / (Gw * Gh);
            if (abs(tj - t0) <= wt && abs(hj - h0) <= wh && abs(wj - w0) <= ww) sel |= 1u << u;
        }
    }
    // emit mask row and ascending list
    uint8_t* mrow = mask + row * nK;
    int32_t* out = q2k_idx + row * nK;
    int n = 0;
    for (int u = 0; u < per_lane; ++u) {
        const int j = u * 32 + lane;
        const bool on = j < nK && ((sel >> u) & 1u);
        if (j < nK) mrow[j] = on ? 1 : 0;
        const uint32_t ballot = __ballot_sync(0xffffffffu, on);
        if (on) out[n + __popc(ballot & ((1u << lane) - 1u))] = j;
        n += __popc(ballot);
    }
    for (int c = n + lane; c < nK; c += 32) out[c] = -1;
    if (lane == 0) q2k_cnt[row] = n;
}

}  // namespace fba

using namespace fba;

extern "C" int fba_sta_index(int Gt, int Gh, int Gw, int wt, int wh, int ww, int32_t* idx, int32_t* cnt,
                             void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!idx || !cnt) return set_error(FBA_ERR_BAD_ARG, "fba_sta_index: null pointer argument");
    if (Gt <= 0 || Gh <= 0 || Gw <= 0 || wt < 0 || wh < 0 || ww < 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_sta_index: bad grid or window");
    const long long n = static_cast<long long>(Gt) * Gh * Gw;
    if (n > 46340) return set_error(FBA_ERR_TOO_LARGE, "fba_sta_index: more than 46340 tiles");
    DeviceGuard guard;
    int rc = guard.bind(idx);
    if (rc != FBA_OK) return rc;
    sta_lists_kernel<<<static_cast<unsigned>((n + 127) / 128), 128, 0, stream>>>(Gt, Gh, Gw, wt, wh, ww, idx, cnt);
    return check_launch("sta_lists_kernel");
}

extern "C" int fba_ssta_scratch_floats(int B, int Hq, int Hkv, int nQ, int nK, uint64_t* n_floats) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || nQ <= 0 || nK <= 0 || !n_floats)
        return set_error(FBA_ERR_BAD_ARG, "fba_ssta_scratch_floats: bad argument");
    *n_floats = (static_cast<uint64_t>(B) * Hq * nQ + static_cast<uint64_t>(B) * Hkv * nK) * 128;
    return FBA_OK;
}

extern "C" int fba_ssta_index(const void* q, const void* k, int B, int Hq, int Hkv, int Sq, int Skv, int q_block,
                              int kv_block, int Gt, int Gh, int Gw, int wt, int wh, int ww, int topk,
                              float* scratch, uint8_t* mask, int32_t* q2k_idx, int32_t* q2k_cnt, int32_t* k2q_idx,
                              int32_t* k2q_cnt, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!q || !k || !scratch || !mask || !q2k_idx || !q2k_cnt)
        return set_error(FBA_ERR_BAD_ARG, "fba_ssta_index: null pointer argument");
    if ((k2q_idx == nullptr) != (k2q_cnt == nullptr))
        return set_error(FBA_ERR_BAD_ARG, "fba_ssta_index: k2q idx and cnt must be given together");
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || Sq <= 0 || Skv <= 0 || q_block <= 0 || kv_block <= 0 ||
        Sq % q_block != 0 || Skv % kv_block != 0 || topk < 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_ssta_index: bad size");
    const int nQ = Sq / q_block, nK = Skv / kv_block;
    // a window extent of -1 selects no tile at all in that dimension: with it the mask is the
    // top-k selection alone (MoBA)
    if (Gt <= 0 || Gh <= 0 || Gw <= 0 || static_cast<long long>(Gt) * Gh * Gw != nK || wt < -1 || wh < -1 || ww < -1)
        return set_error(FBA_ERR_BAD_ARG, "fba_ssta_index: the tile grid must have one tile per key block");
    if (kv_block % q_block != 0 || static_cast<long long>(nQ) * q_block != static_cast<long long>(nK) * kv_block)
        return set_error(FBA_ERR_BAD_ARG,
                         "fba_ssta_index: q_block must divide kv_block and both sequences must cover the same tiles");
    if (nK > 32 * kMaxPerLane) return set_error(FBA_ERR_TOO_LARGE, "fba_ssta_index: more than 1024 key blocks");
    DeviceGuard guard;
    int rc = guard.bind(q);
    if (rc != FBA_OK) return rc;
    float* qp = scratch;
    float* kp = scratch + static_cast<long long>(B) * Hq * nQ * 128;
    block_mean_kernel<<<dim3(nQ, B * Hq), 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(q), qp, Sq, q_block);
    if ((rc = check_launch("block_mean_kernel(q)")) != FBA_OK) return rc;
    block_mean_kernel<<<dim3(nK, B * Hkv), 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(k), kp, Skv, kv_block);
    if ((rc = check_launch("block_mean_kernel(k)")) != FBA_OK) return rc;
    const long long rows = static_cast<long long>(B) * Hq * nQ;
    ssta_select_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, stream>>>(
        qp, kp, Hq, Hkv, nQ, nK, kv_block / q_block, Gt, Gh, Gw, wt, wh, ww, topk, mask, q2k_idx, q2k_cnt, rows);
    if ((rc = check_launch("ssta_select_kernel")) != FBA_OK) return rc;
    if (k2q_idx) rc = fba_build_index(mask, 4, B, Hq, nQ, nK, nullptr, nullptr, k2q_idx, k2q_cnt, stream_);
    return rc;
}
