// Query-major dQ pass of the block-sparse attention backward for sm_100a.
//
// The default backward (fba_bwd.cu) follows the reference's strategy for dQ: the key-major kernel
// computes one 128x128 dQ partial per (key tile, query tile) and reduce-adds it into an fp32
// accumulator (reference flex_block_attn_h100.cu:700-718, 750-764).  This file is the other
// strategy: a second, query-major kernel that recomputes S and dP and accumulates dQ in tensor
// memory, so dQ is written exactly once, in bf16, with no accumulator, no zero-fill, no
// conversion pass and no floating-point reduction whose order depends on scheduling (the result
// is bit-reproducible).  It costs two more GEMMs and a second exp2 pass per tile pair; the
// key-major kernel then runs without its dQ GEMM and drain.
//
// A CTA owns one 128-row query tile of one (batch, head) and walks the query-major list.  Per
// key tile, three 128x128x128 tcgen05 GEMMs:
//     S   = Q K^T        (smem x smem -> TMEM, double-buffered)
//     dP  = dO V^T       (smem x smem -> TMEM)
//     dQ += dS K         (dS bf16 in TMEM x K in smem, MN-major)
// with P = exp2(S * scale * log2e - lse * log2e) and dS = P * (dP - delta) * scale computed by two
// warpgroups (thread = query row, so lse and delta are per-thread scalars; warpgroup h takes key
// columns [64 h, 64 h + 64)).  dS overwrites the S buffer it came from.
// TMEM columns: [0,128) S buffer 0, [128,256) S buffer 1, [256,384) dP, [384,512) dQ.
//
// Warps: 0-7 compute, 8 issues the MMAs, 9 drives TMA.  Shared memory: Q and dO resident (64 KiB),
// two stages of (K tile, V tile) (128 KiB).
#include "fba_common.cuh"

namespace fba {

constexpr int kDqThreads = 320;
constexpr uint32_t kDqSmemQ = 0;
constexpr uint32_t kDqSmemDO = kTileBytes;
constexpr uint32_t kDqSmemKV = 2 * kTileBytes;                 // 2 stages x (K, V)
constexpr uint32_t kDqSmemBars = kDqSmemKV + 4 * kTileBytes;

enum DqBar : uint32_t {
    kDQFull = 0,       // Q and dO landed
    kDKvFull = 1,      // 2
    kDKvEmpty = 3,     // 2
    kDSFull = 5,       // 2: S of an even / odd step is in its buffer
    kDDpFull = 7,
    kDDsReady = 8,     // 256 arrivals: dS written (and dP consumed)
    kDDone = 9,
    kDCount = 10
};
constexpr uint32_t kDqSmemBytes = kDqSmemBars + 8 * kDCount + 16 + 1024;   // + alignment slack
static_assert(kDqSmemBytes <= 232448, "exceeds the 227 KiB shared memory of an sm_100 CTA");

struct DqParams {
    ListDev list;          // query-major: rows = query tiles / rows_div, entries = key tiles / sub
    const float* ld;       // [B*Hq, nMt, 2, 128]: per query tile 128 x (-lse*log2e), then 128 x (-delta*scale)
    uint32_t* status;
    int n_mtiles, Hq, Hkv;
    float scale;
};

__global__ void __launch_bounds__(kDqThreads, 1)
fba_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                  const __grid_constant__ CUtensorMap tm_dq, const DqParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + kDqSmemBars;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kDqSmemBars + 8 * kDCount);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kDqSmemBars + 8 * kDCount + 4);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bq = blockIdx.y;                      // b * Hq + query head
    const int hr = p.Hq / p.Hkv;
    const int bhk = (bq / p.Hq) * p.Hkv + (bq % p.Hq) / hr;
    // Query tile of this CTA.  With a work order (built for the forward's tile pairs) consecutive
    // CTAs take the two tiles of the pairs, longest pair first.
    const int mt = p.list.order
                       ? p.list.order[static_cast<long long>(p.list.bh_stride ? bq : 0) * (gridDim.x >> 1) + (blockIdx.x >> 1)] * 2 +
                             static_cast<int>(blockIdx.x & 1)
                       : static_cast<int>(blockIdx.x);
    if (mt >= p.n_mtiles) return;                   // second half of an odd last pair (uniform per CTA)
    const int sub = p.list.sub;
    const long long lrow = static_cast<long long>(bq) * p.list.bh_stride + mt / p.list.rows_div;
    const int n_total = p.list.cnt[lrow] * sub;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar(kDQFull), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(kDKvFull + s), 1);
            mbar_init(bar(kDKvEmpty + s), 1);
            mbar_init(bar(kDSFull + s), 1);
        }
        mbar_init(bar(kDDpFull), 1);
        mbar_init(bar(kDDsReady), 256);
        mbar_init(bar(kDDone), 1);
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
        tmem_relinquish();
    }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        tma_prefetch_desc(&tm_do);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tDP = tmem + 256, tDQ = tmem + 384;
    auto tS = [&](int b) { return tmem + static_cast<uint32_t>(b) * 128u; };
    const uint32_t sQ = base + kDqSmemQ, sDO = base + kDqSmemDO;
    auto sK = [&](int s) { return base + kDqSmemKV + static_cast<uint32_t>(s) * 2u * kTileBytes; };
    auto sV = [&](int s) { return sK(s) + kTileBytes; };

    if (warp == 9) {
        // ------------------------------------------------------------------ TMA loader
        if (lane == 0 && n_total > 0) {
            mbar_expect_tx(bar(kDQFull), 2 * kTileBytes);
            tma_load_3d(sQ, &tm_q, 0, mt * 128, bq, bar(kDQFull));
            tma_load_3d(sQ + kPanelBytes, &tm_q, 64, mt * 128, bq, bar(kDQFull));
            tma_load_3d(sDO, &tm_do, 0, mt * 128, bq, bar(kDQFull));
            tma_load_3d(sDO + kPanelBytes, &tm_do, 64, mt * 128, bq, bar(kDQFull));
            for (int it = 0; it < n_total; ++it) {
                const int st = it & 1;
                const int e = it / sub;
                const int nt = p.list.idx[lrow * p.list.stride + e] * sub + (it - e * sub);
                if (!mbar_wait(bar(kDKvEmpty + st), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_timeout(p.status, 3, 9, it, 100);
                    break;
                }
                mbar_expect_tx(bar(kDKvFull + st), 2 * kTileBytes);
                tma_load_3d(sK(st), &tm_k, 0, nt * 128, bhk, bar(kDKvFull + st));
                tma_load_3d(sK(st) + kPanelBytes, &tm_k, 64, nt * 128, bhk, bar(kDKvFull + st));
                tma_load_3d(sV(st), &tm_v, 0, nt * 128, bhk, bar(kDKvFull + st));
                tma_load_3d(sV(st) + kPanelBytes, &tm_v, 64, nt * 128, bhk, bar(kDKvFull + st));
            }
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_total > 0) {
            bool ok = true;
            auto wait = [&](uint32_t slot, uint32_t parity, int it, uint32_t tag) {
                if (!ok) return;
                if (!mbar_wait(bar(slot), parity, abort_flag)) {
                    report_timeout(p.status, 3, 8, it, tag);
                    ok = false;
                }
            };
            wait(kDQFull, 0, 0, 200);
            wait(kDKvFull + 0, 0, 0, 201);
            if (ok) {
                tc_fence_after();
                mma_tile_kk(tS(0), sQ, sK(0), false);
                umma_commit(bar(kDSFull + 0));
                mma_tile_kk(tDP, sDO, sV(0), false);
                umma_commit(bar(kDDpFull));
            }
            for (int it = 0; it < n_total && ok; ++it) {
                const int st = it & 1;
                const bool more = it + 1 < n_total;
                if (more) {
                    // S of the next step goes to the other buffer: the dQ GEMM that read dS(it-1)
                    // from it was issued earlier by this thread and therefore runs first.
                    wait(kDKvFull + (st ^ 1), ((it + 1) >> 1) & 1u, it, 210);
                    if (!ok) break;
                    tc_fence_after();
                    mma_tile_kk(tS(st ^ 1), sQ, sK(st ^ 1), false);
                    umma_commit(bar(kDSFull + (st ^ 1)));
                }
                wait(kDDsReady, it & 1u, it, 211);
                if (!ok) break;
                tc_fence_after();
                mma_tile_tm(tDQ, tS(st), tS(st) + 64, sK(st), it > 0);
                umma_commit(bar(kDKvEmpty + st));          // K(it) and V(it) are no longer needed
                if (more) {
                    mma_tile_kk(tDP, sDO, sV(st ^ 1), false);   // dP(it) was consumed before dS(it) was announced
                    umma_commit(bar(kDDpFull));
                }
            }
            if (ok) umma_commit(bar(kDDone));
        }
    } else {
        // ------------------------------------------------------------------ P / dS compute + epilogue
        const int h = warp >> 2;            // key-column half of the tile
        const int quad = warp & 3;
        const int row = quad * 32 + lane;   // query row inside the tile == TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const float c = p.scale * kLog2e;
        const float* ld = p.ld + (static_cast<long long>(bq) * p.n_mtiles + mt) * 256;
        const float lse2 = ld[row];         // -lse * log2e (-inf for a dead or padding row: every P is 0)
        const float dlt = ld[128 + row];    // -delta * scale
        const int g = row >> 4;
        bool ok = true;
        for (int it = 0; it < n_total && ok; ++it) {
            const int st = it & 1;
            if (!mbar_wait(bar(kDSFull + st), (it >> 1) & 1u, abort_flag)) {
                if (lane == 0) report_timeout(p.status, 3, static_cast<uint32_t>(warp), it, 400);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tSb = tS(st) + lane_base + 64u * h;
            float pr[64];
            {
                uint32_t s[64];
                tmem_ld32(tSb, reinterpret_cast<uint32_t(&)[32]>(s[0]));
                tmem_ld32(tSb + 32u, reinterpret_cast<uint32_t(&)[32]>(s[32]));
                tmem_wait_ld();
                bool keep = true;
                if (p.list.msk != nullptr) {
                    const uint32_t w = p.list.msk[lrow * p.list.stride + it / sub];
                    keep = (w >> (8 * h + g)) & 1u;
                }
#pragma unroll
                for (int j = 0; j < 64; ++j)
                    pr[j] = keep ? ex2_approx(fmaf(__uint_as_float(s[j]), c, lse2)) : 0.f;
            }
            if (!mbar_wait(bar(kDDpFull), it & 1u, abort_flag)) {
                if (lane == 0) report_timeout(p.status, 3, static_cast<uint32_t>(warp), it, 401);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t dp[64];
            tmem_ld32(tDP + lane_base + 64u * h, reinterpret_cast<uint32_t(&)[32]>(dp[0]));
            tmem_ld32(tDP + lane_base + 64u * h + 32u, reinterpret_cast<uint32_t(&)[32]>(dp[32]));
            tmem_wait_ld();
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int col = 32 * cc + 2 * j;
                    const float d0 = pr[col] * fmaf(__uint_as_float(dp[col]), p.scale, dlt);
                    const float d1 = pr[col + 1] * fmaf(__uint_as_float(dp[col + 1]), p.scale, dlt);
                    pk[j] = pack_bf16x2(d0, d1);
                }
                tmem_st16(tSb + 16u * cc, pk);     // dS (bf16 pairs) over this warpgroup's own S columns
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(kDDsReady));
        }

        // Epilogue: dQ -> bf16 -> swizzled staging in the Q buffer -> TMA store (rows past Sq are
        // clipped).  Warpgroup h writes columns [64 h, 64 h + 64) = panel h.
        if (n_total > 0 && ok) {
            if (!mbar_wait(bar(kDDone), 0, abort_flag)) {
                if (lane == 0) report_timeout(p.status, 3, static_cast<uint32_t>(warp), 0, 500);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
            uint8_t* stage = base_ptr + kDqSmemQ + static_cast<uint32_t>(h) * kPanelBytes;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t v[32];
                if (n_total > 0) {
                    tmem_ld32(tDQ + lane_base + 64u * h + 32u * cc, v);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 wv;
                    wv.x = pack_bf16x2(__uint_as_float(v[8 * q4 + 0]), __uint_as_float(v[8 * q4 + 1]));
                    wv.y = pack_bf16x2(__uint_as_float(v[8 * q4 + 2]), __uint_as_float(v[8 * q4 + 3]));
                    wv.z = pack_bf16x2(__uint_as_float(v[8 * q4 + 4]), __uint_as_float(v[8 * q4 + 5]));
                    wv.w = pack_bf16x2(__uint_as_float(v[8 * q4 + 6]), __uint_as_float(v[8 * q4 + 7]));
                    const int chunk = cc * 4 + q4;   // 16-byte chunk 0..7 of this panel's 128-byte row
                    *reinterpret_cast<uint4*>(stage + static_cast<uint32_t>(row) * 128u +
                                              (static_cast<uint32_t>(chunk ^ (row & 7)) << 4)) = wv;
                }
            }
            fence_proxy_async_smem();
        }
        named_bar_sync(1, 256);
        if (ok && warp == 0 && lane == 0) {
            tma_store_3d(&tm_dq, 0, mt * 128, bq, sQ);
            tma_store_3d(&tm_dq, 64, mt * 128, bq, sQ + kPanelBytes);
            tma_commit_group();
            tma_wait_group0();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

int launch_bwd_dq(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_do,
                  const CUtensorMap& tm_dq, const fba_list_t& q2k, const float* lse_delta, uint32_t* status,
                  int n_mtiles, long long n_bhq, int Hq, int Hkv, float scale, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(fba_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kDqSmemBytes));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_bwd: cannot raise the dynamic shared memory limit");
    }
    DqParams p;
    p.list = to_dev(q2k);
    p.ld = lse_delta;
    p.status = status;
    p.n_mtiles = n_mtiles;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.scale = scale;
    dim3 grid(q2k.order ? 2 * ((n_mtiles + 1) / 2) : n_mtiles, static_cast<unsigned>(n_bhq));
    timing_mark(3, true, stream);
    fba_bwd_dq_kernel<<<grid, kDqThreads, kDqSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dq, p);
    int rc = check_launch("fba_bwd_dq_kernel");
    timing_mark(3, false, stream);
    return rc;
}

}  // namespace fba
