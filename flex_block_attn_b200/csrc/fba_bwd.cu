// Block-sparse attention backward for sm_100a.
//
// Three kernels, in stream order:
//   1. bwd_prep_kernel      per row (-LSE * log2 e, -scale * sum_d dO * O); the counterpart of
//                           the reference's bwd_attend_prep_ker (flex_block_attn_h100.cu:339-389).
//                           HBM-bound, one pass over O and dO.
//   2. fba_bwd_kernel       key-major main kernel, the counterpart of bwd_attend_ker (.cu:572-802).
//                           A CTA owns one 128-row K/V tile and walks the key-major list of query
//                           tiles.  Per query tile, five 128x128x128 tcgen05 GEMMs:
//                             S^T  = K Q^T          (smem x smem -> TMEM)
//                             dP^T = V dO^T         (smem x smem -> TMEM)
//                             dV  += P^T dO         (P^T bf16 in TMEM x smem)
//                             dQ   = dS K           (dS^T bf16 in smem, MN-major x smem -> TMEM)
//                             dK  += dS^T Q         (dS^T bf16 in smem, K-major x smem)
//                           TMEM columns: [0,128) S^T / P^T, [128,256) dV, [256,384) dP^T then dQ,
//                           [384,512) dK.  dK and dV stay in TMEM for the whole CTA (and across
//                           the query heads of a grouped-query group), so they are written once,
//                           in bf16, with no atomics; the reference reduce-adds fp32 tiles
//                           (.cu:544-570) into zero-filled buffers (.cu:1077-1088).
//                           dQ tiles leave TMEM into registers and are added to an fp32
//                           accumulator with 16-byte vector reductions (red.global.add.v4.f32).
//   3. bwd_dq_convert_kernel  dQ fp32 accumulator (tile-blocked layout) -> bf16 [B,H,Sq,128].
//
// Warp roles of the main kernel (512 threads): warps 0-7 compute P^T and dS^T (thread = key row;
// warps 0-3 take query columns 0-63 of the tile, warps 4-7 columns 64-127), warps 8-11 drain dQ
// from TMEM, warps 12 and 14 issue the MMAs (two independent chains), warp 13 drives TMA.
//
// Shared memory: K, V resident (64 KiB); Q double-buffered with its (lse2, delta) rows (64 + 2 KiB);
// dO double-buffered (64 KiB); dS^T (32 KiB).
#include <stdlib.h>

#include "fba_common.cuh"

#ifndef FBA_BWD_KERNEL_DEFAULT
#define FBA_BWD_KERNEL_DEFAULT 1
#endif

namespace fba {

constexpr int kBwdThreads = 512;  // 4 warpgroups: compute, compute, dQ drain, {MMA, TMA, 2 idle}
constexpr uint32_t kBwdSmemK = 0;
constexpr uint32_t kBwdSmemV = 1 * kTileBytes;
constexpr uint32_t kBwdSmemQ = 2 * kTileBytes;    // 2 stages
constexpr uint32_t kBwdSmemDO = 4 * kTileBytes;   // 2 stages
constexpr uint32_t kBwdSmemDS = 6 * kTileBytes;
constexpr uint32_t kBwdSmemLD = 7 * kTileBytes;     // 2 stages x 128 x (lse2, delta)
constexpr uint32_t kBwdSmemBars = kBwdSmemLD + 2 * 1024;


enum BwdBar : uint32_t {
    kBKvFull = 0,
    kBQFull = 1,      // 2
    kBQEmpty = 3,     // 2
    kBDoFull = 5,     // 2
    kBDoEmpty = 7,    // 2
    kBSFull = 9,
    kBPReady = 10,
    kBDpFull = 11,
    kBDsReady = 12,
    kBDqFull = 13,
    kBDqDrained = 14,
    kBDkvDone = 15,
    kBCount = 16
};
// barriers, then the TMEM base slot and the abort flag
constexpr uint32_t kBwdSmemBytes = kBwdSmemBars + 8 * kBCount + 16;
static_assert(kBwdSmemBytes <= 232448, "exceeds the 227 KiB shared memory of an sm_100 CTA");

// L2 prefetch of the Q / dO tiles a few list entries ahead (1 = on).  Measured 3-4 % slower on
// B200 for both the dense and the random-sparse workloads, so it is off.
#ifndef FBA_BWD_PREFETCH
#define FBA_BWD_PREFETCH 0
#endif
// Pause between two of the 32 vector reductions a drain thread issues per query tile.
#ifndef FBA_RED_SLEEP_NS
#define FBA_RED_SLEEP_NS 32
#endif

struct BwdParams {
    ListDev list;          // key-major: rows = key tiles / rows_div, entries = query tiles / sub
    const float2* ld;      // [B*Hq, nMt, 2, 128]: per query tile 128 x (-lse*log2e), then 128 x (-delta*scale)
    float* dq_accum;       // [B*Hq, nMt, 4 column chunks, 4 row groups, 8, 32, 4] fp32
    uint32_t* status;
    int n_mtiles, Hq, Hkv;
    float scale;           // softmax scale
};

// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bwd_prep_kernel(const __nv_bfloat16* __restrict__ o,
                                                      const __nv_bfloat16* __restrict__ dout,
                                                      const float* __restrict__ lse,
                                                      float2* __restrict__ ld, uint32_t Sq, uint32_t rows_pad,
                                                      uint32_t total_rows, float scale) {
    // A half-warp per row (16 bytes of O and of dO per lane), two rows per half-warp in flight, a
    // grid-stride loop over groups of four rows per warp.  Row counts fit 32 bits (host-checked):
    // 64-bit divisions per row would cost more than the row's memory traffic.
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t half = lane >> 4, l16 = lane & 15;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t base = warp * 4; base < total_rows; base += n_warps * 4) {
        uint32_t w[2];
        bool live[2];
        uint4 a[2], b[2];
        float l[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            w[u] = base + 2 * u + half;             // padded row index (b*h, r)
            const uint32_t bh = w[u] / rows_pad;
            const uint32_t r = w[u] - bh * rows_pad;
            live[u] = w[u] < total_rows && r < Sq;
            a[u] = b[u] = make_uint4(0u, 0u, 0u, 0u);
            l[u] = -INFINITY;
            if (live[u]) {
                const unsigned long long row = static_cast<unsigned long long>(bh) * Sq + r;
                a[u] = reinterpret_cast<const uint4*>(o + row * 128)[l16];
                b[u] = reinterpret_cast<const uint4*>(dout + row * 128)[l16];
                l[u] = lse[row];
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a[u]);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b[u]);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = __bfloat1622float2(a2[j]);
                const float2 y = __bfloat1622float2(b2[j]);
                s = fmaf(x.x, y.x, s);
                s = fmaf(x.y, y.y, s);
            }
#pragma unroll
            for (int m = 8; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);   // within the half-warp
            // Output layout, per 128-row query tile: 128 x (-lse2) followed by 128 x (-delta * scale),
            // so the main kernel fetches four columns' worth of either quantity with one 16-byte
            // shared-memory read.  A row that attended to nothing (LSE = -inf) and the padding rows of
            // the last tile get -inf: every P of such a row is exp2(s * c - inf) = 0, and so is its dS.
            if (l16 == 0 && w[u] < total_rows) {
                float* out = reinterpret_cast<float*>(ld) + static_cast<unsigned long long>(w[u] >> 7) * 256 + (w[u] & 127);
                out[0] = (!live[u] || l[u] == -INFINITY) ? -INFINITY : -l[u] * kLog2e;
                out[128] = live[u] ? -s * scale : 0.f;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// dQ accumulator layout: element (row = 32 w + r, col = 32 cc + 4 j + e) of query tile t sits at
// float offset ((((t * 4 + cc) * 4 + w) * 8 + j) * 32 + r) * 4 + e, i.e. each (column chunk cc,
// row group w) is a contiguous 4 KiB block owned by one drain warp, ordered so that the 32 lanes of a
// vector reduction touch 512 consecutive bytes.
__global__ void __launch_bounds__(256) bwd_dq_convert_kernel(const float* __restrict__ acc,
                                                            __nv_bfloat16* __restrict__ dq, int Sq,
                                                            int n_mtiles) {
    __shared__ uint2 tile[128 * 33];
    const int mt = blockIdx.x;
    const long long bh = blockIdx.y;
    const float4* src = reinterpret_cast<const float4*>(acc) + (bh * n_mtiles + mt) * (32LL * 128);
#pragma unroll 4
    for (int k = 0; k < 16; ++k) {
        const int i = threadIdx.x + 256 * k;
        const int r = i & 31, j = (i >> 5) & 7, w = (i >> 8) & 3, cc = i >> 10;
        const float4 v = src[i];
        uint2 pk;
        pk.x = pack_bf16x2(v.x, v.y);
        pk.y = pack_bf16x2(v.z, v.w);
        tile[(w * 32 + r) * 33 + cc * 8 + j] = pk;
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < 8; ++k) {
        const int i = threadIdx.x + 256 * k;  // (row, 16-byte chunk)
        const int row = i >> 4, c = i & 15;
        const int grow = mt * 128 + row;
        if (grow < Sq) {
            const uint2 a = tile[row * 33 + 2 * c], b = tile[row * 33 + 2 * c + 1];
            uint4 w4 = make_uint4(a.x, a.y, b.x, b.y);
            reinterpret_cast<uint4*>(dq + (bh * Sq + grow) * 128)[c] = w4;
        }
    }
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
                 "f"(d)
                 : "memory");
}
// kWithDq = false: the dK / dV-only variant that runs beside the query-major dQ pass
// (fba_bwd_dq.cu): no dQ GEMM, no drain, no reductions.
template <bool kWithDq>
__global__ void __launch_bounds__(kBwdThreads, 1)
fba_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
               const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
               const BwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    uint8_t* base_ptr = smem_raw;
    const uint32_t bars = base + kBwdSmemBars;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kBwdSmemBars + 8 * kBCount);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kBwdSmemBars + 8 * kBCount + 4);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bhk = blockIdx.y;         // b * Hkv + kv head
    // Key tile of this CTA: the blockIdx.x-th entry of the longest-first order when one is given
    // (CTAs are dispatched in blockIdx order, so the shortest lists of the grid run last).
    const int nt = p.list.order
                       ? p.list.order[static_cast<long long>(p.list.bh_stride ? bhk : 0) * gridDim.x + blockIdx.x]
                       : static_cast<int>(blockIdx.x);
    const int hr = p.Hq / p.Hkv;
    const int bq0 = (bhk / p.Hkv) * p.Hq + (bhk % p.Hkv) * hr;  // first query head of the group
    const int sub = p.list.sub;

    if ((base & 1023u) != 0u) {
        // The swizzled operand panels need a 1024-byte aligned base; report instead of computing garbage.
        if (threadIdx.x == 0) report_timeout(p.status, 2, 99, 0, 999);
        return;
    }

    // List rows of the query heads of this group (hr is small; read on demand).
    auto list_row = [&](int r) {
        return static_cast<long long>(bq0 + r) * p.list.bh_stride + nt / p.list.rows_div;
    };
    int n_total = 0;
    for (int r = 0; r < hr; ++r) n_total += p.list.cnt[list_row(r)] * sub;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar(kBKvFull), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(kBQFull + s), 1);
            mbar_init(bar(kBQEmpty + s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(kBDoFull + s), 1);
            mbar_init(bar(kBDoEmpty + s), 2);   // dV (issuer A) and dP^T (issuer B) both read dO
        }
        mbar_init(bar(kBSFull), 1);
        mbar_init(bar(kBPReady), 256);
        mbar_init(bar(kBDpFull), 1);
        mbar_init(bar(kBDsReady), 256);
        mbar_init(bar(kBDqFull), 1);
        mbar_init(bar(kBDqDrained), 128);
        mbar_init(bar(kBDkvDone), 2);   // last dV (issuer A) and last dK (issuer B)
        mbar_fence_init();
    }
    if (warp == 12) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
        tmem_relinquish();
    }
    if (warp == 13 && lane == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        tma_prefetch_desc(&tm_do);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tST = tmem + 0, tDV = tmem + 128, tDP = tmem + 256, tDK = tmem + 384;
    const uint32_t sK = base + kBwdSmemK, sV = base + kBwdSmemV, sDS = base + kBwdSmemDS;
    auto sDO = [&](int s) { return base + kBwdSmemDO + static_cast<uint32_t>(s) * kTileBytes; };
    auto sQ = [&](int s) { return base + kBwdSmemQ + static_cast<uint32_t>(s) * kTileBytes; };

    // Register budget: 512 threads x 128 at launch (the whole register file); the MMA/TMA
    // warpgroup gives most of its share to the three warpgroups that hold tile rows in registers.
    // The four budgets must not exceed 4 x 128 in total (144 * 3 + 80 = 512), or an increase would
    // wait for registers that are never released.
    if (warp >= 12) {
      reg_dec<80>();
      if (warp == 13) {
        // ------------------------------------------------------------------ TMA loader
        if (lane == 0 && n_total > 0) {
            mbar_expect_tx(bar(kBKvFull), 2 * kTileBytes);
            tma_load_3d(sK, &tm_k, 0, nt * 128, bhk, bar(kBKvFull));
            tma_load_3d(sK + kPanelBytes, &tm_k, 64, nt * 128, bhk, bar(kBKvFull));
            tma_load_3d(sV, &tm_v, 0, nt * 128, bhk, bar(kBKvFull));
            tma_load_3d(sV + kPanelBytes, &tm_v, 64, nt * 128, bhk, bar(kBKvFull));
            // Walk of the (query head, list entry, sub-tile) sequence; a second cursor runs two
            // steps ahead and only asks L2 to fetch those tiles, so that the real loads (which can
            // start only when a stage is released, late in the previous iteration) hit L2.
            struct Cursor {
                int r, e, u, cnt, q0;
                long long lr;
            };
            auto cur_init = [&](Cursor& c) {
                c.r = 0; c.e = 0; c.u = 0;
                c.lr = list_row(0);
                c.cnt = p.list.cnt[c.lr];
                while (c.r < hr && c.cnt == 0) {
                    ++c.r;
                    if (c.r < hr) { c.lr = list_row(c.r); c.cnt = p.list.cnt[c.lr]; }
                }
                c.q0 = c.r < hr ? p.list.idx[c.lr * p.list.stride] * sub : 0;
            };
            auto cur_next = [&](Cursor& c) {
                if (++c.u < sub) return;
                c.u = 0;
                ++c.e;
                while (c.r < hr && c.e >= c.cnt) {
                    ++c.r;
                    c.e = 0;
                    if (c.r < hr) { c.lr = list_row(c.r); c.cnt = p.list.cnt[c.lr]; }
                }
                if (c.r < hr) c.q0 = p.list.idx[c.lr * p.list.stride + c.e] * sub;
            };
            Cursor cur, ahead;
            cur_init(cur);
            cur_init(ahead);
            int n_ahead = 0;
            auto prefetch_to = [&](int target) {
                while (n_ahead < target && n_ahead < n_total) {
                    if (n_ahead > 0) cur_next(ahead);
                    const int qt = ahead.q0 + ahead.u, bq = bq0 + ahead.r;
                    if (FBA_BWD_PREFETCH && n_ahead >= 2) {   // the first two are loaded right away
                        tma_prefetch_l2_3d(&tm_q, 0, qt * 128, bq);
                        tma_prefetch_l2_3d(&tm_q, 64, qt * 128, bq);
                        tma_prefetch_l2_3d(&tm_do, 0, qt * 128, bq);
                        tma_prefetch_l2_3d(&tm_do, 64, qt * 128, bq);
                    }
                    ++n_ahead;
                }
            };
            bool ok = true;
            for (int it = 0; it < n_total && ok; ++it) {
                if (it > 0) cur_next(cur);
                const int st = it & 1;
                const int qt = cur.q0 + cur.u, bq = bq0 + cur.r;
                if (!mbar_wait(bar(kBQEmpty + st), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_timeout(p.status, 2, 13, it, 100);
                    ok = false;
                    break;
                }
                if (it < 64) FBA_TRACE_REC(p.status, 2048 + it * 4 + 0);
                mbar_expect_tx(bar(kBQFull + st), kTileBytes + 1024);
                tma_load_3d(sQ(st), &tm_q, 0, qt * 128, bq, bar(kBQFull + st));
                tma_load_3d(sQ(st) + kPanelBytes, &tm_q, 64, qt * 128, bq, bar(kBQFull + st));
                bulk_load(base + kBwdSmemLD + st * 1024u,
                          p.ld + (static_cast<long long>(bq) * p.n_mtiles + qt) * 128, 1024, bar(kBQFull + st));
                if (!mbar_wait(bar(kBDoEmpty + st), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_timeout(p.status, 2, 13, it, 101);
                    ok = false;
                    break;
                }
                if (it < 64) FBA_TRACE_REC(p.status, 2048 + it * 4 + 1);
                mbar_expect_tx(bar(kBDoFull + st), kTileBytes);
                tma_load_3d(sDO(st), &tm_do, 0, qt * 128, bq, bar(kBDoFull + st));
                tma_load_3d(sDO(st) + kPanelBytes, &tm_do, 64, qt * 128, bq, bar(kBDoFull + st));
                prefetch_to(it + 4);
            }
        }
    } else if (warp == 12) {
        // ------------------------------------------------------------------ MMA issuer A: dV and S^T
        // Two issuing threads share the tensor core.  An issuing thread is blocked while its MMAs
        // execute and while it polls barriers, so with a single thread every wake-up and commit
        // is tensor-core idle time; thread A runs the chain  P ready -> dV -> next S^T  and
        // thread B (warp 14) the chain  dS ready -> dQ -> dK -> (dQ drained) -> next dP^T.
        if (lane == 0 && n_total > 0) {
            bool ok = true;
            auto wait = [&](uint32_t slot, uint32_t parity, int it, uint32_t tag) {
                if (!ok) return;
                if (!mbar_wait(bar(slot), parity, abort_flag)) {
                    report_timeout(p.status, 2, 12, it, tag);
                    ok = false;
                }
            };
            wait(kBKvFull, 0, 0, 200);
            wait(kBQFull + 0, 0, 0, 201);
            if (ok) {
                tc_fence_after();
                mma_tile_kk(tST, sK, sQ(0), false);
                umma_commit(bar(kBSFull));
            }
            for (int it = 0; it < n_total && ok; ++it) {
                const int st = it & 1;
                if (it < 64) FBA_TRACE_REC(p.status, 1024 + it * 8 + 0);
                wait(kBDoFull + st, (it >> 1) & 1u, it, 215);   // dO(it) has landed (normally long before P^T)
                wait(kBPReady, it & 1u, it, 210);
                if (!ok) break;
                tc_fence_after();
                if (it < 64) FBA_TRACE_REC(p.status, 1024 + it * 8 + 1);
                mma_tile_tm(tDV, tST, tST + 64, sDO(st), it > 0);
                umma_commit(bar(kBDoEmpty + st));     // one of the two releases of dO(it)
                if (it + 1 < n_total) {
                    if (it < 64) FBA_TRACE_REC(p.status, 2048 + it * 4 + 2);
                    wait(kBQFull + (st ^ 1), ((it + 1) >> 1) & 1u, it, 211);
                    if (!ok) break;
                    tc_fence_after();
                    if (it < 64) FBA_TRACE_REC(p.status, 1024 + it * 8 + 7);
                    mma_tile_kk(tST, sK, sQ(st ^ 1), false);
                    umma_commit(bar(kBSFull));
                }
                if (it < 64) FBA_TRACE_REC(p.status, 1024 + it * 8 + 2);
            }
            if (ok) umma_commit(bar(kBDkvDone));
        }
      } else if (warp == 14) {
        // ------------------------------------------------------------------ MMA issuer B: dP^T, dQ, dK
        if (lane == 0 && n_total > 0) {
            bool ok = true;
            auto wait = [&](uint32_t slot, uint32_t parity, int it, uint32_t tag) {
                if (!ok) return;
                if (!mbar_wait(bar(slot), parity, abort_flag)) {
                    report_timeout(p.status, 2, 14, it, tag);
                    ok = false;
                }
            };
            wait(kBKvFull, 0, 0, 220);
            wait(kBDoFull + 0, 0, 0, 202);
            if (ok) {
                tc_fence_after();
                mma_tile_kk(tDP, sV, sDO(0), false);
                umma_commit(bar(kBDpFull));
                umma_commit(bar(kBDoEmpty + 0));      // the other release of dO(0)
            }
            for (int it = 0; it < n_total && ok; ++it) {
                const int st = it & 1;
                const uint32_t ph = it & 1u;
                wait(kBDsReady, ph, it, 212);
                if (!ok) break;
                tc_fence_after();
                if (it < 64) FBA_TRACE_REC(p.status, 1024 + it * 8 + 3);
                if (kWithDq) {
                    mma_tile_mm(tDP, sDS, sK, false);     // dQ first: its drain overlaps the dK GEMM
                    umma_commit(bar(kBDqFull));
                }
                mma_tile_km(tDK, sDS, sQ(st), it > 0);
                umma_commit(bar(kBQEmpty + st));
                if (it < 64) FBA_TRACE_REC(p.status, 1024 + it * 8 + 4);
                if (it + 1 < n_total) {
                    wait(kBDoFull + (st ^ 1), ((it + 1) >> 1) & 1u, it, 214);
                    if (kWithDq) wait(kBDqDrained, ph, it, 213);   // else: dP^T(it) was consumed before dS^T(it) was announced
                    if (!ok) break;
                    tc_fence_after();
                    if (it < 64) FBA_TRACE_REC(p.status, 1024 + it * 8 + 5);
                    mma_tile_kk(tDP, sV, sDO(st ^ 1), false);
                    umma_commit(bar(kBDpFull));
                    umma_commit(bar(kBDoEmpty + (st ^ 1)));
                    if (it < 64) FBA_TRACE_REC(p.status, 1024 + it * 8 + 6);
                }
            }
            if (ok) umma_commit(bar(kBDkvDone));
        }
      }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ dQ drain
        reg_inc<144>();
        const int quad = warp & 3;
        const uint32_t tdq = tDP + (static_cast<uint32_t>(quad * 32) << 16);
        int it = 0;
        bool ok = true;
        for (int r = 0; r < hr && ok && kWithDq; ++r) {
            const long long lr = list_row(r);
            const int cnt = p.list.cnt[lr];
            const long long bq = bq0 + r;
            for (int e = 0; e < cnt && ok; ++e) {
                const int q0 = p.list.idx[lr * p.list.stride + e] * sub;
                for (int u = 0; u < sub && ok; ++u, ++it) {
                    if (!mbar_wait(bar(kBDqFull), it & 1u, abort_flag)) {
                        if (lane == 0) report_timeout(p.status, 2, static_cast<uint32_t>(warp), it, 300);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    if (warp == 8 && lane == 0 && it < 64) FBA_TRACE_REC(p.status, it * 8 + 4);
                    float* dst = p.dq_accum + ((bq * p.n_mtiles + (q0 + u)) * 16LL + quad) * 1024;
                    uint32_t v[128];
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
                        tmem_ld32(tdq + 32u * cc, reinterpret_cast<uint32_t(&)[32]>(v[32 * cc]));
                    tmem_wait_ld();
                    tc_fence_before();
                    mbar_arrive(bar(kBDqDrained));
                    if (warp == 8 && lane == 0 && it < 64) FBA_TRACE_REC(p.status, it * 8 + 5);
                    // One 16-byte reduction per lane and 4-column group; consecutive lanes hit
                    // consecutive addresses (512 contiguous bytes per instruction).  The short
                    // sleep spreads the 32 reductions of a tile over the iteration: issued back to
                    // back they fill the memory-instruction queue that the MMA issue also uses.
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            red_add_v4(dst + cc * 4096 + (j * 32 + lane) * 4, __uint_as_float(v[32 * cc + 4 * j]),
                                       __uint_as_float(v[32 * cc + 4 * j + 1]), __uint_as_float(v[32 * cc + 4 * j + 2]),
                                       __uint_as_float(v[32 * cc + 4 * j + 3]));
                            __nanosleep(FBA_RED_SLEEP_NS);
                        }
                    }
                    if (warp == 8 && lane == 0 && it < 64) FBA_TRACE_REC(p.status, it * 8 + 6);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ P^T / dS^T compute
        reg_inc<144>();
        const int h = warp >> 2;           // query-column half of the tile
        const int quad = warp & 3;
        const int row = quad * 32 + lane;  // key row inside the tile == TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const float c = p.scale * kLog2e;
        const float2 sc2 = make_float2(p.scale, p.scale);
        const int mbit0 = 8 * (row >> 6);  // key-half part of the mask bit index
        int it = 0;
        bool ok = true;
        for (int r = 0; r < hr && ok; ++r) {
            const long long lr = list_row(r);
            const int cnt = p.list.cnt[lr];
            for (int e = 0; e < cnt && ok; ++e) {
                const uint32_t w = p.list.msk ? p.list.msk[lr * p.list.stride + e] : 0xffffu;
                for (int u = 0; u < sub && ok; ++u, ++it) {
                    const int st = it & 1;
                    const float4* lse4 = reinterpret_cast<const float4*>(base_ptr + kBwdSmemLD + st * 1024) + 16 * h;
                    const float4* del4 = lse4 + 32;
                    if (!mbar_wait(bar(kBSFull), it & 1u, abort_flag) ||
                        !mbar_wait(bar(kBQFull + st), (it >> 1) & 1u, abort_flag)) {
                        if (lane == 0) report_timeout(p.status, 2, static_cast<uint32_t>(warp), it, 400);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    if (warp == 0 && lane == 0 && it < 64) FBA_TRACE_REC(p.status, it * 8 + 0);
                    float pr[64];
                    {
                        uint32_t s[64];
                        tmem_ld32(tST + lane_base + 64u * h, reinterpret_cast<uint32_t(&)[32]>(s[0]));
                        tmem_ld32(tST + lane_base + 64u * h + 32u, reinterpret_cast<uint32_t(&)[32]>(s[32]));
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float4 l4 = lse4[j];   // -lse2 of columns 4j .. 4j+3
                            const float2 x0 = fma2(make_float2(__uint_as_float(s[4 * j]), __uint_as_float(s[4 * j + 1])),
                                                   make_float2(c, c), make_float2(l4.x, l4.y));
                            const float2 x1 = fma2(make_float2(__uint_as_float(s[4 * j + 2]), __uint_as_float(s[4 * j + 3])),
                                                   make_float2(c, c), make_float2(l4.z, l4.w));
                            pr[4 * j] = ex2_approx(x0.x);
                            pr[4 * j + 1] = ex2_approx(x0.y);
                            pr[4 * j + 2] = ex2_approx(x1.x);
                            pr[4 * j + 3] = ex2_approx(x1.y);
                        }
                    }
                    if (w != 0xffffu) {
#pragma unroll
                        for (int j = 0; j < 64; ++j)
                            if (!((w >> (mbit0 + ((64 * h + j) >> 4))) & 1u)) pr[j] = 0.f;
                    }
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        uint32_t pk[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(pr[32 * cc + 2 * j], pr[32 * cc + 2 * j + 1]);
                        tmem_st16(tST + lane_base + 64u * h + 16u * cc, pk);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(bar(kBPReady));
                    if (warp == 0 && lane == 0 && it < 64) FBA_TRACE_REC(p.status, it * 8 + 1);

                    if (!mbar_wait(bar(kBDpFull), it & 1u, abort_flag)) {
                        if (lane == 0) report_timeout(p.status, 2, static_cast<uint32_t>(warp), it, 401);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    if (warp == 0 && lane == 0 && it < 64) FBA_TRACE_REC(p.status, it * 8 + 2);
                    uint8_t* ds_row = base_ptr + kBwdSmemDS + static_cast<uint32_t>(h) * kPanelBytes +
                                      static_cast<uint32_t>(row) * 128u;
                    uint32_t dp[64];
                    tmem_ld32(tDP + lane_base + 64u * h, reinterpret_cast<uint32_t(&)[32]>(dp[0]));
                    tmem_ld32(tDP + lane_base + 64u * h + 32u, reinterpret_cast<uint32_t(&)[32]>(dp[32]));
                    tmem_wait_ld();
#pragma unroll
                    for (int q8 = 0; q8 < 8; ++q8) {
                        uint32_t wds[4];
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int col = 8 * q8 + 4 * j;
                            const float4 d4 = del4[col >> 2];   // -delta*scale of columns col .. col+3
                            const float2 t0 = fma2(make_float2(__uint_as_float(dp[col]), __uint_as_float(dp[col + 1])),
                                                   sc2, make_float2(d4.x, d4.y));
                            const float2 t1 = fma2(make_float2(__uint_as_float(dp[col + 2]), __uint_as_float(dp[col + 3])),
                                                   sc2, make_float2(d4.z, d4.w));
                            const float2 e0 = mul2(make_float2(pr[col], pr[col + 1]), t0);
                            const float2 e1 = mul2(make_float2(pr[col + 2], pr[col + 3]), t1);
                            wds[2 * j] = pack_bf16x2(e0.x, e0.y);
                            wds[2 * j + 1] = pack_bf16x2(e1.x, e1.y);
                        }
                        *reinterpret_cast<uint4*>(ds_row + (static_cast<uint32_t>(q8 ^ (row & 7)) << 4)) =
                            make_uint4(wds[0], wds[1], wds[2], wds[3]);
                    }
                    fence_proxy_async_smem();
                    tc_fence_before();
                    mbar_arrive(bar(kBDsReady));
                    if (warp == 0 && lane == 0 && it < 64) FBA_TRACE_REC(p.status, it * 8 + 3);
                }
            }
        }

        // Epilogue: warps 0-3 write dV, warps 4-7 write dK (bf16, through swizzled staging + TMA).
        if (n_total > 0 && ok) {
            if (!mbar_wait(bar(kBDkvDone), 0, abort_flag)) {
                if (lane == 0) report_timeout(p.status, 2, static_cast<uint32_t>(warp), 0, 500);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
        }
        const uint32_t stage_off = h == 0 ? kBwdSmemQ : kBwdSmemQ + kTileBytes;
        if (ok) {
            tc_fence_after();
            const uint32_t tsrc = (h == 0 ? tDV : tDK) + lane_base;
            uint8_t* stage = base_ptr + stage_off;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t v[32];
                if (n_total > 0) {
                    tmem_ld32(tsrc + 32u * cc, v);
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
                    const int chunk = cc * 4 + q4;
                    const uint32_t o = static_cast<uint32_t>(chunk >> 3) * kPanelBytes +
                                       static_cast<uint32_t>(row) * 128u +
                                       (static_cast<uint32_t>((chunk & 7) ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4*>(stage + o) = wv;
                }
            }
            fence_proxy_async_smem();
        }
        named_bar_sync(1 + h, 128);
        if (ok && quad == 0 && lane == 0) {
            const CUtensorMap* tm = h == 0 ? &tm_dv : &tm_dk;
            tma_store_3d(tm, 0, nt * 128, bhk, base + stage_off);
            tma_store_3d(tm, 64, nt * 128, bhk, base + stage_off + kPanelBytes);
            tma_commit_group();
            tma_wait_group0();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 12) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace fba

using namespace fba;

extern "C" int fba_bwd_scratch_bytes(int B, int Hq, int Sq, uint64_t* lse_delta_bytes,
                                     uint64_t* dq_accum_bytes) {
    if (B <= 0 || Hq <= 0 || Sq <= 0 || !lse_delta_bytes || !dq_accum_bytes)
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd_scratch_bytes: bad argument");
    const uint64_t rows = static_cast<uint64_t>(B) * Hq * ((Sq + 127) / 128) * 128;
    *lse_delta_bytes = rows * 2 * sizeof(float);
    *dq_accum_bytes = rows * 128 * sizeof(float);
    return FBA_OK;
}

namespace fba {
int launch_bwd_v2(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_do,
                  const CUtensorMap& tm_dk, const CUtensorMap& tm_dv, const fba_list_t& k2q, const float* lse_delta,
                  float* dq_accum, uint32_t* status, int n_mtiles, int n_ntiles, long long n_bhk, int Hq, int Hkv,
                  float scale, cudaStream_t stream);

// Which key-major kernel the default dQ mode runs: 1 = score tile transposed, lane = key row
// (fba_bwd_kernel<1>); 2 = lane = query row (fba_bwd_v2_kernel).  Set by fba_set_bwd_kernel() or, before
// the first call, by the environment variable FBA_BWD_KERNEL.
static int g_bwd_kernel = 0;   // 0 = not chosen yet
static int bwd_kernel_choice() {
    int c = __atomic_load_n(&g_bwd_kernel, __ATOMIC_RELAXED);
    if (c == 0) {
        const char* e = getenv("FBA_BWD_KERNEL");
        c = (e && e[0] == '2' && e[1] == 0) ? 2 : (e && e[0] == '1' && e[1] == 0) ? 1 : FBA_BWD_KERNEL_DEFAULT;
        __atomic_store_n(&g_bwd_kernel, c, __ATOMIC_RELAXED);
    }
    return c;
}

int launch_bwd_dq(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_do,
                  const CUtensorMap& tm_dq, const fba_list_t& q2k, const float* lse_delta, uint32_t* status,
                  int n_mtiles, long long n_bhq, int Hq, int Hkv, float scale, cudaStream_t stream);
}

extern "C" int fba_set_bwd_kernel(int which) {
    if (which != 1 && which != 2) return set_error(FBA_ERR_BAD_ARG, "fba_set_bwd_kernel: which must be 1 or 2");
    const int prev = bwd_kernel_choice();
    __atomic_store_n(&g_bwd_kernel, which, __ATOMIC_RELAXED);
    return prev;
}

extern "C" int fba_bwd_ex(const void* q, const void* k, const void* v, const void* o, const float* lse,
                          const void* dout, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq,
                          int Skv, const fba_list_t* k2q, const fba_list_t* q2k, float softmax_scale, int dq_mode,
                          float* lse_delta, float* dq_accum, uint32_t* status, void* stream_) {
    ProfRange range("fba_bwd");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dq_mode != FBA_DQ_ATOMIC && dq_mode != FBA_DQ_QMAJOR)
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd: dq_mode must be FBA_DQ_ATOMIC or FBA_DQ_QMAJOR");
    const bool qmajor = dq_mode == FBA_DQ_QMAJOR;
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv || !lse_delta || !status ||
        (!qmajor && !dq_accum))
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd: null pointer argument");
    if (qmajor) {
        if (!q2k || !q2k->idx || !q2k->cnt || q2k->stride <= 0 || q2k->rows_per_bh <= 0 || q2k->rows_div <= 0 ||
            q2k->sub <= 0 || (q2k->bh_stride != 0 && q2k->bh_stride != q2k->rows_per_bh))
            return set_error(FBA_ERR_BAD_ARG, "fba_bwd: the query-major dQ pass needs a well-formed q2k list");
        const int nm = (Sq + 127) / 128, nn = (Skv + 127) / 128;
        if (static_cast<long long>(q2k->rows_per_bh) * q2k->rows_div < nm ||
            static_cast<long long>(q2k->stride) * q2k->sub < nn || nn % q2k->sub != 0 || nm % q2k->rows_div != 0)
            return set_error(FBA_ERR_BAD_ARG, "fba_bwd: q2k list does not cover the sequences");
    }
    if (!(softmax_scale > 0.f) || !(softmax_scale < INFINITY))
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd: softmax_scale must be positive and finite");
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd: non-positive size");
    if (Hq % Hkv != 0) return set_error(FBA_ERR_BAD_ARG, "fba_bwd: Hq must be a multiple of Hkv");
    if (Sq < 128 || Skv < 128)
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd: sequence lengths below 128 are not supported");
    if (!k2q || !k2q->idx || !k2q->cnt || k2q->stride <= 0 || k2q->rows_per_bh <= 0 || k2q->rows_div <= 0 ||
        k2q->sub <= 0 || (k2q->bh_stride != 0 && k2q->bh_stride != k2q->rows_per_bh))
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd: malformed k2q list");
    const int n_mtiles = (Sq + 127) / 128;
    const int n_ntiles = (Skv + 127) / 128;
    if (static_cast<long long>(k2q->rows_per_bh) * k2q->rows_div < n_ntiles ||
        static_cast<long long>(k2q->stride) * k2q->sub < n_mtiles)
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd: k2q list does not cover the sequences");
    // An entry stands for `sub` whole query tiles and a list row for `rows_div` whole key tiles: a
    // sequence that ends inside such a group would make the kernel touch scratch past its end.
    if (n_mtiles % k2q->sub != 0 || n_ntiles % k2q->rows_div != 0)
        return set_error(FBA_ERR_BAD_ARG,
                         "fba_bwd: ceil(Sq/128) must be a multiple of k2q->sub and ceil(Skv/128) of k2q->rows_div");
    if (static_cast<long long>(B) * Hq > 65535)
        return set_error(FBA_ERR_TOO_LARGE, "fba_bwd: B * Hq exceeds 65535");

    const long long n_bhq = static_cast<long long>(B) * Hq, n_bhk = static_cast<long long>(B) * Hkv;
    CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, tm_dq;
    int rc;
    DeviceGuard guard;
    if ((rc = guard.bind(q)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_q, q, Sq, n_bhq, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_k, k, Skv, n_bhk, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_v, v, Skv, n_bhk, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_do, dout, Sq, n_bhq, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_dk, dk, Skv, n_bhk, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_dv, dv, Skv, n_bhk, 128)) != FBA_OK) return rc;
    if (qmajor && (rc = make_tmap_bf16(&tm_dq, dq, Sq, n_bhq, 128)) != FBA_OK) return rc;

    const int rows_pad = n_mtiles * 128;
    const long long total_rows = n_bhq * rows_pad;
    {
        if (total_rows > 0x7fffff00LL) return set_error(FBA_ERR_TOO_LARGE, "fba_bwd: more than 2^31 query rows");
        long long blocks = (total_rows + 31) / 32;             // 8 warps x 4 rows per step
        if (blocks > 148 * 16) blocks = 148 * 16;
        bwd_prep_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), lse,
            reinterpret_cast<float2*>(lse_delta), static_cast<uint32_t>(Sq), static_cast<uint32_t>(rows_pad),
            static_cast<uint32_t>(total_rows), softmax_scale);
        if ((rc = check_launch("bwd_prep_kernel")) != FBA_OK) return rc;
    }
    if (!qmajor &&
        cudaMemsetAsync(dq_accum, 0, static_cast<size_t>(total_rows) * 128 * sizeof(float), stream) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_bwd: cudaMemsetAsync failed");
    }
    {
        cudaError_t e = cudaFuncSetAttribute(fba_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kBwdSmemBytes));
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(fba_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kBwdSmemBytes));
        if (e != cudaSuccess) {
            cudaGetLastError();
            return set_error(FBA_ERR_LAUNCH, "fba_bwd: cannot raise the dynamic shared memory limit");
        }
        BwdParams p;
        p.list = to_dev(*k2q);
        p.ld = reinterpret_cast<const float2*>(lse_delta);
        p.dq_accum = dq_accum;
        p.status = status;
        p.n_mtiles = n_mtiles;
        p.Hq = Hq;
        p.Hkv = Hkv;
        p.scale = softmax_scale;
        dim3 grid(n_ntiles, static_cast<unsigned>(n_bhk));
        if (!qmajor && bwd_kernel_choice() == 2) {
            rc = launch_bwd_v2(tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, *k2q, lse_delta, dq_accum, status, n_mtiles,
                               n_ntiles, n_bhk, Hq, Hkv, softmax_scale, stream);
            if (rc != FBA_OK) return rc;
        } else {
            timing_mark(2, true, stream);
            if (qmajor)
                fba_bwd_kernel<false><<<grid, kBwdThreads, kBwdSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, p);
            else
                fba_bwd_kernel<true><<<grid, kBwdThreads, kBwdSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, p);
            rc = check_launch("fba_bwd_kernel");
            timing_mark(2, false, stream);
            if (rc != FBA_OK) return rc;
        }
    }
    if (qmajor)
        return launch_bwd_dq(tm_q, tm_k, tm_v, tm_do, tm_dq, *q2k, lse_delta, status, n_mtiles, n_bhq, Hq, Hkv,
                             softmax_scale, stream);
    {
        dim3 grid(n_mtiles, static_cast<unsigned>(n_bhq));
        bwd_dq_convert_kernel<<<grid, 256, 0, stream>>>(dq_accum, static_cast<__nv_bfloat16*>(dq), Sq, n_mtiles);
        if ((rc = check_launch("bwd_dq_convert_kernel")) != FBA_OK) return rc;
    }
    return FBA_OK;
}

extern "C" int fba_bwd_scaled(const void* q, const void* k, const void* v, const void* o, const float* lse,
                              const void* dout, void* dq, void* dk, void* dv, int B, int Hq, int Hkv,
                              int Sq, int Skv, const fba_list_t* k2q, float softmax_scale, float* lse_delta,
                              float* dq_accum, uint32_t* status, void* stream) {
    return fba_bwd_ex(q, k, v, o, lse, dout, dq, dk, dv, B, Hq, Hkv, Sq, Skv, k2q, nullptr, softmax_scale,
                      FBA_DQ_ATOMIC, lse_delta, dq_accum, status, stream);
}

extern "C" int fba_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                       const void* dout, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq,
                       int Skv, const fba_list_t* k2q, float* lse_delta, float* dq_accum,
                       uint32_t* status, void* stream) {
    return fba_bwd_scaled(q, k, v, o, lse, dout, dq, dk, dv, B, Hq, Hkv, Sq, Skv, k2q, kSoftmaxScale, lse_delta,
                          dq_accum, status, stream);
}

// ------------------------------------------------------------------------------------------
// Backward without caller-provided scratch.
//
// Some hosts of this library may not allocate device memory at the moment they need a backward
// pass: a serving or training process that handed all of its HBM to a fixed arena at start-up, a
// plugin that runs inside someone else's memory pool, or code on a latency-critical path where
// cudaMalloc's implicit device synchronisation is not acceptable.  For them the two scratch
// buffers of fba_bwd live in a fixed device array that is part of the library image.  Every GPU
// whose context loads the library carries this array until the process exits.
//
// Capacity: kStaticScratchRows padded query rows in total (B * Hq * ceil(Sq/128) * 128), each row
// needing 2 floats of (lse, delta) and 128 floats of dQ accumulator.
constexpr unsigned long long kStaticScratchRows = 131072;  // e.g. B*Hq = 8 at Sq = 16384
constexpr unsigned long long kStaticLdBytes = kStaticScratchRows * 2 * sizeof(float);
constexpr unsigned long long kStaticAccBytes = kStaticScratchRows * 128 * sizeof(float);
static __device__ __align__(256) unsigned char g_bwd_static_scratch[kStaticLdBytes + kStaticAccBytes];

constexpr int kMaxDevices = 64;
static unsigned char* g_static_scratch_addr[kMaxDevices];  // device address per device ordinal

extern "C" uint64_t fba_bwd_static_scratch_max_rows(void) { return kStaticScratchRows; }

extern "C" int fba_bwd_static_scratch(const void* q, const void* k, const void* v, const void* o,
                                      const float* lse, const void* dout, void* dq, void* dk, void* dv,
                                      int B, int Hq, int Hkv, int Sq, int Skv, const fba_list_t* k2q,
                                      uint32_t* status, void* stream) {
    if (!q) return set_error(FBA_ERR_BAD_ARG, "fba_bwd_static_scratch: null pointer argument");
    if (B <= 0 || Hq <= 0 || Sq <= 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd_static_scratch: non-positive size");
    const unsigned long long rows =
        static_cast<unsigned long long>(B) * Hq * ((static_cast<unsigned long long>(Sq) + 127) / 128) * 128;
    if (rows > kStaticScratchRows)
        return set_error(FBA_ERR_TOO_LARGE,
                         "fba_bwd_static_scratch: B * Hq * ceil(Sq/128) * 128 exceeds the built-in scratch "
                         "capacity of 131072 rows; use fba_bwd with caller-allocated scratch");
    DeviceGuard guard;
    int rc = guard.bind(q);
    if (rc != FBA_OK) return rc;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_bwd_static_scratch: cannot identify the current device");
    }
    // The array's name is only a host-side handle; the kernels need its device address, which
    // is looked up once per device (with that device current) and cached.
    unsigned char* base = __atomic_load_n(&g_static_scratch_addr[dev], __ATOMIC_ACQUIRE);
    if (!base) {
        void* sym = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&sym, g_bwd_static_scratch);
        if (e != cudaSuccess || !sym) {
            cudaGetLastError();
            return set_error(FBA_ERR_LAUNCH, "fba_bwd_static_scratch: cudaGetSymbolAddress failed");
        }
        base = static_cast<unsigned char*>(sym);
        __atomic_store_n(&g_static_scratch_addr[dev], base, __ATOMIC_RELEASE);
    }
    float* lse_delta = reinterpret_cast<float*>(base);
    float* dq_accum = reinterpret_cast<float*>(base + kStaticLdBytes);
    // fba_bwd overwrites the (lse, delta) region and zero-fills the part of the accumulator it
    // uses before accumulating, so nothing left over from an earlier call is read.
    return fba_bwd(q, k, v, o, lse, dout, dq, dk, dv, B, Hq, Hkv, Sq, Skv, k2q, lse_delta, dq_accum, status,
                   stream);
}
