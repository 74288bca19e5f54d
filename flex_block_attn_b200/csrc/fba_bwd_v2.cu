// Key-major backward main kernel, query-row orientation ("v2"), for sm_100a.
//
// Same job, grid, lists, scratch layouts and results as fba_bwd_kernel<1> (fba_bwd.cu): a CTA owns
// one 128-row K/V tile, walks the key-major list of query tiles, keeps dK and dV in tensor memory
// for its whole life and reduce-adds one 128x128 fp32 dQ partial per query tile into the dQ
// accumulator.  What differs is the orientation of the score tile.  fba_bwd_kernel computes
// S^T = K Q^T (TMEM lane = key row), so every compute thread needs the log-sum-exp and delta of 64
// different query columns per tile pair and fetches them with broadcast shared-memory reads: about
// 1000 of the ~1300 LSU shared-memory wavefronts per tile pair, a quarter of all the shared-memory
// traffic of a kernel that ncu shows to be bound by exactly that.  Here
//     S   = Q K^T          (smem x smem -> TMEM, lane = query row)
//     dP  = dO V^T         (smem x smem -> TMEM)
// so a compute thread owns one query row and its log-sum-exp / delta are two scalars, and
//     P   -> bf16 [q][kv] in shared memory          dV += P^T dO    (A = P, MN-major)
//     dS  -> bf16 [q][kv] over the same buffer      dQ  = dS K      (A = dS, K-major)
//                                                   dK += dS^T Q    (A = dS, MN-major)
// P no longer lives in the S columns of tensor memory, so S of the next query tile can be issued as
// soon as the compute warps have read the current one, instead of after dV.
// TMEM columns: [0,128) S, [128,256) dV, [256,384) dP then dQ, [384,512) dK.
//
// Warp roles (512 threads): warps 0-7 compute (thread = query row; warps 0-3 take key columns 0-63
// of the tile, warps 4-7 columns 64-127), warps 8-11 drain dQ, warp 12 issues S and dV, warp 13
// drives TMA, warp 14 issues dP, dQ and dK.
#include "fba_common.cuh"

namespace fba {

constexpr int kV2Threads = 512;
constexpr uint32_t kV2SmemK = 0;
constexpr uint32_t kV2SmemV = 1 * kTileBytes;
constexpr uint32_t kV2SmemQ = 2 * kTileBytes;     // 2 stages
constexpr uint32_t kV2SmemDO = 4 * kTileBytes;    // 2 stages
constexpr uint32_t kV2SmemPS = 6 * kTileBytes;    // P, then dS
constexpr uint32_t kV2SmemLD = 7 * kTileBytes;    // 2 stages x (128 x lse2, 128 x delta)
constexpr uint32_t kV2SmemBars = kV2SmemLD + 2 * 1024;

enum V2Bar : uint32_t {
    kVKvFull = 0,
    kVQFull = 1,       // 2
    kVQEmpty = 3,      // 2
    kVDoFull = 5,      // 2
    kVDoEmpty = 7,     // 2 (two releases each: dP and dV)
    kVSFull = 9,
    kVSRead = 10,      // 256: the compute warps have loaded S
    kVPReady = 11,     // 256: P is in shared memory
    kVPFree = 12,      // dV has read P
    kVDpFull = 13,
    kVDsReady = 14,    // 256: dS is in shared memory (and dP has been loaded)
    kVDsFree = 15,     // dQ and dK have read dS
    kVDqFull = 16,
    kVDqDrained = 17,  // 128
    kVDkvDone = 18,    // 2
    kVCount = 19
};
constexpr uint32_t kV2SmemBytes = kV2SmemBars + 8 * kVCount + 16;
static_assert(kV2SmemBytes <= 232448, "exceeds the 227 KiB shared memory of an sm_100 CTA");

#ifndef FBA_RED_SLEEP_NS
#define FBA_RED_SLEEP_NS 32
#endif

struct V2Params {
    ListDev list;          // key-major: rows = key tiles / rows_div, entries = query tiles / sub
    const float* ld;       // [B*Hq, nMt, 2, 128]: per query tile 128 x (-lse*log2e), then 128 x (-delta*scale)
    float* dq_accum;       // [B*Hq, nMt, 4 column chunks, 4 row groups, 8, 32, 4] fp32
    uint32_t* status;
    int n_mtiles, Hq, Hkv;
    float scale;
};

__device__ __forceinline__ void v2_red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

__global__ void __launch_bounds__(kV2Threads, 1)
fba_bwd_v2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                  const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                  const V2Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    uint8_t* base_ptr = smem_raw;
    const uint32_t bars = base + kV2SmemBars;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kV2SmemBars + 8 * kVCount);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kV2SmemBars + 8 * kVCount + 4);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bhk = blockIdx.y;         // b * Hkv + kv head
    const int nt = p.list.order
                       ? p.list.order[static_cast<long long>(p.list.bh_stride ? bhk : 0) * gridDim.x + blockIdx.x]
                       : static_cast<int>(blockIdx.x);
    const int hr = p.Hq / p.Hkv;
    const int bq0 = (bhk / p.Hkv) * p.Hq + (bhk % p.Hkv) * hr;  // first query head of the group
    const int sub = p.list.sub;

    if ((base & 1023u) != 0u) {
        if (threadIdx.x == 0) report_timeout(p.status, 5, 99, 0, 999);
        return;
    }

    auto list_row = [&](int r) {
        return static_cast<long long>(bq0 + r) * p.list.bh_stride + nt / p.list.rows_div;
    };
    int n_total = 0;
    for (int r = 0; r < hr; ++r) n_total += p.list.cnt[list_row(r)] * sub;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar(kVKvFull), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(kVQFull + s), 1);
            mbar_init(bar(kVQEmpty + s), 1);
            mbar_init(bar(kVDoFull + s), 1);
            mbar_init(bar(kVDoEmpty + s), 2);
        }
        mbar_init(bar(kVSFull), 1);
        mbar_init(bar(kVSRead), 256);
        mbar_init(bar(kVPReady), 256);
        mbar_init(bar(kVPFree), 1);
        mbar_init(bar(kVDpFull), 1);
        mbar_init(bar(kVDsReady), 256);
        mbar_init(bar(kVDsFree), 1);
        mbar_init(bar(kVDqFull), 1);
        mbar_init(bar(kVDqDrained), 128);
        mbar_init(bar(kVDkvDone), 2);
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
    const uint32_t tS = tmem + 0, tDV = tmem + 128, tDP = tmem + 256, tDK = tmem + 384;
    const uint32_t sK = base + kV2SmemK, sV = base + kV2SmemV, sPS = base + kV2SmemPS;
    auto sDO = [&](int s) { return base + kV2SmemDO + static_cast<uint32_t>(s) * kTileBytes; };
    auto sQ = [&](int s) { return base + kV2SmemQ + static_cast<uint32_t>(s) * kTileBytes; };

    // Register budget as in fba_bwd_kernel: 144 * 3 + 80 = 512 = 4 x 128.
    if (warp >= 12) {
      reg_dec<80>();
      if (warp == 13) {
        // ------------------------------------------------------------------ TMA loader
        if (lane == 0 && n_total > 0) {
            mbar_expect_tx(bar(kVKvFull), 2 * kTileBytes);
            tma_load_3d(sK, &tm_k, 0, nt * 128, bhk, bar(kVKvFull));
            tma_load_3d(sK + kPanelBytes, &tm_k, 64, nt * 128, bhk, bar(kVKvFull));
            tma_load_3d(sV, &tm_v, 0, nt * 128, bhk, bar(kVKvFull));
            tma_load_3d(sV + kPanelBytes, &tm_v, 64, nt * 128, bhk, bar(kVKvFull));
            int r = 0, e = 0, u = 0;
            long long lr = list_row(0);
            int cnt = p.list.cnt[lr];
            while (r < hr && cnt == 0) {
                ++r;
                if (r < hr) { lr = list_row(r); cnt = p.list.cnt[lr]; }
            }
            for (int it = 0; it < n_total; ++it) {
                const int st = it & 1;
                const int qt = p.list.idx[lr * p.list.stride + e] * sub + u, bq = bq0 + r;
                if (!mbar_wait(bar(kVQEmpty + st), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_timeout(p.status, 5, 13, it, 100);
                    break;
                }
                mbar_expect_tx(bar(kVQFull + st), kTileBytes + 1024);
                tma_load_3d(sQ(st), &tm_q, 0, qt * 128, bq, bar(kVQFull + st));
                tma_load_3d(sQ(st) + kPanelBytes, &tm_q, 64, qt * 128, bq, bar(kVQFull + st));
                bulk_load(base + kV2SmemLD + st * 1024u,
                          p.ld + (static_cast<long long>(bq) * p.n_mtiles + qt) * 256, 1024, bar(kVQFull + st));
                if (!mbar_wait(bar(kVDoEmpty + st), ((it >> 1) & 1u) ^ 1u, abort_flag)) {
                    report_timeout(p.status, 5, 13, it, 101);
                    break;
                }
                mbar_expect_tx(bar(kVDoFull + st), kTileBytes);
                tma_load_3d(sDO(st), &tm_do, 0, qt * 128, bq, bar(kVDoFull + st));
                tma_load_3d(sDO(st) + kPanelBytes, &tm_do, 64, qt * 128, bq, bar(kVDoFull + st));
                // advance (query head, list entry, sub-tile)
                if (++u == sub) {
                    u = 0;
                    ++e;
                    while (r < hr && e >= cnt) {
                        ++r;
                        e = 0;
                        if (r < hr) { lr = list_row(r); cnt = p.list.cnt[lr]; }
                    }
                }
            }
        }
      } else if (warp == 12) {
        // ------------------------------------------------------------------ MMA issuer A: S and dV
        if (lane == 0 && n_total > 0) {
            bool ok = true;
            auto wait = [&](uint32_t slot, uint32_t parity, int it, uint32_t tag) {
                if (!ok) return;
                if (!mbar_wait(bar(slot), parity, abort_flag)) {
                    report_timeout(p.status, 5, 12, it, tag);
                    ok = false;
                }
            };
            wait(kVKvFull, 0, 0, 200);
            wait(kVQFull + 0, 0, 0, 201);
            if (ok) {
                tc_fence_after();
                mma_tile_kk(tS, sQ(0), sK, false);
                umma_commit(bar(kVSFull));
            }
            for (int it = 0; it < n_total && ok; ++it) {
                const int st = it & 1;
                const bool more = it + 1 < n_total;
                bool s_issued = false;
                auto issue_next_s = [&]() {
                    tc_fence_after();
                    mma_tile_kk(tS, sQ(st ^ 1), sK, false);
                    umma_commit(bar(kVSFull));
                    s_issued = true;
                };
                // S of the next query tile only needs the next Q tile and the S columns, which are
                // free once the compute warps have loaded S of this tile: issue it ahead of dV if
                // both are already there.
                if (more && mbar_try_wait(bar(kVQFull + (st ^ 1)), ((it + 1) >> 1) & 1u) &&
                    mbar_try_wait(bar(kVSRead), it & 1u))
                    issue_next_s();
                wait(kVDoFull + st, (it >> 1) & 1u, it, 215);
                wait(kVPReady, it & 1u, it, 210);
                if (!ok) break;
                tc_fence_after();
                mma_tile_mm(tDV, sPS, sDO(st), it > 0);        // dV += P^T dO
                umma_commit(bar(kVPFree));
                umma_commit(bar(kVDoEmpty + st));              // one of the two releases of dO(it)
                if (more && !s_issued) {
                    wait(kVQFull + (st ^ 1), ((it + 1) >> 1) & 1u, it, 211);
                    wait(kVSRead, it & 1u, it, 212);
                    if (!ok) break;
                    issue_next_s();
                }
            }
            if (ok) umma_commit(bar(kVDkvDone));
        }
      } else if (warp == 14) {
        // ------------------------------------------------------------------ MMA issuer B: dP, dQ, dK
        if (lane == 0 && n_total > 0) {
            bool ok = true;
            auto wait = [&](uint32_t slot, uint32_t parity, int it, uint32_t tag) {
                if (!ok) return;
                if (!mbar_wait(bar(slot), parity, abort_flag)) {
                    report_timeout(p.status, 5, 14, it, tag);
                    ok = false;
                }
            };
            wait(kVKvFull, 0, 0, 220);
            wait(kVDoFull + 0, 0, 0, 202);
            if (ok) {
                tc_fence_after();
                mma_tile_kk(tDP, sDO(0), sV, false);
                umma_commit(bar(kVDpFull));
                umma_commit(bar(kVDoEmpty + 0));               // the other release of dO(0)
            }
            for (int it = 0; it < n_total && ok; ++it) {
                const int st = it & 1;
                const uint32_t ph = it & 1u;
                wait(kVDsReady, ph, it, 213);
                if (!ok) break;
                tc_fence_after();
                mma_tile_km(tDP, sPS, sK, false);              // dQ = dS K (first: its drain overlaps dK)
                umma_commit(bar(kVDqFull));
                mma_tile_mm(tDK, sPS, sQ(st), it > 0);         // dK += dS^T Q
                umma_commit(bar(kVQEmpty + st));
                umma_commit(bar(kVDsFree));
                if (it + 1 < n_total) {
                    wait(kVDoFull + (st ^ 1), ((it + 1) >> 1) & 1u, it, 214);
                    wait(kVDqDrained, ph, it, 216);
                    if (!ok) break;
                    tc_fence_after();
                    mma_tile_kk(tDP, sDO(st ^ 1), sV, false);
                    umma_commit(bar(kVDpFull));
                    umma_commit(bar(kVDoEmpty + (st ^ 1)));
                }
            }
            if (ok) umma_commit(bar(kVDkvDone));
        }
      }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ dQ drain
        reg_inc<144>();
        const int quad = warp & 3;
        const uint32_t tdq = tDP + (static_cast<uint32_t>(quad * 32) << 16);
        int it = 0;
        bool ok = true;
        for (int r = 0; r < hr && ok; ++r) {
            const long long lr = list_row(r);
            const int cnt = p.list.cnt[lr];
            const long long bq = bq0 + r;
            for (int e = 0; e < cnt && ok; ++e) {
                const int q0 = p.list.idx[lr * p.list.stride + e] * sub;
                for (int u = 0; u < sub && ok; ++u, ++it) {
                    if (!mbar_wait(bar(kVDqFull), it & 1u, abort_flag)) {
                        if (lane == 0) report_timeout(p.status, 5, static_cast<uint32_t>(warp), it, 300);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    float* dst = p.dq_accum + ((bq * p.n_mtiles + (q0 + u)) * 16LL + quad) * 1024;
                    uint32_t v[128];
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
                        tmem_ld32(tdq + 32u * cc, reinterpret_cast<uint32_t(&)[32]>(v[32 * cc]));
                    tmem_wait_ld();
                    tc_fence_before();
                    mbar_arrive(bar(kVDqDrained));
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            v2_red_add_v4(dst + cc * 4096 + (j * 32 + lane) * 4, __uint_as_float(v[32 * cc + 4 * j]),
                                          __uint_as_float(v[32 * cc + 4 * j + 1]), __uint_as_float(v[32 * cc + 4 * j + 2]),
                                          __uint_as_float(v[32 * cc + 4 * j + 3]));
                            __nanosleep(FBA_RED_SLEEP_NS);
                        }
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ P / dS compute
        reg_inc<144>();
        const int h = warp >> 2;           // key-column half of the tile
        const int quad = warp & 3;
        const int row = quad * 32 + lane;  // query row inside the tile == TMEM lane (epilogue: key row)
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const float c = p.scale * kLog2e;
        const int g = row >> 4;            // 16-row query group of the sub-tile mask
        uint8_t* ps_row = base_ptr + kV2SmemPS + static_cast<uint32_t>(h) * kPanelBytes + static_cast<uint32_t>(row) * 128u;
        int it = 0;
        bool ok = true;
        for (int r = 0; r < hr && ok; ++r) {
            const long long lr = list_row(r);
            const int cnt = p.list.cnt[lr];
            for (int e = 0; e < cnt && ok; ++e) {
                const uint32_t w = p.list.msk ? p.list.msk[lr * p.list.stride + e] : 0xffffu;
                const bool keep = (w >> (8 * h + g)) & 1u;
                for (int u = 0; u < sub && ok; ++u, ++it) {
                    const int st = it & 1;
                    if (!mbar_wait(bar(kVSFull), it & 1u, abort_flag) ||
                        !mbar_wait(bar(kVQFull + st), (it >> 1) & 1u, abort_flag)) {
                        if (lane == 0) report_timeout(p.status, 5, static_cast<uint32_t>(warp), it, 400);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    const float* ld = reinterpret_cast<const float*>(base_ptr + kV2SmemLD + st * 1024);
                    const float lse2 = ld[row];          // -lse * log2e of this query row (-inf: dead / padding row)
                    const float dlt = ld[128 + row];     // -delta * scale
                    float pr[64];
                    {
                        uint32_t s[64];
                        tmem_ld32(tS + lane_base + 64u * h, reinterpret_cast<uint32_t(&)[32]>(s[0]));
                        tmem_ld32(tS + lane_base + 64u * h + 32u, reinterpret_cast<uint32_t(&)[32]>(s[32]));
                        tmem_wait_ld();
                        tc_fence_before();
                        mbar_arrive(bar(kVSRead));       // the S columns may be overwritten by the next tile's S
#pragma unroll
                        for (int j = 0; j < 64; ++j)
                            pr[j] = keep ? ex2_approx(fmaf(__uint_as_float(s[j]), c, lse2)) : 0.f;
                    }
                    // P -> shared memory, once dQ and dK of the previous tile have read dS from there.
                    if (it > 0 && !mbar_wait(bar(kVDsFree), (it - 1) & 1u, abort_flag)) {
                        if (lane == 0) report_timeout(p.status, 5, static_cast<uint32_t>(warp), it, 402);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
#pragma unroll
                    for (int q8 = 0; q8 < 8; ++q8) {
                        uint4 wv;
                        wv.x = pack_bf16x2(pr[8 * q8 + 0], pr[8 * q8 + 1]);
                        wv.y = pack_bf16x2(pr[8 * q8 + 2], pr[8 * q8 + 3]);
                        wv.z = pack_bf16x2(pr[8 * q8 + 4], pr[8 * q8 + 5]);
                        wv.w = pack_bf16x2(pr[8 * q8 + 6], pr[8 * q8 + 7]);
                        *reinterpret_cast<uint4*>(ps_row + (static_cast<uint32_t>(q8 ^ (row & 7)) << 4)) = wv;
                    }
                    fence_proxy_async_smem();
                    mbar_arrive(bar(kVPReady));

                    if (!mbar_wait(bar(kVDpFull), it & 1u, abort_flag)) {
                        if (lane == 0) report_timeout(p.status, 5, static_cast<uint32_t>(warp), it, 401);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t dsw[32];
                    {
                        uint32_t dp[64];
                        tmem_ld32(tDP + lane_base + 64u * h, reinterpret_cast<uint32_t(&)[32]>(dp[0]));
                        tmem_ld32(tDP + lane_base + 64u * h + 32u, reinterpret_cast<uint32_t(&)[32]>(dp[32]));
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float d0 = pr[2 * j] * fmaf(__uint_as_float(dp[2 * j]), p.scale, dlt);
                            const float d1 = pr[2 * j + 1] * fmaf(__uint_as_float(dp[2 * j + 1]), p.scale, dlt);
                            dsw[j] = pack_bf16x2(d0, d1);
                        }
                    }
                    // dS over P, once dV has read P.
                    if (!mbar_wait(bar(kVPFree), it & 1u, abort_flag)) {
                        if (lane == 0) report_timeout(p.status, 5, static_cast<uint32_t>(warp), it, 403);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
#pragma unroll
                    for (int q8 = 0; q8 < 8; ++q8)
                        *reinterpret_cast<uint4*>(ps_row + (static_cast<uint32_t>(q8 ^ (row & 7)) << 4)) =
                            make_uint4(dsw[4 * q8], dsw[4 * q8 + 1], dsw[4 * q8 + 2], dsw[4 * q8 + 3]);
                    fence_proxy_async_smem();
                    tc_fence_before();
                    mbar_arrive(bar(kVDsReady));
                }
            }
        }

        // Epilogue: warps 0-3 write dV, warps 4-7 write dK (bf16, through swizzled staging + TMA);
        // here `row` is the key row (TMEM lane of the dK / dV accumulators).
        if (n_total > 0 && ok) {
            if (!mbar_wait(bar(kVDkvDone), 0, abort_flag)) {
                if (lane == 0) report_timeout(p.status, 5, static_cast<uint32_t>(warp), 0, 500);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
        }
        const uint32_t stage_off = h == 0 ? kV2SmemQ : kV2SmemQ + kTileBytes;
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

int launch_bwd_v2(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_do,
                  const CUtensorMap& tm_dk, const CUtensorMap& tm_dv, const fba_list_t& k2q, const float* lse_delta,
                  float* dq_accum, uint32_t* status, int n_mtiles, int n_ntiles, long long n_bhk, int Hq, int Hkv,
                  float scale, cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(fba_bwd_v2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kV2SmemBytes));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_bwd: cannot raise the dynamic shared memory limit");
    }
    V2Params p;
    p.list = to_dev(k2q);
    p.ld = lse_delta;
    p.dq_accum = dq_accum;
    p.status = status;
    p.n_mtiles = n_mtiles;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.scale = scale;
    dim3 grid(n_ntiles, static_cast<unsigned>(n_bhk));
    timing_mark(2, true, stream);
    fba_bwd_v2_kernel<<<grid, kV2Threads, kV2SmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dk, tm_dv, p);
    int rc = check_launch("fba_bwd_v2_kernel");
    timing_mark(2, false, stream);
    return rc;
}

}  // namespace fba
