// Block-sparse attention forward for sm_100a.
//
// Computes what the reference's fwd_attend_ker (flex_block_attn_h100.cu:52-318) computes --
// O = softmax(QK^T / sqrt(128) restricted to the active blocks) V and the row log-sum-exp -- but
// is organised around Blackwell's tensor memory instead of Hopper register accumulators:
//
//   * a CTA owns two 128-row query tiles (A and B) of one (batch, head) and ping-pongs between
//     them, so the tensor core works on one tile while the softmax warps work on the other;
//   * one thread per query tile issues that tile's tcgen05.mma.  S = Q K^T goes to TMEM (128 fp32 columns per tile),
//     the softmax warps read it with tcgen05.ld (one thread = one row, so row max / row sum need
//     no shuffles), write P back as bf16 into the same columns, and O += P V consumes P
//     straight from TMEM; O (128 fp32 columns per tile) never leaves TMEM until the epilogue.
//     TMEM columns: [0,128) S/P of tile A, [128,256) S/P of tile B, [256,384) O_A, [384,512) O_B;
//   * one thread streams only the listed K / V tiles through a 5-stage shared-memory ring with
//     TMA + mbarrier; the list comes from the compaction kernel, not from scanning the mask;
//   * rescaling of O is lazy (only when the running row max grew by more than 2^8), done by the
//     softmax warps between two MMAs of their tile;
//   * optionally a fixed fraction of the exponentials is evaluated by a polynomial on the FMA pipe
//     to unload the special-function unit (FBA_FWD_POLY_PAIRS).
//
// If both query tiles map to the same list row they share every K / V stage; otherwise each tile
// streams its own list ("split" mode) in a fixed interleaving that loader and issuer both follow.
#include "fba_common.cuh"

namespace fba {

constexpr int kFwdThreads = 384;  // warpgroup 0: softmax A, 1: softmax B, 2: {MMA A, TMA, MMA B, idle}
constexpr int kFwdStages = 5;
constexpr uint32_t kFwdSmemQ = 0;
constexpr uint32_t kFwdSmemRing = 2 * kTileBytes;
constexpr uint32_t kFwdSmemBars = kFwdSmemRing + kFwdStages * kTileBytes;
constexpr uint32_t kFwdSmemBytes = kFwdSmemBars + 256 + 1024;  // + alignment slack

// Of every 16 pairs of exponentials, this many are evaluated by ex2_poly2 on the FMA pipe and the
// rest by the special-function unit (16 ex2 / clk / SM, which would otherwise cap the kernel at
// the tensor core's own time for a 128-wide head).
#ifndef FBA_FWD_POLY_PAIRS
#define FBA_FWD_POLY_PAIRS 0
#endif

// P is handed to the MMA issuer in this many pieces per 128-key step, so that O += P V starts while
// the later exponentials are still being computed.
constexpr int kFwdPieces = 4;
constexpr int kFwdPiecePairs = 64 / kFwdPieces;   // bf16x2 words (= TMEM columns) per piece

struct FwdParams {
    ListDev list;
    float* lse;            // may be null: no log-sum-exp is written (inference)
    uint32_t* status;
    int n_mtiles, Sq, Hq, Hkv;
    float scale_log2;      // softmax scale * log2(e)
};

// Barrier slots (8 bytes each) inside the barrier block.
enum FwdBar : uint32_t {
    kBarQFull = 0,                         // 2
    kBarRingFull = 2,                      // kFwdStages
    kBarRingEmpty = 2 + kFwdStages,        // kFwdStages
    kBarSFull = 2 + 2 * kFwdStages,        // 2
    kBarP = 4 + 2 * kFwdStages,            // 2 x 4: piece q of tile t's P is in TMEM (slot 4 t + q)
    kBarTurn = 12 + 2 * kFwdStages,        // 2: the other tile's issuer has issued its block
    kBarODone = 14 + 2 * kFwdStages,       // 2
    kBarCount = 16 + 2 * kFwdStages
};
static_assert(8 * kBarCount + 16 <= 256, "barrier block overflows its 256-byte slot");
static_assert(kFwdSmemBytes <= 232448, "exceeds the 227 KiB shared memory of an sm_100 CTA");

// One piece (8 / kFwdPieces k-steps of 16 keys) of O += P V.
__device__ __forceinline__ void mma_pv_piece(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_smem, int piece,
                                             bool accumulate) {
    const uint32_t b = desc_lo_mnmajor(v_smem);
    constexpr int kSteps = 8 / kFwdPieces;
#pragma unroll
    for (int k = 0; k < kSteps; ++k) {
        const int kk = piece * kSteps + k;
        umma_ts(d_tmem, p_tmem + static_cast<uint32_t>(kk) * 8u, b + kstep_mnmajor(kk), kIdescKM,
                (accumulate || kk > 0) ? 1u : 0u);
    }
}

__global__ void __launch_bounds__(kFwdThreads, 1)
fba_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               const FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + kFwdSmemBars;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kFwdSmemBars + 8 * kBarCount);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kFwdSmemBars + 8 * kBarCount + 4);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    // Work item of this CTA: the blockIdx.x-th entry of the (batch, head)'s longest-first order when
    // one is given (CTAs are dispatched in blockIdx order, so the shortest items of the grid run
    // last and the tail of the launch stays short), else blockIdx.x itself.
    const int pair = p.list.order
                         ? p.list.order[static_cast<long long>(p.list.bh_stride ? bh : 0) * gridDim.x + blockIdx.x]
                         : static_cast<int>(blockIdx.x);
    const int hr = p.Hq / p.Hkv;
    const int bhk = (bh / p.Hq) * p.Hkv + (bh % p.Hq) / hr;

    // Per-tile list rows and lengths (identical in every thread).
    const int mt0 = 2 * pair, mt1 = 2 * pair + 1;
    const bool tile1_valid = mt1 < p.n_mtiles;
    const long long lrow0 = static_cast<long long>(bh) * p.list.bh_stride + mt0 / p.list.rows_div;
    const long long lrow1 = static_cast<long long>(bh) * p.list.bh_stride + (tile1_valid ? mt1 / p.list.rows_div : 0);
    const int sub = p.list.sub;
    const int n0 = p.list.cnt[lrow0] * sub;
    const int n1 = tile1_valid ? p.list.cnt[lrow1] * sub : 0;
    const bool shared_mode = tile1_valid && lrow0 == lrow1;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar(kBarQFull + 0), 1);
        mbar_init(bar(kBarQFull + 1), 1);
        for (int s = 0; s < kFwdStages; ++s) {
            mbar_init(bar(kBarRingFull + s), 1);
            mbar_init(bar(kBarRingEmpty + s), 2);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar(kBarSFull + t), 1);
            for (int q = 0; q < kFwdPieces; ++q) mbar_init(bar(kBarP + 4 * t + q), 128);
            mbar_init(bar(kBarTurn + t), 1);
            mbar_init(bar(kBarODone + t), 1);
        }
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
        tma_prefetch_desc(&tm_o);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t sQ0 = base + kFwdSmemQ, sQ1 = base + kFwdSmemQ + kTileBytes;
    auto ring = [&](int s) { return base + kFwdSmemRing + static_cast<uint32_t>(s) * kTileBytes; };
    auto kv_tile_of = [&](int t, int i) {
        const int e = i / sub;
        return p.list.idx[(t ? lrow1 : lrow0) * p.list.stride + e] * sub + (i - e * sub);
    };

    if (warp >= 8) {
        // Register pool of the CTA = 384 threads x 168 at launch = 3 x 128 x 168.  The budgets set
        // below must not add up to more than that (216 + 216 + 72 = 504), or the increase would
        // wait for registers that are never released.
        reg_dec<72>();
        if (warp == 9) {
            // -------------------------------------------------------------- TMA loader
            if (lane == 0) {
                bool ok = true;
                uint32_t prod = 0;
                if (n0 > 0) {
                    mbar_expect_tx(bar(kBarQFull + 0), kTileBytes);
                    tma_load_3d(sQ0, &tm_q, 0, mt0 * 128, bh, bar(kBarQFull + 0));
                    tma_load_3d(sQ0 + kPanelBytes, &tm_q, 64, mt0 * 128, bh, bar(kBarQFull + 0));
                }
                if (n1 > 0) {
                    mbar_expect_tx(bar(kBarQFull + 1), kTileBytes);
                    tma_load_3d(sQ1, &tm_q, 0, mt1 * 128, bh, bar(kBarQFull + 1));
                    tma_load_3d(sQ1 + kPanelBytes, &tm_q, 64, mt1 * 128, bh, bar(kBarQFull + 1));
                }
                auto load = [&](const CUtensorMap* tm, int kv_tile, uint32_t tag) {
                    if (!ok) return;
                    const int s = prod % kFwdStages;
                    const uint32_t parity = ((prod / kFwdStages) & 1u) ^ 1u;
                    if (!mbar_wait(bar(kBarRingEmpty + s), parity, abort_flag)) {
                        report_timeout(p.status, 1, 9, prod, tag);
                        ok = false;
                        return;
                    }
                    mbar_expect_tx(bar(kBarRingFull + s), kTileBytes);
                    tma_load_3d(ring(s), tm, 0, kv_tile * 128, bhk, bar(kBarRingFull + s));
                    tma_load_3d(ring(s) + kPanelBytes, tm, 64, kv_tile * 128, bhk, bar(kBarRingFull + s));
                    ++prod;
                };
                const int ln[2] = {n0, shared_mode ? 0 : n1};
                const int nmax = ln[0] > ln[1] ? ln[0] : ln[1];
                for (int t = 0; t < 2; ++t)
                    if (ln[t] > 0) load(&tm_k, kv_tile_of(t, 0), 100 + t);
                for (int i = 0; i < nmax && ok; ++i) {
                    for (int t = 0; t < 2; ++t) {
                        if (i < ln[t]) {
                            load(&tm_v, kv_tile_of(t, i), 200 + t);
                            if (i + 1 < ln[t]) load(&tm_k, kv_tile_of(t, i + 1), 100 + t);
                        }
                    }
                }
            }
        } else if (warp == 8 || warp == 10) {
            // -------------------------------------------------------------- MMA issuers
            // One issuing thread per query tile (warp 8: tile A, warp 10: tile B).  A tile's chain
            // S -> softmax -> P V -> next S is serial, and the issuing thread is blocked while its
            // MMAs execute and while it polls barriers; with one thread per tile those bubbles are
            // filled by the other tile's MMAs.
            const int t = warp == 8 ? 0 : 1;
            const int nt = t ? n1 : n0;
            if (lane == 0 && nt > 0) {
                bool ok = true;
                const uint32_t sQt = t ? sQ1 : sQ0;
                const uint32_t tS = tmem + static_cast<uint32_t>(t) * 128u;
                const uint32_t tO = tmem + 256u + static_cast<uint32_t>(t) * 128u;
                const int ln1 = shared_mode ? 0 : n1;   // what the loader streams for tile B
                // Position of an operand in the loader's global order -> ring slot and parity.
                auto wait_full = [&](uint32_t pos, uint32_t tag) -> int {
                    const int s = pos % kFwdStages;
                    if (!mbar_wait(bar(kBarRingFull + s), (pos / kFwdStages) & 1u, abort_flag)) {
                        report_timeout(p.status, 1, static_cast<uint32_t>(warp), pos, tag);
                        ok = false;
                    }
                    return s;
                };
                // Every ring slot needs two releases per use: one from each tile's issuer when the
                // tiles share the stream, both from the only consumer otherwise.
                auto release = [&](int s) {
                    umma_commit(bar(kBarRingEmpty + s));
                    if (!shared_mode) umma_commit(bar(kBarRingEmpty + s));
                };
                // Loader order: K(A,0) K(B,0), then per step i: V(A,i) K(A,i+1) V(B,i) K(B,i+1).
                uint32_t g = (n0 > 0 ? 1u : 0u) + (ln1 > 0 ? 1u : 0u);   // loads before step 0
                const uint32_t pos_k0 = (t == 1 && !shared_mode) ? (n0 > 0 ? 1u : 0u) : 0u;
                if (!mbar_wait(bar(kBarQFull + t), 0, abort_flag)) {
                    report_timeout(p.status, 1, static_cast<uint32_t>(warp), 0, 300 + t);
                    ok = false;
                }
                int slot_k = wait_full(pos_k0, 310 + t);
                if (ok) {
                    tc_fence_after();
                    mma_tile_kk(tS, sQt, ring(slot_k), false);
                    umma_commit(bar(kBarSFull + t));
                    release(slot_k);
                }
                for (int i = 0; i < nt && ok; ++i) {
                    const uint32_t a_v = (i < n0), a_k = (i + 1 < n0), b_v = (i < ln1), b_k = (i + 1 < ln1);
                    const bool own_a = t == 0 || shared_mode;
                    const uint32_t pos_v = own_a ? g : g + a_v + a_k;
                    const uint32_t pos_k = pos_v + 1;
                    g += a_v + a_k + b_v + b_k;
                    const bool more = i + 1 < nt;
                    // Both operands of this step were requested long ago; check them before the
                    // wait for P so that nothing but the MMAs follows it.
                    const int slot_v = wait_full(pos_v, 330 + t);
                    if (more) slot_k = wait_full(pos_k, 340 + t);
                    if (!ok) break;
                    if (i < 64) FBA_TRACE_REC(p.status, 1024 + i * 8 + t * 4 + 0);
                    if (!mbar_wait(bar(kBarP + 4 * t), i & 1u, abort_flag)) {
                        report_timeout(p.status, 1, static_cast<uint32_t>(warp), i, 320 + t);
                        ok = false;
                        break;
                    }
                    // Blocks are issued in the fixed order A(0) B(0) A(1) B(1) ...: that keeps the
                    // two tiles half a period apart, so one tile's softmax always overlaps the
                    // other tile's MMAs instead of both softmaxes competing for the same units.
                    const bool wait_turn = t == 0 ? (i >= 1 && i - 1 < n1) : (i < n0);
                    if (wait_turn && !mbar_wait(bar(kBarTurn + t), (t == 0 ? i - 1 : i) & 1u, abort_flag)) {
                        report_timeout(p.status, 1, static_cast<uint32_t>(warp), i, 350 + t);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (i < 64) FBA_TRACE_REC(p.status, 1024 + i * 8 + t * 4 + 1);
                    mma_pv_piece(tO, tS, ring(slot_v), 0, i > 0);
#pragma unroll
                    for (int q = 1; q < kFwdPieces; ++q) {
                        if (ok && !mbar_wait(bar(kBarP + 4 * t + q), i & 1u, abort_flag)) {
                            report_timeout(p.status, 1, static_cast<uint32_t>(warp), i, 325 + t);
                            ok = false;
                        }
                        if (ok) {
                            tc_fence_after();
                            mma_pv_piece(tO, tS, ring(slot_v), q, true);
                        }
                    }
                    if (!ok) break;
                    if (more) {
                        mma_tile_kk(tS, sQt, ring(slot_k), false);
                        umma_commit(bar(kBarSFull + t));
                        mbar_arrive(bar(kBarTurn + (t ^ 1)));
                        release(slot_v);
                        release(slot_k);
                    } else {
                        umma_commit(bar(kBarODone + t));
                        mbar_arrive(bar(kBarTurn + (t ^ 1)));
                        release(slot_v);
                    }
                    if (i < 64) FBA_TRACE_REC(p.status, 1024 + i * 8 + t * 4 + 2);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        reg_inc<216>();
        const int t = warp >> 2;                       // 0: tile A, 1: tile B
        const int row = (warp & 3) * 32 + lane;        // row inside the tile == TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + lane_base + static_cast<uint32_t>(t) * 128u;
        const uint32_t tO = tmem + lane_base + 256u + static_cast<uint32_t>(t) * 128u;
        const int mt = t ? mt1 : mt0;
        const int nt = t ? n1 : n0;
        const long long lrow = t ? lrow1 : lrow0;
        const uint32_t sQt = t ? sQ1 : sQ0;
        const bool tile_valid = mt < p.n_mtiles;
        const float c = p.scale_log2;
        const int g = row >> 4;
        const bool tracer = (warp & 3) == 0 && lane == 0;

        float off = 0.f;        // exponent offset (scaled-by-c row max the exponentials refer to)
        bool have_off = false;  // false until the row has seen a finite score
        float2 l2a = make_float2(0.f, 0.f), l2b = make_float2(0.f, 0.f);
        bool ok = true;

        for (int i = 0; i < nt && ok; ++i) {
            if (!mbar_wait(bar(kBarSFull + t), i & 1u, abort_flag)) {
                if (lane == 0) report_timeout(p.status, 1, static_cast<uint32_t>(warp), i, 400 + t);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (tracer && i < 64) FBA_TRACE_REC(p.status, i * 8 + t * 4 + 0);
            uint32_t u[128];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc)
                tmem_ld32(tS + 32u * cc, reinterpret_cast<uint32_t(&)[32]>(u[32 * cc]));
            tmem_wait_ld();
            if (tracer && i < 64) FBA_TRACE_REC(p.status, i * 8 + t * 4 + 1);

            if (p.list.msk != nullptr) {
                const uint32_t w = p.list.msk[lrow * p.list.stride + i / sub];
                if (w != 0xffffu) {
                    const bool keep0 = (w >> g) & 1u, keep1 = (w >> (8 + g)) & 1u;
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        if (!keep0) u[j] = 0xff800000u;
                        if (!keep1) u[64 + j] = 0xff800000u;
                    }
                }
            }
            // Row maximum: eight independent chains of two-input maxima.
            float mm[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) mm[j] = __uint_as_float(u[j]);
#pragma unroll
            for (int j = 8; j < 128; ++j) mm[j & 7] = fmaxf(mm[j & 7], __uint_as_float(u[j]));
            const float mx = fmaxf(fmaxf(fmaxf(mm[0], mm[1]), fmaxf(mm[2], mm[3])),
                                   fmaxf(fmaxf(mm[4], mm[5]), fmaxf(mm[6], mm[7])));
            if (tracer && i < 64) FBA_TRACE_REC(p.status, i * 8 + t * 4 + 2);

            float alpha = 1.f;
            const float cand = mx * c;
            if (!have_off) {
                if (mx > -INFINITY) {
                    off = cand;
                    have_off = true;
                }
            } else if (cand - off > 8.f) {
                alpha = ex2_approx(off - cand);
                off = cand;
            }
            if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // Rescale this warp's 32 rows of O.  The previous P V of this tile has completed
                // (the commit that released S covers it) and the next one waits for the P barriers.
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t v[32];
                    tmem_ld32(tO + 32u * cc, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
                    tmem_st32(tO + 32u * cc, v);
                }
            }
            l2a.x *= alpha;
            l2a.y *= alpha;
            l2b.x *= alpha;
            l2b.y *= alpha;
            const float neg_off = have_off ? -off : 0.f;
            // P goes to TMEM in pieces (keys in ascending order); a piece is announced to the
            // issuer once its TMEM store has completed.
            uint32_t pk[64];
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                // (plain scalar fused multiply-adds: the packed f32x2 forms measured ~3 % slower here)
                float2 x;
                x.x = fmaf(__uint_as_float(u[2 * j]), c, neg_off);
                x.y = fmaf(__uint_as_float(u[2 * j + 1]), c, neg_off);
                float2 e;
                if ((j & 15) < FBA_FWD_POLY_PAIRS) {
                    e = ex2_poly2(x);
                } else {
                    e.x = ex2_approx(x.x);
                    e.y = ex2_approx(x.y);
                }
                if (j & 1) {
                    l2b.x += e.x;
                    l2b.y += e.y;
                } else {
                    l2a.x += e.x;
                    l2a.y += e.y;
                }
                pk[j] = pack_bf16x2(e.x, e.y);
                if (j % kFwdPiecePairs == kFwdPiecePairs - 1) {
                    const int q = j / kFwdPiecePairs;
                    tmem_st16(tS + 16u * q, reinterpret_cast<uint32_t(&)[16]>(pk[16 * q]));
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(bar(kBarP + 4 * t + q));
                    if (q == 0 && tracer && i < 64) FBA_TRACE_REC(p.status, 3072 + i * 4 + t);
                }
            }
            if (tracer && i < 64) FBA_TRACE_REC(p.status, i * 8 + t * 4 + 3);
        }
        const float l = (l2a.x + l2a.y) + (l2b.x + l2b.y);

        // Epilogue: O / l -> bf16 -> swizzled staging in this tile's Q buffer -> TMA store.
        if (tile_valid) {
            if (nt > 0 && ok) {
                if (!mbar_wait(bar(kBarODone + t), 0, abort_flag)) {
                    if (lane == 0) report_timeout(p.status, 1, static_cast<uint32_t>(warp), 0, 500 + t);
                    ok = false;
                }
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                tc_fence_after();
                const float inv_l = l > 0.f ? 1.f / l : 0.f;
                uint8_t* stage = base_ptr + kFwdSmemQ + static_cast<uint32_t>(t) * kTileBytes;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t v[32];
                    if (nt > 0) {
                        tmem_ld32(tO + 32u * cc, v);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = 0u;
                    }
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 w;
                        w.x = pack_bf16x2(__uint_as_float(v[8 * q4 + 0]) * inv_l, __uint_as_float(v[8 * q4 + 1]) * inv_l);
                        w.y = pack_bf16x2(__uint_as_float(v[8 * q4 + 2]) * inv_l, __uint_as_float(v[8 * q4 + 3]) * inv_l);
                        w.z = pack_bf16x2(__uint_as_float(v[8 * q4 + 4]) * inv_l, __uint_as_float(v[8 * q4 + 5]) * inv_l);
                        w.w = pack_bf16x2(__uint_as_float(v[8 * q4 + 6]) * inv_l, __uint_as_float(v[8 * q4 + 7]) * inv_l);
                        const int chunk = cc * 4 + q4;  // 16-byte chunk 0..15 of the 256-byte row
                        const uint32_t o = static_cast<uint32_t>(chunk >> 3) * kPanelBytes +
                                           static_cast<uint32_t>(row) * 128u +
                                           (static_cast<uint32_t>((chunk & 7) ^ (row & 7)) << 4);
                        *reinterpret_cast<uint4*>(stage + o) = w;
                    }
                }
                const int grow = mt * 128 + row;
                if (p.lse != nullptr && grow < p.Sq)
                    p.lse[static_cast<long long>(bh) * p.Sq + grow] =
                        l > 0.f ? (off + lg2_approx(l)) * kLn2 : -INFINITY;
                fence_proxy_async_smem();
            }
            named_bar_sync(1 + t, 128);
            if (ok && (warp & 3) == 0 && lane == 0) {
                tma_store_3d(&tm_o, 0, mt * 128, bh, sQt);
                tma_store_3d(&tm_o, 64, mt * 128, bh, sQt + kPanelBytes);
                tma_commit_group();
                tma_wait_group0();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace fba

using namespace fba;

static int check_list(const fba_list_t* l, const char* who) {
    if (!l || !l->idx || !l->cnt) return set_error(FBA_ERR_BAD_ARG, who);
    if (l->stride <= 0 || l->rows_per_bh <= 0 || l->rows_div <= 0 || l->sub <= 0 ||
        (l->bh_stride != 0 && l->bh_stride != l->rows_per_bh))
        return set_error(FBA_ERR_BAD_ARG, who);
    return FBA_OK;
}

static int fwd_impl(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Hq,
                    int Hkv, int Sq, int Skv, const fba_list_t* q2k, float softmax_scale, uint32_t* status,
                    void* stream_) {
    ProfRange range("fba_fwd");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!q || !k || !v || !o || !status)
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd: null pointer argument");
    if (!(softmax_scale > 0.f) || !(softmax_scale < INFINITY))
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd: softmax_scale must be positive and finite");
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd: non-positive size");
    if (Hq % Hkv != 0) return set_error(FBA_ERR_BAD_ARG, "fba_fwd: Hq must be a multiple of Hkv");
    if (Sq < 128 || Skv < 128)
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd: sequence lengths below 128 are not supported");
    int rc = check_list(q2k, "fba_fwd: malformed q2k list");
    if (rc != FBA_OK) return rc;
    const int n_mtiles = (Sq + 127) / 128;
    const int n_ntiles = (Skv + 127) / 128;
    if (static_cast<long long>(q2k->rows_per_bh) * q2k->rows_div < n_mtiles ||
        static_cast<long long>(q2k->stride) * q2k->sub < n_ntiles)
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd: q2k list does not cover the sequences");
    // An entry stands for `sub` whole key tiles and a list row for `rows_div` whole query tiles: a
    // sequence that ends inside such a group would make the kernel touch tiles past its end.
    if (n_ntiles % q2k->sub != 0 || n_mtiles % q2k->rows_div != 0)
        return set_error(FBA_ERR_BAD_ARG,
                         "fba_fwd: ceil(Skv/128) must be a multiple of q2k->sub and ceil(Sq/128) of q2k->rows_div");
    if (static_cast<long long>(B) * Hq > 65535)
        return set_error(FBA_ERR_TOO_LARGE, "fba_fwd: B * Hq exceeds 65535");
    DeviceGuard guard;
    if ((rc = guard.bind(q)) != FBA_OK) return rc;

    CUtensorMap tm_q, tm_k, tm_v, tm_o;
    if ((rc = make_tmap_bf16(&tm_q, q, Sq, static_cast<long long>(B) * Hq, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_k, k, Skv, static_cast<long long>(B) * Hkv, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_v, v, Skv, static_cast<long long>(B) * Hkv, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_o, o, Sq, static_cast<long long>(B) * Hq, 128)) != FBA_OK) return rc;

    {
        cudaError_t e = cudaFuncSetAttribute(fba_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kFwdSmemBytes));
        if (e != cudaSuccess) {
            cudaGetLastError();
            return set_error(FBA_ERR_LAUNCH, "fba_fwd: cannot raise the dynamic shared memory limit");
        }
    }
    FwdParams p;
    p.list = to_dev(*q2k);
    p.lse = lse;
    p.status = status;
    p.n_mtiles = n_mtiles;
    p.Sq = Sq;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.scale_log2 = softmax_scale * kLog2e;
    dim3 grid((n_mtiles + 1) / 2, B * Hq);
    timing_mark(1, true, stream);
    fba_fwd_kernel<<<grid, kFwdThreads, kFwdSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_o, p);
    rc = check_launch("fba_fwd_kernel");
    timing_mark(1, false, stream);
    return rc;
}

extern "C" int fba_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Hq,
                       int Hkv, int Sq, int Skv, const fba_list_t* q2k, uint32_t* status, void* stream) {
    if (!lse) return set_error(FBA_ERR_BAD_ARG, "fba_fwd: null pointer argument");
    return fwd_impl(q, k, v, o, lse, B, Hq, Hkv, Sq, Skv, q2k, kSoftmaxScale, status, stream);
}

extern "C" int fba_fwd_scaled(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                              int Hq, int Hkv, int Sq, int Skv, const fba_list_t* q2k,
                              float softmax_scale, uint32_t* status, void* stream) {
    return fwd_impl(q, k, v, o, lse, B, Hq, Hkv, Sq, Skv, q2k, softmax_scale, status, stream);
}
