// Inference forward with an 8-bit (e4m3) key / value cache, for sm_100a.
//
// No counterpart in the reference (its kernels are bf16 only, flex_block_attn_h100.cu:854-858).  The
// computation is fba_fwd's -- O = softmax(scale * Q K^T on the listed blocks) V -- with K and V
// stored as e4m3 bytes plus fp32 scales (one per (batch, kv head, block of `scale_block` rows)), so
// the K / V stream is half as wide and both GEMMs run as tcgen05.mma.kind::f8f6f4 (32 elements per
// instruction instead of 16):
//   * K8 is [B, Hkv, Skv, 128] bytes; V8 is stored TRANSPOSED, [B, Hkv, 128, Skv] bytes, so that both
//     GEMMs take K-major shared-memory operands (the cache is written once, its layout is free);
//   * Q arrives in bf16; the softmax warps quantise their own row to e4m3 with a per-row scale when
//     the tile lands (thread = row, so the row scale is a per-thread factor of the score);
//   * S = Q8 K8^T in TMEM; the exponent's multiplier is softmax_scale * log2e * q_scale[row] *
//     k_scale[block], so dequantisation costs nothing;
//   * P is written back to TMEM as e4m3 (four per column) times v_scale[block] / max_block v_scale,
//     O += P8 V8^T accumulates in fp32 in TMEM, and the head's largest V scale is applied once in the
//     epilogue; the row sum uses the unquantised P.
// Structure, roles, barriers and the two-tile ping-pong are those of fba_fwd_kernel (fba_fwd.cu).
//
// fba_quantize_kv_e4m3 is the matching cache writer (amax / 448 scaling per block).
#include "fba_common.cuh"

namespace fba {

constexpr int kF8Threads = 384;
constexpr int kF8Stages = 6;
constexpr uint32_t kTile8Bytes = 16384;                       // [128 rows][128 e4m3], 128-byte pitch, swizzled
constexpr uint32_t kF8SmemQ = 0;                              // 2 x bf16 Q tile (later: O staging)
constexpr uint32_t kF8SmemQ8 = 2 * kTileBytes;                // 2 x e4m3 Q tile
constexpr uint32_t kF8SmemRing = kF8SmemQ8 + 2 * kTile8Bytes;
constexpr uint32_t kF8SmemBars = kF8SmemRing + kF8Stages * kTile8Bytes;
constexpr uint32_t kF8SmemBytes = kF8SmemBars + 256 + 1024;   // + alignment slack
constexpr uint32_t kIdescF8 = umma_idesc_e4m3(128, 128, 0, 0);
constexpr float kInvE4m3Max = 1.0f / 448.0f;   // scale = amax * this (one fp32 multiplication, reproducible anywhere)

enum F8Bar : uint32_t {
    kF8QFull = 0,                          // 2: bf16 Q tile landed
    kF8Q8 = 2,                             // 2: e4m3 Q tile written (128 arrivals)
    kF8RingFull = 4,                       // kF8Stages
    kF8RingEmpty = 4 + kF8Stages,          // kF8Stages
    kF8SFull = 4 + 2 * kF8Stages,          // 2
    kF8P = 6 + 2 * kF8Stages,              // 2 x 4
    kF8Turn = 14 + 2 * kF8Stages,          // 2
    kF8ODone = 16 + 2 * kF8Stages,         // 2
    kF8Count = 18 + 2 * kF8Stages
};
static_assert(8 * kF8Count + 16 <= 256, "barrier block overflows its 256-byte slot");
static_assert(kF8SmemBytes <= 232448, "exceeds the 227 KiB shared memory of an sm_100 CTA");

struct F8Params {
    ListDev list;
    const float* k_scale;   // [B*Hkv, n_sblocks]
    const float* v_scale;   // [B*Hkv, n_sblocks]
    float* lse;             // may be null
    uint32_t* status;
    int n_mtiles, Sq, Hq, Hkv, n_sblocks, tiles_per_sblock;
    float scale_log2;
};

__global__ void __launch_bounds__(kF8Threads, 1)
fba_fwd_fp8_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k8,
                   const __grid_constant__ CUtensorMap tm_v8t, const __grid_constant__ CUtensorMap tm_o,
                   const F8Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + kF8SmemBars;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + kF8SmemBars + 8 * kF8Count);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kF8SmemBars + 8 * kF8Count + 4);
    auto bar = [&](uint32_t slot) { return bars + 8u * slot; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int pair = p.list.order
                         ? p.list.order[static_cast<long long>(p.list.bh_stride ? bh : 0) * gridDim.x + blockIdx.x]
                         : static_cast<int>(blockIdx.x);
    const int hr = p.Hq / p.Hkv;
    const int bhk = (bh / p.Hq) * p.Hkv + (bh % p.Hq) / hr;

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
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar(kF8QFull + t), 1);
            mbar_init(bar(kF8Q8 + t), 128);
            mbar_init(bar(kF8SFull + t), 1);
            for (int q = 0; q < 4; ++q) mbar_init(bar(kF8P + 4 * t + q), 128);
            mbar_init(bar(kF8Turn + t), 1);
            mbar_init(bar(kF8ODone + t), 1);
        }
        for (int s = 0; s < kF8Stages; ++s) {
            mbar_init(bar(kF8RingFull + s), 1);
            mbar_init(bar(kF8RingEmpty + s), 2);
        }
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
        tmem_relinquish();
    }
    if (warp == 9 && lane == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k8);
        tma_prefetch_desc(&tm_v8t);
        tma_prefetch_desc(&tm_o);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t sQ0 = base + kF8SmemQ, sQ1 = base + kF8SmemQ + kTileBytes;
    auto sQ8 = [&](int t) { return base + kF8SmemQ8 + static_cast<uint32_t>(t) * kTile8Bytes; };
    auto ring = [&](int s) { return base + kF8SmemRing + static_cast<uint32_t>(s) * kTile8Bytes; };
    auto kv_tile_of = [&](int t, int i) {
        const int e = i / sub;
        return p.list.idx[(t ? lrow1 : lrow0) * p.list.stride + e] * sub + (i - e * sub);
    };

    if (warp >= 8) {
        reg_dec<72>();
        if (warp == 9) {
            // -------------------------------------------------------------- TMA loader
            if (lane == 0) {
                bool ok = true;
                uint32_t prod = 0;
                if (n0 > 0) {
                    mbar_expect_tx(bar(kF8QFull + 0), kTileBytes);
                    tma_load_3d(sQ0, &tm_q, 0, mt0 * 128, bh, bar(kF8QFull + 0));
                    tma_load_3d(sQ0 + kPanelBytes, &tm_q, 64, mt0 * 128, bh, bar(kF8QFull + 0));
                }
                if (n1 > 0) {
                    mbar_expect_tx(bar(kF8QFull + 1), kTileBytes);
                    tma_load_3d(sQ1, &tm_q, 0, mt1 * 128, bh, bar(kF8QFull + 1));
                    tma_load_3d(sQ1 + kPanelBytes, &tm_q, 64, mt1 * 128, bh, bar(kF8QFull + 1));
                }
                auto load = [&](bool is_v, int kv_tile, uint32_t tag) {
                    if (!ok) return;
                    const int s = prod % kF8Stages;
                    const uint32_t parity = ((prod / kF8Stages) & 1u) ^ 1u;
                    if (!mbar_wait(bar(kF8RingEmpty + s), parity, abort_flag)) {
                        report_timeout(p.status, 4, 9, prod, tag);
                        ok = false;
                        return;
                    }
                    mbar_expect_tx(bar(kF8RingFull + s), kTile8Bytes);
                    if (is_v)   // V8^T: 128 rows of d, 128 key bytes starting at the tile's first key
                        tma_load_3d(ring(s), &tm_v8t, kv_tile * 128, 0, bhk, bar(kF8RingFull + s));
                    else        // K8: 128 key rows of 128 bytes
                        tma_load_3d(ring(s), &tm_k8, 0, kv_tile * 128, bhk, bar(kF8RingFull + s));
                    ++prod;
                };
                const int ln[2] = {n0, shared_mode ? 0 : n1};
                const int nmax = ln[0] > ln[1] ? ln[0] : ln[1];
                for (int t = 0; t < 2; ++t)
                    if (ln[t] > 0) load(false, kv_tile_of(t, 0), 100 + t);
                for (int i = 0; i < nmax && ok; ++i) {
                    for (int t = 0; t < 2; ++t) {
                        if (i < ln[t]) {
                            load(true, kv_tile_of(t, i), 200 + t);
                            if (i + 1 < ln[t]) load(false, kv_tile_of(t, i + 1), 100 + t);
                        }
                    }
                }
            }
        } else if (warp == 8 || warp == 10) {
            // -------------------------------------------------------------- MMA issuers (one per tile)
            const int t = warp == 8 ? 0 : 1;
            const int nt = t ? n1 : n0;
            if (lane == 0 && nt > 0) {
                bool ok = true;
                const uint32_t aQ = desc_lo_kmajor(sQ8(t));
                const uint32_t tS = tmem + static_cast<uint32_t>(t) * 128u;
                const uint32_t tO = tmem + 256u + static_cast<uint32_t>(t) * 128u;
                const int ln1 = shared_mode ? 0 : n1;
                auto wait_full = [&](uint32_t pos, uint32_t tag) -> int {
                    const int s = pos % kF8Stages;
                    if (!mbar_wait(bar(kF8RingFull + s), (pos / kF8Stages) & 1u, abort_flag)) {
                        report_timeout(p.status, 4, static_cast<uint32_t>(warp), pos, tag);
                        ok = false;
                    }
                    return s;
                };
                auto release = [&](int s) {
                    umma_commit(bar(kF8RingEmpty + s));
                    if (!shared_mode) umma_commit(bar(kF8RingEmpty + s));
                };
                auto mma_s = [&](int slot_k) {   // S = Q8 K8^T: four 32-element k steps of 32 bytes
                    const uint32_t b = desc_lo_kmajor(ring(slot_k));
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) umma_ss_f8(tS, aQ + 2u * kk, b + 2u * kk, kIdescF8, kk > 0 ? 1u : 0u);
                };
                uint32_t g = (n0 > 0 ? 1u : 0u) + (ln1 > 0 ? 1u : 0u);
                const uint32_t pos_k0 = (t == 1 && !shared_mode) ? (n0 > 0 ? 1u : 0u) : 0u;
                if (!mbar_wait(bar(kF8Q8 + t), 0, abort_flag)) {
                    report_timeout(p.status, 4, static_cast<uint32_t>(warp), 0, 300 + t);
                    ok = false;
                }
                int slot_k = wait_full(pos_k0, 310 + t);
                if (ok) {
                    tc_fence_after();
                    mma_s(slot_k);
                    umma_commit(bar(kF8SFull + t));
                    release(slot_k);
                }
                for (int i = 0; i < nt && ok; ++i) {
                    const uint32_t a_v = (i < n0), a_k = (i + 1 < n0), b_v = (i < ln1), b_k = (i + 1 < ln1);
                    const bool own_a = t == 0 || shared_mode;
                    const uint32_t pos_v = own_a ? g : g + a_v + a_k;
                    const uint32_t pos_k = pos_v + 1;
                    g += a_v + a_k + b_v + b_k;
                    const bool more = i + 1 < nt;
                    const int slot_v = wait_full(pos_v, 330 + t);
                    if (more) slot_k = wait_full(pos_k, 340 + t);
                    if (!ok) break;
                    const bool wait_turn = t == 0 ? (i >= 1 && i - 1 < n1) : (i < n0);
                    const uint32_t bV = desc_lo_kmajor(ring(slot_v));
                    for (int q = 0; q < 4 && ok; ++q) {
                        if (!mbar_wait(bar(kF8P + 4 * t + q), i & 1u, abort_flag)) {
                            report_timeout(p.status, 4, static_cast<uint32_t>(warp), i, 320 + t);
                            ok = false;
                            break;
                        }
                        if (q == 0 && wait_turn &&
                            !mbar_wait(bar(kF8Turn + t), (t == 0 ? i - 1 : i) & 1u, abort_flag)) {
                            report_timeout(p.status, 4, static_cast<uint32_t>(warp), i, 350 + t);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        // O += P8[:, 32 q .. 32 q + 31] V8^T[.., same keys]: one 32-key step
                        umma_ts_f8(tO, tS + 8u * q, bV + 2u * q, kIdescF8, (i > 0 || q > 0) ? 1u : 0u);
                    }
                    if (!ok) break;
                    if (more) {
                        mma_s(slot_k);
                        umma_commit(bar(kF8SFull + t));
                        mbar_arrive(bar(kF8Turn + (t ^ 1)));
                        release(slot_v);
                        release(slot_k);
                    } else {
                        umma_commit(bar(kF8ODone + t));
                        mbar_arrive(bar(kF8Turn + (t ^ 1)));
                        release(slot_v);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        reg_inc<216>();
        const int t = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + lane_base + static_cast<uint32_t>(t) * 128u;
        const uint32_t tO = tmem + lane_base + 256u + static_cast<uint32_t>(t) * 128u;
        const int mt = t ? mt1 : mt0;
        const int nt = t ? n1 : n0;
        const long long lrow = t ? lrow1 : lrow0;
        const uint32_t sQt = t ? sQ1 : sQ0;
        const bool tile_valid = mt < p.n_mtiles;
        const int g = row >> 4;
        const float* ks = p.k_scale + static_cast<long long>(bhk) * p.n_sblocks;
        const float* vs = p.v_scale + static_cast<long long>(bhk) * p.n_sblocks;

        float off = 0.f;
        bool have_off = false;
        float2 l2a = make_float2(0.f, 0.f), l2b = make_float2(0.f, 0.f);
        bool ok = true;
        float c_row = 0.f;        // softmax_scale * log2e * (this row's Q scale)
        float vs_ref = 1.f;       // the head's largest V scale

        if (nt > 0) {
            // Largest V scale of this kv head (P is multiplied by v_scale[block] / vs_ref <= 1 before
            // it is quantised, so one factor remains for the epilogue).
            float m = 0.f;
            for (int b = lane; b < p.n_sblocks; b += 32) m = fmaxf(m, vs[b]);
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
            vs_ref = m > 0.f ? m : 1.f;

            // Quantise this thread's Q row: bf16 (swizzled panels) -> e4m3 (swizzled [128][128 B]).
            if (!mbar_wait(bar(kF8QFull + t), 0, abort_flag)) {
                if (lane == 0) report_timeout(p.status, 4, static_cast<uint32_t>(warp), 0, 390 + t);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                const uint8_t* qrow = base_ptr + kF8SmemQ + static_cast<uint32_t>(t) * kTileBytes + static_cast<uint32_t>(row) * 128u;
                uint4 w[16];
                float amax = 0.f;
#pragma unroll
                for (int ch = 0; ch < 16; ++ch) {
                    w[ch] = *reinterpret_cast<const uint4*>(qrow + static_cast<uint32_t>(ch >> 3) * kPanelBytes +
                                                            (static_cast<uint32_t>((ch & 7) ^ (row & 7)) << 4));
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w[ch]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __bfloat1622float2(h2[j]);
                        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                    }
                }
                const float qs = amax > 0.f ? amax * kInvE4m3Max : 1.f;
                const float inv = 1.f / qs;
                c_row = p.scale_log2 * qs;
                uint8_t* q8row = base_ptr + kF8SmemQ8 + static_cast<uint32_t>(t) * kTile8Bytes + static_cast<uint32_t>(row) * 128u;
#pragma unroll
                for (int j = 0; j < 8; ++j) {      // 16 output bytes = 16 elements = two input chunks
                    uint32_t o4[4];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w[2 * j + u]);
                        const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
                        const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
                        o4[2 * u] = pack_e4m3x4(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
                        o4[2 * u + 1] = pack_e4m3x4(f2.x * inv, f2.y * inv, f3.x * inv, f3.y * inv);
                    }
                    *reinterpret_cast<uint4*>(q8row + (static_cast<uint32_t>(j ^ (row & 7)) << 4)) =
                        make_uint4(o4[0], o4[1], o4[2], o4[3]);
                }
                fence_proxy_async_smem();
                mbar_arrive(bar(kF8Q8 + t));
            }
        }

        for (int i = 0; i < nt && ok; ++i) {
            if (!mbar_wait(bar(kF8SFull + t), i & 1u, abort_flag)) {
                if (lane == 0) report_timeout(p.status, 4, static_cast<uint32_t>(warp), i, 400 + t);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t u[128];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc)
                tmem_ld32(tS + 32u * cc, reinterpret_cast<uint32_t(&)[32]>(u[32 * cc]));
            tmem_wait_ld();

            const int sblk = kv_tile_of(t, i) / p.tiles_per_sblock;
            const float c = c_row * ks[sblk];           // dequantising multiplier of this step's scores
            const float pv = vs[sblk] / vs_ref;         // relative V scale folded into P

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
            float mm[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) mm[j] = __uint_as_float(u[j]);
#pragma unroll
            for (int j = 8; j < 128; ++j) mm[j & 7] = fmaxf(mm[j & 7], __uint_as_float(u[j]));
            const float mx = fmaxf(fmaxf(fmaxf(mm[0], mm[1]), fmaxf(mm[2], mm[3])),
                                   fmaxf(fmaxf(mm[4], mm[5]), fmaxf(mm[6], mm[7])));

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
            // P goes to TMEM as e4m3 times the relative V scale pv <= 1, which is folded into the
            // exponent (exp2(x + log2 pv) = pv * exp2(x)); the row sum wants the unscaled P, so this
            // step's sum of scaled values is divided by pv once.  Four keys per column, four pieces
            // of 32 keys; a piece is announced once its TMEM store has completed.
            const float neg_off = (have_off ? -off : 0.f) + lg2_approx(pv);
            float2 sa = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
            uint32_t pk[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                float e[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) e[x] = ex2_approx(fmaf(__uint_as_float(u[4 * j + x]), c, neg_off));
                if (j & 1) {
                    sb.x += e[0] + e[2];
                    sb.y += e[1] + e[3];
                } else {
                    sa.x += e[0] + e[2];
                    sa.y += e[1] + e[3];
                }
                pk[j] = pack_e4m3x4(e[0], e[1], e[2], e[3]);
                if ((j & 7) == 7) {
                    const int q = j >> 3;
                    tmem_st8(tS + 8u * q, reinterpret_cast<uint32_t(&)[8]>(pk[8 * q]));
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(bar(kF8P + 4 * t + q));
                }
            }
            const float inv_pv = 1.f / pv;
            l2a.x = fmaf(sa.x, inv_pv, l2a.x);
            l2a.y = fmaf(sa.y, inv_pv, l2a.y);
            l2b.x = fmaf(sb.x, inv_pv, l2b.x);
            l2b.y = fmaf(sb.y, inv_pv, l2b.y);
        }
        const float l = (l2a.x + l2a.y) + (l2b.x + l2b.y);

        if (tile_valid) {
            if (nt > 0 && ok) {
                if (!mbar_wait(bar(kF8ODone + t), 0, abort_flag)) {
                    if (lane == 0) report_timeout(p.status, 4, static_cast<uint32_t>(warp), 0, 500 + t);
                    ok = false;
                }
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                tc_fence_after();
                const float inv_l = l > 0.f ? vs_ref / l : 0.f;
                uint8_t* stage = base_ptr + kF8SmemQ + static_cast<uint32_t>(t) * kTileBytes;
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
                        const int chunk = cc * 4 + q4;
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

// ------------------------------------------------------------------------------------------
// Cache writer: bf16 [n_bh, S, 128] -> e4m3 with one fp32 scale per (bh, block of `block` rows),
// scale = amax * fp32(1/448) (1 for an all-zero block), value = x * (1 / scale).  transposed == 0 writes
// [n_bh, S, 128]; transposed != 0 writes [n_bh, 128, S] (the layout the forward wants for V).
// One CTA per (128-row tile, bh); the block's amax is recomputed per tile from the whole block
// (blocks are a few tiles), so there is no second pass over a scratch buffer.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_kv_kernel(const __nv_bfloat16* __restrict__ x,
                                                         uint8_t* __restrict__ x8, float* __restrict__ scales,
                                                         int S, int block, int transposed) {
    __shared__ float red[8];
    __shared__ uint32_t tile[128 * 33];      // [128 rows][128 bytes] + 4 bytes of padding per row
    const int tile_idx = blockIdx.x, bh = blockIdx.y;
    const int tiles_per_block = block / 128;
    const int sblk = tile_idx / tiles_per_block;
    const int n_sblocks = S / block;
    const __nv_bfloat16* xb = x + (static_cast<long long>(bh) * S + static_cast<long long>(sblk) * block) * 128;
    float amax = 0.f;
    for (int i = threadIdx.x; i < block * 16; i += 256) {      // 16-byte chunks of the block
        const uint4 w = reinterpret_cast<const uint4*>(xb)[i];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h2[j]);
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) amax = fmaxf(amax, red[j]);
    const float scale = amax > 0.f ? amax * kInvE4m3Max : 1.f;
    const float inv = 1.f / scale;
    if (threadIdx.x == 0 && tile_idx % tiles_per_block == 0) scales[static_cast<long long>(bh) * n_sblocks + sblk] = scale;

    const int r0 = tile_idx * 128;
    const __nv_bfloat16* xt = x + (static_cast<long long>(bh) * S + r0) * 128;
    for (int i = threadIdx.x; i < 128 * 16; i += 256) {         // (row, 8-element chunk)
        const int r = i >> 4, ch = i & 15;
        const uint4 w = reinterpret_cast<const uint4*>(xt)[i];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
        const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
        const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
        tile[r * 33 + 2 * ch] = pack_e4m3x4(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
        tile[r * 33 + 2 * ch + 1] = pack_e4m3x4(f2.x * inv, f2.y * inv, f3.x * inv, f3.y * inv);
    }
    __syncthreads();
    const uint8_t* tb = reinterpret_cast<const uint8_t*>(tile);
    if (!transposed) {
        uint32_t* out = reinterpret_cast<uint32_t*>(x8 + (static_cast<long long>(bh) * S + r0) * 128);
        for (int i = threadIdx.x; i < 128 * 32; i += 256) out[i] = tile[(i >> 5) * 33 + (i & 31)];
    } else {
        // out[d][r0 + r] = tile[r][d]: a warp writes 128 consecutive bytes of one d row
        for (int i = threadIdx.x; i < 128 * 32; i += 256) {
            const int d = i >> 5, r4 = (i & 31) * 4;
            uint32_t v = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) v |= static_cast<uint32_t>(tb[(r4 + j) * 132 + d]) << (8 * j);
            *reinterpret_cast<uint32_t*>(x8 + (static_cast<long long>(bh) * 128 + d) * S + r0 + r4) = v;
        }
    }
}

}  // namespace fba

using namespace fba;

extern "C" int fba_quantize_kv_e4m3(const void* x, uint8_t* x8, float* scales, int n_bh, int S, int scale_block,
                                    int transposed, void* stream) {
    if (!x || !x8 || !scales) return set_error(FBA_ERR_BAD_ARG, "fba_quantize_kv_e4m3: null pointer argument");
    if (n_bh <= 0 || S <= 0 || scale_block <= 0 || scale_block % 128 != 0 || S % scale_block != 0)
        return set_error(FBA_ERR_BAD_ARG,
                         "fba_quantize_kv_e4m3: scale_block must be a multiple of 128 that divides the sequence length");
    if (n_bh > 65535) return set_error(FBA_ERR_TOO_LARGE, "fba_quantize_kv_e4m3: more than 65535 (batch, head) slices");
    DeviceGuard guard;
    int rc = guard.bind(x);
    if (rc != FBA_OK) return rc;
    quantize_kv_kernel<<<dim3(S / 128, n_bh), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), x8, scales, S, scale_block, transposed);
    return check_launch("quantize_kv_kernel");
}

extern "C" int fba_fwd_fp8kv(const void* q, const uint8_t* k8, const uint8_t* v8t, const float* k_scale,
                             const float* v_scale, int scale_block, void* o, float* lse, int B, int Hq, int Hkv,
                             int Sq, int Skv, const fba_list_t* q2k, float softmax_scale, uint32_t* status,
                             void* stream_) {
    ProfRange range("fba_fwd_fp8kv");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!q || !k8 || !v8t || !k_scale || !v_scale || !o || !status)
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd_fp8kv: null pointer argument");
    if (!(softmax_scale > 0.f) || !(softmax_scale < INFINITY))
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd_fp8kv: softmax_scale must be positive and finite");
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || Hq % Hkv != 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd_fp8kv: bad size");
    if (Sq < 128 || Skv < 128)
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd_fp8kv: sequence lengths below 128 are not supported");
    if (scale_block <= 0 || scale_block % 128 != 0 || Skv % scale_block != 0)
        return set_error(FBA_ERR_BAD_ARG,
                         "fba_fwd_fp8kv: scale_block must be a multiple of 128 that divides the key length");
    if (!q2k || !q2k->idx || !q2k->cnt || q2k->stride <= 0 || q2k->rows_per_bh <= 0 || q2k->rows_div <= 0 ||
        q2k->sub <= 0 || (q2k->bh_stride != 0 && q2k->bh_stride != q2k->rows_per_bh))
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd_fp8kv: malformed q2k list");
    const int n_mtiles = (Sq + 127) / 128, n_ntiles = Skv / 128;
    if (static_cast<long long>(q2k->rows_per_bh) * q2k->rows_div < n_mtiles ||
        static_cast<long long>(q2k->stride) * q2k->sub < n_ntiles || n_ntiles % q2k->sub != 0 ||
        n_mtiles % q2k->rows_div != 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_fwd_fp8kv: q2k list does not cover the sequences");
    if (static_cast<long long>(B) * Hq > 65535)
        return set_error(FBA_ERR_TOO_LARGE, "fba_fwd_fp8kv: B * Hq exceeds 65535");
    DeviceGuard guard;
    int rc = guard.bind(q);
    if (rc != FBA_OK) return rc;
    CUtensorMap tm_q, tm_k8, tm_v8t, tm_o;
    if ((rc = make_tmap_bf16(&tm_q, q, Sq, static_cast<long long>(B) * Hq, 128)) != FBA_OK) return rc;
    if ((rc = make_tmap_u8(&tm_k8, k8, 128, Skv, static_cast<long long>(B) * Hkv)) != FBA_OK) return rc;
    if ((rc = make_tmap_u8(&tm_v8t, v8t, Skv, 128, static_cast<long long>(B) * Hkv)) != FBA_OK) return rc;
    if ((rc = make_tmap_bf16(&tm_o, o, Sq, static_cast<long long>(B) * Hq, 128)) != FBA_OK) return rc;
    cudaError_t e = cudaFuncSetAttribute(fba_fwd_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kF8SmemBytes));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_fwd_fp8kv: cannot raise the dynamic shared memory limit");
    }
    F8Params p;
    p.list = to_dev(*q2k);
    p.k_scale = k_scale;
    p.v_scale = v_scale;
    p.lse = lse;
    p.status = status;
    p.n_mtiles = n_mtiles;
    p.Sq = Sq;
    p.Hq = Hq;
    p.Hkv = Hkv;
    p.n_sblocks = Skv / scale_block;
    p.tiles_per_sblock = scale_block / 128;
    p.scale_log2 = softmax_scale * kLog2e;
    dim3 grid((n_mtiles + 1) / 2, B * Hq);
    timing_mark(1, true, stream);
    fba_fwd_fp8_kernel<<<grid, kF8Threads, kF8SmemBytes, stream>>>(tm_q, tm_k8, tm_v8t, tm_o, p);
    rc = check_launch("fba_fwd_fp8_kernel");
    timing_mark(1, false, stream);
    return rc;
}
