// Block-mask -> index-list compaction.
//
// The reference keeps the bool block mask and has every attention CTA scan a whole mask row (or,
// in backward, a row of the transposed copy made by flex_block_attn_interface.py:85-86) to find
// its active tiles (flex_block_attn_h100.cu:107-121, 131-149, 642-699).  Here one pass turns the
// mask into ascending index lists, query-major and key-major, which the attention kernels walk.
//
// One warp owns one list row.  It reads 32 predicate values per step, ballots, and each active
// lane writes its column index at (running count + popc(lower lanes)).  Output order is therefore
// ascending and independent of scheduling: bit-identical to a nonzero()-based restatement.
// This is byte/integer work bounded by HBM/L2 bandwidth; it is tiny next to the attention
// kernels (a [2,24,540,180] mask is 4.7 MB).
#include "fba_internal.cuh"

namespace fba {

// Predicate over the raw block mask.  TRANSPOSED reads mask[bh][col][row].
template <bool TRANSPOSED>
struct BlockPred {
    const uint8_t* mask;
    long long bh_stride;  // bytes between (batch, head) slices, 0 for a shared 2-D mask
    int nQ, nK;
    __device__ __forceinline__ uint32_t operator()(int bh, int row, int col) const {
        const uint8_t* m = mask + static_cast<long long>(bh) * bh_stride;
        const int qi = TRANSPOSED ? col : row;
        const int kj = TRANSPOSED ? row : col;
        return m[static_cast<long long>(qi) * nK + kj] ? 1u : 0u;
    }
};

// Predicate over 128x128 token tiles: 16-bit word, bit (8*h + g) set iff 16-row query group g of
// query tile mt attends to 64-row key half h of key tile nt.  Groups / halves past the end of a
// sequence read as "not attended", so ragged last tiles need no special case downstream.
template <bool TRANSPOSED>
struct TilePred {
    const uint8_t* mask;
    long long bh_stride;
    int nQ, nK, q_block, kv_block, Sq, Skv;
    __device__ __forceinline__ uint32_t operator()(int bh, int row, int col) const {
        const uint8_t* m = mask + static_cast<long long>(bh) * bh_stride;
        const int mt = TRANSPOSED ? col : row;
        const int nt = TRANSPOSED ? row : col;
        uint32_t w = 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kcol = nt * 128 + h * 64;
            if (kcol >= Skv) continue;
            const int kj = kcol / kv_block;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const int qrow = mt * 128 + g * 16;
                if (qrow >= Sq) continue;
                if (m[static_cast<long long>(qrow / q_block) * nK + kj]) w |= 1u << (8 * h + g);
            }
        }
        return w;
    }
};

template <class Pred>
__global__ void __launch_bounds__(256) compact_rows_kernel(Pred pred, int rows, int cols,
                                                           long long total_rows,
                                                           int32_t* __restrict__ idx,
                                                           int32_t* __restrict__ cnt,
                                                           uint16_t* __restrict__ msk) {
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (warp >= total_rows) return;
    const int lane = threadIdx.x & 31;
    const int bh = static_cast<int>(warp / rows);
    const int row = static_cast<int>(warp % rows);
    int32_t* out_idx = idx + warp * cols;
    uint16_t* out_msk = msk ? msk + warp * cols : nullptr;
    int n = 0;
    for (int c0 = 0; c0 < cols; c0 += 32) {
        const int c = c0 + lane;
        const uint32_t w = (c < cols) ? pred(bh, row, c) : 0u;
        const uint32_t ballot = __ballot_sync(0xffffffffu, w != 0u);
        if (w != 0u) {
            const int pos = n + __popc(ballot & ((1u << lane) - 1u));
            out_idx[pos] = c;
            if (out_msk) out_msk[pos] = static_cast<uint16_t>(w);
        }
        n += __popc(ballot);
    }
    for (int c = n + lane; c < cols; c += 32) {
        out_idx[c] = -1;
        if (out_msk) out_msk[c] = 0;
    }
    if (lane == 0) cnt[warp] = n;
}

template <class Pred>
static int launch_compact(const Pred& pred, int n_bh, int rows, int cols, int32_t* idx, int32_t* cnt,
                          uint16_t* msk, cudaStream_t stream) {
    const long long total = static_cast<long long>(n_bh) * rows;
    if (total == 0 || cols == 0) return FBA_OK;
    const long long blocks = (total * 32 + 255) / 256;
    if (blocks > 0x7fffffffLL) return set_error(FBA_ERR_TOO_LARGE, "mask too large");
    compact_rows_kernel<Pred><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(pred, rows, cols,
                                                                                total, idx, cnt, msk);
    return check_launch("compact_rows_kernel");
}

}  // namespace fba

using namespace fba;

extern "C" int fba_build_index(const uint8_t* mask, int mask_dim, int B, int H, int nQ, int nK,
                               int32_t* q2k_idx, int32_t* q2k_cnt, int32_t* k2q_idx,
                               int32_t* k2q_cnt, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!mask) return set_error(FBA_ERR_BAD_ARG, "fba_build_index: mask is null");
    if (mask_dim != 2 && mask_dim != 4)
        return set_error(FBA_ERR_BAD_ARG, "fba_build_index: mask_dim must be 2 or 4");
    if (nQ <= 0 || nK <= 0 || (mask_dim == 4 && (B <= 0 || H <= 0)))
        return set_error(FBA_ERR_BAD_ARG, "fba_build_index: non-positive size");
    if ((q2k_idx == nullptr) != (q2k_cnt == nullptr) || (k2q_idx == nullptr) != (k2q_cnt == nullptr))
        return set_error(FBA_ERR_BAD_ARG, "fba_build_index: idx and cnt must be given together");
    const int n_bh = mask_dim == 4 ? B * H : 1;
    const long long bh_stride = mask_dim == 4 ? static_cast<long long>(nQ) * nK : 0;
    DeviceGuard guard;
    int rc = guard.bind(mask);
    if (rc != FBA_OK) return rc;
    if (q2k_idx) {
        BlockPred<false> p{mask, bh_stride, nQ, nK};
        rc = launch_compact(p, n_bh, nQ, nK, q2k_idx, q2k_cnt, nullptr, stream);
        if (rc != FBA_OK) return rc;
    }
    if (k2q_idx) {
        BlockPred<true> p{mask, bh_stride, nQ, nK};
        rc = launch_compact(p, n_bh, nK, nQ, k2q_idx, k2q_cnt, nullptr, stream);
    }
    return rc;
}

extern "C" int fba_build_tile_lists(const uint8_t* mask, int mask_dim, int B, int H, int nQ, int nK,
                                    int q_block, int kv_block, int Sq, int Skv, int32_t* fwd_idx,
                                    int32_t* fwd_cnt, uint16_t* fwd_msk, int32_t* bwd_idx,
                                    int32_t* bwd_cnt, uint16_t* bwd_msk, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!mask) return set_error(FBA_ERR_BAD_ARG, "fba_build_tile_lists: mask is null");
    if (mask_dim != 2 && mask_dim != 4)
        return set_error(FBA_ERR_BAD_ARG, "fba_build_tile_lists: mask_dim must be 2 or 4");
    if (nQ <= 0 || nK <= 0 || (mask_dim == 4 && (B <= 0 || H <= 0)))
        return set_error(FBA_ERR_BAD_ARG, "fba_build_tile_lists: non-positive size");
    if (q_block <= 0 || q_block % 16 != 0 || kv_block <= 0 || kv_block % 64 != 0)
        return set_error(FBA_ERR_BAD_ARG,
                         "fba_build_tile_lists: q_block must be a multiple of 16 and kv_block of 64");
    if (static_cast<long long>(q_block) * nQ != Sq || static_cast<long long>(kv_block) * nK != Skv)
        return set_error(FBA_ERR_BAD_ARG, "fba_build_tile_lists: block size * block count != length");
    const bool want_fwd = fwd_idx || fwd_cnt || fwd_msk;
    const bool want_bwd = bwd_idx || bwd_cnt || bwd_msk;
    if ((want_fwd && !(fwd_idx && fwd_cnt && fwd_msk)) || (want_bwd && !(bwd_idx && bwd_cnt && bwd_msk)))
        return set_error(FBA_ERR_BAD_ARG, "fba_build_tile_lists: idx, cnt and msk go together");
    const int n_bh = mask_dim == 4 ? B * H : 1;
    const long long bh_stride = mask_dim == 4 ? static_cast<long long>(nQ) * nK : 0;
    const int nMt = (Sq + 127) / 128, nNt = (Skv + 127) / 128;
    DeviceGuard guard;
    int rc = guard.bind(mask);
    if (rc != FBA_OK) return rc;
    if (want_fwd) {
        TilePred<false> p{mask, bh_stride, nQ, nK, q_block, kv_block, Sq, Skv};
        rc = launch_compact(p, n_bh, nMt, nNt, fwd_idx, fwd_cnt, fwd_msk, stream);
        if (rc != FBA_OK) return rc;
    }
    if (want_bwd) {
        TilePred<true> p{mask, bh_stride, nQ, nK, q_block, kv_block, Sq, Skv};
        rc = launch_compact(p, n_bh, nNt, nMt, bwd_idx, bwd_cnt, bwd_msk, stream);
    }
    return rc;
}

// ------------------------------------------------------------------------------------------
// Work-item order.
//
// The attention grids have one CTA per work item (forward: a pair of 128-row query tiles; backward:
// one 128-row key tile) and list lengths differ from item to item, so the last wave of a launch
// idles SMs while the longest items finish.  CTAs are dispatched in blockIdx order: handing the
// items of each (batch, head) out longest first leaves the shortest for the end.  The order is the
// stable descending argsort of the item's work (the sum of the list lengths it walks): integer,
// deterministic, bit-identical to argsort(stable=True, descending=True).
//
// One CTA per order row; the keys sit in shared memory and every thread ranks its items by
// counting the items that sort before them (n^2 / 256 comparisons per thread, n = a few hundred).
namespace fba {

constexpr int kOrderMaxItems = 12288;   // keys of one order row must fit 48 KiB of shared memory

__global__ void __launch_bounds__(256) work_order_kernel(const int32_t* __restrict__ cnt, int bh_stride,
                                                         int rows_div, int n_tiles, int tiles_per_item,
                                                         int heads_per_item, int n_items,
                                                         int32_t* __restrict__ order) {
    extern __shared__ int32_t key[];
    const int g = blockIdx.x;
    for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
        int k = 0;
        for (int r = 0; r < heads_per_item; ++r) {
            const long long base = static_cast<long long>(g * heads_per_item + r) * bh_stride;
            for (int u = 0; u < tiles_per_item; ++u) {
                const int tile = i * tiles_per_item + u;
                if (tile < n_tiles) k += cnt[base + tile / rows_div];
            }
        }
        key[i] = k;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
        const int ki = key[i];
        int rank = 0;
        for (int j = 0; j < n_items; ++j) {
            const int kj = key[j];
            rank += (kj > ki || (kj == ki && j < i)) ? 1 : 0;
        }
        order[static_cast<long long>(g) * n_items + rank] = i;
    }
}

static int launch_order(const fba_list_t* l, const char* who, int n_order_rows, int n_tiles, int tiles_per_item,
                        int heads_per_item, int32_t* order, cudaStream_t stream) {
    if (!l || !l->cnt || !order) return set_error(FBA_ERR_BAD_ARG, who);
    if (l->rows_per_bh <= 0 || l->rows_div <= 0 || (l->bh_stride != 0 && l->bh_stride != l->rows_per_bh) ||
        static_cast<long long>(l->rows_per_bh) * l->rows_div < n_tiles)
        return set_error(FBA_ERR_BAD_ARG, who);
    const int n_items = (n_tiles + tiles_per_item - 1) / tiles_per_item;
    if (n_items > kOrderMaxItems)
        return set_error(FBA_ERR_TOO_LARGE, "work order: more than 12288 work items per (batch, head); pass order = NULL");
    DeviceGuard guard;
    int rc = guard.bind(order);
    if (rc != FBA_OK) return rc;
    work_order_kernel<<<static_cast<unsigned>(n_order_rows), 256, n_items * sizeof(int32_t), stream>>>(
        l->cnt, l->bh_stride, l->rows_div, n_tiles, tiles_per_item, heads_per_item, n_items, order);
    return check_launch("work_order_kernel");
}

}  // namespace fba

extern "C" int fba_fwd_order(const fba_list_t* q2k, int B, int Hq, int Sq, int32_t* order, void* stream) {
    if (B <= 0 || Hq <= 0 || Sq <= 0) return set_error(FBA_ERR_BAD_ARG, "fba_fwd_order: non-positive size");
    const int rows = (q2k && q2k->bh_stride) ? B * Hq : 1;
    return launch_order(q2k, "fba_fwd_order: malformed q2k list or null order", rows, (Sq + 127) / 128, 2, 1, order,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int fba_bwd_order(const fba_list_t* k2q, int B, int Hq, int Hkv, int Skv, int32_t* order, void* stream) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Skv <= 0 || Hq % Hkv != 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_bwd_order: bad size");
    const bool per_head = k2q && k2q->bh_stride;
    return launch_order(k2q, "fba_bwd_order: malformed k2q list or null order", per_head ? B * Hkv : 1,
                        (Skv + 127) / 128, 1, per_head ? Hq / Hkv : 1, order, static_cast<cudaStream_t>(stream));
}
