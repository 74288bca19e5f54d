// Sequence <-> head exchange fused with the token reorder, over peer memory (NVLink).
//
// The reference is single-GPU; its callers hold activations as [B, S, H, 128] in raster (t, h, w)
// token order (reference benchmark/dynamic/random/scripts/random_fwd.py:58-60).  With the sequence
// sharded over P GPUs, attention needs [B, H/P, S, 128] on every GPU, in tile-major token order for
// sliding-tile masks.  Instead of "transpose + permute locally, then all-to-all, then unpack", one
// kernel per GPU reads its local rows once and stores every 256-byte row straight into its final
// place in the owning GPU's buffer (plain peer stores; the receiver runs nothing).  The way back
// (O, and the gradients) is the same kernel with the roles of the two layouts swapped.
//
// The kernel contains no waits.  Ordering against the consumers on the other GPUs is the
// caller's: a cross-GPU barrier before the call (everyone is done reading the destination
// buffers) and one after it (all rows have landed).
#include <string.h>

#include "fba_internal.cuh"

namespace fba {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
    uint4* p[kMaxPeers];
};

struct TokenGrid {
    int T, H, W, tt, th, tw;   // latent grid and tile extents
    // raster position of tile-major position s
    __device__ __forceinline__ int raster_of(int s) const {
        const int per_tile = tt * th * tw;
        const int tile = s / per_tile, in = s - tile * per_tile;
        const int gw = W / tw, gh = H / th;
        const int tw_i = tile % gw, th_i = (tile / gw) % gh, tt_i = tile / (gw * gh);
        const int w_in = in % tw, h_in = (in / tw) % th, t_in = in / (tw * th);
        return ((tt_i * tt + t_in) * H + (th_i * th + h_in)) * W + (tw_i * tw + w_in);
    }
    // tile-major position of raster position r
    __device__ __forceinline__ int tile_major_of(int r) const {
        const int w = r % W, h = (r / W) % H, t = r / (W * H);
        const int gw = W / tw, gh = H / th;
        const int tile = ((t / tt) * gh + (h / th)) * gw + (w / tw);
        const int in = ((t % tt) * th + (h % th)) * tw + (w % tw);
        return tile * (tt * th * tw) + in;
    }
};

// to_head: src = this rank's [B, S/P, H, 128] raster chunk (global raster rows rank*S/P ...);
//          row (b, s_l, h) goes to rank h / (H/P), buffer [B, H/P, S, 128], row tile_major_of(s).
// else:    src = this rank's [B, H/P, S, 128] tile-major heads;
//          row (b, h_l, s) goes to rank raster_of(s) / (S/P), buffer [B, S/P, H, 128].
__global__ void __launch_bounds__(256) peer_exchange_kernel(const uint4* __restrict__ src, PeerPtrs peers, int n_ranks,
                                                           int rank, int B, int H, int S, TokenGrid grid, bool to_head) {
    // All row counts fit 32 bits (checked by the host); only byte offsets need 64.
    const uint32_t Hl = H / n_ranks, Sl = S / n_ranks, uH = H, uS = S;
    const uint32_t total = static_cast<uint32_t>(B) * (to_head ? Sl * uH : Hl * uS);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t half = lane >> 4, l16 = lane & 15;   // a warp moves two 256-byte rows at a time, 16 bytes per lane
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    constexpr uint32_t kUnroll = 4;                 // rows in flight per half-warp; a warp step is 8 rows
    // The rows are enumerated so that the eight rows of a warp step form a 2 KiB contiguous run at
    // the DESTINATION (eight consecutive tokens of one head on the way to the heads, eight
    // consecutive heads of one token on the way back) while the eight warps of a CTA together read
    // 16 KiB of neighbouring source rows.  That needs whole groups of eight along the walked
    // dimension; otherwise the rows are taken in source order.
    const bool runs = to_head ? (Sl % 8 == 0) : (Hl % 8 == 0);
    // With tiles that are a multiple of eight tokens wide, a group of eight consecutive raster
    // tokens starting at a multiple of eight is also consecutive in tile-major order.
    const bool run_contig = grid.tw % 8 == 0 && (rank * Sl) % 8 == 0;
    for (uint32_t base = warp * (2 * kUnroll); base < total; base += n_warps * (2 * kUnroll)) {
        uint4 v[kUnroll];
        uint4* dst[kUnroll];
        if (runs) {
            const uint32_t g = base >> 3;           // base is a multiple of 8: the whole step shares g
            if (to_head) {
                const uint32_t h = g % uH, t = g / uH;
                const uint32_t s8 = t % (Sl >> 3), b = t / (Sl >> 3);
                const uint32_t dest = h / Hl;
                const uint32_t r0 = rank * Sl + s8 * 8;
                const uint32_t p0 = run_contig ? grid.tile_major_of(r0) : 0u;
                const unsigned long long srow0 = (static_cast<unsigned long long>(b) * Sl + s8 * 8) * uH + h;
                const unsigned long long drow0 = (static_cast<unsigned long long>(b) * Hl + (h - dest * Hl)) * uS;
#pragma unroll
                for (uint32_t u = 0; u < kUnroll; ++u) {
                    const uint32_t i = 2 * u + half;
                    const uint32_t pos = run_contig ? p0 + i : static_cast<uint32_t>(grid.tile_major_of(r0 + i));
                    v[u] = src[(srow0 + static_cast<unsigned long long>(i) * uH) * 16 + l16];
                    dst[u] = peers.p[dest] + (drow0 + pos) * 16 + l16;
                }
            } else {
                const uint32_t s_ = g % uS, t = g / uS;
                const uint32_t hl8 = t % (Hl >> 3), b = t / (Hl >> 3);
                const uint32_t r = grid.raster_of(s_);
                const uint32_t dest = r / Sl;
                const unsigned long long srow0 = (static_cast<unsigned long long>(b) * Hl + hl8 * 8) * uS + s_;
                const unsigned long long drow0 =
                    (static_cast<unsigned long long>(b) * Sl + (r - dest * Sl)) * uH + rank * Hl + hl8 * 8;
#pragma unroll
                for (uint32_t u = 0; u < kUnroll; ++u) {
                    const uint32_t i = 2 * u + half;
                    v[u] = src[(srow0 + static_cast<unsigned long long>(i) * uS) * 16 + l16];
                    dst[u] = peers.p[dest] + (drow0 + i) * 16 + l16;
                }
            }
        } else {
#pragma unroll
            for (uint32_t u = 0; u < kUnroll; ++u) {
                const uint32_t e = base + 2 * u + half;   // source row index
                dst[u] = nullptr;
                if (e >= total) continue;
                uint32_t dest;
                unsigned long long drow;
                if (to_head) {
                    const uint32_t h = e % uH, t = e / uH;
                    const uint32_t sl = t % Sl, b = t / Sl;
                    dest = h / Hl;
                    drow = (static_cast<unsigned long long>(b) * Hl + (h - dest * Hl)) * uS +
                           grid.tile_major_of(rank * Sl + sl);
                } else {
                    const uint32_t s_ = e % uS, t = e / uS;
                    const uint32_t hl = t % Hl, b = t / Hl;
                    const uint32_t r = grid.raster_of(s_);
                    dest = r / Sl;
                    drow = (static_cast<unsigned long long>(b) * Sl + (r - dest * Sl)) * uH + rank * Hl + hl;
                }
                v[u] = src[static_cast<unsigned long long>(e) * 16 + l16];
                dst[u] = peers.p[dest] + drow * 16 + l16;
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < kUnroll; ++u)
            if (dst[u] != nullptr) *dst[u] = v[u];
    }
}

}  // namespace fba

using namespace fba;

extern "C" int fba_peer_alloc(uint64_t bytes, void** ptr) {
    if (!ptr || bytes == 0) return set_error(FBA_ERR_BAD_ARG, "fba_peer_alloc: bad argument");
    *ptr = nullptr;
    if (cudaMalloc(ptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        *ptr = nullptr;
        return set_error(FBA_ERR_LAUNCH, "fba_peer_alloc: cudaMalloc failed");
    }
    return FBA_OK;
}

extern "C" int fba_peer_free(void* ptr) {
    if (!ptr) return FBA_OK;
    if (cudaFree(ptr) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_peer_free: cudaFree failed");
    }
    return FBA_OK;
}

extern "C" int fba_peer_export(const void* ptr, unsigned char* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!ptr || !handle64) return set_error(FBA_ERR_BAD_ARG, "fba_peer_export: null argument");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_peer_export: cudaIpcGetMemHandle failed");
    }
    memcpy(handle64, &h, 64);
    return FBA_OK;
}

extern "C" int fba_peer_open(const unsigned char* handle64, void** ptr) {
    if (!handle64 || !ptr) return set_error(FBA_ERR_BAD_ARG, "fba_peer_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    *ptr = nullptr;
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        *ptr = nullptr;
        return set_error(FBA_ERR_LAUNCH, "fba_peer_open: cudaIpcOpenMemHandle failed (no peer access?)");
    }
    return FBA_OK;
}

extern "C" int fba_peer_close(void* ptr) {
    if (!ptr) return FBA_OK;
    if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_peer_close: cudaIpcCloseMemHandle failed");
    }
    return FBA_OK;
}

extern "C" int fba_peer_exchange(const void* src, void* const* peers, int n_ranks, int rank, int B, int H, int T,
                                 int Hh, int W, int tt, int th, int tw, int to_head, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!src || !peers) return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: null argument");
    if (n_ranks <= 0 || n_ranks > kMaxPeers || rank < 0 || rank >= n_ranks)
        return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: bad rank / world size (at most 16 ranks)");
    if (B <= 0 || H <= 0 || T <= 0 || Hh <= 0 || W <= 0 || tt <= 0 || th <= 0 || tw <= 0 || T % tt || Hh % th || W % tw)
        return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: the grid must be a positive multiple of the tile");
    const long long S = static_cast<long long>(T) * Hh * W;
    if (S > 0x7fffffffLL) return set_error(FBA_ERR_TOO_LARGE, "fba_peer_exchange: sequence too long");
    if (H % n_ranks || S % n_ranks)
        return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: heads and sequence must divide over the ranks");
    if (reinterpret_cast<uintptr_t>(src) % 16 != 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: source must be 16-byte aligned");
    PeerPtrs pp;
    for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = nullptr;
    for (int i = 0; i < n_ranks; ++i) {
        if (!peers[i]) return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: null peer buffer");
        if (peers[i] == src) return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: source aliases a destination");
        if (reinterpret_cast<uintptr_t>(peers[i]) % 16 != 0)
            return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: destinations must be 16-byte aligned");
        pp.p[i] = static_cast<uint4*>(peers[i]);
    }
    DeviceGuard guard;
    {
        // The local destination must not overlap the source: rows would be read after a store of
        // this same launch had overwritten them.  (The other ranks' buffers live in other devices'
        // memory and cannot overlap a local source.)
        const unsigned long long bytes = static_cast<unsigned long long>(B) * H * S / n_ranks * 256ull;
        const uintptr_t s0 = reinterpret_cast<uintptr_t>(src), d0 = reinterpret_cast<uintptr_t>(peers[rank]);
        if (s0 < d0 + bytes && d0 < s0 + bytes)
            return set_error(FBA_ERR_BAD_ARG, "fba_peer_exchange: source overlaps the local destination buffer");
    }
    int rc = guard.bind(src);
    if (rc != FBA_OK) return rc;
    // Persistent grid: a few CTAs per SM, each warp strides over groups of rows.
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_peer_exchange: cannot query the device");
    }
    const long long rows = static_cast<long long>(B) * H * S / n_ranks;
    if (rows > 0x7fffffffLL) return set_error(FBA_ERR_TOO_LARGE, "fba_peer_exchange: more than 2^31 rows per rank");
    long long blocks = (rows + 63) / 64;                       // 8 warps x 8 rows per step
    if (blocks > 8LL * sms) blocks = 8LL * sms;
    TokenGrid g{T, Hh, W, tt, th, tw};
    peer_exchange_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint4*>(src), pp, n_ranks, rank, B, H, static_cast<int>(S), g, to_head != 0);
    return check_launch("peer_exchange_kernel");
}

// Layout change on one GPU: the reference's callers hold activations as [B, S, H, 128] in raster
// (t, h, w) token order and transpose to [B, H, S, 128] before the call (reference
// benchmark/dynamic/random/scripts/random_fwd.py:58-60); sliding-tile masks additionally want the
// tokens in tile-major order.  This is the exchange above with a single rank: one HBM-bound pass,
// one 256-byte row read and written per token and head, in either direction.
extern "C" int fba_tile_major(const void* src, void* dst, int B, int Hn, int T, int H, int W, int tt, int th, int tw,
                              int to_tile_major, void* stream) {
    if (!src || !dst || src == dst) return set_error(FBA_ERR_BAD_ARG, "fba_tile_major: bad pointer argument");
    if (B <= 0 || Hn <= 0 || T <= 0 || H <= 0 || W <= 0 || tt <= 0 || th <= 0 || tw <= 0 || T % tt || H % th || W % tw)
        return set_error(FBA_ERR_BAD_ARG, "fba_tile_major: the grid must be a positive multiple of the tile");
    void* peers[1] = {dst};
    return fba_peer_exchange(src, peers, 1, 0, B, Hn, T, H, W, tt, th, tw, to_tile_major, stream);
}
