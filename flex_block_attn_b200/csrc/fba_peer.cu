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
    const int Hl = H / n_ranks, Sl = S / n_ranks;
    const long long total = to_head ? static_cast<long long>(B) * Sl * H : static_cast<long long>(B) * Hl * S;
    const int lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;   // a warp moves two 256-byte rows per step, 16 bytes per lane
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    constexpr int kUnroll = 4;                      // rows in flight per half-warp
    for (long long base = warp * (2 * kUnroll); base < total; base += n_warps * (2 * kUnroll)) {
        uint4 v[kUnroll];
        uint4* dst[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const long long row = base + 2 * u + half;
            dst[u] = nullptr;
            if (row >= total) continue;
            v[u] = src[row * 16 + l16];
            int dest;
            long long drow;
            if (to_head) {
                const int h = static_cast<int>(row % H);
                const int sl = static_cast<int>((row / H) % Sl);
                const long long b = row / (static_cast<long long>(H) * Sl);
                dest = h / Hl;
                drow = (b * Hl + (h - dest * Hl)) * S + grid.tile_major_of(rank * Sl + sl);
            } else {
                const int s = static_cast<int>(row % S);
                const int hl = static_cast<int>((row / S) % Hl);
                const long long b = row / (static_cast<long long>(S) * Hl);
                const int r = grid.raster_of(s);
                dest = r / Sl;
                drow = (b * Sl + (r - dest * Sl)) * H + rank * Hl + hl;
            }
            dst[u] = peers.p[dest] + drow * 16 + l16;
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
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
    int rc = bind_device_of(src);
    if (rc != FBA_OK) return rc;
    // Persistent grid: a few CTAs per SM, each warp strides over groups of rows.
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return set_error(FBA_ERR_LAUNCH, "fba_peer_exchange: cannot query the device");
    }
    const long long rows = static_cast<long long>(B) * H * S / n_ranks;
    long long blocks = (rows + 63) / 64;                       // 8 warps x 8 rows per step
    if (blocks > 8LL * sms) blocks = 8LL * sms;
    TokenGrid g{T, Hh, W, tt, th, tw};
    peer_exchange_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint4*>(src), pp, n_ranks, rank, B, H, static_cast<int>(S), g, to_head != 0);
    return check_launch("peer_exchange_kernel");
}
