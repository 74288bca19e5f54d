// Entry points with the call shape of the reference extension (reference attn.cpp:12-21:
// attention_forward(q, k, v, q_block_size, kv_block_size, block_mask, small_block_mask,
// use_small_block_mode) -> {o, lse} and attention_backward(q, k, v, o, lse, do, ...same...) ->
// {dq, dk, dv}), so that a binder can replace `attn_forward` / `attn_backward` one for one.
//
// The reference allocates its outputs and temporaries through torch inside the extension
// (flex_block_attn_h100.cu:862-876, 1077-1093).  A C ABI cannot, so the caller passes the outputs
// and ONE workspace whose size fba_attn_workspace_bytes() reports; the index lists, their work
// orders and (backward) the two scratch arrays are carved out of it.  Everything is stream-ordered
// and nothing is allocated.
#include "fba_internal.cuh"

namespace fba {

struct AttnWs {
    uint64_t idx, cnt, msk, order, mask, lse_delta, dq_accum, total;
    int n_bh, nQ, nK, nMt, nNt, list_rows, list_cols, order_rows, order_items;
    bool aligned;
};

static uint64_t carve(uint64_t& off, uint64_t bytes) {
    const uint64_t at = off;
    off += (bytes + 255) & ~static_cast<uint64_t>(255);
    return at;
}

static int plan(AttnWs& w, int B, int Hq, int Hkv, int Sq, int Skv, int q_block, int kv_block, int mask_dim,
                bool backward, const char* who) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || Hq % Hkv != 0) return set_error(FBA_ERR_BAD_ARG, who);
    if (mask_dim != 2 && mask_dim != 4) return set_error(FBA_ERR_BAD_ARG, "block_mask dim must be 2/4");
    if (q_block <= 0 || q_block % 16 != 0 || kv_block <= 0 || kv_block % 64 != 0 ||
        (kv_block % q_block != 0 && q_block % kv_block != 0))
        return set_error(FBA_ERR_BAD_ARG,
                         "q_block_size must be a multiple of 16, kv_block_size of 64, and one must divide the other");
    if (Sq % q_block != 0 || Skv % kv_block != 0)
        return set_error(FBA_ERR_BAD_ARG, "sequence lengths must be multiples of their block sizes");
    w.aligned = q_block % 128 == 0 && kv_block % 128 == 0;
    w.n_bh = mask_dim == 4 ? B * Hq : 1;
    w.nQ = Sq / q_block;
    w.nK = Skv / kv_block;
    w.nMt = (Sq + 127) / 128;
    w.nNt = (Skv + 127) / 128;
    if (!backward) {
        w.list_rows = w.aligned ? w.nQ : w.nMt;
        w.list_cols = w.aligned ? w.nK : w.nNt;
        w.order_rows = mask_dim == 4 ? B * Hq : 1;
        w.order_items = (w.nMt + 1) / 2;
    } else {
        w.list_rows = w.aligned ? w.nK : w.nNt;
        w.list_cols = w.aligned ? w.nQ : w.nMt;
        w.order_rows = mask_dim == 4 ? B * Hkv : 1;
        w.order_items = w.nNt;
    }
    const uint64_t rows = static_cast<uint64_t>(w.n_bh) * w.list_rows;
    uint64_t off = 0;
    w.idx = carve(off, rows * w.list_cols * sizeof(int32_t));
    w.cnt = carve(off, rows * sizeof(int32_t));
    w.msk = w.aligned ? 0 : carve(off, rows * w.list_cols * sizeof(uint16_t));
    w.order = carve(off, static_cast<uint64_t>(w.order_rows) * w.order_items * sizeof(int32_t));
    w.mask = w.lse_delta = w.dq_accum = 0;
    if (backward) {
        if (!w.aligned) w.mask = carve(off, static_cast<uint64_t>(w.n_bh) * w.nQ * w.nK);
        uint64_t n1 = 0, n2 = 0;
        int rc = fba_bwd_scratch_bytes(B, Hq, Sq, &n1, &n2);
        if (rc != FBA_OK) return rc;
        w.lse_delta = carve(off, n1);
        w.dq_accum = carve(off, n2);
    }
    w.total = off;
    return FBA_OK;
}

// out[bh][q][k] = in[bh][k][q]
__global__ void __launch_bounds__(256) untranspose_mask_kernel(const uint8_t* __restrict__ in,
                                                               uint8_t* __restrict__ out, int nQ, int nK,
                                                               long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long per = static_cast<long long>(nQ) * nK;
    const long long bh = i / per;
    const int r = static_cast<int>(i - bh * per);
    const int qi = r / nK, kj = r - qi * nK;
    out[i] = in[bh * per + static_cast<long long>(kj) * nQ + qi];
}

}  // namespace fba

using namespace fba;

extern "C" int fba_attn_workspace_bytes(int B, int Hq, int Hkv, int Sq, int Skv, int q_block_size,
                                        int kv_block_size, int mask_dim, int backward, uint64_t* bytes) {
    if (!bytes) return set_error(FBA_ERR_BAD_ARG, "fba_attn_workspace_bytes: null argument");
    AttnWs w;
    int rc = plan(w, B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, mask_dim, backward != 0,
                  "fba_attn_workspace_bytes: bad size");
    if (rc != FBA_OK) return rc;
    *bytes = w.total;
    return FBA_OK;
}

extern "C" int fba_attn_forward(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Hq,
                                int Hkv, int Sq, int Skv, int q_block_size, int kv_block_size,
                                const uint8_t* block_mask, const uint8_t* small_block_mask, int mask_dim,
                                int use_small_block_mode, void* workspace, uint64_t workspace_bytes,
                                uint32_t* status, void* stream) {
    ProfRange range("fba_attn_forward");
    const uint8_t* mask = (use_small_block_mode && small_block_mask) ? small_block_mask : block_mask;
    if (!q || !k || !v || !o || !lse || !mask || !workspace || !status)
        return set_error(FBA_ERR_BAD_ARG, "fba_attn_forward: null pointer argument");
    AttnWs w;
    int rc = plan(w, B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, mask_dim, false, "fba_attn_forward: bad size");
    if (rc != FBA_OK) return rc;
    if (workspace_bytes < w.total)
        return set_error(FBA_ERR_BAD_ARG, "fba_attn_forward: workspace smaller than fba_attn_workspace_bytes() reports");
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_attn_forward: workspace must be 256-byte aligned");
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int32_t* idx = reinterpret_cast<int32_t*>(ws + w.idx);
    int32_t* cnt = reinterpret_cast<int32_t*>(ws + w.cnt);
    uint16_t* msk = w.aligned ? nullptr : reinterpret_cast<uint16_t*>(ws + w.msk);
    int32_t* order = reinterpret_cast<int32_t*>(ws + w.order);
    if (w.aligned)
        rc = fba_build_index(mask, mask_dim, B, Hq, w.nQ, w.nK, idx, cnt, nullptr, nullptr, stream);
    else
        rc = fba_build_tile_lists(mask, mask_dim, B, Hq, w.nQ, w.nK, q_block_size, kv_block_size, Sq, Skv, idx, cnt,
                                  msk, nullptr, nullptr, nullptr, stream);
    if (rc != FBA_OK) return rc;
    fba_list_t l;
    l.idx = idx;
    l.cnt = cnt;
    l.msk = msk;
    l.stride = w.list_cols;
    l.rows_per_bh = w.list_rows;
    l.bh_stride = mask_dim == 4 ? w.list_rows : 0;
    l.rows_div = w.aligned ? q_block_size / 128 : 1;
    l.sub = w.aligned ? kv_block_size / 128 : 1;
    l.order = nullptr;
    if ((rc = fba_fwd_order(&l, B, Hq, Sq, order, stream)) != FBA_OK) return rc;
    l.order = order;
    return fba_fwd(q, k, v, o, lse, B, Hq, Hkv, Sq, Skv, &l, status, stream);
}

extern "C" int fba_attn_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                 const void* dout, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq,
                                 int Skv, int q_block_size, int kv_block_size, const uint8_t* block_mask_t,
                                 const uint8_t* small_block_mask_t, int mask_dim, int use_small_block_mode,
                                 void* workspace, uint64_t workspace_bytes, uint32_t* status, void* stream_) {
    ProfRange range("fba_attn_backward");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const uint8_t* mask_t = (use_small_block_mode && small_block_mask_t) ? small_block_mask_t : block_mask_t;
    if (!q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv || !mask_t || !workspace || !status)
        return set_error(FBA_ERR_BAD_ARG, "fba_attn_backward: null pointer argument");
    AttnWs w;
    int rc = plan(w, B, Hq, Hkv, Sq, Skv, q_block_size, kv_block_size, mask_dim, true, "fba_attn_backward: bad size");
    if (rc != FBA_OK) return rc;
    if (workspace_bytes < w.total)
        return set_error(FBA_ERR_BAD_ARG, "fba_attn_backward: workspace smaller than fba_attn_workspace_bytes() reports");
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return set_error(FBA_ERR_BAD_ARG, "fba_attn_backward: workspace must be 256-byte aligned");
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int32_t* idx = reinterpret_cast<int32_t*>(ws + w.idx);
    int32_t* cnt = reinterpret_cast<int32_t*>(ws + w.cnt);
    uint16_t* msk = w.aligned ? nullptr : reinterpret_cast<uint16_t*>(ws + w.msk);
    int32_t* order = reinterpret_cast<int32_t*>(ws + w.order);
    if (w.aligned) {
        // The masks arrive transposed ([.., nK, nQ], reference flex_block_attn_interface.py:85-86): the
        // query-major compaction of the transposed mask is the key-major list.
        rc = fba_build_index(mask_t, mask_dim, B, Hq, w.nK, w.nQ, idx, cnt, nullptr, nullptr, stream_);
    } else {
        DeviceGuard guard;
        if ((rc = guard.bind(mask_t)) != FBA_OK) return rc;
        uint8_t* mask = ws + w.mask;
        const long long total = static_cast<long long>(w.n_bh) * w.nQ * w.nK;
        untranspose_mask_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(mask_t, mask, w.nQ,
                                                                                                 w.nK, total);
        if ((rc = check_launch("untranspose_mask_kernel")) != FBA_OK) return rc;
        rc = fba_build_tile_lists(mask, mask_dim, B, Hq, w.nQ, w.nK, q_block_size, kv_block_size, Sq, Skv, nullptr,
                                  nullptr, nullptr, idx, cnt, msk, stream_);
    }
    if (rc != FBA_OK) return rc;
    fba_list_t l;
    l.idx = idx;
    l.cnt = cnt;
    l.msk = msk;
    l.stride = w.list_cols;
    l.rows_per_bh = w.list_rows;
    l.bh_stride = mask_dim == 4 ? w.list_rows : 0;
    l.rows_div = w.aligned ? kv_block_size / 128 : 1;
    l.sub = w.aligned ? q_block_size / 128 : 1;
    l.order = nullptr;
    if ((rc = fba_bwd_order(&l, B, Hq, Hkv, Skv, order, stream_)) != FBA_OK) return rc;
    l.order = order;
    return fba_bwd(q, k, v, o, lse, dout, dq, dk, dv, B, Hq, Hkv, Sq, Skv, &l, reinterpret_cast<float*>(ws + w.lse_delta),
                   reinterpret_cast<float*>(ws + w.dq_accum), status, stream_);
}
