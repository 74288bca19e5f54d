/*
 * C ABI of the B200 (sm_100a) block-sparse attention library, libfba_b200.so.
 *
 * This is the boundary the Python autograd layer binds with ctypes.  It stands where the reference
 * project's pybind module `flex_block_attn_cuda` stood (reference attn.cpp:24-32, which exports
 * attn_forward / attn_backward and forwards to attention_forward / attention_backward in
 * flex_block_attn/flex_block_attn_h100.cu:810 and :1009).  Differences from that boundary, all
 * deliberate:
 *   - plain pointers and sizes only; the caller owns every buffer (no hidden allocation);
 *   - the work is stream-ordered on the stream passed in, with no device-wide synchronisation
 *     (the reference synchronises the device around every launch, .cu:882, 1004, 1113, 1212, 1263);
 *   - errors are integer status codes, never C++ exceptions; fba_last_error() gives the text;
 *   - the bool block mask is first compacted into index lists (fba_build_index /
 *     fba_build_tile_lists) which the attention kernels walk, instead of being scanned inside
 *     the attention kernels (reference .cu:107-121, 131-149, 642-699).
 *
 * Tensor layouts (all contiguous, device memory):
 *   q, o, dout, dq : bf16 [B, Hq,  Sq,  128]
 *   k, v, dk, dv   : bf16 [B, Hkv, Skv, 128]      Hq % Hkv == 0, head h reads kv head h / (Hq/Hkv)
 *   lse            : fp32 [B, Hq, Sq]   natural-log sum-exp of the scaled scores of each row
 *                    (-inf for a row that attends to nothing; its output row is 0)
 *   block mask     : uint8 (bool) [nQ, nK] (mask_dim 2, shared by every batch and head) or
 *                    [B, Hq, nQ, nK] (mask_dim 4); non-zero = attend
 * The softmax scale is 1/sqrt(128) (the reference's constant, .cu:177) unless an entry point takes one
 * explicitly; head_dim is fixed at 128 (.cu:833).
 *
 * Devices: every entry point that takes tensor pointers runs on the device that owns them and puts the
 * calling thread's previous CUDA context back before it returns (a thread that had none is left
 * without one), so a call has no effect on the caller's device selection.  Host threads may call
 * concurrently; fba_last_error() and the timing hook are per thread.
 *
 * Fixed limits (FBA_ERR_BAD_ARG / FBA_ERR_TOO_LARGE otherwise): head_dim 128; Sq >= 128 and Skv >= 128
 * (the reference also accepts a sequence of one 64-row block, flex_block_attn_interface.py:19; pad
 * such inputs to 128 rows with the extra keys masked off); B * Hq <= 65535 (grid y dimension).
 *
 * List format ("list" = fba_list_t): for list row r, entries idx[r * stride + e], e < cnt[r], are
 * ascending; unused slots hold -1.  `rows_per_bh` is the number of list rows of one (batch, head);
 * `bh_stride` is rows_per_bh for a per-head list and 0 for a list shared by all heads.
 * `rows_div` consecutive 128-row tiles share one list row and every entry stands for `sub`
 * consecutive 128-row tiles of the other sequence; `msk` (nullable) carries one 16-bit word per
 * entry: bit (8 * h + g) says whether 16-row query group g (0..7) of the 128-row query tile
 * attends to 64-row half h (0..1) of the 128-row key tile.
 */
#ifndef FBA_H_
#define FBA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FBA_ABI_VERSION 2
#define FBA_HEAD_DIM 128
#define FBA_TILE 128

/* Status codes (0 = success; negative = error). */
#define FBA_OK 0
#define FBA_ERR_BAD_ARG (-1)        /* null pointer, bad size, unsupported block size ... */
#define FBA_ERR_LAUNCH (-2)         /* CUDA reported an error at or before the launch */
#define FBA_ERR_DRIVER (-3)         /* could not resolve / run cuTensorMapEncodeTiled */
#define FBA_ERR_TIMEOUT (-4)        /* a bounded device-side wait gave up (see status words) */
#define FBA_ERR_TOO_LARGE (-5)      /* problem exceeds a documented fixed limit */

typedef struct fba_list {
    const int32_t* idx;   /* [rows_total, stride] */
    const int32_t* cnt;   /* [rows_total] */
    const uint16_t* msk;  /* [rows_total, stride] or NULL (every entry fully dense) */
    int32_t stride;       /* entries per list row */
    int32_t rows_per_bh;  /* list rows belonging to one (batch, head) */
    int32_t bh_stride;    /* rows_per_bh, or 0 when one list serves every (batch, head) */
    int32_t rows_div;     /* 128-row tiles per list row */
    int32_t sub;          /* 128-row tiles per entry */
    const int32_t* order; /* NULL, or the work-item order from fba_fwd_order / fba_bwd_order */
} fba_list_t;

int fba_abi_version(void);
/* Text of the most recent error on the calling thread ("" if none). */
const char* fba_last_error(void);

/*
 * Read the 8 status words the attention kernels write when a bounded device-side wait gives up
 * (synchronises `stream`).  FBA_OK if none did; otherwise FBA_ERR_TIMEOUT with the place in
 * fba_last_error(), and the words are cleared.  No counterpart in the reference, whose kernels spin
 * without a limit (its whole error handling is CHECK_CUDA_ERROR after the launch,
 * flex_block_attn_h100.cu:1003, 1262).  Call it where the host synchronises anyway (once per step).
 */
int fba_check_status(uint32_t* status, void* stream);
/*
 * Self-test of that path: one toy CTA waits, with a budget of `limit_cycles` SM clocks, on a barrier
 * nobody arrives at; the wait runs out, the kernel records (kernel 9, role 1, tag 777) in `status`
 * and ends normally.  fba_check_status() afterwards returns FBA_ERR_TIMEOUT.  `waited_cycles`
 * (device pointer, nullable) receives the clocks the wait took.
 */
int fba_selftest_wait_timeout(uint32_t* status, int64_t limit_cycles, uint64_t* waited_cycles, void* stream);

/* Number of kernels this library has launched in this process (all threads). */
uint64_t fba_launch_count(void);
/*
 * Measurement hook (no counterpart in the reference, which times whole calls from Python with
 * do_bench, benchmark/dynamic/random/scripts/random_fwd.py:161-166).  After
 * fba_set_timing_events(which, e0, e1) the calling thread's later fba_fwd (which = 1) or fba_bwd
 * (which = 2) calls record the CUDA events e0 / e1 (cudaEvent_t) on their stream immediately
 * before / after the main attention kernel, so its duration can be read without the small
 * helper kernels around it; which = 3 selects the query-major dQ kernel of FBA_DQ_QMAJOR.
 * which = 0 switches the hook off.
 */
int fba_set_timing_events(int which, void* start_event, void* stop_event);

/*
 * Block-mask -> index-list compaction (integer work, bit-exact against a nonzero()-based
 * restatement).  Replaces the per-call mask pooling and transposes of the reference's Python layer
 * (flex_block_attn/flex_block_attn_interface.py:38-66, 85-86) and the in-kernel mask scans.
 *   q2k_idx int32 [R, nK], q2k_cnt int32 [R]    R  = nQ (mask_dim 2) or B*H*nQ (mask_dim 4)
 *   k2q_idx int32 [Rk, nQ], k2q_cnt int32 [Rk]  Rk = nK (mask_dim 2) or B*H*nK
 * Either pair may be NULL to skip that direction.
 */
int fba_build_index(const uint8_t* mask, int mask_dim, int B, int H, int nQ, int nK,
                    int32_t* q2k_idx, int32_t* q2k_cnt, int32_t* k2q_idx, int32_t* k2q_cnt,
                    void* stream);

/*
 * 128x128-tile lists with 16-bit sub-tile masks, for block sizes that are not multiples of 128
 * (any q_block % 16 == 0, kv_block % 64 == 0).  nMt = ceil(Sq/128), nNt = ceil(Skv/128).
 *   fwd_idx int32 [R, nNt], fwd_cnt int32 [R], fwd_msk uint16 [R, nNt]   R  = nMt or B*H*nMt
 *   bwd_idx int32 [Rk, nMt], bwd_cnt int32 [Rk], bwd_msk uint16 [Rk, nMt] Rk = nNt or B*H*nNt
 * Either triple may be NULL.
 */
int fba_build_tile_lists(const uint8_t* mask, int mask_dim, int B, int H, int nQ, int nK,
                         int q_block, int kv_block, int Sq, int Skv, int32_t* fwd_idx,
                         int32_t* fwd_cnt, uint16_t* fwd_msk, int32_t* bwd_idx, int32_t* bwd_cnt,
                         uint16_t* bwd_msk, void* stream);

/*
 * Work-item order for the attention grids (no counterpart in the reference, whose CTAs take
 * blockIdx order, flex_block_attn_h100.cu:924).  The forward launches one CTA per pair of 128-row
 * query tiles, the backward one per 128-row key tile; list lengths differ, so both hand the items
 * of each (batch, head) out longest first when `list->order` is set.  The order is the stable
 * descending argsort of the item's work (sum of the list lengths it walks; backward: over the query
 * heads of the kv head's group), integer and deterministic.
 *   fba_fwd_order: order int32 [R, ceil(ceil(Sq/128)/2)],  R = B*Hq  (per-head list) or 1 (shared)
 *   fba_bwd_order: order int32 [R, ceil(Skv/128)],         R = B*Hkv (per-head list) or 1 (shared)
 * At most 12288 items per row (FBA_ERR_TOO_LARGE beyond; leave `order` NULL then).
 */
int fba_fwd_order(const fba_list_t* q2k, int B, int Hq, int Sq, int32_t* order, void* stream);
int fba_bwd_order(const fba_list_t* k2q, int B, int Hq, int Hkv, int Skv, int32_t* order, void* stream);

/*
 * Mask builders that emit lists directly (no counterpart in the reference: it advertises sliding-
 * tile, MoBA and hybrid SSTA masks, README.md:54-55, but its __init__.py:7-12 leaves them out).
 *
 * fba_sta_index: 3-D sliding-tile window over a Gt x Gh x Gw grid of tiles (tile id =
 * (t*Gh + h)*Gw + w; tile i attends tile j iff |dt|<=wt, |dh|<=wh, |dw|<=ww).  Writes the shared
 * (2-D) list idx int32 [n, n], cnt int32 [n], n = Gt*Gh*Gw; the relation is symmetric, so the same
 * list is both the query-major and the key-major one.  Equal to fba_build_index on the bool mask.
 *
 * fba_ssta_index: per (batch, head) the STA window of the tile containing each query block,
 * united with the `topk` key blocks of largest (mean of the query block) . (mean of the key block).
 * One key block = one tile (Gt*Gh*Gw == Skv/kv_block), q_block divides kv_block.  Writes the bool
 * mask uint8 [B, Hq, nQ, nK], the query-major list (q2k_idx int32 [B*Hq*nQ, nK], q2k_cnt) and,
 * if given, the key-major list.  `scratch` holds fba_ssta_scratch_floats() floats.
 * A window extent of -1 (wt = wh = ww = -1) switches the window off: the mask is then the top-k
 * selection alone, i.e. a MoBA mask (use the grid 1 x 1 x nK).
 */
int fba_sta_index(int Gt, int Gh, int Gw, int wt, int wh, int ww, int32_t* idx, int32_t* cnt,
                  void* stream);
int fba_ssta_scratch_floats(int B, int Hq, int Hkv, int nQ, int nK, uint64_t* n_floats);
int fba_ssta_index(const void* q, const void* k, int B, int Hq, int Hkv, int Sq, int Skv, int q_block,
                   int kv_block, int Gt, int Gh, int Gw, int wt, int wh, int ww, int topk,
                   float* scratch, uint8_t* mask, int32_t* q2k_idx, int32_t* q2k_cnt,
                   int32_t* k2q_idx, int32_t* k2q_cnt, void* stream);

/*
 * Layout change around the operator, one pass: bf16 [B, S, Hn, 128] with tokens in raster (t, h, w)
 * order over a T x H x W grid  <->  bf16 [B, Hn, S, 128] with tokens in tile-major order (tiles of
 * tt x th x tw tokens, tiles in raster order).  Replaces the transpose the reference's callers do
 * before the call (benchmark/dynamic/random/scripts/random_fwd.py:58-60) plus the token reorder
 * sliding-tile masks assume.  to_tile_major != 0: src is [B,S,Hn,128], dst [B,Hn,S,128]; else the
 * inverse.  src and dst must not overlap.
 */
int fba_tile_major(const void* src, void* dst, int B, int Hn, int T, int H, int W, int tt, int th, int tw,
                   int to_tile_major, void* stream);

/*
 * Forward (replaces attention_forward, reference .cu:810-1007, and fwd_attend_ker, .cu:52-318).
 * `q2k` is the query-major list.  `status` points at 8 zero-initialised uint32 words in device
 * memory; word 0 becomes non-zero if a bounded wait inside the kernel gave up (then the outputs
 * are undefined), words 1.. say where.
 */
int fba_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Hq,
            int Hkv, int Sq, int Skv, const fba_list_t* q2k, uint32_t* status, void* stream);
/*
 * fba_fwd with a caller-chosen softmax scale (no counterpart in the reference, whose kernels fix
 * 1/sqrt(128), flex_block_attn_h100.cu:201): scores are softmax_scale * q k^T; softmax_scale
 * must be positive and finite.  lse may be NULL: then no log-sum-exp is written (inference-only
 * forward).  fba_fwd(...) == fba_fwd_scaled(..., 1/sqrt(128), ...) with lse required.
 */
int fba_fwd_scaled(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Hq,
                   int Hkv, int Sq, int Skv, const fba_list_t* q2k, float softmax_scale,
                   uint32_t* status, void* stream);

/*
 * Inference forward over an 8-bit key / value cache (no counterpart in the reference, which is bf16
 * only, flex_block_attn_h100.cu:854-858).
 *
 * fba_quantize_kv_e4m3 writes the cache: x bf16 [n_bh, S, 128] -> e4m3 bytes with one fp32 scale per
 * (bh, block of `scale_block` rows), scale = max|x| * fp32(1/448) over the block (1 for an all-zero
 * block), byte = e4m3(x * (1 / scale)), round to nearest even, saturating.  transposed == 0: x8 is [n_bh, S, 128] (use for K);
 * transposed != 0: x8 is [n_bh, 128, S] (use for V).  scales: fp32 [n_bh, S / scale_block].
 * scale_block must be a multiple of 128 and divide S.
 *
 * fba_fwd_fp8kv: o = softmax(softmax_scale * q K^T on the listed blocks) V with K = k8 * k_scale,
 * V = v8t^T * v_scale; q and o are bf16 like fba_fwd's, lse may be NULL.  Both GEMMs run in e4m3 on the
 * tensor cores: q is quantised per row and the probabilities per element inside the kernel, so the
 * result differs from the bf16 forward on the dequantised cache by 8-bit rounding of q and P
 * (cosine >= 0.999 against the oracle on the dequantised cache on the tested shapes).  Skv must be a multiple of scale_block.
 */
int fba_quantize_kv_e4m3(const void* x, uint8_t* x8, float* scales, int n_bh, int S, int scale_block,
                         int transposed, void* stream);
int fba_fwd_fp8kv(const void* q, const uint8_t* k8, const uint8_t* v8t, const float* k_scale,
                  const float* v_scale, int scale_block, void* o, float* lse, int B, int Hq, int Hkv, int Sq,
                  int Skv, const fba_list_t* q2k, float softmax_scale, uint32_t* status, void* stream);

/*
 * Backward (replaces attention_backward, reference .cu:1009-1267, bwd_attend_prep_ker .cu:339-389
 * and bwd_attend_ker .cu:572-802).  Gradients come back in bf16.
 *   k2q      : key-major list (entries are query tiles)
 *   lse_delta: scratch fp32 [B*Hq, nMt*128, 2]   (nMt = ceil(Sq/128))
 *   dq_accum : scratch fp32 [B*Hq, nMt*128, 128]; zeroed by this call
 * Both scratch buffers are caller-allocated; fba_bwd_scratch_bytes() gives their sizes.
 */
int fba_bwd_scratch_bytes(int B, int Hq, int Sq, uint64_t* lse_delta_bytes,
                          uint64_t* dq_accum_bytes);
int fba_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
            const void* dout, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq,
            int Skv, const fba_list_t* k2q, float* lse_delta, float* dq_accum, uint32_t* status,
            void* stream);
/* fba_bwd for a forward that ran with fba_fwd_scaled: pass the same softmax_scale. */
int fba_bwd_scaled(const void* q, const void* k, const void* v, const void* o, const float* lse,
                   const void* dout, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq,
                   int Skv, const fba_list_t* k2q, float softmax_scale, float* lse_delta,
                   float* dq_accum, uint32_t* status, void* stream);

/*
 * Backward with a choice of dQ strategy (the reference has only the first: its key-major kernel
 * reduce-adds fp32 dQ tiles into global memory, flex_block_attn_h100.cu:700-718, 750-764).
 *   FBA_DQ_ATOMIC  the key-major kernel adds each 128x128 dQ partial into the fp32 accumulator
 *                  `dq_accum` with vector reductions; a conversion pass writes bf16 dQ.  `q2k` is
 *                  not used (may be NULL).  dQ sums arrive in scheduling order: equal to fp32
 *                  rounding, not bit-reproducible.
 *   FBA_DQ_QMAJOR  a second, query-major kernel walks `q2k`, recomputes S and dP and accumulates
 *                  dQ in tensor memory; the key-major kernel computes only dK and dV.  dQ is written
 *                  once, in bf16, bit-reproducibly; `dq_accum` is not used (may be NULL) and only the
 *                  small `lse_delta` scratch is needed.  Two more GEMMs per tile pair.
 * fba_bwd_scaled(...) == fba_bwd_ex(..., q2k = NULL, ..., FBA_DQ_ATOMIC, ...).
 */
#define FBA_DQ_ATOMIC 0
#define FBA_DQ_QMAJOR 1
/*
 * Two interchangeable key-major kernels exist for FBA_DQ_ATOMIC (same results to fp32 summation
 * order in dK / dV, same scratch): 1 keeps the score tile transposed (tensor-memory lane = key row,
 * P^T feeds dV straight from tensor memory), 2 keeps it upright (lane = query row: per-row log-sum-exp
 * and delta are scalars, P and dS go through shared memory).  1 is the default because it measures
 * 4-5 % faster on B200; `FBA_BWD_KERNEL=2` in the environment, or this call, selects the other.
 * Returns the previous choice (1 or 2), or FBA_ERR_BAD_ARG.  Process-wide.
 */
int fba_set_bwd_kernel(int which);
int fba_bwd_ex(const void* q, const void* k, const void* v, const void* o, const float* lse,
               const void* dout, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq, int Skv,
               const fba_list_t* k2q, const fba_list_t* q2k, float softmax_scale, int dq_mode,
               float* lse_delta, float* dq_accum, uint32_t* status, void* stream);

/*
 * The reference extension's own call shape (reference attn.cpp:12-21 and
 * flex_block_attn_h100.cu:810-818, 1009-1021): q, k, v (+ o, lse, dO), the two block sizes, the bool
 * block mask(s) and use_small_block_mode in; o, lse / dq, dk, dv out.  Where the reference allocates
 * its results and temporaries through torch inside the call (.cu:862-876, 1077-1093), the caller
 * here passes the outputs and one 256-byte-aligned device workspace of fba_attn_workspace_bytes();
 * mask compaction, work order and (backward) scratch all live there.  Stream-ordered; nothing is
 * allocated.
 *   block_mask / small_block_mask: uint8 (bool), mask_dim 2 or 4.  As in the reference,
 *     small_block_mask is the mask at [Sq/q_block, Skv/kv_block] granularity and is the one used when
 *     use_small_block_mode != 0 (block_mask, the pooled mask, is not needed then and may be NULL);
 *     otherwise block_mask is used.
 *   fba_attn_backward takes the masks TRANSPOSED ([.., Skv/kv_block, Sq/q_block]) like the reference
 *     (flex_block_attn_interface.py:85-86).
 *   lse: fp32 [B, Hq, Sq], natural log (the reference stores -sqrt(128) * LSE in [B, H, Sq, 1]).
 */
int fba_attn_workspace_bytes(int B, int Hq, int Hkv, int Sq, int Skv, int q_block_size, int kv_block_size,
                             int mask_dim, int backward, uint64_t* bytes);
int fba_attn_forward(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Hq, int Hkv,
                     int Sq, int Skv, int q_block_size, int kv_block_size, const uint8_t* block_mask,
                     const uint8_t* small_block_mask, int mask_dim, int use_small_block_mode, void* workspace,
                     uint64_t workspace_bytes, uint32_t* status, void* stream);
int fba_attn_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                      const void* dout, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq, int Skv,
                      int q_block_size, int kv_block_size, const uint8_t* block_mask_t,
                      const uint8_t* small_block_mask_t, int mask_dim, int use_small_block_mode, void* workspace,
                      uint64_t workspace_bytes, uint32_t* status, void* stream);

/*
 * Backward for callers that cannot allocate device memory (no counterpart in the reference, whose
 * extension allocates everything it needs through torch, .cu:1077-1093).
 *
 * Same computation and results as fba_bwd, but the two scratch buffers come from a fixed array
 * built into the library instead of from the caller: meant for hosts whose HBM is fully owned by
 * a pre-sized arena or a foreign memory pool, or that must avoid cudaMalloc's device-wide
 * synchronisation on a latency-critical path.  The call itself allocates nothing.
 *   - Limit: B * Hq * ceil(Sq/128) * 128 <= fba_bwd_static_scratch_max_rows() (131072 rows, i.e.
 *     about 65 MiB that every GPU loading this library keeps resident until the process exits).
 *     Larger problems return FBA_ERR_TOO_LARGE; use fba_bwd for those.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress with that device current); make that first call outside any stream
 *     capture.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left;
 *     each call rewrites / zero-fills the part it uses before reading it.  Two calls whose
 *     kernels may overlap on the GPU (different streams, or several host threads) race on it:
 *     serialise them.
 */
uint64_t fba_bwd_static_scratch_max_rows(void);
int fba_bwd_static_scratch(const void* q, const void* k, const void* v, const void* o,
                           const float* lse, const void* dout, void* dq, void* dk, void* dv, int B,
                           int Hq, int Hkv, int Sq, int Skv, const fba_list_t* k2q, uint32_t* status,
                           void* stream);

/*
 * Sequence <-> head exchange over peer memory, fused with the token reorder (no counterpart in the
 * reference, which is single-GPU; its callers' layouts are benchmark/dynamic/random/scripts/
 * random_fwd.py:58-60).  With the sequence of a [B, S, H, 128] raster-order (t, h, w) activation
 * sharded over n_ranks GPUs (rank r holds rows r*S/n .. (r+1)*S/n), every GPU needs
 * [B, H/n, S, 128] for its heads, tokens in tile-major order (tiles of tt x th x tw; 1 x 1 x 1
 * keeps raster order).  fba_peer_exchange reads the local tensor once and stores each 256-byte
 * row into its final place in the owning GPU's destination buffer:
 *   to_head != 0: src [B, S/n, H, 128] raster chunk  -> peers[h / (H/n)] as [B, H/n, S, 128] tile-major
 *   to_head == 0: src [B, H/n, S, 128] tile-major    -> peers[owner of the raster row] as [B, S/n, H, 128]
 * peers[i] is rank i's destination buffer as addressable from THIS process (peers[rank] is the
 * local one).  The kernel waits on nothing; the caller orders it against the other GPUs with a
 * barrier before (destinations no longer read) and after (rows have landed).
 *
 * Destination buffers are plain cudaMalloc memory shared through CUDA IPC:
 *   fba_peer_alloc / fba_peer_free   on the owning process (current device),
 *   fba_peer_export                  64-byte handle to send to the other processes,
 *   fba_peer_open / fba_peer_close   map / unmap another process's buffer (enables peer access).
 */
int fba_peer_alloc(uint64_t bytes, void** ptr);
int fba_peer_free(void* ptr);
int fba_peer_export(const void* ptr, unsigned char* handle64);
int fba_peer_open(const unsigned char* handle64, void** ptr);
int fba_peer_close(void* ptr);
int fba_peer_exchange(const void* src, void* const* peers, int n_ranks, int rank, int B, int H, int T,
                      int Hh, int W, int tt, int th, int tw, int to_head, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FBA_H_ */
