// Shared pieces of the paged decode walk: launch arguments, the per-warp KV tile
// pipeline (cp.async ring in shared memory) and the page-id prefetcher.
#pragma once

#include "hkb_common.cuh"

namespace hkb {

// Stages of the walk a measurement build can leave out, to see what each costs (the mask of
// hkb_paged_decode_ablate; the reference's ablate=("page","kload","vload","qk","softmax","pv"),
// python/hk/ops/paged.py:524-533). A walk with any of them set computes nothing meaningful.
constexpr int ABL_PAGE = 1;      // page ids are not read from the block table (tile t reads block t mod pool)
constexpr int ABL_KLOAD = 2;     // K tiles are not copied
constexpr int ABL_VLOAD = 4;     // V tiles are not copied
constexpr int ABL_QK = 8;        // no S = K Q^T products
constexpr int ABL_SOFTMAX = 16;  // no maximum / exponential / sum
constexpr int ABL_PV = 32;       // no O += V^T P^T products

struct DecodeArgs {
  __nv_bfloat16* out;
  int64_t out_stride_tok, out_stride_head;
  const __nv_bfloat16* q;
  int64_t q_stride_tok, q_stride_head;
  const uint8_t* k;  // cache bases; strides below are in BYTES
  const uint8_t* v;
  int64_t k_stride_block, k_stride_token, k_stride_head;
  int64_t v_stride_block, v_stride_token, v_stride_head;
  int num_blocks;  // page ids are clamped to [0, num_blocks)
  const int* block_table;
  int64_t table_stride;
  int max_pages;
  const int* seq_lens;
  const int* q_start;
  int num_q_heads, num_kv_heads, group;
  int tiles_per_page;  // block_size / 16
  float scale;
  const float* k_scale;
  const float* v_scale;
  int num_splits;
  float* part_out;
  float* part_lse;
  // The decode step in one launch (stream kernel only; null = off):
  int* arrivals;                 // fold-on-arrival counters, ARRIVAL_INTS a (plane, sequence), zero between launches
  const __nv_bfloat16* new_k;    // the step's new token of every sequence, written into the cache by the ring
  const __nv_bfloat16* new_v;    // that walks the sequence's last tile, before it fetches that tile
  int64_t new_k_stride_tok, new_k_stride_head, new_v_stride_tok, new_v_stride_head;   // elements
  const void* slots;
  int slot_is_i64;
  int block_size;
  int xsplit;   // the caches are in the x-split layout (XSplitLoader); strides then describe blocks and heads only
};

// The range of 16-token tiles split `split` of a sequence with `n_tiles` tiles walks:
// contiguous, ceil(n_tiles / splits) each, as hk-dsl cuts it (python/hk/ops/paged.py:552-559).
__device__ __forceinline__ void split_range(int n_tiles, int splits, int split, int& lo, int& hi) {
  const int per = max((n_tiles + splits - 1) / splits, 1);
  lo = min(n_tiles, split * per);
  hi = min(n_tiles, lo + per);
}

// One warp's view of the KV stream of a (sequence, kv head): issues the cp.async
// copies of tile `t` (K rows then V rows) into ring stage `stage`. Page ids come
// from `PageIds`, which keeps 32 ids a batch in registers, one batch ahead, so that
// the table read is never on the critical path of a copy.
template <int ROWB, bool UNIT32 = false>   // UNIT32: the 32-byte-unit layout of fp8 rows (tile_off_f8)
struct TileLoader {
  static constexpr int CPR = ROWB / 16;              // 16-byte chunks per row
  static constexpr int TILE_BYTES = TILE_TOKENS * ROWB;
  static constexpr int ITERS = TILE_TOKENS * CPR / 32;   // copies a lane issues a tile
  static constexpr int RPI = 32 / CPR;               // rows the warp covers an iteration
  static constexpr int NPAT = 8 / RPI;               // distinct swizzle patterns over the iterations
  const uint8_t* kbase;  // + kv head offset
  const uint8_t* vbase;
  int64_t ksb, kst, vsb, vst;
  int tiles_per_page, num_blocks;
  // per-lane constants (set by `prepare`): where this lane's chunk sits in a row group
  uint32_t dst[NPAT];    // shared-memory offset of iteration q (mod NPAT), without it * 512
  int lane_k, lane_v;    // global offset of the lane's chunk in iteration 0
  bool k_flat, v_flat;   // the 16 rows of a tile are contiguous in global memory

  __device__ __forceinline__ void prepare(int lane) {
    const int rl = lane / CPR, c = lane % CPR;
#pragma unroll
    for (int q = 0; q < NPAT; ++q)
      dst[q] = UNIT32 ? tile_off_f8<UNIT32 ? ROWB : 128>(RPI * q + rl, c) - RPI * q * ROWB : tile_off<ROWB>(RPI * q + rl, c) - RPI * q * ROWB;
    lane_k = rl * (int)kst + c * 16;
    lane_v = rl * (int)vst + c * 16;
    k_flat = kst == ROWB;
    v_flat = vst == ROWB;
  }

  __device__ __forceinline__ void copy_tile(uint32_t smem_tile, const uint8_t* p, int64_t st, int lane_off,
                                            bool flat) const {
    p += lane_off;
    if (flat) {   // iteration it is 512 bytes on: immediates
#pragma unroll
      for (int it = 0; it < ITERS; ++it) cp_async16(smem_tile + dst[it % NPAT] + it * (RPI * ROWB), p + it * 512);
    } else {
      const int64_t step = RPI * st;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) cp_async16(smem_tile + dst[it % NPAT] + it * (RPI * ROWB), p + it * step);
    }
  }

  __device__ __forceinline__ void tile_ptrs(int tile, int page_id, const uint8_t*& kp, const uint8_t*& vp) const {
    const int id = min(max(page_id, 0), num_blocks - 1);
    kp = kbase + (int64_t)id * ksb;
    vp = vbase + (int64_t)id * vsb;
    if (tiles_per_page != 1) {   // a page of several 16-token tiles
      const int sub = tile % tiles_per_page;
      kp += (int64_t)(sub * TILE_TOKENS) * kst;
      vp += (int64_t)(sub * TILE_TOKENS) * vst;
    }
  }

  // The K tile alone (which = 0) or the V tile alone (which = 1): for rings two warps fill.
  __device__ __forceinline__ void issue_one(uint32_t smem_stage, int tile, int page_id, int lane, int which) const {
    const uint8_t *kp, *vp;
    tile_ptrs(tile, page_id, kp, vp);
    if (which) copy_tile(smem_stage + TILE_BYTES, vp, vst, lane_v, v_flat);
    else copy_tile(smem_stage, kp, kst, lane_k, k_flat);
  }

  __device__ __forceinline__ void issue(uint32_t smem_stage, int tile, int page_id, int lane) const {
    const uint8_t *kp, *vp;
    tile_ptrs(tile, page_id, kp, vp);
    copy_tile(smem_stage, kp, kst, lane_k, k_flat);
    copy_tile(smem_stage + TILE_BYTES, vp, vst, lane_v, v_flat);
  }
};

// The same interface over vLLM's older "x-split" cache layout, read in place
// (python/hk/ops/paged_prefill.py:768-772, `rocm_views`): K is (blocks, kv_heads, head_dim / x, page, x)
// with x = 8 sixteen-bit elements -- a token's row is head_dim / 8 chunks of 16 bytes, page * 16 bytes
// apart -- and V is (blocks, kv_heads, head_dim, page): V^T, a dim's tokens contiguous. Both tiles
// land in shared memory as they are stored. K: [chunk][16 tokens][16 bytes] -- the eight rows of an
// ldmatrix (eight tokens of one chunk) are 128 contiguous bytes, so no swizzle is needed, and a
// lane's copies go from consecutive addresses to consecutive addresses (scattering each lane's 16
// bytes to its token's row, the TileLoader arrangement, measured 1.75x the L2 sectors and 5.3
// against 6.4 TB/s). V: [dim][16 tokens] in 32-byte rows (the two 16-byte halves of a row swapped
// on every other group of four rows, which keeps the eight rows of an ldmatrix on distinct
// banks), read by the second product without a transpose.
template <int D>
struct XSplitLoader {
  static constexpr int ROWB = D * 2;
  static constexpr int TILE_BYTES = TILE_TOKENS * ROWB;      // K tile and V^T tile: 4 KB each at head_dim 128
  const uint8_t* kbase;
  const uint8_t* vbase;
  int64_t ksb, kst, vsb, vst;   // ksb / vsb: bytes between blocks; kst / vst are not used (the layout fixes them)
  int tiles_per_page, num_blocks;
  uint32_t kdst, vdst;          // this lane's shared-memory offsets in iteration 0
  int klane, vlane;             // and its global offsets

  __device__ __forceinline__ void prepare(int lane) {
    // K: a chunk index c is 16 tokens x 16 bytes contiguous; a half-warp takes one chunk, token r = lane % 16
    kdst = (uint32_t)(lane * 16);                // + 512 it: chunk c = 2 it + lane / 16 at 256 c + 16 r
    klane = (lane & 15) * 16;
    // V^T: a dim row is 32 bytes (16 tokens); two lanes a row, 16 rows an iteration
    const int d = lane >> 1, h = lane & 1;
    vdst = (uint32_t)(d * 32 + ((h ^ ((d >> 2) & 1)) << 4));
    vlane = h * 16;
  }
  __device__ __forceinline__ void tile_ptrs(int tile, int page_id, const uint8_t*& kp, const uint8_t*& vp) const {
    const int id = min(max(page_id, 0), num_blocks - 1);
    const int sub = tiles_per_page != 1 ? tile % tiles_per_page : 0;
    kp = kbase + (int64_t)id * ksb + sub * (TILE_TOKENS * 16);
    vp = vbase + (int64_t)id * vsb + sub * (TILE_TOKENS * 2);
  }
  __device__ __forceinline__ void issue_k(uint32_t dst, const uint8_t* kp, int lane) const {
    const int chunk_stride = tiles_per_page * TILE_TOKENS * 16;      // page tokens x 16 bytes
#pragma unroll
    for (int it = 0; it < D / 16; ++it) {                            // D / 8 chunks, two an iteration
      const int c = 2 * it + (lane >> 4);
      cp_async16(dst + kdst + it * 512, kp + (int64_t)c * chunk_stride + klane);
    }
  }
  __device__ __forceinline__ void issue_v(uint32_t dst, const uint8_t* vp, int lane) const {
    const int dim_stride = tiles_per_page * TILE_TOKENS * 2;         // page tokens x 2 bytes
#pragma unroll
    for (int it = 0; it < D / 16; ++it) {                            // 16 dim rows an iteration
      const int d = it * 16 + (lane >> 1);
      cp_async16(dst + it * 512 + vdst, vp + (int64_t)d * dim_stride + vlane);
    }
  }
  __device__ __forceinline__ void issue_one(uint32_t smem_stage, int tile, int page_id, int lane, int which) const {
    const uint8_t *kp, *vp;
    tile_ptrs(tile, page_id, kp, vp);
    if (which) issue_v(smem_stage + TILE_BYTES, vp, lane);
    else issue_k(smem_stage, kp, lane);
  }
  __device__ __forceinline__ void issue(uint32_t smem_stage, int tile, int page_id, int lane) const {
    const uint8_t *kp, *vp;
    tile_ptrs(tile, page_id, kp, vp);
    issue_k(smem_stage, kp, lane);
    issue_v(smem_stage + TILE_BYTES, vp, lane);
  }
};

struct PageIds {
  const int* row;  // this sequence's block-table row
  int max_pages, tiles_per_page, t_hi;
  int base;        // first tile of the batch held in `cur`
  int cur, nxt;

  __device__ __forceinline__ int fetch(int first_tile, int lane) const {
    const int t = first_tile + lane;
    if (t >= t_hi) return 0;
    const int p = min(t / tiles_per_page, max_pages - 1);
    return __ldg(row + p);
  }
  __device__ __forceinline__ void init(int t_lo, int lane) {
    base = t_lo;
    cur = fetch(base, lane);
    nxt = fetch(base + 32, lane);
  }
  // Page id of tile `t`; tiles are asked for in increasing order.
  __device__ __forceinline__ int get(int t, int lane) {
    if (t - base >= 32) {
      base += 32;
      cur = nxt;
      nxt = fetch(base + 32, lane);
    }
    return __shfl_sync(0xffffffffu, cur, t - base);
  }
};

}  // namespace hkb
