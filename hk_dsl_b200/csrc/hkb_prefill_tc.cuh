// Paged prefill on the fifth-generation tensor cores: tcgen05.mma with accumulators in tensor
// memory (TMEM). head_dim 128, bf16 or fp16 caches.
//
// What it computes is hk-dsl's paged prefill (python/hk/ops/paged_prefill.py:59-620): causal
// attention of a request's new tokens over its paged cache, the grid a host-built work list of
// (request, query tile) items (paged_prefill.py:879-968).
//
// The grid is persistent: one CTA an SM, each walking its share of the (work item, head pass) pairs
// (dealt out in rounds, every other round backwards: the list is sorted by keys, so the CTAs' sums
// come out even). Barrier phases simply run on from item to item, so the producers fetch the next
// item's query rows and first K/V blocks, and the MMA warps issue its first scores, while the softmax
// warps are still in the epilogue of the current one. An item is 2 query tiles of 128 rows each -- a
// tile is T = 128 / GP consecutive tokens of GP query heads of one kv head, so both tiles and all
// their heads share every K/V block the CTA stages -- and its keys are walked in blocks of 128:
//
//   producers (2 warps)  gather the block's eight 16-token pages through the block table into a ring
//                        of 32 KB shared-memory slots (one warp the K blocks, one the V blocks,
//                        alternating in the ring): sixteen TMA tile copies a block
//                        (cp.async.bulk.tensor over a 4-D map of the cache, 16 tokens x 64 dims a
//                        copy, 128-byte swizzle, completion counted in bytes on the slot's
//                        mbarrier), one lane a copy. The block that holds the last keys -- where
//                        rows past the end must read as zeros -- and caches no tensor map describes
//                        go through cp.async with the same swizzle, a proxy fence and an arrive.
//                        The V warp also brings the query tiles (TMA over a 3-D map of q), once
//                        the products of the item before have read the old ones;
//   MMA warp (1 thread)  S = Q K^T (8 tcgen05.mma of 128 x 128 x 16, Q and K from shared memory)
//                        into the tile's 128 score columns of TMEM, and O += P V (8 tcgen05.mma of
//                        128 x 128 x 16, P from TMEM, V from shared memory read MN-major) into its
//                        128 accumulator columns; the two tiles take turns on the tensor pipe: a
//                        tile's P V product and its next block's scores are issued as soon as its
//                        softmax warps hand P over, while the other tile's warps are in their
//                        exponentials; completion is signalled by tcgen05.commit onto mbarriers;
//   softmax (2 x 4 warps) a thread owns one query row: it reads its 128 scores from TMEM
//                        (tcgen05.ld), masks the diagonal block, keeps the running maximum lazily
//                        (the accumulator is rescaled only when a block's maximum exceeds the
//                        reference by 2^8), writes P as packed 16-bit pairs over the scores it has
//                        read (tcgen05.st) and arrives; no shuffles: a row is a TMEM lane. After
//                        an item's last block it normalises the accumulator and writes the rows
//                        out through staging rows of its own in shared memory.
//
// All 512 TMEM columns are in use (two accumulators, two score tiles), which is why P lives where
// the scores were. Every wait is bounded: a barrier that does not flip within about a second sets
// an error word (hkb_prefill_tc_error) and the CTA winds down -- its copies drained, its TMEM
// freed -- instead of spinning.
#pragma once

#include <cuda.h>   // CUtensorMap (the type only: the encoder is fetched through the runtime)

#include "hkb_common.cuh"

namespace hkb {
namespace tc {

constexpr int KVB = 128;                      // keys a block
constexpr int ROWS = 128;                     // rows of a query tile = TMEM lanes
constexpr int D = 128;                        // head_dim
constexpr int HALF_BYTES_Q = ROWS * 128;      // 64 dims of 128 rows, 128-byte rows
constexpr int Q_BYTES = 2 * HALF_BYTES_Q;     // one query tile: 32 KB
constexpr int HALF_BYTES_KV = KVB * 128;      // 64 dims of 128 tokens
constexpr int SLOT_BYTES = 2 * HALF_BYTES_KV; // a K or a V block: 32 KB
constexpr int NSLOT = 4;                      // ring slots: K blocks in the even ones, V blocks in the odd ones
constexpr int SOFTMAX_WARPS = 8, MMA_WARP = 8, K_WARP = 9, V_WARP = 10, WARPS = 11;
constexpr int THREADS = WARPS * 32;
// fp8 caches: of a block's eight 16-token tiles the kind's own producer warp widens the first FP8_MAIN; below 8
// a third producer warp takes the rest of both kinds. Measured at 8 x 2048: two warps (8) 544-548 TFLOP/s,
// three (6 + 2) 511, four (two a kind, 13 warps: the CTA is rounded up to 16 warps of 128 registers and the
// softmax warps spill) 516 -- the widening does not get faster with more warps, so two it is.
constexpr int FP8_MAIN = 8;
__host__ __device__ constexpr int threads_of(bool fp8) { return fp8 && FP8_MAIN < 8 ? THREADS + 32 : THREADS; }
constexpr int TMEM_COLS = 512;
// TMEM columns: O of tile 0 and 1, then the scores of tile 0 and 1 (P is written over the scores)
__host__ __device__ constexpr int o_col(int tile) { return tile * 128; }
__host__ __device__ constexpr int s_col(int tile) { return 256 + tile * 128; }

struct Bars {                                  // mbarriers, 8 bytes each
  uint64_t full[NSLOT], empty[NSLOT];
  uint64_t s_full[2], p_full[2], o_done[2], q_full[2], q_empty[2], q_ready[2];
  uint32_t tmem_base;
  int abort;
};
constexpr int EPI_BYTES = SOFTMAX_WARPS * 4096;   // the epilogue's staging: 32 half rows of 128 bytes a softmax warp (fp8 caches:
                                                  // 32 quarter rows of 64 bytes; the upper 16 KB are the producers' staging rings)
constexpr int FP8_STAGE_TILES = 4;                // 16-token fp8 tiles (2 KB) in a producer's staging ring: three in flight, one being widened
                                                  // (seven in flight measured the same: the producers are not waiting for their copies)
static_assert((FP8_MAIN < 8 ? 3 : 2) * FP8_STAGE_TILES * 2048 <= EPI_BYTES / 2, "the producers' staging rings live in the upper half of the epilogue's space");
constexpr int SMEM_BYTES = 1024 /*alignment slack*/ + 2 * Q_BYTES + NSLOT * SLOT_BYTES + EPI_BYTES + 1024 /*Bars*/;
static_assert(sizeof(Bars) <= 1024, "barrier block");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory of one SM");

__device__ int g_error;   // first failure code of any CTA since it was last cleared (0: none)

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ long long now() {   // the SM's cycle counter
  long long t;
  asm volatile("mov.u64 %0, %%clock64;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(bar) : "memory");
}
// one arrival that also announces `bytes` of asynchronous copies to come (the phase completes when they have landed)
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}\n" ::"r"(bar), "r"(bytes) : "memory");
}
// One TMA tile copy, global -> this CTA's shared memory, bytes counted on `bar`. No multicast. The
// innermost coordinate times the element size is a multiple of 16 bytes (0 or 64 elements here).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {   // volatile: keeps its place in the instruction stream
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Wait for the phase of `parity` to complete; gives up (and raises the CTA's abort flag) after
// about 2^31 clocks, or as soon as another thread of the CTA has given up.
// NAP: sleep ~64 ns between polls. A polling warp takes issue slots from the warps of its scheduler; where
// the waits are long and another role is short of issue slots (fp8 caches: the producers' conversion), the
// waiters step aside.
template <bool NAP = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort, int code) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = now();
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if (NAP) __nanosleep(64);
    if (*abort) return false;
    if (now() - t0 > (1ll << 31)) {
      *abort = code;
      atomicCAS(&g_error, 0, code);
      return false;
    }
  }
}
// The same for a whole warp: every lane polls, and all lanes take the same way out (the TMEM loads
// and stores that follow are warp-collective).
template <bool NAP = false>
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort, int code) {
  const bool ok = mbar_wait<NAP>(bar, parity, abort, code);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t addr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 consecutive fp32 columns of this thread's TMEM lane: two 32-column loads in flight, one wait
__device__ __forceinline__ void tmem_ld64(uint32_t addr, float (&v)[64]) {
  uint32_t r[64];
#pragma unroll
  for (int h = 0; h < 2; ++h)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[32 * h + 0]), "=r"(r[32 * h + 1]), "=r"(r[32 * h + 2]), "=r"(r[32 * h + 3]), "=r"(r[32 * h + 4]), "=r"(r[32 * h + 5]),
          "=r"(r[32 * h + 6]), "=r"(r[32 * h + 7]), "=r"(r[32 * h + 8]), "=r"(r[32 * h + 9]), "=r"(r[32 * h + 10]), "=r"(r[32 * h + 11]),
          "=r"(r[32 * h + 12]), "=r"(r[32 * h + 13]), "=r"(r[32 * h + 14]), "=r"(r[32 * h + 15]), "=r"(r[32 * h + 16]), "=r"(r[32 * h + 17]),
          "=r"(r[32 * h + 18]), "=r"(r[32 * h + 19]), "=r"(r[32 * h + 20]), "=r"(r[32 * h + 21]), "=r"(r[32 * h + 22]), "=r"(r[32 * h + 23]),
          "=r"(r[32 * h + 24]), "=r"(r[32 * h + 25]), "=r"(r[32 * h + 26]), "=r"(r[32 * h + 27]), "=r"(r[32 * h + 28]), "=r"(r[32 * h + 29]),
          "=r"(r[32 * h + 30]), "=r"(r[32 * h + 31])
        : "r"(addr + 32 * h) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// max of three (one instruction on sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a tile whose rows are 128 bytes, 8-row groups 1024 bytes
// apart, 16-byte chunks XOR-swizzled by the row (the 128-byte swizzle): start address, leading
// and stride byte offsets in 16-byte units, descriptor version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lead_bytes) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)((lead_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: fp32 accumulate, A and B both bf16 (1) or f16 (0), A K-major,
// B K-major or MN-major, N / 8 and M / 16.
__host__ __device__ constexpr uint32_t instr_desc(bool f16, bool b_mn_major, int n) {
  return (1u << 4) | ((f16 ? 0u : 1u) << 7) | ((f16 ? 0u : 1u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
}

struct Args {
  __nv_bfloat16* out;
  int64_t out_stride_tok, out_stride_head;
  const __nv_bfloat16* q;
  int64_t q_stride_tok, q_stride_head;
  const uint8_t* k;
  const uint8_t* v;
  int64_t k_stride_block, k_stride_token, k_stride_head;   // bytes
  int64_t v_stride_block, v_stride_token, v_stride_head;
  int num_blocks;
  const int* block_table;
  int64_t table_stride;
  int max_pages;
  const int* seq_lens;
  const int* q_start;
  const int* work;
  int num_work;
  int num_q_heads, num_kv_heads, group, tiles_per_page;
  float scale;
  const float* k_scale;     // fp8 caches: the per-tensor scales (device floats); else unused
  const float* v_scale;
  int tma;                  // K and V blocks by TMA (the two tensor maps are valid)
  int tma_q;                // the query tiles by TMA (the query map is valid)
  int k_pos[3], v_pos[3];   // which coordinate of the map (1..3) is the token, the kv head, the block
  int q_pos[2];             // which coordinate of the query map (1..2) is the token, the head
  unsigned long long* trace;   // TRACE builds only: 32 cycle counters a CTA (see Lap), else unused
};

// Where a CTA's cycles go, for the traced build (hkb_paged_prefill_trace): one thread of each role
// adds the clocks between consecutive laps to a counter. Slots: softmax of tile g at 8 g + {0 wait
// for the scores, 1 TMEM loads and maximum, 2 exponentials, 3 wait for the previous product (and the
// rescale), 4 P store and arrive, 5 epilogue}; MMA warp 16 wait for Q, 17 wait for K, 18 issue of the
// first score products, 19 wait for V, 20 / 22 wait for P of tile 0 / 1, 21 issue of the P V products,
// 23 issue of the next block's scores;
// producers 24 + 4 w + {0 wait for a free slot, 1 issue of the copies, 2 wait for copies to land};
// 31 the CTA's whole time.
template <bool TRACE>
struct Lap {
  long long t;
  __device__ __forceinline__ Lap() : t(TRACE ? now() : 0) {}
  __device__ __forceinline__ void operator()(unsigned long long& acc) {
    if (TRACE) { const long long n = now(); acc += (unsigned long long)(n - t); t = n; }
  }
};

// Half of a 128-token block (64 rows: four 16-token pages) of K or of V into a ring slot, by one
// producer warp: 64 rows x 16 chunks of 16 bytes, 32 copies a lane. Rows at or past `kv_limit` are
// zero-filled, never read.
__device__ __forceinline__ void fill_half(const Args& a, uint32_t slot, const uint8_t* base, int64_t sb, int64_t st,
                                          const int* table_row, int kv0, int kv_limit, int lane) {
  // the four 16-token tiles: page id and offset of each, one lane a tile
  int my_id = 0, my_sub = 0;
  if (lane < 4) {
    const int tile = kv0 / TILE_TOKENS + lane;
    if (tile * TILE_TOKENS < kv_limit) {
      const int page = min(tile / a.tiles_per_page, a.max_pages - 1);
      my_id = min(max(__ldg(table_row + page), 0), a.num_blocks - 1);
      my_sub = tile % a.tiles_per_page;
    }
  }
  const int c = lane & 15, hi = lane >> 4;
  // where this lane's chunk lands inside an 8-row group, for the four row phases it meets
  uint32_t x[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) x[q] = (uint32_t)((c >> 3) * HALF_BYTES_KV + (((c & 7) ^ ((2 * q + hi) & 7)) << 4));
  const uint32_t dst0 = slot + (uint32_t)((kv0 % KVB) + hi) * 128;
  const int64_t lane_off = (int64_t)hi * st + c * 16, step = 2 * st;
  if (kv0 + 64 <= kv_limit) {                     // every row is a key: nothing to predicate
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int id = __shfl_sync(0xffffffffu, my_id, t), sub = __shfl_sync(0xffffffffu, my_sub, t);
      const uint8_t* p = base + (int64_t)id * sb + (int64_t)(sub * TILE_TOKENS) * st + lane_off;
#pragma unroll
      for (int it = 0; it < 8; ++it) cp_async16(dst0 + (t * 16 + it * 2) * 128 + x[it & 3], p + it * step);
    }
  } else {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int id = __shfl_sync(0xffffffffu, my_id, t), sub = __shfl_sync(0xffffffffu, my_sub, t);
      const uint8_t* p = base + (int64_t)id * sb + (int64_t)(sub * TILE_TOKENS) * st + lane_off;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const uint32_t dst = dst0 + (t * 16 + it * 2) * 128 + x[it & 3];
        if (kv0 + t * 16 + it * 2 + hi < kv_limit) cp_async16(dst, p + it * step);
        else asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(dst), "r"(0u) : "memory");
      }
    }
  }
}

// fp8-e4m3 caches: a producer warp brings its blocks 16 tokens (a 2 KB tile) at a time -- cp.async into
// a staging ring of its own (FP8_STAGE_TILES tiles: all but one in flight while that one is converted),
// then shared memory -> registers -> f16 (cvt.rn.f16x2.e4m3x2, exact; the per-tensor scale is applied to
// the scores and to the output, not here) -> the ring slot, where the 16-bit path's copies would have
// landed. A lane owns a 16-byte chunk (16 dims) of four rows of every tile and reads back only what it
// copied itself, so the staging needs no barrier. Rows at or past the keys' end are zeros, never read.
// (Measured on the way, TFLOP/s at 8 x 2048: loading into registers instead of staging, with the
// conversion unrolled over several tiles to keep loads in flight, 250-490; widening by byte permutes,
// shifts and one packed multiply by 2^8 instead of the convert instruction -- 5 instructions a pair of
// values against 2 -- 426 against 548: the producers are bound by the instructions they issue.)
__device__ __forceinline__ uint32_t fp8x2_to_f16x2(uint32_t two_bytes) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h2) : "h"((uint16_t)two_bytes));
  return h2;
}

// One half (64 columns) of a score row: causal mask, then either the maximum (MATH = 0) or the
// exponentials, their sum and the packed 16-bit P (MATH = 1).
template <bool F16>
__device__ __forceinline__ float half_max(float (&s)[64], bool masked, bool valid, int key0, int pos) {
  if (masked) {
#pragma unroll
    for (int i = 0; i < 64; ++i)
      if (!valid || key0 + i > pos) s[i] = -INFINITY;
  }
  float mq[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {          // four independent chains of three-input max
    mq[c] = max3(s[16 * c], s[16 * c + 1], s[16 * c + 2]);
#pragma unroll
    for (int i = 3; i < 15; i += 2) mq[c] = max3(mq[c], s[16 * c + i], s[16 * c + i + 1]);
    mq[c] = fmaxf(mq[c], s[16 * c + 15]);
  }
  return fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
}
// 2^x on the FMA pipe, for x <= 8 or so: x = n + f with n the nearest integer (the add of 1.5 * 2^23
// leaves n in the low mantissa bits), a cubic for 2^f on [-0.5, 0.5] (fitted for the smallest largest
// relative error, 7.5e-5 -- P is rounded to 16 bits, 2e-3, after it), n added to the exponent field.
// The MUFU unit does 16 exponentials a clock an SM, as long as the tensor core takes for the two
// products they feed: a share of them done here takes that unit off the critical path.
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -126.f);                         // a masked score (-inf) comes out as 2^-126: nothing
  const float shifted = x + 12582912.f;
  const float f = x - (shifted - 12582912.f);
  const float p = fmaf(fmaf(fmaf(0.0551716685f, f, 0.2426111251f), f, 0.6932609677f), f, 0.9999280572f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(shifted) << 23));
}
// which pairs of a row take the polynomial: one in POLY_EVERY (0: none). Measured with the libraries run in
// turn on one B200 (TFLOP/s at 1 x 8192 / 8 x 2048 / 32 x 512): none 1070-1080 / 758-770 / 318-388; every 3rd
// 1011-1027 / 677-688 / 322-341; 4th 1042-1061 / 727-764 / 360-366; 5th 1081-1086 / 821-826 / 392-404;
// 6th 1061-1063 / 729-736 / 361-371; 7th 1084-1089 / 746-750 / 368-381; 8th 1092-1108 / 843-855 / 408-410;
// 10th 1114-1116 / 843-850 / 414; 12th 1105 / 840-845 / 410; 16th 1108-1111 / 832-841 / 396-406. Not a smooth
// curve: where the polynomial's nine dependent instructions fall among the MUFU pairs decides how well the
// row's instruction stream packs.
constexpr int POLY_EVERY = 10;

template <bool F16>
__device__ __forceinline__ float half_exp(float (&s)[64], bool masked, bool valid, int key0, int pos, float qs, float off,
                                          uint32_t (&p)[32]) {
  if (masked) {
#pragma unroll
    for (int i = 0; i < 64; ++i)
      if (!valid || key0 + i > pos) s[i] = -INFINITY;
  }
  // p = exp2(s * qs - m): packed fp32 pairs for the multiply-add and the sums (four chains), one
  // MUFU a value, a packed convert a pair
  const uint64_t qs2 = pack2(qs, qs), off2 = pack2(off, off);
  uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float x0, x1;
    unpack2(fma2(pack2(s[2 * i], s[2 * i + 1]), qs2, off2), x0, x1);
    const bool poly = POLY_EVERY > 0 && (i % (POLY_EVERY > 0 ? POLY_EVERY : 1)) == (POLY_EVERY > 0 ? POLY_EVERY : 1) - 1;
    const float p0 = poly ? poly_exp2(x0) : fast_exp2(x0), p1 = poly ? poly_exp2(x1) : fast_exp2(x1);
    acc[i & 3] = add2(acc[i & 3], pack2(p0, p1));
    if (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(p[i]) : "f"(p1), "f"(p0));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;\n" : "=r"(p[i]) : "f"(p1), "f"(p0));
  }
  float a0, a1;
  unpack2(add2(add2(acc[0], acc[1]), add2(acc[2], acc[3])), a0, a1);
  return a0 + a1;
}

// One work item as every role of the CTA sees it.
struct Item {
  int req, row0, q0, q_len, seq_len, ctx, kvh, hbase;
  int nblk0, nblk1;   // key blocks each query tile attends to (tile 1 may be empty)
  int kv_limit;       // keys the item reads
  int n;              // blocks the CTA walks: max of the two
  // by select, not by index: the item stays in registers
  __device__ __forceinline__ int nblk(int t) const { return t ? nblk1 : nblk0; }
};

// F16: the products' operands (Q, K, V, P) are f16, else bf16. FP8: the caches are fp8-e4m3 -- the
// producers convert them to f16 on their way into the ring, the query rows (bf16) are converted to f16
// as they are staged, so F16 is set; the output stays bf16 and carries v_scale, the scores carry k_scale.
template <int GP, bool F16, bool TRACE = false, bool FP8 = false>
__global__ void __launch_bounds__(threads_of(FP8), 1) prefill_tc_kernel(const Args a, const __grid_constant__ CUtensorMap kmap,
                                                                const __grid_constant__ CUtensorMap vmap,
                                                                const __grid_constant__ CUtensorMap qmap) {
  extern __shared__ uint8_t raw_smem[];
  unsigned long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};      // this thread's lap counters (TRACE builds)
  const long long t_begin = TRACE ? now() : 0;
  constexpr int T = ROWS / GP;                 // tokens of one query tile
  constexpr bool OUT_F16 = F16 && !FP8;
  static_assert(!FP8 || F16, "an fp8 cache is widened to f16");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t base = (smem_u32(raw_smem) + 1023u) & ~1023u;
  uint8_t* gen = raw_smem + (base - smem_u32(raw_smem));
  const uint32_t q_smem = base;                              // two query tiles
  const uint32_t ring = base + 2 * Q_BYTES;
  const uint32_t epi = ring + NSLOT * SLOT_BYTES;            // the epilogue's staging rows: 4 KB a softmax warp
  Bars* bars = reinterpret_cast<Bars*>(gen + 2 * Q_BYTES + NSLOT * SLOT_BYTES + EPI_BYTES);
  const uint32_t bars_u = epi + EPI_BYTES;
#define HKB_BAR(field) (bars_u + (uint32_t)offsetof(Bars, field))
  volatile int* abort = &bars->abort;

  // ---- the CTA's items: the grid is persistent (at most one CTA an SM); the (work item, head pass)
  // pairs, work-major -- the list is sorted by keys, so consecutive pairs cost the same -- are dealt out
  // in rounds of gridDim.x, every other round backwards, which evens the CTAs' sums out ----
  const int passes = a.group / GP;
  const int planes = a.num_kv_heads * passes;
  const int total = a.num_work * planes;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  // 0: no more rounds; 1: nothing of this round for this CTA (or an item without rows); 2: `it` is set
  auto item_at = [&](int round, Item& it) -> int {
    if ((long long)round * G >= total) return 0;
    const int idx = round * G + ((round & 1) ? G - 1 - cta : cta);
    if (idx >= total) return 1;
    const int w = idx / planes, plane = idx - w * planes;
    it.kvh = plane / passes;
    it.hbase = it.kvh * a.group + (plane % passes) * GP;
    it.req = __ldg(a.work + 2 * w); it.row0 = __ldg(a.work + 2 * w + 1);
    it.q0 = __ldg(a.q_start + it.req); it.q_len = __ldg(a.q_start + it.req + 1) - it.q0;
    it.seq_len = __ldg(a.seq_lens + it.req);
    it.ctx = it.seq_len - it.q_len;
    if (it.q_len <= 0 || it.row0 >= it.q_len || it.ctx < 0) return 1;
    const int lim0 = min(it.seq_len, it.ctx + min(it.row0 + T, it.q_len));
    const int lim1 = it.row0 + T < it.q_len ? min(it.seq_len, it.ctx + min(it.row0 + 2 * T, it.q_len)) : 0;
    it.nblk0 = (lim0 + KVB - 1) / KVB;
    it.nblk1 = (lim1 + KVB - 1) / KVB;
    it.kv_limit = min(it.seq_len, it.ctx + min(it.row0 + 2 * T, it.q_len));
    it.n = max(it.nblk0, it.nblk1);
    return 2;
  };

  // ---- set-up: barriers and TMEM ----
  if (threadIdx.x == 0) {
    for (int i = 0; i < NSLOT; ++i) { mbar_init(HKB_BAR(full) + 8 * i, FP8 && FP8_MAIN < 8 ? 2 : 1); mbar_init(HKB_BAR(empty) + 8 * i, 1); }   // (fp8 with a third producer: a slot is filled by two warps)
    for (int i = 0; i < 2; ++i) {
      mbar_init(HKB_BAR(s_full) + 8 * i, 1); mbar_init(HKB_BAR(p_full) + 8 * i, ROWS);
      mbar_init(HKB_BAR(o_done) + 8 * i, 1); mbar_init(HKB_BAR(q_full) + 8 * i, a.tma_q ? 1 : ROWS);
      mbar_init(HKB_BAR(q_empty) + 8 * i, 1); mbar_init(HKB_BAR(q_ready) + 8 * i, ROWS);
    }
    bars->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(HKB_BAR(tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  // Barrier phases run on across items. Every role counts for itself, and all count alike: `blocks[t]`
  // the key blocks of tile t so far (s_full, p_full, o_done complete once a block), `items[t]` the items
  // in which tile t had rows (q_full, q_empty complete once an item), `kcnt` / `vcnt` the K / V blocks
  // through the ring (block c of a kind sits in slot 2 (c % 2) + kind, on the slot's lap c / 2).
  bool ok = true;
  Item it;
  if (warp < SOFTMAX_WARPS) {
    // ================= softmax: thread = one query row of tile g =================
    const int g = warp >> 2, row = (warp & 3) * 32 + lane;
    // whether output rows can be written as 16-byte vectors (else as 4-byte words)
    const bool out16 = ((reinterpret_cast<uintptr_t>(a.out) | (uintptr_t)(a.out_stride_tok * 2) | (uintptr_t)(a.out_stride_head * 2)) & 15) == 0;
    if (TRACE) tr[7] = (unsigned long long)(now() - t_begin);   // set-up: barriers, TMEM, the CTA-wide barrier
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_addr + s_col(g);
    const float qs = a.scale * LOG2E * (FP8 ? __ldg(a.k_scale) : 1.f);
    const float out_scale = FP8 ? __ldg(a.v_scale) : 1.f;
    int blocks = 0, items = 0;
    Item nxt;
    int got_nxt = item_at(0, nxt);
    for (int round = 1; ok && got_nxt; ++round) {
      // the item after this one is looked up now: its three dependent loads are long done when it is needed
      it = nxt;
      const int got = got_nxt;
      got_nxt = item_at(round, nxt);
      if (got == 1 || it.nblk(g) == 0) continue;
      const int row0 = it.row0, q_len = it.q_len, q0 = it.q0, hbase = it.hbase;
      Lap<TRACE> lap_q;
      if (!a.tma_q) {
        // No tensor map for the queries: this tile's warps stage its rows themselves -- row r is head
        // r / T, token r % T of the tile -- once the products of the item before have read the old ones.
        if (items > 0) {
          ok = warp_wait<FP8>(HKB_BAR(q_empty) + 8 * g, (items - 1) & 1, abort, 9);
          if (!ok) break;
        }
        uint4 qv[16];
#pragma unroll
        for (int x16 = 0; x16 < 16; ++x16) {                      // all sixteen loads in flight, then the stores
          const int x = x16 * ROWS + (warp & 3) * 32 + lane, r = x >> 4, c = x & 15;
          const int tk = min(row0 + g * T + r % T, q_len - 1);  // rows past the request: any finite row will do, they are masked
          qv[x16] = ldg_stream16(a.q + (int64_t)(q0 + tk) * a.q_stride_tok + (int64_t)(hbase + r / T) * a.q_stride_head + c * 8);
        }
#pragma unroll
        for (int x16 = 0; x16 < 16; ++x16) {
          const int x = x16 * ROWS + (warp & 3) * 32 + lane, r = x >> 4, c = x & 15;
          const uint32_t dst = q_smem + g * Q_BYTES + (c >> 3) * HALF_BYTES_Q + r * 128 + (((c & 7) ^ (r & 7)) << 4);
          if (FP8) {   // bf16 query rows beside an f16 cache tile: to f16, clamped to its range
            uint32_t* w = reinterpret_cast<uint32_t*>(&qv[x16]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float lo = fminf(fmaxf(bf16lo(w[i]), -65504.f), 65504.f), hi = fminf(fmaxf(bf16hi(w[i]), -65504.f), 65504.f);
              asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(w[i]) : "f"(hi), "f"(lo));
            }
          }
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(dst), "r"(qv[x16].x), "r"(qv[x16].y), "r"(qv[x16].z), "r"(qv[x16].w) : "memory");
        }
        fence_async_smem();
        mbar_arrive(HKB_BAR(q_full) + 8 * g);
      } else if (FP8) {
        // The rows came by TMA as they are in memory, bf16, under the item before's tail; the products run
        // on f16 beside the widened cache: each thread converts the sixteen chunks it would have staged, in
        // place, and the MMA warp waits for all 128 threads (q_ready) instead of for the copy.
        ok = warp_wait<FP8>(HKB_BAR(q_full) + 8 * g, items & 1, abort, 8);
        if (!ok) break;
        uint4 qv[16];
#pragma unroll
        for (int x16 = 0; x16 < 16; ++x16) {
          const int x = x16 * ROWS + (warp & 3) * 32 + lane, r = x >> 4, c = x & 15;
          qv[x16] = lds128(q_smem + g * Q_BYTES + (c >> 3) * HALF_BYTES_Q + r * 128 + (((c & 7) ^ (r & 7)) << 4));
        }
#pragma unroll
        for (int x16 = 0; x16 < 16; ++x16) {
          const int x = x16 * ROWS + (warp & 3) * 32 + lane, r = x >> 4, c = x & 15;
          uint32_t* w = reinterpret_cast<uint32_t*>(&qv[x16]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = fminf(fmaxf(bf16lo(w[i]), -65504.f), 65504.f), hi = fminf(fmaxf(bf16hi(w[i]), -65504.f), 65504.f);
            asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(w[i]) : "f"(hi), "f"(lo));
          }
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(q_smem + g * Q_BYTES + (c >> 3) * HALF_BYTES_Q + r * 128 + (((c & 7) ^ (r & 7)) << 4)),
                       "r"(qv[x16].x), "r"(qv[x16].y), "r"(qv[x16].z), "r"(qv[x16].w) : "memory");
        }
        fence_async_smem();
        mbar_arrive(HKB_BAR(q_ready) + 8 * g);
      }
      ++items;
      lap_q(tr[6]);
      const int tok = row0 + g * T + row % T;
      const bool valid = tok < q_len;
      const int pos = it.ctx + tok;                           // the last key this row sees
      float m = -INFINITY, l = 0.f;
      const int nb = it.nblk(g);
      for (int j = 0; j < nb && ok; ++j) {
        Lap<TRACE> lap;
        ok = warp_wait<FP8>(HKB_BAR(s_full) + 8 * g, (blocks + j) & 1, abort, 1);
        if (!ok) break;
        lap(tr[0]);
        tc_fence_after();
        const int kv0 = j * KVB;
        const bool masked = !valid || kv0 + KVB - 1 > pos;     // the diagonal block, or a row past the request
        float s[64];
        // pass 1: the row maximum over both halves
        tmem_ld64(s_addr, s);
        float mx = half_max<F16>(s, masked, valid, kv0, pos);
        tmem_ld64(s_addr + 64, s);
        mx = fmaxf(mx, half_max<F16>(s, masked, valid, kv0 + 64, pos)) * qs;     // qs > 0
        lap(tr[1]);
        // lazy reference: it moves only when a block's maximum exceeds it by 2^8 (P <= 256 fits 16 bits)
        const bool need = mx > m + 8.f;
        const bool any_need = __any_sync(0xffffffffu, need);
        float alpha = 1.f;
        if (need) {
          alpha = fast_exp2(m - mx);                           // m = -inf the first time: 0
          m = mx;
        }
        const float off = (m == -INFINITY) ? 0.f : -m;
        // pass 2: the second half is still in registers; P of keys 64..127 goes to columns 32..63, which
        // held scores of the first half -- read again below before anything is written there
        uint32_t p_hi[32], p_lo[32];
        float sum = half_exp<F16>(s, false, valid, kv0 + 64, pos, qs, off, p_hi);
        tmem_ld64(s_addr, s);
        sum += half_exp<F16>(s, masked, valid, kv0, pos, qs, off, p_lo);
        l = l * alpha + sum;
        if (TRACE) asm volatile("" ::"r"(p_lo[0]), "r"(p_hi[31]), "f"(l));   // the math is done before the lap is taken
        lap(tr[2]);
        if (j > 0) {
          // the tile's previous product has landed: O may be touched, and stays untouched until P arrives
          ok = warp_wait<FP8>(HKB_BAR(o_done) + 8 * g, (blocks + j - 1) & 1, abort, 2);
          if (!ok) break;
          tc_fence_after();
          if (any_need) {
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
              float o[32];
              uint32_t w[32];
              tmem_ld32(lane_addr + o_col(g) + c0, o);
#pragma unroll
              for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(o[i] * alpha);
              tmem_st32(lane_addr + o_col(g) + c0, w);
            }
          }
        }
        lap(tr[3]);
        tmem_st32(s_addr, p_lo);                                // P over the first 64 columns of the scores
        tmem_st32(s_addr + 32, p_hi);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(HKB_BAR(p_full) + 8 * g);
        lap(tr[4]);
      }
      if (!ok) break;
      Lap<TRACE> lap_end;
      ok = warp_wait<FP8>(HKB_BAR(o_done) + 8 * g, (blocks + nb - 1) & 1, abort, 3);
      if (!ok) break;
      blocks += nb;
      tc_fence_after();
      const float inv = (l > 0.f ? 1.f / l : 0.f) * out_scale;
      // Each thread parks half of its output row (64 dims = 128 bytes; a quarter in the fp8 build; 16-byte
      // chunks XOR-ed by the row so that the 32 rows of a warp do not collide on banks) in the warp's staging rows, then the warp -- which owns exactly
      // these 32 rows -- writes them out 512 bytes an instruction; then the next part. The accumulator
      // is free for the next item as soon as its last part has been read: the first P of that item is
      // handed over after this, by these same threads.
      // (fp8 caches: half of the staging space belongs to the producers, so a quarter of a row at a time)
      constexpr int PASS_DIMS = FP8 ? 32 : 64, ROWE = PASS_DIMS * 2, CPRE = ROWE / 16;   // dims, bytes, 16-byte chunks of a staged row
      const uint32_t stage = epi + (uint32_t)warp * (32u * ROWE);
      const int wswz = CPRE == 8 ? (lane & 7) : ((lane >> 1) & 3);     // a 64-byte row: two rows share a 128-byte bank line
#pragma unroll 1
      for (int pass = 0; pass < D / PASS_DIMS; ++pass) {
#pragma unroll
        for (int c32 = 0; c32 < PASS_DIMS / 32; ++c32) {
          float o[32];
          tmem_ld32(lane_addr + o_col(g) + pass * PASS_DIMS + c32 * 32, o);
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (OUT_F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(w[i]) : "f"(o[2 * i + 1] * inv), "f"(o[2 * i] * inv));
            else asm("cvt.rn.bf16x2.f32 %0, %1, %2;\n" : "=r"(w[i]) : "f"(o[2 * i + 1] * inv), "f"(o[2 * i] * inv));
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = c32 * 4 + q4;                     // 16-byte chunk of the staged row
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(stage + lane * ROWE + ((chunk ^ wswz) << 4)),
                         "r"(w[4 * q4]), "r"(w[4 * q4 + 1]), "r"(w[4 * q4 + 2]), "r"(w[4 * q4 + 3]) : "memory");
          }
        }
        __syncwarp();
#pragma unroll 4
        for (int x = 0; x < CPRE; ++x) {
          const int rr = x * (32 / CPRE) + lane / CPRE, chunk = lane % CPRE;        // row of the warp, chunk of the staged row
          const int r_tile = (warp & 3) * 32 + rr;
          const int tk = row0 + g * T + r_tile % T;
          const int rswz = CPRE == 8 ? (rr & 7) : ((rr >> 1) & 3);
          const uint4 v = lds128(stage + rr * ROWE + ((chunk ^ rswz) << 4));
          if (tk < q_len) {
            __nv_bfloat16* dst = a.out + (int64_t)(q0 + tk) * a.out_stride_tok + (int64_t)(hbase + r_tile / T) * a.out_stride_head +
                                 pass * PASS_DIMS + chunk * 8;
            if (out16) *reinterpret_cast<uint4*>(dst) = v;
            else {
              uint32_t* d32 = reinterpret_cast<uint32_t*>(dst);
              d32[0] = v.x; d32[1] = v.y; d32[2] = v.z; d32[3] = v.w;
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      lap_end(tr[5]);
    }
    if (TRACE && row == 0)
      for (int i = 0; i < 8; ++i) a.trace[(size_t)cta * 32 + 8 * g + i] = tr[i];
  } else if (warp == MMA_WARP) {
    // ================= MMA issue: one thread; the whole warp keeps step at the barriers =================
    // (One warp for both tiles: a second issuing warp, one a tile, was measured -- 800 against 1000
    // TFLOP/s on a long prompt. A tcgen05.mma of 128 x 128 x 16 takes the tensor pipe ~85 clocks here
    // whoever issues it, and two threads' products interleave on the pipe without order.)
    constexpr uint32_t IDESC_S = instr_desc(F16, false, KVB), IDESC_PV = instr_desc(F16, true, D);
    int blocks0 = 0, blocks1 = 0, items0 = 0, items1 = 0, kcnt = 0, vcnt = 0;   // scalars: the two tiles' loops are unrolled
    auto slot_of = [](int kind, int c) { return 2 * (c & 1) + kind; };
    // S_t = Q_t K^T for the K block in ring slot `slot`: eight products (two 64-dim halves x four 16-dim
    // steps) into the tile's score columns; the tile's query rows are free after the item's last one
    // Every matrix descriptor the kernel will ever use, once: the query tiles and the four ring slots do
    // not move. The issuing thread then has nothing to compute between two products -- building the
    // 64-bit descriptors in the loop, a dozen dependent instructions a product on ONE thread, was what
    // an "86-clock tcgen05.mma" mostly consisted of.
    uint64_t qd0[8], qd1[8], kd0[8], kd1[8], vd0[8], vd1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int h = i >> 2, ks = i & 3;          // S: two 64-dim halves x four 16-dim steps (32 bytes inside the 128-byte row)
      qd0[i] = smem_desc(q_smem + h * HALF_BYTES_Q + ks * 32, 16);
      qd1[i] = smem_desc(q_smem + Q_BYTES + h * HALF_BYTES_Q + ks * 32, 16);
      kd0[i] = smem_desc(ring + h * HALF_BYTES_KV + ks * 32, 16);                      // K blocks sit in slots 0 and 2
      kd1[i] = smem_desc(ring + 2 * SLOT_BYTES + h * HALF_BYTES_KV + ks * 32, 16);
      vd0[i] = smem_desc(ring + SLOT_BYTES + i * 16 * 128, HALF_BYTES_KV);             // V blocks in slots 1 and 3: 16 tokens a step
      vd1[i] = smem_desc(ring + 3 * SLOT_BYTES + i * 16 * 128, HALF_BYTES_KV);
    }
    // S_t = Q_t K^T for the K block in ring slot `slot`: eight products into the tile's score columns; the
    // tile's query rows are free after the item's last one
    auto scores = [&](int t, int slot, bool last) {
      const bool hi = slot >= 2;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        umma_ss(tmem + s_col(t), t ? qd1[i] : qd0[i], hi ? kd1[i] : kd0[i], IDESC_S, i ? 1u : 0u);
      tc_commit(HKB_BAR(s_full) + 8 * t);
      if (last) tc_commit(HKB_BAR(q_empty) + 8 * t);
    };
    auto wait_block = [&](int kind, int c, int code) {     // block c of K (kind 0) or V (kind 1) has landed
      ok = warp_wait<FP8>(HKB_BAR(full) + 8 * slot_of(kind, c), (c >> 1) & 1, abort, code);
      tc_fence_after();
    };
    Item nxt;
    int got_nxt = item_at(0, nxt);
    for (int round = 1; ok && got_nxt; ++round) {
      it = nxt;
      const int got = got_nxt;
      got_nxt = item_at(round, nxt);
      if (got == 1) continue;
      const int n = it.n;
      Lap<TRACE> lap;
      // the tiles' query rows are in place
      const uint32_t q_bar = FP8 && a.tma_q ? HKB_BAR(q_ready) : HKB_BAR(q_full);   // fp8: the rows as converted in place
      if (it.nblk0 > 0) ok = warp_wait<FP8>(q_bar, items0 & 1, abort, 8);
      if (ok && it.nblk1 > 0) ok = warp_wait<FP8>(q_bar + 8, items1 & 1, abort, 8);
      if (!ok) break;
      lap(tr[0]);
      wait_block(0, kcnt, 4);
      if (!ok) break;
      lap(tr[1]);
      if (lane == 0) {
        if (it.nblk0 > 0) scores(0, slot_of(0, kcnt), it.nblk0 == 1);
        if (it.nblk1 > 0) scores(1, slot_of(0, kcnt), it.nblk1 == 1);
        // the first K block's slot is handed back at once
        tc_commit(HKB_BAR(empty) + 8 * slot_of(0, kcnt));
      }
      __syncwarp();
      lap(tr[2]);
      for (int j = 0; j < n && ok; ++j) {
        wait_block(1, vcnt + j, 5);                    // V_j
        if (!ok) break;
        lap(tr[3]);
        if (j + 1 < n) wait_block(0, kcnt + j + 1, 4);     // K_{j+1}
        if (!ok) break;
        lap(tr[1]);
        const bool v_hi = slot_of(1, vcnt + j) == 3;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!ok || j >= it.nblk(t)) continue;
          // P of the block; for an item's first block this also says the tile's warps have read the
          // accumulator of the item before out of TMEM (they arrive here after their epilogue)
          ok = warp_wait<FP8>(HKB_BAR(p_full) + 8 * t, ((t ? blocks1 : blocks0) + j) & 1, abort, 6);
          if (!ok) continue;
          lap(tr[t ? 6 : 4]);
          tc_fence_after();
          if (lane == 0) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)           // 16 tokens a step: 8 TMEM columns of P, 16 rows of V
              umma_ts(tmem + o_col(t), tmem + s_col(t) + ks * 8, v_hi ? vd1[ks] : vd0[ks], IDESC_PV, (j | ks) ? 1u : 0u);
            tc_commit(HKB_BAR(o_done) + 8 * t);
            // the block's last P V product has been issued: the V slot goes back now, before the scores that
            // follow (a commit covers every product issued so far; the scores do not read V, and waiting for
            // them too handed the slot back ~700 clocks later, with the MMA warp then waiting for the next V)
            if (t == 1 || j >= it.nblk1) tc_commit(HKB_BAR(empty) + 8 * slot_of(1, vcnt + j));
          }
          if (TRACE) { __syncwarp(); lap(tr[5]); }
          // the tile's next scores go over the P just consumed: the tensor pipe runs products in the order issued
          if (lane == 0 && j + 1 < it.nblk(t)) scores(t, slot_of(0, kcnt + j + 1), j + 2 == it.nblk(t));
          __syncwarp();
          lap(tr[TRACE ? 7 : 5]);
        }
        if (ok && lane == 0) {
          if (j + 1 < n) tc_commit(HKB_BAR(empty) + 8 * slot_of(0, kcnt + j + 1));   // K_{j+1}
        }
        __syncwarp();
      }
      kcnt += n; vcnt += n;
      blocks0 += it.nblk0; blocks1 += it.nblk1;
      items0 += it.nblk0 > 0; items1 += it.nblk1 > 0;
    }
    if (TRACE && lane == 0)
      for (int i = 0; i < 8; ++i) a.trace[(size_t)cta * 32 + 16 + i] = tr[i];
  } else {
    // ================= producers: warp K_WARP brings the K blocks, warp V_WARP the V blocks =================
    const int which = (warp - K_WARP) & 1;   // 0: K, 1: V
    const int part = (warp - K_WARP) >> 1;   // fp8 caches only: 1 = the third producer, which helps with both kinds
    const int64_t sb = which ? a.v_stride_block : a.k_stride_block, st = which ? a.v_stride_token : a.k_stride_token;
    const void* map = which ? static_cast<const void*>(&vmap) : static_cast<const void*>(&kmap);
    const int p_tok = which ? a.v_pos[0] : a.k_pos[0], p_head = which ? a.v_pos[1] : a.k_pos[1];   // the block id takes the third
    int cnt = 0, items0 = 0, items1 = 0;
    Item nxt;
    int got_nxt = item_at(0, nxt);
    for (int round = 1; ok && got_nxt; ++round) {
      it = nxt;
      const int got = got_nxt;
      got_nxt = item_at(round, nxt);
      if (got == 1) continue;
      const int n = it.n, kvh = it.kvh, kv_limit = it.kv_limit;
      const uint8_t* src = (which ? a.v + (int64_t)kvh * a.v_stride_head : a.k + (int64_t)kvh * a.k_stride_head);
      const int* table_row = a.block_table + (int64_t)it.req * a.table_stride;
      // page ids of a block's eight 16-token tiles, fetched one block ahead of their use (raw: the clamp
      // waits for the load, so it is applied where the id is used)
      auto page_ids = [&](int kv0, int& id, int& sub) {
        id = 0; sub = 0;
        if (lane < 8 && kv0 < kv_limit) {
          const int tile = kv0 / TILE_TOKENS + lane;
          const int page = min(tile / a.tiles_per_page, a.max_pages - 1);
          id = __ldg(table_row + page);
          sub = tile % a.tiles_per_page;
        }
      };
      int next_id, next_sub;
      page_ids(0, next_id, next_sub);
      if (a.tma_q && which == 1 && part == 0) {
        // the V warp has nothing to do until the first scores exist: it brings the query tiles, one copy a
        // (tile, head, 64-dim half): T token rows of 128 bytes, landing where row h * T + token belongs --
        // once the products of the item before have read the old ones
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!ok || it.nblk(t) == 0) continue;
          const int before = t ? items1 : items0;
          if (before > 0) {
            ok = warp_wait(HKB_BAR(q_empty) + 8 * t, (before - 1) & 1, abort, 9);
            if (!ok) continue;
          }
          if (t) ++items1; else ++items0;
          if (lane == 0) mbar_arrive_expect_tx(HKB_BAR(q_full) + 8 * t, Q_BYTES);
          __syncwarp();
          for (int x = lane; x < 2 * GP; x += 32) {
            const int h = x >> 1, half = x & 1;
            const int tok = it.q0 + it.row0 + t * T, head = it.hbase + h;
            tma_load_3d(q_smem + t * Q_BYTES + half * HALF_BYTES_Q + h * T * 128, &qmap, HKB_BAR(q_full) + 8 * t, half * 64,
                        a.q_pos[0] == 1 ? tok : head, a.q_pos[0] == 1 ? head : tok);
          }
        }
        if (!ok) break;
      }
      if constexpr (FP8) {
        // the item's tiles as one stream: tile x = block x / 8, 16-token tile x % 8
        // Of a block's eight 16-token tiles the kind's own warp takes the first MAIN, a third producer (if MAIN < 8)
        // the rest of both kinds: its stream a block is K tiles MAIN.., then V tiles MAIN.. . A slot is complete
        // when every warp that fills it has arrived.
        constexpr int TPB = KVB / TILE_TOKENS, MAIN = FP8_MAIN, REST = TPB - MAIN > 0 ? TPB - MAIN : 1;
        const int per_blk = part ? 2 * REST : MAIN;        // this warp's tiles a block
        const uint32_t stg = epi + EPI_BYTES / 2 + (uint32_t)(warp - K_WARP) * (FP8_STAGE_TILES * 2048u);
        // A lane owns one 16-byte chunk (16 dims) of four rows of every tile. 16-byte accesses are served a
        // quarter warp at a time, so eight consecutive lanes must fall on eight different 16-byte bank groups:
        // a quarter warp takes the four chunks of one 64-dim half of two adjacent rows -- the 128-byte swizzle
        // of the slot puts an even and an odd row's chunks on complementary groups, and the staging rows swap
        // their halves on odd rows for the same reason.
        const int gq = lane & 3, rp = (lane >> 2) & 1, hq = (lane >> 3) & 1, rq = lane >> 4;
        const int g = hq * 4 + gq;                         // the row's 16-byte fp8 chunk: dims 16 g .. + 15
        const int row0 = 2 * rq + rp;                      // rows row0 + 4 y of the tile, y = 0..3
        const int c0 = 2 * gq;                             // the first of the two 16-byte f16 chunks its 16 dims become
        const uint32_t lane_stg = (uint32_t)row0 * 128 + (uint32_t)((g ^ (rp * 4)) << 4);
        const uint32_t lane_dst = (uint32_t)hq * HALF_BYTES_KV + (uint32_t)row0 * 128;
        // r & 7 of rows row0, row0 + 4, ...: row0 or row0 + 4, so the two chunks' places inside a row take two values each
        const uint32_t xa0 = (uint32_t)((c0 ^ row0) << 4), xa1 = (uint32_t)(((c0 + 1) ^ row0) << 4);
        const uint32_t xb0 = (uint32_t)((c0 ^ (row0 + 4)) << 4), xb1 = (uint32_t)(((c0 + 1) ^ (row0 + 4)) << 4);
        const int tiles = n * per_blk;                     // this warp's tiles of the item, as one stream
        // tile x of the stream: which kind (0 K, 1 V) and which tile of the block
        auto kind_of = [&](int r) { return part ? r / REST : which; };
        auto tile_of = [&](int r) { return part ? MAIN + r % REST : r; };
        int id_cur = next_id, sub_cur = next_sub, blk_cur = 0;    // lanes 0..7: the page ids of block blk_cur, and of the one after
        page_ids(KVB, next_id, next_sub);
        auto issue = [&](int x) {
          const int jb = x / per_blk, r = x % per_blk, kind = kind_of(r), t = tile_of(r);
          if (jb != blk_cur) { id_cur = next_id; sub_cur = next_sub; blk_cur = jb; page_ids((jb + 1) * KVB, next_id, next_sub); }
          const int id = min(max(__shfl_sync(0xffffffffu, id_cur, t), 0), a.num_blocks - 1), sub = __shfl_sync(0xffffffffu, sub_cur, t);
          const int64_t sbk = kind ? a.v_stride_block : a.k_stride_block, stk = kind ? a.v_stride_token : a.k_stride_token;
          const uint8_t* tp = (kind ? a.v + (int64_t)kvh * a.v_stride_head : a.k + (int64_t)kvh * a.k_stride_head) +
                              (int64_t)id * sbk + (int64_t)(sub * TILE_TOKENS + row0) * stk + g * 16;
          const uint32_t buf = stg + (uint32_t)(x % FP8_STAGE_TILES) * 2048u + lane_stg;
          const int tok0 = jb * KVB + t * TILE_TOKENS;
#pragma unroll
          for (int y = 0; y < 4; ++y) {
            if (tok0 + 4 * y + row0 < kv_limit) cp_async16(buf + y * 512, tp + (int64_t)(4 * y) * stk);
            else asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(buf + y * 512), "r"(0u) : "memory");
          }
        };
        for (int x = 0; x < FP8_STAGE_TILES - 1; ++x) { if (x < tiles) issue(x); cp_async_commit(); }
        uint32_t slot_addr = 0, bar = 0;
#pragma unroll 1
        for (int x = 0; x < tiles && ok; ++x) {
          Lap<TRACE> tick;
          if (x + FP8_STAGE_TILES - 1 < tiles) issue(x + FP8_STAGE_TILES - 1);
          cp_async_commit();                               // a group a tile (empty ones at the end): tile x is the oldest one pending
          tick(tr[1]);
          cp_async_wait<FP8_STAGE_TILES - 1>();
          tick(tr[2]);
          const int r = x % per_blk, kind = kind_of(r), t = tile_of(r);
          const bool first = part ? r % REST == 0 : r == 0, last = part ? r % REST == REST - 1 : r == MAIN - 1;
          if (first) {                                     // the first tile this warp puts into the kind's slot of this block
            const int slot = 2 * (cnt & 1) + kind, lap = cnt >> 1;
            slot_addr = ring + slot * SLOT_BYTES; bar = HKB_BAR(full) + 8 * slot;
            tick(tr[1]);
            if (lap > 0) ok = warp_wait(HKB_BAR(empty) + 8 * slot, (lap - 1) & 1, abort, 7);
            if (!ok) break;
            tick(tr[0]);
          }
          const uint32_t buf = stg + (uint32_t)(x % FP8_STAGE_TILES) * 2048u + lane_stg;
          const uint32_t dst = slot_addr + lane_dst + (uint32_t)(t * TILE_TOKENS) * 128;
          uint4 v4[4];      // the four rows' loads first (they keep their order among themselves, as do the stores)
#pragma unroll
          for (int y = 0; y < 4; ++y) v4[y] = lds128(buf + y * 512);
#pragma unroll
          for (int y = 0; y < 4; ++y) {
            const uint32_t w[4] = {v4[y].x, v4[y].y, v4[y].z, v4[y].w};
            uint32_t h[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) { h[2 * i] = fp8x2_to_f16x2(w[i]); h[2 * i + 1] = fp8x2_to_f16x2(w[i] >> 16); }
            const uint32_t row = dst + (uint32_t)(4 * y) * 128;
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(row + ((y & 1) ? xb0 : xa0)), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(row + ((y & 1) ? xb1 : xa1)), "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]) : "memory");
          }
          if (last) {      // this warp's share of the slot is in place
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar);
          }
          if (r == per_blk - 1) ++cnt;
          tick(tr[3]);
        }
      } else
      for (int j = 0; j < n && ok; ++j, ++cnt) {
        const int slot = 2 * (cnt & 1) + which, lap = cnt >> 1;
        const uint32_t slot_addr = ring + slot * SLOT_BYTES, bar = HKB_BAR(full) + 8 * slot;
        int id = next_id, sub = next_sub;
        page_ids((j + 1) * KVB, next_id, next_sub);
        const int kv0 = j * KVB;
        Lap<TRACE> tick;
        if (lap > 0) ok = warp_wait(HKB_BAR(empty) + 8 * slot, (lap - 1) & 1, abort, 7);
        if (!ok) break;
        tick(tr[0]);
        if (a.tma && kv0 + KVB <= kv_limit) {
          // all 128 rows are keys: 8 pages x 2 halves = 16 tile copies, one a lane
          const int t = (lane >> 1) & 7;
          id = __shfl_sync(0xffffffffu, id, t);
          sub = __shfl_sync(0xffffffffu, sub, t);
          if (lane == 0) mbar_arrive_expect_tx(bar, SLOT_BYTES);
          __syncwarp();
          if (lane < 16) {
            // coordinates 1..3 of the map are the token, the kv head and the block in the order the cache's
            // strides put them (selects, not an indexed array: that would live in local memory)
            id = min(max(id, 0), a.num_blocks - 1);
            const int tok = sub * TILE_TOKENS;
            const int c1 = p_tok == 1 ? tok : p_head == 1 ? kvh : id;
            const int c2 = p_tok == 2 ? tok : p_head == 2 ? kvh : id;
            const int c3 = p_tok == 3 ? tok : p_head == 3 ? kvh : id;
            tma_load_4d(slot_addr + (lane & 1) * HALF_BYTES_KV + t * TILE_TOKENS * 128, map, bar, (lane & 1) * 64, c1, c2, c3);
          }
          tick(tr[1]);
        } else {
          // the block with the last keys (rows past them are zero-filled), or no tensor map: cp.async
          fill_half(a, slot_addr, src, sb, st, table_row, kv0, kv_limit, lane);
          fill_half(a, slot_addr, src, sb, st, table_row, kv0 + 64, kv_limit, lane);
          cp_async_commit();
          tick(tr[1]);
          cp_async_wait<0>();
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar);
        }
        tick(tr[2]);
      }
    }
    cp_async_wait<0>();
    if (TRACE && lane == 0 && part == 0)
      for (int i = 0; i < (FP8 && which == 0 ? 4 : 3); ++i) a.trace[(size_t)cta * 32 + 24 + 4 * which + i] = tr[i];   // (fp8, K: + the widening)
  }

  // ---- wind-down ----
  tc_fence_before();
  __syncthreads();
  if (TRACE && threadIdx.x == 0) a.trace[(size_t)cta * 32 + 31] = (unsigned long long)(now() - t_begin);
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
#undef HKB_BAR
}

}  // namespace tc
}  // namespace hkb
