// Paged prefill: causal attention of a request's new tokens (a chunk, or a whole prompt)
// over its paged KV cache -- the cached prefix plus the chunk itself, already written.
//
// What it computes is hk-dsl's paged prefill (python/hk/ops/paged_prefill.py:1-27, 59-620):
// `ctx` tokens of the sequence are in the cache from before, the `q_len` new ones attend to
// all ctx + q_len causally, query row i sitting at position ctx + i; a query tile belongs to
// one request and its rows end where the request's do; the grid is a work list built on the
// host, one entry a (request, query tile), so a ragged batch launches once.
//
// Schedule (sm_100a, legacy tensor path): one CTA a (work item, kv head [x head chunk]) of 4
// warps, two CTAs an SM; a warp owns two units, a unit being a 16-row query tile of ONE query
// head, so every K and V fragment it reads from shared memory feeds two mma tiles; the 8 units
// of a CTA are the GP heads of the GQA group times 8 / GP consecutive 16-token tiles, so one
// staged K/V block serves the whole group. Query rows sit in shared memory and are re-read as A
// fragments each block (the registers go to the two 16 x head_dim accumulators). K/V blocks of 64 tokens (4 pages of
// 16) come through the page table into a 2-stage cp.async ring, XOR-swizzled for ldmatrix (fp8
// tiles land in a raw ring and the warp that fetched a tile widens it to bf16, exactly);
// S = Q K^T and O += P V are mma.sync.m16n8k16 bf16 with P reused from the S accumulators;
// online softmax in exp2 with a lazy reference. This is a dense contraction whose roofline
// is the tensor pipe; mma.sync is the baseline form of it, not the tcgen05 form.
#include "hkb_walk_mma.cuh"
#include "hkb_prefill_tc.cuh"

#include <cstdlib>
#include <cstring>

extern thread_local int hkb_tls_cuda_error;

namespace hkb {

struct PrefillArgs {
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
  const int* work;   // (request, first query row of the tile inside the request) pairs
  int num_q_heads, num_kv_heads, group, tiles_per_page;
  float scale;
  const float* k_scale;   // fp8 caches: per-tensor dequantisation scales (device pointers), else NULL
  const float* v_scale;
};

template <int D, int GP, bool FP8, bool F16 = false>
struct Prefill {
  static_assert(!(FP8 && F16), "an fp8 cache goes with bf16 activations");
  // head_dim 256: a unit's 16 x 256 accumulator is 128 registers, so a warp owns one unit and a CTA has 8 warps
  static constexpr int WARPS = D == 256 ? 8 : 4;
  static constexpr int UNITS = 8;                     // (16-row query tile, query head) pairs a CTA: two a warp
  static constexpr int UPW = UNITS / WARPS;
  static constexpr int TOK_TILES = UNITS / GP;        // 16-token query tiles a CTA
  static constexpr int BT = 16 * TOK_TILES;           // query tokens a CTA
  static constexpr int KV_TILES = 4;                  // 16-token KV tiles a stage: one a warp to fill
  static constexpr int KVB = 16 * KV_TILES;
  static constexpr int NST = 2;
  static constexpr int ROWB = D * 2;                 // a row as the mma reads it (bf16)
  static constexpr int ROWC = FP8 ? D : D * 2;        // a row as it sits in the cache
  static constexpr int KD = D / 16;
  using Loader = TileLoader<ROWC>;
  static constexpr int TILE_BYTES = TILE_TOKENS * ROWB;
  static constexpr int RAW_TILE_BYTES = Loader::TILE_BYTES;
  static constexpr int Q_BYTES = UNITS * TILE_BYTES;  // the CTA's query rows, read back as A fragments every block
  static constexpr int STAGE_BYTES = KV_TILES * 2 * TILE_BYTES;
  static constexpr int RAW_STAGE_BYTES = FP8 ? KV_TILES * 2 * RAW_TILE_BYTES : 0;   // fp8 tiles land here first
  // one landing buffer is enough: a warp widens the tiles it fetched and only then fetches the next block's
  // into the same place (two would not fit beside head_dim 256's query rows and stages)
  static constexpr int SMEM_BYTES = Q_BYTES + NST * STAGE_BYTES + RAW_STAGE_BYTES;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory of one SM");
  static constexpr float RESCALE_LOG2 = 8.f;

  // A warp fills the K and the V tile of its 16 tokens of a stage; rows at or past `kv_limit` are
  // zero-filled instead of read, so nothing past the keys this CTA may attend to enters shared memory.
  __device__ static __forceinline__ void fill(const PrefillArgs& a, const Loader& ld, uint32_t stage, int kv0,
                                              int kv_limit, const int* table_row, int warp, int lane) {
    const int t = WARPS == 4 ? warp : warp >> 1;     // 4 warps: K and V of tile `warp`; 8 warps: one of the two
    const int tok0 = kv0 + 16 * t;
    const int valid = min(16, kv_limit - tok0);      // rows of this tile that hold attendable keys
    int id = 0, sub = 0;
    if (valid > 0) {
      const int tile = tok0 / TILE_TOKENS;
      const int page = min(tile / a.tiles_per_page, a.max_pages - 1);
      id = min(max(__ldg(table_row + page), 0), a.num_blocks - 1);
      sub = tile % a.tiles_per_page;
    }
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      if (WARPS == 8 && which != (warp & 1)) continue;
      const uint32_t dst = stage + (t * 2 + which) * (FP8 ? RAW_TILE_BYTES : TILE_BYTES);
      const int64_t sb = which ? ld.vsb : ld.ksb, st = which ? ld.vst : ld.kst;
      const uint8_t* p = (which ? ld.vbase : ld.kbase) + (int64_t)id * sb + (int64_t)(sub * TILE_TOKENS) * st;
#pragma unroll
      for (int it = 0; it < Loader::ITERS; ++it) {
        const int x = it * 32 + lane;
        const int r = x / Loader::CPR, c = x % Loader::CPR;
        const uint32_t d = dst + tile_off<ROWC>(r, c);
        if (r < valid) cp_async16(d, p + (int64_t)r * st + c * 16);
        else asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(d), "r"(0u) : "memory");
      }
    }
  }

  __device__ static __forceinline__ void run(const PrefillArgs& a, uint8_t* smem) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int passes = a.group / GP;
    const int kvh = blockIdx.y / passes;
    const int hbase = kvh * a.group + (blockIdx.y % passes) * GP;
    // a work item covers 2 * BT query rows (what the tensor-memory kernel takes in one CTA): two CTAs here
    const int item = blockIdx.x >> 1;
    const int req = __ldg(a.work + 2 * item), row0 = __ldg(a.work + 2 * item + 1) + (blockIdx.x & 1) * BT;
    const int q0 = __ldg(a.q_start + req), q1 = __ldg(a.q_start + req + 1);
    const int q_len = q1 - q0;
    const int seq_len = __ldg(a.seq_lens + req);
    const int ctx = seq_len - q_len;
    if (q_len <= 0 || row0 >= q_len || ctx < 0) return;
    const int rows_cta = min(BT, q_len - row0);                 // query rows of this request the CTA covers
    const int kv_limit = min(seq_len, ctx + row0 + rows_cta);   // keys any of them may attend to
    const int n_blocks = (kv_limit + KVB - 1) / KVB;

    // The warp's two units: unit u is query head u % GP of the CTA's heads and 16-token tile u / GP.
    // Thread rows inside a unit: tokens wrow0 + {lane/4, lane/4 + 8}.
    int hq[UPW], wrow0[UPW], posA[UPW], posB[UPW], limit[UPW];
    bool live[UPW];
#pragma unroll
    for (int i = 0; i < UPW; ++i) {
      const int u = warp * UPW + i;
      hq[i] = hbase + u % GP;
      wrow0[i] = row0 + 16 * (u / GP);
      posA[i] = ctx + wrow0[i] + (lane >> 2);
      posB[i] = posA[i] + 8;
      live[i] = wrow0[i] < q_len;                               // a unit whose 16 rows are all past the request idles
      limit[i] = min(kv_limit, ctx + min(wrow0[i] + 16, q_len));   // keys past every row of the unit need no work
    }

    const uint32_t qsm = smem_u32(smem);
    const uint32_t ring = qsm + Q_BYTES;
    const uint32_t raw = ring + NST * STAGE_BYTES;   // fp8 only: where the copies land before they are widened
    const uint32_t land = FP8 ? raw : ring;
    constexpr int LAND_BYTES = FP8 ? 0 : STAGE_BYTES;   // fp8: the one landing buffer

    // Stage the warp's query rows (rows past the request: zeros) in the swizzled layout ldmatrix reads.
    const bool q16 = ((reinterpret_cast<uintptr_t>(a.q) | (uintptr_t)(a.q_stride_tok * 2) | (uintptr_t)(a.q_stride_head * 2)) & 15) == 0;
#pragma unroll
    for (int i = 0; i < UPW; ++i) {
      const uint32_t qt = qsm + (warp * UPW + i) * TILE_BYTES;
      for (int x = lane; x < 16 * (ROWB / 16); x += 32) {
        const int r = x / (ROWB / 16), c = x % (ROWB / 16);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (wrow0[i] + r < q_len) {
          const __nv_bfloat16* src = a.q + (int64_t)(q0 + wrow0[i] + r) * a.q_stride_tok + (int64_t)hq[i] * a.q_stride_head + c * 8;
          if (q16) v = __ldg(reinterpret_cast<const uint4*>(src));
          else {
            const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src);
            v = make_uint4(__ldg(s32), __ldg(s32 + 1), __ldg(s32 + 2), __ldg(s32 + 3));
          }
        }
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(qt + tile_off<ROWB>(r, c)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
      }
    }

    float o[UPW][2 * KD][4];
    float m[UPW][2], l[UPW][2];
#pragma unroll
    for (int i = 0; i < UPW; ++i) {
#pragma unroll
      for (int nt = 0; nt < 2 * KD; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][nt][e] = 0.f;
      m[i][0] = m[i][1] = -INFINITY;
      l[i][0] = l[i][1] = 0.f;
    }
    float qs = a.scale * LOG2E;
    float vs = 1.f;
    if (FP8) { qs *= __ldg(a.k_scale); vs = __ldg(a.v_scale); }

    Loader ld;
    ld.kbase = a.k + (int64_t)kvh * a.k_stride_head;
    ld.vbase = a.v + (int64_t)kvh * a.v_stride_head;
    ld.ksb = a.k_stride_block; ld.kst = a.k_stride_token;
    ld.vsb = a.v_stride_block; ld.vst = a.v_stride_token;
    ld.tiles_per_page = a.tiles_per_page; ld.num_blocks = a.num_blocks;
    const int* table_row = a.block_table + (int64_t)req * a.table_stride;

    // Where this lane's ldmatrix rows sit inside a 16-token tile: A (query rows, row-major), B for S
    // (key rows), B for O (value rows, read transposed). The offset of 16-dim chunk kc is the chunk-0
    // offset XOR (kc << 5): the swizzle XORs the 16-byte chunk index with the row, and 2 kc only
    // touches bits the lane's own part of the index leaves alone -- one register a kind, not KD.
    const uint32_t qoff0 = tile_off<ROWB>(lane & 15, lane >> 4);
    const uint32_t koff0 = tile_off<ROWB>(((lane >> 4) & 1) * 8 + (lane & 7), (lane >> 3) & 1);
    const uint32_t voff0 = tile_off<ROWB>(((lane >> 3) & 1) * 8 + (lane & 7), lane >> 4);

    fill(a, ld, land, 0, kv_limit, table_row, warp, lane);
    cp_async_commit();
    for (int b = 0; b < n_blocks; ++b) {
      cp_async_wait<0>();
      if (FP8) {
        // the warp that fetched a tile widens it to bf16 (exact) into block b's stage. Every warp
        // is past its work on block b-2, the stage's previous tenant (the barrier of iteration b-1).
        __syncwarp();
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          if (WARPS == 8 && which != (warp & 1)) continue;          // eight warps: each fetched one tile (fill)
          const int tile = WARPS == 8 ? warp : warp * 2 + which;
          WalkMMA<D, true, 1, 4, 4>::widen(raw + tile * RAW_TILE_BYTES, ring + (b & 1) * STAGE_BYTES + tile * TILE_BYTES, lane);
        }
        __syncwarp();   // the landing tiles are read: the next block's copies may overwrite them
      }
      __syncthreads();   // block b has landed for every warp (and, the first time, the query rows); block b-1's stage is free
      if (b + 1 < n_blocks) fill(a, ld, land + ((b + 1) & 1) * LAND_BYTES, (b + 1) * KVB, kv_limit, table_row, warp, lane);
      cp_async_commit();
      const uint32_t stage = ring + (b & 1) * STAGE_BYTES;
      const int kv0 = b * KVB;
      bool on[UPW];
      bool any = false;
#pragma unroll
      for (int i = 0; i < UPW; ++i) { on[i] = live[i] && kv0 < limit[i]; any |= on[i]; }
      if (!any) continue;

      // S = Q K^T for the block's 64 keys and both units: every K fragment feeds two query tiles,
      // 16 independent accumulator tiles. Keys past kv_limit are zero rows in the stage; keys past
      // a row's own position are masked below.
      float sc[UPW][2 * KV_TILES][4];
#pragma unroll
      for (int i = 0; i < UPW; ++i)
#pragma unroll
        for (int nt = 0; nt < 2 * KV_TILES; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) sc[i][nt][e] = 0.f;
#pragma unroll
      for (int kc = 0; kc < KD; ++kc) {
        uint32_t qa[UPW][4];
#pragma unroll
        for (int i = 0; i < UPW; ++i) ldmatrix_x4(qa[i], qsm + (warp * UPW + i) * TILE_BYTES + (qoff0 ^ (kc << 5)));
#pragma unroll
        for (int t = 0; t < KV_TILES; ++t) {
          uint32_t kb[4];
          ldmatrix_x4(kb, stage + (t * 2) * TILE_BYTES + (koff0 ^ (kc << 5)));
          const uint32_t b0[2] = {kb[0], kb[1]}, b1[2] = {kb[2], kb[3]};
#pragma unroll
          for (int i = 0; i < UPW; ++i) {
            mma16<F16>(sc[i][2 * t], qa[i], b0);
            mma16<F16>(sc[i][2 * t + 1], qa[i], b1);
          }
        }
      }
      uint32_t pa[UPW][KV_TILES][4];
#pragma unroll
      for (int i = 0; i < UPW; ++i) {
        // causal mask (key j is seen by the row at position p iff j <= p), row maxima. Scores stay
        // unscaled: the exponent below is exp2(s * qs - m) in one fma, m kept in scaled units.
        if (!on[i] || kv0 + KVB - 1 > ctx + wrow0[i]) {   // an idle unit, or a block that reaches past the unit's first row
#pragma unroll
          for (int nt = 0; nt < 2 * KV_TILES; ++nt) {
            const int j = kv0 + nt * 8 + 2 * (lane & 3);
            if (!on[i] || j > posA[i]) sc[i][nt][0] = -INFINITY;
            if (!on[i] || j + 1 > posA[i]) sc[i][nt][1] = -INFINITY;
            if (!on[i] || j > posB[i]) sc[i][nt][2] = -INFINITY;
            if (!on[i] || j + 1 > posB[i]) sc[i][nt][3] = -INFINITY;
          }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2 * KV_TILES; ++nt) {
          mx[0] = fmaxf(mx[0], fmaxf(sc[i][nt][0], sc[i][nt][1]));
          mx[1] = fmaxf(mx[1], fmaxf(sc[i][nt][2], sc[i][nt][3]));
        }
#pragma unroll
        for (int x = 1; x < 4; x <<= 1) {
          mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], x));
          mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], x));
        }
        mx[0] *= qs; mx[1] *= qs;            // qs > 0: the maximum of the scaled scores
        // lazy reference: rescale only when a block's maximum exceeds it by 2^RESCALE_LOG2
        if (__any_sync(0xffffffffu, mx[0] > m[i][0] + RESCALE_LOG2 || mx[1] > m[i][1] + RESCALE_LOG2)) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float m_new = fmaxf(m[i][c], mx[c]);
            const float alpha = fast_exp2(m[i][c] - ((m_new == -INFINITY) ? 0.f : m_new));
            l[i][c] *= alpha;
#pragma unroll
            for (int nt = 0; nt < 2 * KD; ++nt) { o[i][nt][2 * c] *= alpha; o[i][nt][2 * c + 1] *= alpha; }
            m[i][c] = m_new;
          }
        }
        const float sa = (m[i][0] == -INFINITY) ? 0.f : -m[i][0], sb = (m[i][1] == -INFINITY) ? 0.f : -m[i][1];
#pragma unroll
        for (int t = 0; t < KV_TILES; ++t) {
          const float p00 = fast_exp2(fmaf(sc[i][2 * t][0], qs, sa)), p01 = fast_exp2(fmaf(sc[i][2 * t][1], qs, sa));
          const float p02 = fast_exp2(fmaf(sc[i][2 * t][2], qs, sb)), p03 = fast_exp2(fmaf(sc[i][2 * t][3], qs, sb));
          const float p10 = fast_exp2(fmaf(sc[i][2 * t + 1][0], qs, sa)), p11 = fast_exp2(fmaf(sc[i][2 * t + 1][1], qs, sa));
          const float p12 = fast_exp2(fmaf(sc[i][2 * t + 1][2], qs, sb)), p13 = fast_exp2(fmaf(sc[i][2 * t + 1][3], qs, sb));
          l[i][0] += (p00 + p01) + (p10 + p11);
          l[i][1] += (p02 + p03) + (p12 + p13);
          pa[i][t][0] = pack16x2<F16>(p00, p01);   // (row A, keys 0-7 pair)
          pa[i][t][1] = pack16x2<F16>(p02, p03);   // (row B, keys 0-7 pair)
          pa[i][t][2] = pack16x2<F16>(p10, p11);   // (row A, keys 8-15 pair)
          pa[i][t][3] = pack16x2<F16>(p12, p13);   // (row B, keys 8-15 pair)
        }
      }
      // O += P V: B = V^T read transposed from the row-major V tiles; every V fragment feeds both units
#pragma unroll
      for (int t = 0; t < KV_TILES; ++t) {
#pragma unroll
        for (int dt = 0; dt < KD; ++dt) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, stage + (t * 2 + 1) * TILE_BYTES + (voff0 ^ (dt << 5)));
          const uint32_t b0[2] = {vb[0], vb[1]}, b1[2] = {vb[2], vb[3]};
#pragma unroll
          for (int i = 0; i < UPW; ++i) {
            mma16<F16>(o[i][2 * dt], pa[i][t], b0);
            mma16<F16>(o[i][2 * dt + 1], pa[i][t], b1);
          }
        }
      }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < UPW; ++i) {
      if (!live[i]) continue;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int x = 1; x < 4; x <<= 1) l[i][c] += __shfl_xor_sync(0xffffffffu, l[i][c], x);
      const int rA = wrow0[i] + (lane >> 2), rB = rA + 8;
      const bool vA = rA < q_len, vB = rB < q_len;
      const float iA = l[i][0] > 0.f ? vs / l[i][0] : 0.f, iB = l[i][1] > 0.f ? vs / l[i][1] : 0.f;
      __nv_bfloat16* oA = a.out + (int64_t)(q0 + rA) * a.out_stride_tok + (int64_t)hq[i] * a.out_stride_head;
      __nv_bfloat16* oB = a.out + (int64_t)(q0 + rB) * a.out_stride_tok + (int64_t)hq[i] * a.out_stride_head;
#pragma unroll
      for (int nt = 0; nt < 2 * KD; ++nt) {
        const int d = nt * 8 + 2 * (lane & 3);
        if (vA) *reinterpret_cast<uint32_t*>(oA + d) = pack16x2<F16>(o[i][nt][0] * iA, o[i][nt][1] * iA);
        if (vB) *reinterpret_cast<uint32_t*>(oB + d) = pack16x2<F16>(o[i][nt][2] * iB, o[i][nt][3] * iB);
      }
    }
  }
};

template <int D, int GP, bool FP8, bool F16>
__global__ void __launch_bounds__(D == 256 ? 256 : 128, D == 256 ? 1 : 2) prefill_kernel(const PrefillArgs a) {
  extern __shared__ __align__(128) uint8_t hkb_smem[];
  Prefill<D, GP, FP8, F16>::run(a, hkb_smem);
}

template <int D, int GP, bool FP8, bool F16>
static int launch_prefill(const PrefillArgs& a, int num_work, cudaStream_t st) {
  static bool armed[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  constexpr int smem = Prefill<D, GP, FP8, F16>::SMEM_BYTES;
  if (e == cudaSuccess && dev >= 0 && dev < 64 && !armed[dev]) {
    e = cudaFuncSetAttribute(prefill_kernel<D, GP, FP8, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) armed[dev] = true;
  }
  if (e == cudaSuccess) {
    dim3 grid(2 * num_work, a.num_kv_heads * (a.group / GP));
    prefill_kernel<D, GP, FP8, F16><<<grid, Prefill<D, GP, FP8, F16>::WARPS * 32, smem, st>>>(a);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}

template <int D, bool FP8, bool F16 = false>
static int dispatch_prefill(const PrefillArgs& a, int num_work, cudaStream_t st) {
  // heads of the GQA group a CTA serves: the largest of 8, 4, 2, 1 that divides the group
  if (a.group % 8 == 0) return launch_prefill<D, 8, FP8, F16>(a, num_work, st);
  if (a.group % 4 == 0) return launch_prefill<D, 4, FP8, F16>(a, num_work, st);
  if (a.group % 2 == 0) return launch_prefill<D, 2, FP8, F16>(a, num_work, st);
  return launch_prefill<D, 1, FP8, F16>(a, num_work, st);
}

// ---- the tensor-memory form (head_dim 128, 16-bit caches) ----

// cuTensorMapEncodeTiled, fetched through the runtime so that the library links against no driver stub.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn tensor_map_encoder() {
  static const EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// A 4-D tensor map of one paged cache (16-bit elements): head_dim innermost, then the token, kv-head
// and block axes in order of increasing stride (whatever the layout: head-major pages, token-major
// pages, K and V side by side). A copy is a box of 64 dims x 16 tokens of one head of one block, laid
// down with the 128-byte swizzle. `pos` receives the coordinate index of (token, head, block). False
// if the driver has no encoder or refuses the layout: the kernel then gathers with cp.async.
static bool make_cache_map(CUtensorMap* m, const hkb_cache_t& c, int block_size, int num_kv_heads, int pos[3]) {
  const EncodeTiledFn encode = tensor_map_encoder();
  if (!encode) return false;
  struct Axis { cuuint64_t size, stride; int role; } ax[3] = {
      {(cuuint64_t)block_size, (cuuint64_t)c.stride_token * 2, 0},
      {(cuuint64_t)num_kv_heads, (cuuint64_t)c.stride_head * 2, 1},
      {(cuuint64_t)c.num_blocks, (cuuint64_t)c.stride_block * 2, 2}};
  for (int i = 0; i < 3; ++i)
    if (c.stride_token < 0 || c.stride_head < 0 || c.stride_block < 0 || ax[i].stride % 16 || ax[i].stride >= (1ull << 40) ||
        ax[i].size == 0 || ax[i].size > (1ull << 32))
      return false;
  for (int i = 0; i < 3; ++i)          // three entries: a hand-rolled sort by stride
    for (int j = i + 1; j < 3; ++j)
      if (ax[j].stride < ax[i].stride) { const Axis t = ax[i]; ax[i] = ax[j]; ax[j] = t; }
  cuuint64_t dims[4] = {128, ax[0].size, ax[1].size, ax[2].size};
  cuuint64_t strides[3] = {ax[0].stride, ax[1].stride, ax[2].stride};
  cuuint32_t box[4] = {64, 1, 1, 1}, elem[4] = {1, 1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    pos[ax[i].role] = i + 1;
    if (ax[i].role == 0) box[i + 1] = TILE_TOKENS;
  }
  return encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, c.ptr, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A 3-D tensor map of the queries (tokens, heads, 128 dims, 16-bit), the token and head axes in order of
// increasing stride; a copy is a box of 64 dims x `tile_tokens` tokens of one head. `pos`: the
// coordinate index of (token, head).
static bool make_query_map(CUtensorMap* m, const void* q, int64_t stride_tok, int64_t stride_head, int64_t num_tokens,
                           int num_q_heads, int tile_tokens, int pos[2]) {
  const EncodeTiledFn encode = tensor_map_encoder();
  if (!encode || stride_tok <= 0 || stride_head <= 0 || num_tokens <= 0) return false;
  struct Axis { cuuint64_t size, stride; int role; } ax[2] = {{(cuuint64_t)num_tokens, (cuuint64_t)stride_tok * 2, 0},
                                                              {(cuuint64_t)num_q_heads, (cuuint64_t)stride_head * 2, 1}};
  if (ax[1].stride < ax[0].stride) { const Axis t = ax[0]; ax[0] = ax[1]; ax[1] = t; }
  for (int i = 0; i < 2; ++i)
    if (ax[i].stride % 16 || ax[i].stride >= (1ull << 40) || ax[i].size > (1ull << 32)) return false;
  cuuint64_t dims[3] = {128, ax[0].size, ax[1].size};
  cuuint64_t strides[2] = {ax[0].stride, ax[1].stride};
  cuuint32_t box[3] = {64, 1, 1}, elem[3] = {1, 1, 1};
  for (int i = 0; i < 2; ++i) {
    pos[ax[i].role] = i + 1;
    if (ax[i].role == 0) box[i + 1] = (cuuint32_t)tile_tokens;
  }
  return encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int GP, bool F16, bool TRACE = false, bool FP8 = false>
static int launch_prefill_tc(const tc::Args& a, const CUtensorMap& kmap, const CUtensorMap& vmap, const CUtensorMap& qmap,
                             int num_work, cudaStream_t st) {
  static bool armed[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess && dev >= 0 && dev < 64 && !armed[dev]) {
    e = cudaFuncSetAttribute(tc::prefill_tc_kernel<GP, F16, TRACE, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
    if (e == cudaSuccess) armed[dev] = true;
  }
  if (e == cudaSuccess) {
    // a persistent grid: one CTA an SM at most, each walks its share of the (work item, head pass) pairs
    const long long total = (long long)num_work * a.num_kv_heads * (a.group / GP);
    int sms = hkb_sm_count(-1);
    if (sms <= 0) sms = 148;
    dim3 grid((unsigned)(total < sms ? total : sms));
    tc::prefill_tc_kernel<GP, F16, TRACE, FP8><<<grid, tc::threads_of(FP8), tc::SMEM_BYTES, st>>>(a, kmap, vmap, qmap);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}

template <bool F16, bool FP8 = false>
static int dispatch_prefill_tc(const tc::Args& a, const CUtensorMap& kmap, const CUtensorMap& vmap, const CUtensorMap& qmap,
                               int num_work, cudaStream_t st) {
  if (a.group % 8 == 0) return launch_prefill_tc<8, F16, false, FP8>(a, kmap, vmap, qmap, num_work, st);
  if (a.group % 4 == 0) return launch_prefill_tc<4, F16, false, FP8>(a, kmap, vmap, qmap, num_work, st);
  if (a.group % 2 == 0) return launch_prefill_tc<2, F16, false, FP8>(a, kmap, vmap, qmap, num_work, st);
  return launch_prefill_tc<1, F16, false, FP8>(a, kmap, vmap, qmap, num_work, st);
}

}  // namespace hkb

// 256 query rows (tokens x the heads of the GQA group a CTA serves) a work item, whichever kernel runs.
extern "C" int hkb_prefill_tile_rows(int num_q_heads, int num_kv_heads) {
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return 0;
  const int g = num_q_heads / num_kv_heads;
  const int gp = g % 8 == 0 ? 8 : g % 4 == 0 ? 4 : g % 2 == 0 ? 2 : 1;
  return 256 / gp;
}

extern "C" int hkb_prefill_uses_tcgen05(int head_dim, int kv_dtype) {
  const char* v = std::getenv("HKB_PREFILL_MMA_SYNC");
  if (v && v[0] == '1') return 0;
  return head_dim == 128 && (kv_dtype == HKB_KV_BF16 || kv_dtype == HKB_KV_F16 || kv_dtype == HKB_KV_FP8_E4M3) ? 1 : 0;
}

extern "C" int hkb_prefill_tc_error(int clear) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, hkb::tc::g_error, sizeof(int)) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
  if (clear && code) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(hkb::tc::g_error, &zero, sizeof(int)) != cudaSuccess) (void)cudaGetLastError();
  }
  return code;
}

namespace { thread_local unsigned long long* g_trace_for_next_call = nullptr; }

extern "C" int hkb_paged_prefill(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                                 const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                                 hkb_cache_t kc, hkb_cache_t vc,
                                 const int32_t* block_table, int64_t table_stride, int max_pages,
                                 const int32_t* seq_lens, const int32_t* q_start,
                                 const int32_t* work, int num_work, int num_tokens,
                                 int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                                 float scale, int kv_dtype, const float* k_scale, const float* v_scale,
                                 void* stream) {
  using namespace hkb;
  if (num_work < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_tokens < 0) return HKB_ERR_SIZE;
  if (num_work == 0) return HKB_OK;
  if (!out || !q || !kc.ptr || !vc.ptr || !block_table || !seq_lens || !q_start || !work) return HKB_ERR_NULL;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return HKB_ERR_HEAD_DIM;
  if (block_size <= 0 || block_size % TILE_TOKENS) return HKB_ERR_BLOCK_SIZE;
  if (num_q_heads % num_kv_heads || num_q_heads / num_kv_heads > HKB_MAX_GROUP) return HKB_ERR_GROUP;
  if (kv_dtype != HKB_KV_BF16 && kv_dtype != HKB_KV_FP8_E4M3 && kv_dtype != HKB_KV_F16) return HKB_ERR_DTYPE;
  const bool fp8 = kv_dtype == HKB_KV_FP8_E4M3;
  if (fp8 && (!k_scale || !v_scale)) return HKB_ERR_SCALE;
  const int es = fp8 ? 1 : 2;
  if (max_pages < 1 || kc.num_blocks < 1 || vc.num_blocks < 1) return HKB_ERR_SIZE;
  const int group = num_q_heads / num_kv_heads;
  if ((int64_t)num_kv_heads * group > 65535) return HKB_ERR_SIZE;
  const int64_t kv_strides = kc.stride_block | kc.stride_token | kc.stride_head | vc.stride_block | vc.stride_token | vc.stride_head;
  if ((kv_strides * es) % 16) return HKB_ERR_STRIDE;
  if ((q_stride_tok | q_stride_head | out_stride_tok | out_stride_head) % 2) return HKB_ERR_STRIDE;
  if (((uintptr_t)kc.ptr | (uintptr_t)vc.ptr) % 16 || ((uintptr_t)q | (uintptr_t)out) % 4) return HKB_ERR_ALIGN;

  PrefillArgs a;
  a.out = (__nv_bfloat16*)out; a.out_stride_tok = out_stride_tok; a.out_stride_head = out_stride_head;
  a.q = (const __nv_bfloat16*)q; a.q_stride_tok = q_stride_tok; a.q_stride_head = q_stride_head;
  a.k = (const uint8_t*)kc.ptr; a.v = (const uint8_t*)vc.ptr;
  a.k_stride_block = kc.stride_block * es; a.k_stride_token = kc.stride_token * es; a.k_stride_head = kc.stride_head * es;
  a.v_stride_block = vc.stride_block * es; a.v_stride_token = vc.stride_token * es; a.v_stride_head = vc.stride_head * es;
  const int64_t nb = kc.num_blocks < vc.num_blocks ? kc.num_blocks : vc.num_blocks;
  a.num_blocks = nb > 0x7fffffff ? 0x7fffffff : (int)nb;
  a.block_table = block_table; a.table_stride = table_stride; a.max_pages = max_pages;
  a.seq_lens = seq_lens; a.q_start = q_start; a.work = work;
  a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads; a.group = group;
  a.tiles_per_page = block_size / TILE_TOKENS;
  a.scale = scale;
  a.k_scale = fp8 ? k_scale : nullptr;
  a.v_scale = fp8 ? v_scale : nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  // head_dim 128 on a 16-bit cache: the tcgen05 / TMEM kernel, when every query row can be read in
  // 16-byte chunks (it stages them with vector loads); the mma.sync kernel otherwise
  if (hkb_prefill_uses_tcgen05(head_dim, kv_dtype) && (uintptr_t)q % 16 == 0 && (q_stride_tok | q_stride_head) % 8 == 0) {
    tc::Args t;
    t.out = a.out; t.out_stride_tok = a.out_stride_tok; t.out_stride_head = a.out_stride_head;
    t.q = a.q; t.q_stride_tok = a.q_stride_tok; t.q_stride_head = a.q_stride_head;
    t.k = a.k; t.v = a.v;
    t.k_stride_block = a.k_stride_block; t.k_stride_token = a.k_stride_token; t.k_stride_head = a.k_stride_head;
    t.v_stride_block = a.v_stride_block; t.v_stride_token = a.v_stride_token; t.v_stride_head = a.v_stride_head;
    t.num_blocks = a.num_blocks; t.block_table = a.block_table; t.table_stride = a.table_stride; t.max_pages = a.max_pages;
    t.seq_lens = a.seq_lens; t.q_start = a.q_start; t.work = a.work; t.num_work = num_work;
    t.num_q_heads = a.num_q_heads; t.num_kv_heads = a.num_kv_heads; t.group = a.group; t.tiles_per_page = a.tiles_per_page;
    t.scale = a.scale;
    t.k_scale = a.k_scale; t.v_scale = a.v_scale;
    t.trace = g_trace_for_next_call;
    // K and V blocks come by TMA where a tensor map describes the cache (HKB_PREFILL_NO_TMA=1: the cp.async gather, the comparison arm)
    alignas(64) CUtensorMap kmap, vmap, qmap;
    const char* no_tma = std::getenv("HKB_PREFILL_NO_TMA");
    const int gp = group % 8 == 0 ? 8 : group % 4 == 0 ? 4 : group % 2 == 0 ? 2 : 1;
    // a query tile that runs past the tensor's last token reads zeros there (the map knows num_tokens);
    // rows past a request's own tokens belong to the next request and are masked
    const int64_t q_tokens = num_tokens;
    // (an fp8 cache is widened by the producers on its way in: no tile copies for K and V; the query tiles still come by TMA)
    const bool tma_ok = !(no_tma && no_tma[0] == '1');
    t.tma_q = tma_ok && make_query_map(&qmap, q, q_stride_tok, q_stride_head, q_tokens, num_q_heads, 128 / gp, t.q_pos);
    t.tma = t.tma_q && !fp8 && make_cache_map(&kmap, kc, block_size, num_kv_heads, t.k_pos) &&
            make_cache_map(&vmap, vc, block_size, num_kv_heads, t.v_pos);
    if (!t.tma) {
      memset(&kmap, 0, sizeof(kmap)); memset(&vmap, 0, sizeof(vmap));
      for (int i = 0; i < 3; ++i) t.k_pos[i] = t.v_pos[i] = i + 1;
      if (!fp8) t.tma_q = 0;      // 16-bit caches: all three by TMA, or none (the comparison arm)
    }
    if (!t.tma_q) {
      memset(&qmap, 0, sizeof(qmap));
      t.q_pos[0] = 1; t.q_pos[1] = 2;
    }
    if (t.trace) {   // the traced build: the headline shape only (a bf16 or an fp8 cache, a GQA group of 4)
      if (kv_dtype == HKB_KV_F16 || group % 4 || group % 8 == 0) return HKB_ERR_UNSUPPORTED;
      return fp8 ? launch_prefill_tc<4, true, true, true>(t, kmap, vmap, qmap, num_work, st)
                 : launch_prefill_tc<4, false, true>(t, kmap, vmap, qmap, num_work, st);
    }
    if (fp8) return dispatch_prefill_tc<true, true>(t, kmap, vmap, qmap, num_work, st);
    return kv_dtype == HKB_KV_F16 ? dispatch_prefill_tc<true>(t, kmap, vmap, qmap, num_work, st)
                                  : dispatch_prefill_tc<false>(t, kmap, vmap, qmap, num_work, st);
  }
  if (fp8) {
    if (head_dim == 256) return dispatch_prefill<256, true>(a, num_work, st);
    return head_dim == 128 ? dispatch_prefill<128, true>(a, num_work, st) : dispatch_prefill<64, true>(a, num_work, st);
  }
  if (kv_dtype == HKB_KV_F16) {
    if (head_dim == 256) return dispatch_prefill<256, false, true>(a, num_work, st);
    return head_dim == 128 ? dispatch_prefill<128, false, true>(a, num_work, st) : dispatch_prefill<64, false, true>(a, num_work, st);
  }
  if (head_dim == 256) return dispatch_prefill<256, false>(a, num_work, st);
  return head_dim == 128 ? dispatch_prefill<128, false>(a, num_work, st) : dispatch_prefill<64, false>(a, num_work, st);
}

// hkb_paged_prefill on the traced build of the tensor-memory kernel: every CTA (work item x kv head,
// CTA index = kv-head index * num_work + work index) leaves 32 cycle counters in `trace` -- where
// the softmax warps, the MMA warp and the producers spent their clocks. Measurement only.
extern "C" int hkb_paged_prefill_trace(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                                       const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                                       hkb_cache_t kc, hkb_cache_t vc,
                                       const int32_t* block_table, int64_t table_stride, int max_pages,
                                       const int32_t* seq_lens, const int32_t* q_start,
                                       const int32_t* work, int num_work, int num_tokens,
                                       int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                                       float scale, int kv_dtype, const float* k_scale, const float* v_scale,
                                       unsigned long long* trace, void* stream) {
  if (!trace) return HKB_ERR_NULL;
  if (!hkb_prefill_uses_tcgen05(head_dim, kv_dtype)) return HKB_ERR_UNSUPPORTED;
  g_trace_for_next_call = trace;
  const int rc = hkb_paged_prefill(out, out_stride_tok, out_stride_head, q, q_stride_tok, q_stride_head, kc, vc, block_table,
                                   table_stride, max_pages, seq_lens, q_start, work, num_work, num_tokens, num_q_heads,
                                   num_kv_heads, head_dim, block_size, scale, kv_dtype, k_scale, v_scale, stream);
  g_trace_for_next_call = nullptr;
  return rc;
}
