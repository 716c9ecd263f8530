// The decode walk on CUDA cores, for GQA groups below 8 (up to 4 query heads a CTA
// pass): one CTA per (sequence, kv head [x head chunk], kv split).
//
// What it computes is hk-dsl's fused walk (python/hk/ops/paged.py:544-662): scores
// scaled by scale*log2(e), tail rows past seq_len masked, online softmax in exp2,
// O += P V, then either the answer (one split) or a normalised partial and its lse.
//
// How it is laid out for B200:
//   * every warp walks its own contiguous share of the split's 16-token tiles through
//     its own ring of NST shared-memory stages filled by 16-byte cp.async copies
//     (K tile then V tile a stage), so WARPS * (NST-1) tiles are in flight a CTA and
//     no CTA-wide barrier sits in the loop;
//   * inside a warp, 8 lanes share a token and split head_dim between them, 4 tokens
//     a step, 4 steps a tile. Each 8-lane group is its own online-softmax stream
//     (its own m, l and partial O for the tokens it saw), so the only cross-lane
//     traffic in the loop is the 3-step butterfly that completes the dot products;
//   * the WARPS*4 streams of a CTA are folded once at the end through shared memory.
#pragma once

#include "hkb_decode.cuh"

namespace hkb {

template <int D, bool FP8, int GH, int WARPS, int NST>
struct WalkCC {
  static constexpr int ES = FP8 ? 1 : 2;
  static constexpr int ROWB = D * ES;
  static constexpr int CPR = ROWB / 16;
  static constexpr int NP = CPR / 8;    // 16-byte pieces of a row a lane owns
  static constexpr int EPP = 16 / ES;   // elements a piece
  static constexpr int DPL = NP * EPP;  // head_dim elements a lane owns (= D / 8)
  using Loader = TileLoader<ROWB>;
  static constexpr int STAGE_BYTES = 2 * Loader::TILE_BYTES;
  static constexpr int STREAMS = WARPS * 4;
  static constexpr int PIPE_BYTES = WARPS * NST * STAGE_BYTES;
  static constexpr int FOLD_BYTES = STREAMS * GH * (D + 2) * 4;
  static constexpr int SMEM_BYTES = PIPE_BYTES > FOLD_BYTES ? PIPE_BYTES : FOLD_BYTES;
  static_assert(NP >= 1, "a row must be at least 128 bytes");

  // head_dim index of element e of piece p for lane-in-group j
  __device__ static __forceinline__ int dim_of(int j, int p, int e) { return (j + 8 * p) * EPP + e; }

  // One 16-byte piece -> EPP floats as EPP/2 packed pairs (element 2i in the low half).
  __device__ static __forceinline__ void unpack_piece(const uint4& x, uint64_t* f2) {
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
    if (!FP8) {
#pragma unroll
      for (int i = 0; i < 4; ++i) f2[i] = pack2(bf16lo(w[i]), bf16hi(w[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = e4m3x2_to_float2((uint16_t)(w[i] & 0xffffu));
        const float2 b = e4m3x2_to_float2((uint16_t)(w[i] >> 16));
        f2[2 * i] = pack2(a.x, a.y);
        f2[2 * i + 1] = pack2(b.x, b.y);
      }
    }
  }

  template <bool LAST>
  __device__ static __forceinline__ void tile(uint32_t stage, int tok0, int seq_len, int g, int j,
                                              const uint64_t (&q2)[GH][DPL / 2], float (&m)[GH], float (&l)[GH],
                                              uint64_t (&o2)[GH][DPL / 2]) {
    float s[4][GH];
    // scores of this lane's 4 tokens over its DPL dims: packed FMAs over (even, odd) dims
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 4 + g;
      uint64_t k2[DPL / 2];
#pragma unroll
      for (int p = 0; p < NP; ++p) unpack_piece(lds128(stage + tile_off<ROWB>(r, j + 8 * p)), k2 + p * (EPP / 2));
#pragma unroll
      for (int h = 0; h < GH; ++h) {
        uint64_t acc = 0ull;  // (+0.f, +0.f)
#pragma unroll
        for (int e = 0; e < DPL / 2; ++e) acc = fma2(k2[e], q2[h][e], acc);
        float a0, a1;
        unpack2(acc, a0, a1);
        s[i][h] = a0 + a1;
      }
    }
    // complete the dot products over the 8 lanes of the group
#pragma unroll
    for (int x = 1; x < 8; x <<= 1)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int h = 0; h < GH; ++h) s[i][h] += __shfl_xor_sync(0xffffffffu, s[i][h], x);

    bool live[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      live[i] = !LAST || (tok0 + i * 4 + g < seq_len);
      if (LAST && !live[i])
#pragma unroll
        for (int h = 0; h < GH; ++h) s[i][h] = -INFINITY;
    }
    // online softmax of this stream, head by head
#pragma unroll
    for (int h = 0; h < GH; ++h) {
      const float mx = fmaxf(fmaxf(s[0][h], s[1][h]), fmaxf(s[2][h], s[3][h]));
      const float m_new = fmaxf(m[h], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // nothing seen yet: keep exp2 finite
      if (m_new != m[h]) {
        const float alpha = fast_exp2(m[h] - m_use);
        l[h] *= alpha;
        const uint64_t a2 = pack2(alpha, alpha);
#pragma unroll
        for (int e = 0; e < DPL / 2; ++e) o2[h][e] = mul2(o2[h][e], a2);
        m[h] = m_new;
      }
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) { s[i][h] = fast_exp2(s[i][h] - m_use); sum += s[i][h]; }
      l[h] += sum;
    }
    // O += P V
    const uint32_t vst = stage + Loader::TILE_BYTES;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 4 + g;
      uint64_t v2[DPL / 2];
#pragma unroll
      for (int p = 0; p < NP; ++p) unpack_piece(lds128(vst + tile_off<ROWB>(r, j + 8 * p)), v2 + p * (EPP / 2));
      if (LAST && !live[i]) continue;  // rows past the end may hold anything, NaN included
#pragma unroll
      for (int h = 0; h < GH; ++h) {
        const uint64_t p2 = pack2(s[i][h], s[i][h]);
#pragma unroll
        for (int e = 0; e < DPL / 2; ++e) o2[h][e] = fma2(p2, v2[e], o2[h][e]);
      }
    }
  }

  __device__ static __forceinline__ void run(const DecodeArgs& a, uint8_t* smem) {
    const int split = blockIdx.x, seq = blockIdx.z;
    const int chunks = (a.group + GH - 1) / GH;
    const int kvh = blockIdx.y / chunks;
    const int h0 = (blockIdx.y % chunks) * GH;          // first head of this pass inside the group
    const int nh = min(GH, a.group - h0);
    const int hq0 = kvh * a.group + h0;                 // its query head index
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 3, j = lane & 7;

    int row = seq;
    if (a.q_start) {
      row = __ldg(a.q_start + seq);
      if (__ldg(a.q_start + seq + 1) <= row) return;    // no query: write nothing
    }
    const int seq_len = max(__ldg(a.seq_lens + seq), 0);
    const int n_tiles = (seq_len + TILE_TOKENS - 1) / TILE_TOKENS;
    int lo, hi;
    split_range(n_tiles, a.num_splits, split, lo, hi);
    const bool partial = a.num_splits > 1;
    float* po = partial ? a.part_out + ((int64_t)(seq * a.num_splits + split) * a.num_q_heads + hq0) * D : nullptr;
    float* pl = partial ? a.part_lse + (int64_t)(seq * a.num_splits + split) * a.num_q_heads + hq0 : nullptr;

    if (lo >= hi) {  // nothing to read: an empty split, or a padded request
      if (partial) {
        if (threadIdx.x < nh) pl[threadIdx.x] = -INFINITY;
      } else {
        for (int x = threadIdx.x; x < nh * D; x += WARPS * 32)
          a.out[(int64_t)row * a.out_stride_tok + (int64_t)(hq0 + x / D) * a.out_stride_head + x % D] =
              __float2bfloat16(0.f);
      }
      return;
    }

    // this warp's contiguous share of the split
    const int per_w = (hi - lo + WARPS - 1) / WARPS;
    const int t_lo = min(hi, lo + warp * per_w);
    const int t_hi = min(hi, t_lo + per_w);
    const int n = t_hi - t_lo;

    float qs = a.scale * LOG2E;
    float vs = 1.f;
    if (FP8) { qs *= __ldg(a.k_scale); vs = __ldg(a.v_scale); }

    uint64_t q2[GH][DPL / 2], o2[GH][DPL / 2];
    float m[GH], l[GH];
#pragma unroll
    for (int h = 0; h < GH; ++h) {
      m[h] = -INFINITY; l[h] = 0.f;
      const __nv_bfloat16* qp = a.q + (int64_t)row * a.q_stride_tok + (int64_t)(hq0 + h) * a.q_stride_head;
#pragma unroll
      for (int p = 0; p < NP; ++p)
#pragma unroll
        for (int e = 0; e < EPP; e += 8) {
          uint4 x = make_uint4(0, 0, 0, 0);
          if (h < nh) x = __ldg(reinterpret_cast<const uint4*>(qp + dim_of(j, p, e)));
          const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) q2[h][(p * EPP + e) / 2 + i] = pack2(bf16lo(w[i]) * qs, bf16hi(w[i]) * qs);
        }
#pragma unroll
      for (int e = 0; e < DPL / 2; ++e) o2[h][e] = 0ull;
    }

    Loader ld;
    ld.kbase = a.k + (int64_t)kvh * a.k_stride_head;
    ld.vbase = a.v + (int64_t)kvh * a.v_stride_head;
    ld.ksb = a.k_stride_block; ld.kst = a.k_stride_token;
    ld.vsb = a.v_stride_block; ld.vst = a.v_stride_token;
    ld.tiles_per_page = a.tiles_per_page; ld.num_blocks = a.num_blocks;
    PageIds ids;
    ids.row = a.block_table + (int64_t)seq * a.table_stride;
    ids.max_pages = a.max_pages; ids.tiles_per_page = a.tiles_per_page; ids.t_hi = t_hi;
    ids.init(t_lo, lane);

    const uint32_t ring = smem_u32(smem) + warp * (NST * STAGE_BYTES);
#pragma unroll
    for (int k = 0; k < NST - 1; ++k) {
      if (k < n) ld.issue(ring + k * STAGE_BYTES, t_lo + k, ids.get(t_lo + k, lane), lane);
      cp_async_commit();
    }
    for (int k = 0; k < n; ++k) {
      cp_async_wait<NST - 2>();
      __syncwarp();
      const int kn = k + NST - 1;
      if (kn < n) ld.issue(ring + (kn % NST) * STAGE_BYTES, t_lo + kn, ids.get(t_lo + kn, lane), lane);
      cp_async_commit();
      const uint32_t stage = ring + (k % NST) * STAGE_BYTES;
      const int t = t_lo + k;
      if (t == n_tiles - 1) tile<true>(stage, t * TILE_TOKENS, seq_len, g, j, q2, m, l, o2);
      else tile<false>(stage, t * TILE_TOKENS, seq_len, g, j, q2, m, l, o2);
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its ring: the fold reuses the memory

    // fold the CTA's streams
    float* fo = reinterpret_cast<float*>(smem);            // [STREAMS][GH][D]
    float* fml = fo + STREAMS * GH * D;                    // [STREAMS][GH][2]
    const int stream = warp * 4 + g;
#pragma unroll
    for (int h = 0; h < GH; ++h) {
#pragma unroll
      for (int p = 0; p < NP; ++p)
#pragma unroll
        for (int e = 0; e < EPP; e += 2) {
          float x0, x1;
          unpack2(o2[h][(p * EPP + e) / 2], x0, x1);
          *reinterpret_cast<float2*>(&fo[(stream * GH + h) * D + dim_of(j, p, e)]) = make_float2(x0, x1);
        }
      if (j == 0) { fml[(stream * GH + h) * 2] = m[h]; fml[(stream * GH + h) * 2 + 1] = l[h]; }
    }
    __syncthreads();
    for (int x = threadIdx.x; x < nh * D; x += WARPS * 32) {
      const int h = x / D, d = x % D;
      float mm = -INFINITY;
#pragma unroll
      for (int sidx = 0; sidx < STREAMS; ++sidx) mm = fmaxf(mm, fml[(sidx * GH + h) * 2]);
      float num = 0.f, den = 0.f;
      if (mm != -INFINITY) {
#pragma unroll
        for (int sidx = 0; sidx < STREAMS; ++sidx) {
          const float w = fast_exp2(fml[(sidx * GH + h) * 2] - mm);  // 0 for a stream that saw nothing
          num = fmaf(w, fo[(sidx * GH + h) * D + d], num);
          den = fmaf(w, fml[(sidx * GH + h) * 2 + 1], den);
        }
      }
      const float val = den > 0.f ? num / den * vs : 0.f;
      if (partial) {
        po[h * D + d] = val;
        if (d == 0) pl[h] = den > 0.f ? (mm + log2f(den)) * LN2 : -INFINITY;
      } else {
        a.out[(int64_t)row * a.out_stride_tok + (int64_t)(hq0 + h) * a.out_stride_head + d] = __float2bfloat16(val);
      }
    }
  }
};

template <int D, bool FP8, int GH, int WARPS, int NST>
__global__ void __launch_bounds__(WARPS * 32) walk_cc_kernel(const DecodeArgs a) {
  extern __shared__ __align__(128) uint8_t hkb_smem[];
  WalkCC<D, FP8, GH, WARPS, NST>::run(a, hkb_smem);
}

}  // namespace hkb
