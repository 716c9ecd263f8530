// The decode walk on CUDA cores, for small GQA groups (up to 4 query heads a CTA
// pass; hkb_walk_uses_mma says which groups come here): one CTA per (sequence, kv head [x head chunk], kv split).
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
  static constexpr float RESCALE_LOG2 = 8.f;   // how far a tile's maximum may exceed the reference

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
    // This lane's 16-byte pieces: row r = 4 i + g, chunk (j ^ (r & 7)) + 8 p. r & 7 is 4 (i & 1) + g,
    // so two lane-constant bases (even / odd i) plus compile-time offsets address all of them.
    const uint32_t xe = stage + g * ROWB + ((j ^ g) << 4);
    const uint32_t xo = stage + g * ROWB + ((j ^ (4 + g)) << 4);
    // scores of this lane's 4 tokens over its DPL dims: packed FMAs over (even, odd) dims;
    // kept as pairs over tokens (2 i2, 2 i2 + 1) for the packed adds below
    uint64_t s2[2][GH];
#pragma unroll
    for (int i2 = 0; i2 < 2; ++i2) {
      float sa[2][GH];
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        const int i = 2 * i2 + ii;
        uint64_t k2[DPL / 2];
#pragma unroll
        for (int p = 0; p < NP; ++p)
          unpack_piece(lds128((ii ? xo : xe) + i * 4 * ROWB + p * 128), k2 + p * (EPP / 2));
#pragma unroll
        for (int h = 0; h < GH; ++h) {
          uint64_t acc = 0ull;  // (+0.f, +0.f)
#pragma unroll
          for (int e = 0; e < DPL / 2; ++e) acc = fma2(k2[e], q2[h][e], acc);
          float a0, a1;
          unpack2(acc, a0, a1);
          sa[ii][h] = a0 + a1;
        }
      }
#pragma unroll
      for (int h = 0; h < GH; ++h) s2[i2][h] = pack2(sa[0][h], sa[1][h]);
    }
    // complete the dot products over the 8 lanes of the group (shuffle halves, add pairs)
#pragma unroll
    for (int x = 1; x < 8; x <<= 1)
#pragma unroll
      for (int i2 = 0; i2 < 2; ++i2)
#pragma unroll
        for (int h = 0; h < GH; ++h) {
          float a0, a1;
          unpack2(s2[i2][h], a0, a1);
          s2[i2][h] = add2(s2[i2][h], pack2(__shfl_xor_sync(0xffffffffu, a0, x), __shfl_xor_sync(0xffffffffu, a1, x)));
        }

    float s[4][GH];
#pragma unroll
    for (int i2 = 0; i2 < 2; ++i2)
#pragma unroll
      for (int h = 0; h < GH; ++h) unpack2(s2[i2][h], s[2 * i2][h], s[2 * i2 + 1][h]);
    bool live[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      live[i] = !LAST || (tok0 + i * 4 + g < seq_len);
      if (LAST && !live[i])
#pragma unroll
        for (int h = 0; h < GH; ++h) s[i][h] = -INFINITY;
    }
    // online softmax of this stream with a LAZY reference: m[h] is the reference the running
    // sums are scaled to, not the exact running maximum. It moves (and the sums are rescaled,
    // all heads in ONE branch) only when a tile's maximum exceeds it by more than 2^RESCALE_LOG2,
    // so after a stream's first tiles the branch is almost never taken; until then
    // probabilities are at most 2^RESCALE_LOG2, far inside fp32. out = O / l is unchanged.
    bool moved = false;
    float mx[GH];
#pragma unroll
    for (int h = 0; h < GH; ++h) {
      mx[h] = fmaxf(fmaxf(s[0][h], s[1][h]), fmaxf(s[2][h], s[3][h]));
      moved |= mx[h] > m[h] + RESCALE_LOG2;
    }
    if (moved) {
#pragma unroll
      for (int h = 0; h < GH; ++h) {
        const float m_new = fmaxf(m[h], mx[h]);
        const float safe = (m_new == -INFINITY) ? 0.f : m_new;   // nothing seen yet: keep exp2 finite
        const float alpha = fast_exp2(m[h] - safe);              // 1 for a head whose reference stays
        l[h] *= alpha;
        const uint64_t a2 = pack2(alpha, alpha);
#pragma unroll
        for (int e = 0; e < DPL / 2; ++e) o2[h][e] = mul2(o2[h][e], a2);
        m[h] = m_new;
      }
    }
#pragma unroll
    for (int h = 0; h < GH; ++h) {
      const float safe = (m[h] == -INFINITY) ? 0.f : m[h];
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) { s[i][h] = fast_exp2(s[i][h] - safe); sum += s[i][h]; }
      l[h] += sum;
    }
    // O += P V
    const uint32_t ve = xe + Loader::TILE_BYTES, vo = xo + Loader::TILE_BYTES;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint64_t v2[DPL / 2];
#pragma unroll
      for (int p = 0; p < NP; ++p)
        unpack_piece(lds128(((i & 1) ? vo : ve) + i * 4 * ROWB + p * 128), v2 + p * (EPP / 2));
      if (LAST && !live[i]) continue;  // rows past the end may hold anything, NaN included
#pragma unroll
      for (int h = 0; h < GH; ++h) {
        const uint64_t p2 = pack2(s[i][h], s[i][h]);
#pragma unroll
        for (int e = 0; e < DPL / 2; ++e) o2[h][e] = fma2(p2, v2[e], o2[h][e]);
      }
    }
  }

  // ---- the same compute as a per-warp stream (hkb_walk_stream.cuh drives it) ----------
  static constexpr int HEADS = GH;                       // query heads a warp
  static constexpr int MIN_CTAS = 2;                     // CTAs an SM the stream kernel is compiled and launched for
  static constexpr int WPR = 1;                          // warps a ring
  static constexpr int RING_SMEM = NST * STAGE_BYTES;    // one ring
  static constexpr int STAGES = NST;
  static constexpr int HEAD_DIM = D;
  __host__ __device__ static constexpr int passes(int group) { return (group + GH - 1) / GH; }

  struct State {
    uint64_t q2[GH][DPL / 2], o2[GH][DPL / 2];
    float m[GH], l[GH];
  };

  // Load the query rows of `nh` heads from hq0 on (scaled by qs) and clear the running state.
  __device__ static __forceinline__ void begin(State& st, const DecodeArgs& a, int row, int hq0, int nh, int lane,
                                               float qs) {
    const int j = lane & 7;
#pragma unroll
    for (int h = 0; h < GH; ++h) {
      st.m[h] = -INFINITY; st.l[h] = 0.f;
      const __nv_bfloat16* qp = a.q + (int64_t)row * a.q_stride_tok + (int64_t)(hq0 + h) * a.q_stride_head;
#pragma unroll
      for (int p = 0; p < NP; ++p)
#pragma unroll
        for (int e = 0; e < EPP; e += 8) {
          uint4 x = make_uint4(0, 0, 0, 0);
          if (h < nh) x = __ldg(reinterpret_cast<const uint4*>(qp + dim_of(j, p, e)));
          const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) st.q2[h][(p * EPP + e) / 2 + i] = pack2(bf16lo(w[i]) * qs, bf16hi(w[i]) * qs);
        }
#pragma unroll
      for (int e = 0; e < DPL / 2; ++e) st.o2[h][e] = 0ull;
    }
  }

  __device__ static __forceinline__ void step(State& st, uint32_t warp_smem, int stage_idx, int tok0, int seq_len,
                                              bool last, int lane, float /*qs*/) {
    const uint32_t stage = warp_smem + stage_idx * STAGE_BYTES;
    if (last) tile<true>(stage, tok0, seq_len, lane >> 3, lane & 7, st.q2, st.m, st.l, st.o2);
    else tile<false>(stage, tok0, seq_len, lane >> 3, lane & 7, st.q2, st.m, st.l, st.o2);
  }

  // Fold the warp's four 8-lane streams with shuffles and write the normalised partial of
  // `nh` heads to po[h * D + d] and its natural-log lse to pl[h].
  __device__ static __forceinline__ void end(const State& st, int lane, int nh, float vs, float* po, float* pl) {
    const int g = lane >> 3, j = lane & 7;
#pragma unroll
    for (int h = 0; h < GH; ++h) {
      float mm = fmaxf(st.m[h], __shfl_xor_sync(0xffffffffu, st.m[h], 8));
      mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 16));
      const float w = (st.m[h] == -INFINITY) ? 0.f : fast_exp2(st.m[h] - mm);
      float lt = st.l[h] * w;
      lt += __shfl_xor_sync(0xffffffffu, lt, 8);
      lt += __shfl_xor_sync(0xffffffffu, lt, 16);
      const float inv = lt > 0.f ? vs / lt : 0.f;
      float o[DPL];
#pragma unroll
      for (int e = 0; e < DPL / 2; ++e) {
        float x0, x1;
        unpack2(st.o2[h][e], x0, x1);
        x0 *= w; x1 *= w;
        x0 += __shfl_xor_sync(0xffffffffu, x0, 8); x1 += __shfl_xor_sync(0xffffffffu, x1, 8);
        x0 += __shfl_xor_sync(0xffffffffu, x0, 16); x1 += __shfl_xor_sync(0xffffffffu, x1, 16);
        o[2 * e] = x0 * inv; o[2 * e + 1] = x1 * inv;
      }
      if (g == 0 && h < nh) {
#pragma unroll
        for (int p = 0; p < NP; ++p)
#pragma unroll
          for (int e = 0; e < EPP; e += 4)
            *reinterpret_cast<float4*>(po + h * D + dim_of(j, p, e)) =
                make_float4(o[p * EPP + e], o[p * EPP + e + 1], o[p * EPP + e + 2], o[p * EPP + e + 3]);
        if (j == 0) pl[h] = lt > 0.f ? (mm + log2f(lt)) * LN2 : -INFINITY;
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
    ld.prepare(lane);
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
    int sc = 0, sl = NST - 1;   // ring stages of the compute and of the loader
    for (int k = 0; k < n; ++k) {
      cp_async_wait<NST - 2>();
      __syncwarp();
      const int kn = k + NST - 1;
      if (kn < n) ld.issue(ring + sl * STAGE_BYTES, t_lo + kn, ids.get(t_lo + kn, lane), lane);
      cp_async_commit();
      const uint32_t stage = ring + sc * STAGE_BYTES;
      sc = sc + 1 == NST ? 0 : sc + 1;
      sl = sl + 1 == NST ? 0 : sl + 1;
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

// The stream's CUDA-core worker: a ring shared by WPR_ warps, each holding GW query heads of
// the kv head (registers for 2 heads instead of 4 let twice the warps live on an SM, which is
// what hides this path's dependent-issue latency); warp 0 of the ring fills the K tiles, warp
// 1 the V tiles.
template <int D, bool FP8, int GW, int WPR_, int NST>
struct StreamCC : WalkCC<D, FP8, GW, 1, NST> {
  static constexpr int WPR = WPR_;
  static constexpr int PASS_HEADS = GW * WPR_;          // query heads a ring serves a pass
  __host__ __device__ static constexpr int passes(int group) { return (group + PASS_HEADS - 1) / PASS_HEADS; }
};

// The stream's worker for four query heads a kv head (the GQA-4 shapes): WalkCC's tile with the
// dot products completed by a TRANSPOSED reduction instead of a butterfly.
//
// A butterfly leaves all 16 (token, head) scores of a step in all 8 lanes of a group: 48
// shuffles, and every lane repeats the same softmax arithmetic. Here each exchange halves what
// a lane keeps -- 8, 4, 2 values over the xor-4, xor-2, xor-1 partners: 14 shuffles -- so a lane
// ends with the two scores of ONE token for ONE pair of heads, does the softmax for those two,
// and the 16 probabilities the P V product needs come back with 14 shuffles. To make "keep one
// half, send the other" a compile-time register choice, a lane's register order is permuted
// by its own lane bits: token register i holds token i ^ (j >> 1) of the step, head register hh
// holds head hh ^ (2 (j & 1)). The reference maximum m and the partial sum l are kept per lane
// for its own head pair (2 (j & 1), 2 (j & 1) + 1) and its own token slot.
template <int D, bool FP8, int NST>
struct StreamCC4 : WalkCC<D, FP8, 4, 1, NST> {
  using B = WalkCC<D, FP8, 4, 1, NST>;
  static constexpr int WPR = 1;
  static constexpr int PASS_HEADS = 4;
  static constexpr int DPL = B::DPL, NP = B::NP, EPP = B::EPP, ROWB = B::ROWB;
  __host__ __device__ static constexpr int passes(int group) { return (group + 3) / 4; }

  struct State {
    uint64_t q2[4][DPL / 2], o2[4][DPL / 2];
    float m[2], l[2];
    uint32_t rowoff[4];   // shared-memory offset of token register i's first piece inside a tile
  };

  __device__ static __forceinline__ void begin(State& st, const DecodeArgs& a, int row, int hq0, int nh, int lane,
                                               float qs) {
    const int g = lane >> 3, j = lane & 7;
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      const int ha = hh ^ (2 * (j & 1));
      const __nv_bfloat16* qp = a.q + (int64_t)row * a.q_stride_tok + (int64_t)(hq0 + ha) * a.q_stride_head;
#pragma unroll
      for (int p = 0; p < NP; ++p)
#pragma unroll
        for (int e = 0; e < EPP; e += 8) {
          uint4 x = make_uint4(0, 0, 0, 0);
          if (ha < nh) x = __ldg(reinterpret_cast<const uint4*>(qp + B::dim_of(j, p, e)));
          const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) st.q2[hh][(p * EPP + e) / 2 + i] = pack2(bf16lo(w[i]) * qs, bf16hi(w[i]) * qs);
        }
#pragma unroll
      for (int e = 0; e < DPL / 2; ++e) st.o2[hh][e] = 0ull;
    }
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) st.rowoff[i] = tile_off<ROWB>(4 * (i ^ (j >> 1)) + g, j);
  }

  template <bool LAST>
  __device__ static __forceinline__ void tile4(State& st, uint32_t stage, int tok0, int seq_len, int lane) {
    const int g = lane >> 3, j = lane & 7;
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint64_t k2[DPL / 2];
#pragma unroll
      for (int p = 0; p < NP; ++p) B::unpack_piece(lds128(stage + st.rowoff[i] + p * 128), k2 + p * (EPP / 2));
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) {
        uint64_t acc = 0ull;
#pragma unroll
        for (int e = 0; e < DPL / 2; ++e) acc = fma2(k2[e], st.q2[hh][e], acc);
        float a0, a1;
        unpack2(acc, a0, a1);
        s[i][hh] = a0 + a1;
      }
    }
    // transposed reduction over the 8 lanes: keep the low half of the registers, send the high half
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) s[i][hh] += __shfl_xor_sync(0xffffffffu, s[i + 2][hh], 4);
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) s[0][hh] += __shfl_xor_sync(0xffffffffu, s[1][hh], 2);
    float sa = s[0][0] + __shfl_xor_sync(0xffffffffu, s[0][2], 1);
    float sb = s[0][1] + __shfl_xor_sync(0xffffffffu, s[0][3], 1);
    // sa, sb: token (j >> 1) of the step, heads 2 (j & 1) and 2 (j & 1) + 1
    if (LAST && tok0 + 4 * (j >> 1) + g >= seq_len) { sa = -INFINITY; sb = -INFINITY; }
    float ma = fmaxf(sa, __shfl_xor_sync(0xffffffffu, sa, 2));
    float mb = fmaxf(sb, __shfl_xor_sync(0xffffffffu, sb, 2));
    ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 4));
    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 4));
    // lazy reference (see WalkCC::tile): one warp-uniform branch for the rare rescale
    const bool moved = ma > st.m[0] + B::RESCALE_LOG2 || mb > st.m[1] + B::RESCALE_LOG2;
    if (__any_sync(0xffffffffu, moved)) {
      const float na = fmaxf(st.m[0], ma), nb = fmaxf(st.m[1], mb);
      const float al_a = fast_exp2(st.m[0] - ((na == -INFINITY) ? 0.f : na));
      const float al_b = fast_exp2(st.m[1] - ((nb == -INFINITY) ? 0.f : nb));
      st.l[0] *= al_a; st.l[1] *= al_b;
      st.m[0] = na; st.m[1] = nb;
      const float al[4] = {al_a, al_b, __shfl_xor_sync(0xffffffffu, al_a, 1), __shfl_xor_sync(0xffffffffu, al_b, 1)};
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) {
        const uint64_t a2 = pack2(al[hh], al[hh]);
#pragma unroll
        for (int e = 0; e < DPL / 2; ++e) st.o2[hh][e] = mul2(st.o2[hh][e], a2);
      }
    }
    const float pa = fast_exp2(sa - ((st.m[0] == -INFINITY) ? 0.f : st.m[0]));
    const float pb = fast_exp2(sb - ((st.m[1] == -INFINITY) ? 0.f : st.m[1]));
    st.l[0] += pa;
    st.l[1] += pb;
    // O += P V: the probabilities of this lane's token registers come from the lanes that own them
    const uint32_t vst = stage + B::Loader::TILE_BYTES;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint64_t v2[DPL / 2];
#pragma unroll
      for (int p = 0; p < NP; ++p) B::unpack_piece(lds128(vst + st.rowoff[i] + p * 128), v2 + p * (EPP / 2));
      float pr[4];
#pragma unroll
      for (int hh = 0; hh < 4; ++hh)
        pr[hh] = (i == 0 && hh < 2) ? ((hh & 1) ? pb : pa)
                                    : __shfl_xor_sync(0xffffffffu, (hh & 1) ? pb : pa, (i << 1) | (hh >> 1));
      if (LAST && tok0 + 4 * (i ^ (j >> 1)) + g >= seq_len) continue;   // rows past the end may hold NaN
#pragma unroll
      for (int hh = 0; hh < 4; ++hh) {
        const uint64_t p2 = pack2(pr[hh], pr[hh]);
#pragma unroll
        for (int e = 0; e < DPL / 2; ++e) st.o2[hh][e] = fma2(p2, v2[e], st.o2[hh][e]);
      }
    }
  }

  __device__ static __forceinline__ void step(State& st, uint32_t warp_smem, int stage_idx, int tok0, int seq_len,
                                              bool last, int lane, float /*qs*/) {
    const uint32_t stage = warp_smem + stage_idx * B::STAGE_BYTES;
    if (last) tile4<true>(st, stage, tok0, seq_len, lane);
    else tile4<false>(st, stage, tok0, seq_len, lane);
  }

  // Fold the 4 token slots of a group and the warp's 4 groups, write the normalised partial.
  __device__ static __forceinline__ void end(const State& st, int lane, int nh, float vs, float* po, float* pl) {
    const int g = lane >> 3, j = lane & 7;
    float w[2], lt[2], mm[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      mm[c] = fmaxf(st.m[c], __shfl_xor_sync(0xffffffffu, st.m[c], 8));
      mm[c] = fmaxf(mm[c], __shfl_xor_sync(0xffffffffu, mm[c], 16));
      w[c] = (st.m[c] == -INFINITY) ? 0.f : fast_exp2(st.m[c] - mm[c]);
      lt[c] = st.l[c] * w[c];
#pragma unroll
      for (int x = 2; x < 32; x <<= 1) lt[c] += __shfl_xor_sync(0xffffffffu, lt[c], x);   // token slots, then groups
    }
    const float wh[4] = {w[0], w[1], __shfl_xor_sync(0xffffffffu, w[0], 1), __shfl_xor_sync(0xffffffffu, w[1], 1)};
    const float lh[4] = {lt[0], lt[1], __shfl_xor_sync(0xffffffffu, lt[0], 1), __shfl_xor_sync(0xffffffffu, lt[1], 1)};
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      const int ha = hh ^ (2 * (j & 1));
      const float inv = lh[hh] > 0.f ? vs / lh[hh] : 0.f;
      float o[DPL];
#pragma unroll
      for (int e = 0; e < DPL / 2; ++e) {
        float x0, x1;
        unpack2(st.o2[hh][e], x0, x1);
        x0 *= wh[hh]; x1 *= wh[hh];
        x0 += __shfl_xor_sync(0xffffffffu, x0, 8); x1 += __shfl_xor_sync(0xffffffffu, x1, 8);
        x0 += __shfl_xor_sync(0xffffffffu, x0, 16); x1 += __shfl_xor_sync(0xffffffffu, x1, 16);
        o[2 * e] = x0 * inv; o[2 * e + 1] = x1 * inv;
      }
      if (g == 0 && ha < nh) {
#pragma unroll
        for (int p = 0; p < NP; ++p)
#pragma unroll
          for (int e = 0; e < EPP; e += 4)
            *reinterpret_cast<float4*>(po + ha * D + B::dim_of(j, p, e)) =
                make_float4(o[p * EPP + e], o[p * EPP + e + 1], o[p * EPP + e + 2], o[p * EPP + e + 3]);
      }
    }
    if (g == 0 && (j >> 1) == 0) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int ha = 2 * (j & 1) + c;
        if (ha < nh) pl[ha] = lt[c] > 0.f ? (mm[c] + log2f(lt[c])) * LN2 : -INFINITY;
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
