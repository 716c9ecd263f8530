// The decode walk on tensor cores, for GQA groups up to 16 (a group under 8 leaves columns
// of zeros; hkb_walk_uses_mma says from which group on that is still the faster walk): one CTA per
// (sequence, kv head, kv split), the group's query heads as the N=8 columns of
// mma.sync.m16n8k16 tiles (NT = 1 for a group of 8, 2 for 9..16).
//
// The contraction is written transposed, as hk-dsl's walk is (python/hk/ops/paged.py:77-83,
// 590-638): S^T[kv, q] = K[kv, :] . Q[q, :] puts a 16-token tile on M and the heads on N,
// and O^T[d, q] += V^T[d, kv] . P^T[kv, q] puts head_dim on M. A 16-token KV tile is then
// exactly one A operand of the first product and the K dimension of the second, and a
// group of 8 wastes no tensor-core lanes.
//
// The memory side is the CUDA-core walk's: every warp streams its own contiguous share
// of the split's tiles through its own cp.async ring; the CTA's WARPS online-softmax
// streams are folded once at the end. fp8 tiles are widened to bf16 in a per-warp
// shared-memory tile first (exact: e4m3 fits bf16), so both dtypes share the mma code.
#pragma once

#include <type_traits>

#include "hkb_decode.cuh"

namespace hkb {

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// The 16-bit type of the activations and of a 16-bit cache: bf16, or fp16 (F16) for a model served
// in float16. Same fragments, same loads; the mma instruction, the packing of P and the output differ.
template <bool F16>
__device__ __forceinline__ void mma16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  if (F16) mma_f16(c, a, b); else mma_bf16(c, a, b);
}
template <bool F16>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) { return F16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi); }
template <bool F16>
__device__ __forceinline__ void store16(__nv_bfloat16* p, float x) {
  if (F16) *reinterpret_cast<__half*>(p) = __float2half_rn(x); else *p = __float2bfloat16(x);
}

// VT: the caches are in the x-split layout (XSplitLoader): the V tile sits in shared memory as V^T.
template <int D, bool FP8, int NT, int WARPS, int NST, bool F16 = false, bool VT = false>
struct WalkMMA {
  static_assert(!(FP8 && F16), "an fp8 cache goes with bf16 activations");
  static_assert(!(VT && FP8), "the x-split layout is read for 16-bit caches");
  static constexpr int ES = FP8 ? 1 : 2;
  static constexpr int ROWB = D * ES;     // bytes of a row as it sits in the cache
  static constexpr int ROWB16 = D * 2;    // bytes of a row as the mma reads it
  using Loader = typename std::conditional<VT, XSplitLoader<D>, TileLoader<ROWB>>::type;
  static constexpr int STAGE_BYTES = 2 * Loader::TILE_BYTES;
  static constexpr int TILE16_BYTES = TILE_TOKENS * ROWB16;
  static constexpr int WIDEN_BYTES = FP8 ? 2 * TILE16_BYTES : 0;  // per warp
  static constexpr int KD = D / 16;       // 16-wide chunks of head_dim
  static constexpr int HEADS = NT * 8;          // query heads a CTA pass holds columns for
  static constexpr float RESCALE_LOG2 = 8.f;    // how far a tile's maximum may exceed the softmax reference
  static constexpr int PIPE_BYTES = WARPS * (NST * STAGE_BYTES + WIDEN_BYTES);
  static constexpr int FOLD_BYTES = WARPS * HEADS * (D + 2) * 4;
  static constexpr int SMEM_BYTES = PIPE_BYTES > FOLD_BYTES ? PIPE_BYTES : FOLD_BYTES;

  // fp8 tile (rows of D bytes) -> bf16 tile (rows of 2D bytes), both swizzled.
  __device__ static __forceinline__ void widen(uint32_t src, uint32_t dst, int lane) {
    constexpr int CPR = ROWB / 16;
#pragma unroll
    for (int it = 0; it < TILE_TOKENS * CPR / 32; ++it) {
      const int x = it * 32 + lane;
      const int r = x / CPR, c = x % CPR;
      const uint4 v = lds128(src + tile_off<ROWB>(r, c));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = e4m3x2_to_float2((uint16_t)(w[i] & 0xffffu));
        const float2 b = e4m3x2_to_float2((uint16_t)(w[i] >> 16));
        o[2 * i] = pack_bf16x2(a.x, a.y);
        o[2 * i + 1] = pack_bf16x2(b.x, b.y);
      }
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(dst + tile_off<ROWB16>(r, 2 * c)), "r"(o[0]),
                   "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(dst + tile_off<ROWB16>(r, 2 * c + 1)), "r"(o[4]),
                   "r"(o[5]), "r"(o[6]), "r"(o[7]) : "memory");
    }
  }

  // ABL: stages left out for attribution runs (hkb_paged_decode_ablate), a mask of ABL_* bits; 0 = the walk.
  template <bool LAST, int ABL = 0>
  __device__ static __forceinline__ void tile(uint32_t ktile, uint32_t vtile, int tok0, int seq_len, int lane,
                                              float qs, const uint32_t (&qb)[NT][KD][2], float (&m)[NT][2],
                                              float (&l)[NT][2], float (&o)[NT][KD][4]) {
    float sc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[nt][i] = (ABL & ABL_QK) ? __uint_as_float(ktile + i) * 1e-30f : 0.f;
    // S^T = K Q^T: A = the K tile (tokens x 16 dims), B = Q^T
    if (!(ABL & ABL_QK)) {
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int kc = 0; kc < KD; ++kc) {
        uint32_t a[4];
        // the x-split K tile is [chunk][16 tokens][16 bytes]; the usual one token rows, chunks swizzled
        ldmatrix_x4(a, ktile + (VT ? (kc * 2 + (lane >> 4)) * 256 + r * 16 : tile_off<ROWB16>(r, kc * 2 + (lane >> 4))));
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma16<F16>(sc[nt], a, qb[nt][kc]);
      }
    }
    const int tA = tok0 + (lane >> 2), tB = tA + 8;  // the two tokens this lane holds scores of
    uint32_t pb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (ABL & ABL_SOFTMAX) {   // no maximum, no exponential, no sum: the scores go on as they are
        pb[nt][0] = movmatrix_trans(pack16x2<F16>(sc[nt][0], sc[nt][1]));
        pb[nt][1] = movmatrix_trans(pack16x2<F16>(sc[nt][2], sc[nt][3]));
        continue;
      }
      // scores stay unscaled: the exponent is exp2(s * qs - m) in one fma, m kept in scaled units
      if (LAST) {
        if (tA >= seq_len) { sc[nt][0] = -INFINITY; sc[nt][1] = -INFINITY; }
        if (tB >= seq_len) { sc[nt][2] = -INFINITY; sc[nt][3] = -INFINITY; }
      }
      // column (head) maxima over the tile's 16 tokens: 2 local rows, then the 8 row groups
      float mx[2] = {fmaxf(sc[nt][0], sc[nt][2]), fmaxf(sc[nt][1], sc[nt][3])};
#pragma unroll
      for (int x = 4; x < 32; x <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], x));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], x));
      }
      mx[0] *= qs; mx[1] *= qs;   // qs > 0
      // lazy reference: the running maximum moves (and the accumulators are rescaled) only when a
      // tile's maximum exceeds it by 2^RESCALE_LOG2 -- one warp-uniform branch, rarely taken
      if (__any_sync(0xffffffffu, mx[0] > m[nt][0] + RESCALE_LOG2 || mx[1] > m[nt][1] + RESCALE_LOG2)) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float m_new = fmaxf(m[nt][c], mx[c]);
          const float alpha = fast_exp2(m[nt][c] - ((m_new == -INFINITY) ? 0.f : m_new));
          l[nt][c] *= alpha;
#pragma unroll
          for (int dt = 0; dt < KD; ++dt) { o[nt][dt][c] *= alpha; o[nt][dt][c + 2] *= alpha; }
          m[nt][c] = m_new;
        }
      }
      const float mu0 = (m[nt][0] == -INFINITY) ? 0.f : -m[nt][0], mu1 = (m[nt][1] == -INFINITY) ? 0.f : -m[nt][1];
      const float p0 = fast_exp2(fmaf(sc[nt][0], qs, mu0)), p1 = fast_exp2(fmaf(sc[nt][1], qs, mu1));
      const float p2 = fast_exp2(fmaf(sc[nt][2], qs, mu0)), p3 = fast_exp2(fmaf(sc[nt][3], qs, mu1));
      l[nt][0] += p0 + p2;
      l[nt][1] += p1 + p3;
      // [token, head] fragments -> [head, token] = the B operand of the second product
      pb[nt][0] = movmatrix_trans(pack16x2<F16>(p0, p1));
      pb[nt][1] = movmatrix_trans(pack16x2<F16>(p2, p3));
    }
    // O^T += V^T P^T: A = V^T (16 dims x tokens), read transposed from the row-major V tile -- or, where
    // the cache stores V^T, straight from the [dim][16 tokens] tile: matrix m of the ldmatrix is dims
    // 8 (m & 1) .. + 7, tokens 8 (m >> 1) .. + 7
    if (!(ABL & ABL_PV)) {
      if (VT) {
        const int dl = (lane & 7) + ((lane >> 3) & 1) * 8, th = lane >> 4;
#pragma unroll
        for (int dt = 0; dt < KD; ++dt) {
          const int d = dt * 16 + dl;
          uint32_t a[4];
          ldmatrix_x4(a, vtile + d * 32 + ((th ^ ((d >> 2) & 1)) << 4));
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma16<F16>(o[nt][dt], a, pb[nt]);
        }
      } else {
        const int r = (lane & 7) + (lane >> 4) * 8;
#pragma unroll
        for (int dt = 0; dt < KD; ++dt) {
          uint32_t a[4];
          ldmatrix_x4_trans(a, vtile + tile_off<ROWB16>(r, dt * 2 + ((lane >> 3) & 1)));
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma16<F16>(o[nt][dt], a, pb[nt]);
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) o[nt][0][0] += __uint_as_float(pb[nt][0] ^ pb[nt][1]) * 1e-30f;   // keeps P alive
    }
  }

  // Zero the V rows of a tail tile that lie past seq_len: P is 0 there, but 0 * NaN is NaN.
  __device__ static __forceinline__ void scrub_tail(uint32_t vtile, int tok0, int seq_len, int lane) {
    if (VT) {   // V^T tile: tokens are the columns of every dim row
      const int live = seq_len - tok0;                       // 1..15 live tokens here
      for (int x = lane; x < D * 2; x += 32) {               // (dim row, 16-byte half): 8 tokens each
        const int d = x >> 1, h = x & 1;
        const uint32_t addr = vtile + d * 32 + ((h ^ ((d >> 2) & 1)) << 4);
        const int first = live - h * 8;                      // tokens of this half at or past `first` are dead
        if (first >= 8) continue;
        uint4 v = lds128(addr);
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (2 * i >= first) w[i] = 0u;
          else if (2 * i + 1 >= first) w[i] &= 0xffffu;
        }
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
      }
      return;
    }
    constexpr int CPR = ROWB16 / 16;
    for (int x = lane; x < TILE_TOKENS * CPR; x += 32) {
      const int r = x / CPR, c = x % CPR;
      if (tok0 + r >= seq_len)
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(vtile + tile_off<ROWB16>(r, c)), "r"(0u) : "memory");
    }
  }

  // ---- the same compute as a per-warp stream (hkb_walk_stream.cuh drives it) ----------
  static constexpr int RING_SMEM = NST * STAGE_BYTES + WIDEN_BYTES;
  static constexpr int WPR = 1;                 // warps a ring
  static constexpr int PASS_HEADS = HEADS;      // query heads a ring serves a pass
  static constexpr int STAGES = NST;
  static constexpr int HEAD_DIM = D;
  static constexpr int MIN_CTAS = (D == 256 || WARPS >= 6) ? 1 : 2;   // CTAs an SM the stream kernel is compiled and launched for (one, where a CTA has six rings or more)
  __host__ __device__ static constexpr int passes(int) { return 1; }

  struct State {
    uint32_t qb[NT][KD][2];
    float m[NT][2], l[NT][2], o[NT][KD][4];
  };

  __device__ static __forceinline__ void begin(State& st, const DecodeArgs& a, int row, int hq0, int nh, int lane,
                                               float /*qs*/) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int h = nt * 8 + (lane >> 2);
      const uint32_t* qp = reinterpret_cast<const uint32_t*>(
          a.q + (int64_t)row * a.q_stride_tok + (int64_t)(hq0 + h) * a.q_stride_head);
#pragma unroll
      for (int kc = 0; kc < KD; ++kc) {
        st.qb[nt][kc][0] = h < nh ? __ldg(qp + kc * 8 + (lane & 3)) : 0u;
        st.qb[nt][kc][1] = h < nh ? __ldg(qp + kc * 8 + 4 + (lane & 3)) : 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) st.o[nt][kc][i] = 0.f;
      }
      st.m[nt][0] = st.m[nt][1] = -INFINITY;
      st.l[nt][0] = st.l[nt][1] = 0.f;
    }
  }

  template <int ABL = 0>
  __device__ static __forceinline__ void step(State& st, uint32_t warp_smem, int stage_idx, int tok0, int seq_len,
                                              bool last, int lane, float qs) {
    const uint32_t stage = warp_smem + stage_idx * STAGE_BYTES;
    uint32_t ktile = stage, vtile = stage + Loader::TILE_BYTES;
    if (FP8) {
      const uint32_t wide = warp_smem + NST * STAGE_BYTES;
      widen(stage, wide, lane);
      widen(stage + Loader::TILE_BYTES, wide + TILE16_BYTES, lane);
      ktile = wide; vtile = wide + TILE16_BYTES;
      __syncwarp();
    }
    if (last) {
      scrub_tail(vtile, tok0, seq_len, lane);
      __syncwarp();
      tile<true, ABL>(ktile, vtile, tok0, seq_len, lane, qs, st.qb, st.m, st.l, st.o);
    } else {
      tile<false, ABL>(ktile, vtile, tok0, seq_len, lane, qs, st.qb, st.m, st.l, st.o);
    }
  }

  // The warp is one online-softmax stream: complete l over the 8 row groups and write the
  // normalised partial of `nh` heads to po[h * D + d] and its natural-log lse to pl[h].
  __device__ static __forceinline__ void end(const State& st, int lane, int nh, float vs, float* po, float* pl) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float lt = st.l[nt][c];
#pragma unroll
        for (int x = 4; x < 32; x <<= 1) lt += __shfl_xor_sync(0xffffffffu, lt, x);
        const int h = nt * 8 + 2 * (lane & 3) + c;
        const float inv = lt > 0.f ? vs / lt : 0.f;
        if (h < nh) {
#pragma unroll
          for (int dt = 0; dt < KD; ++dt) {
            po[h * D + dt * 16 + (lane >> 2)] = st.o[nt][dt][c] * inv;
            po[h * D + dt * 16 + 8 + (lane >> 2)] = st.o[nt][dt][c + 2] * inv;
          }
          if ((lane >> 2) == 0) pl[h] = lt > 0.f ? (st.m[nt][c] + log2f(lt)) * LN2 : -INFINITY;
        }
      }
  }

  __device__ static __forceinline__ void run(const DecodeArgs& a, uint8_t* smem) {
    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int nh = a.group;  // <= HEADS
    const int hq0 = kvh * a.group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int row = seq;
    if (a.q_start) {
      row = __ldg(a.q_start + seq);
      if (__ldg(a.q_start + seq + 1) <= row) return;
    }
    const int seq_len = max(__ldg(a.seq_lens + seq), 0);
    const int n_tiles = (seq_len + TILE_TOKENS - 1) / TILE_TOKENS;
    int lo, hi;
    split_range(n_tiles, a.num_splits, split, lo, hi);
    const bool partial = a.num_splits > 1;
    float* po = partial ? a.part_out + ((int64_t)(seq * a.num_splits + split) * a.num_q_heads + hq0) * D : nullptr;
    float* pl = partial ? a.part_lse + (int64_t)(seq * a.num_splits + split) * a.num_q_heads + hq0 : nullptr;

    if (lo >= hi) {
      if (partial) {
        if (threadIdx.x < nh) pl[threadIdx.x] = -INFINITY;
      } else {
        for (int x = threadIdx.x; x < nh * D; x += WARPS * 32)
          store16<F16>(a.out + (int64_t)row * a.out_stride_tok + (int64_t)(hq0 + x / D) * a.out_stride_head + x % D, 0.f);
      }
      return;
    }
    const int per_w = (hi - lo + WARPS - 1) / WARPS;
    const int t_lo = min(hi, lo + warp * per_w);
    const int t_hi = min(hi, t_lo + per_w);
    const int n = t_hi - t_lo;

    float qs = a.scale * LOG2E;
    float vs = 1.f;
    if (FP8) { qs *= __ldg(a.k_scale); vs = __ldg(a.v_scale); }

    // Q^T fragments: b0 = Q[head lane/4][16 kc + 2 (lane%4) + {0,1}], b1 = the same 8 dims on
    uint32_t qb[NT][KD][2];
    float m[NT][2], l[NT][2], o[NT][KD][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int h = nt * 8 + (lane >> 2);
      const uint32_t* qp = reinterpret_cast<const uint32_t*>(
          a.q + (int64_t)row * a.q_stride_tok + (int64_t)(hq0 + h) * a.q_stride_head);
#pragma unroll
      for (int kc = 0; kc < KD; ++kc) {
        qb[nt][kc][0] = h < nh ? __ldg(qp + kc * 8 + (lane & 3)) : 0u;
        qb[nt][kc][1] = h < nh ? __ldg(qp + kc * 8 + 4 + (lane & 3)) : 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) o[nt][kc][i] = 0.f;
      }
      m[nt][0] = m[nt][1] = -INFINITY;
      l[nt][0] = l[nt][1] = 0.f;
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

    const uint32_t ring = smem_u32(smem) + warp * (NST * STAGE_BYTES + WIDEN_BYTES);
    const uint32_t wide = ring + NST * STAGE_BYTES;
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
      uint32_t ktile = stage, vtile = stage + Loader::TILE_BYTES;
      if (FP8) {
        widen(stage, wide, lane);
        widen(stage + Loader::TILE_BYTES, wide + TILE16_BYTES, lane);
        ktile = wide; vtile = wide + TILE16_BYTES;
        __syncwarp();
      }
      const int t = t_lo + k;
      if (t == n_tiles - 1) {
        scrub_tail(vtile, t * TILE_TOKENS, seq_len, lane);
        __syncwarp();
        tile<true>(ktile, vtile, t * TILE_TOKENS, seq_len, lane, qs, qb, m, l, o);
      } else {
        tile<false>(ktile, vtile, t * TILE_TOKENS, seq_len, lane, qs, qb, m, l, o);
      }
    }
    cp_async_wait<0>();
    // each lane summed only its own two token rows: complete l over the 8 row groups
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int x = 4; x < 32; x <<= 1) l[nt][c] += __shfl_xor_sync(0xffffffffu, l[nt][c], x);
    __syncthreads();

    float* fo = reinterpret_cast<float*>(smem);   // [WARPS][HEADS][D]
    float* fml = fo + WARPS * HEADS * D;          // [WARPS][HEADS][2]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int h = nt * 8 + 2 * (lane & 3) + c;
#pragma unroll
        for (int dt = 0; dt < KD; ++dt) {
          fo[(warp * HEADS + h) * D + dt * 16 + (lane >> 2)] = o[nt][dt][c];
          fo[(warp * HEADS + h) * D + dt * 16 + 8 + (lane >> 2)] = o[nt][dt][c + 2];
        }
        if ((lane >> 2) == 0) { fml[(warp * HEADS + h) * 2] = m[nt][c]; fml[(warp * HEADS + h) * 2 + 1] = l[nt][c]; }
      }
    __syncthreads();
    for (int x = threadIdx.x; x < nh * D; x += WARPS * 32) {
      const int h = x / D, d = x % D;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, fml[(w * HEADS + h) * 2]);
      float num = 0.f, den = 0.f;
      if (mm != -INFINITY) {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
          const float wt = fast_exp2(fml[(w * HEADS + h) * 2] - mm);
          num = fmaf(wt, fo[(w * HEADS + h) * D + d], num);
          den = fmaf(wt, fml[(w * HEADS + h) * 2 + 1], den);
        }
      }
      const float val = den > 0.f ? num / den * vs : 0.f;
      if (partial) {
        po[h * D + d] = val;
        if (d == 0) pl[h] = den > 0.f ? (mm + log2f(den)) * LN2 : -INFINITY;
      } else {
        store16<F16>(a.out + (int64_t)row * a.out_stride_tok + (int64_t)(hq0 + h) * a.out_stride_head + d, val);
      }
    }
  }
};

// ---------------------------------------------------------------------------------
// The stream worker for fp8-e4m3 caches: the dequant fused into the fragment loads.
// ---------------------------------------------------------------------------------
// WalkMMA above widens an fp8 tile to a bf16 tile in shared memory before the mma reads it:
// a second pass over every byte. Here the mma fragments are built straight from the fp8 tile:
// cvt.rn.f16x2.e4m3x2 turns two adjacent bytes into one f16x2 register exactly, and
// mma.sync.m16n8k16 runs in f16 (q converted bf16 -> f16, exact in f16's range; P rounded to
// f16, three more mantissa bits than bf16). Two permutations make the bytes fall into place:
//   * K (A operand of S^T = K Q^T, tokens x dims): a lane reads 8 consecutive bytes of rows g
//     and g+8 (one 64-bit load each) and uses byte pairs (0,1),(2,3) as the k columns
//     (2t,2t+1),(2t+8,2t+9) of one 16-dim chunk and (4,5),(6,7) as those of the next. The
//     contraction runs over dims, so any order will do as long as Q's fragments use the same:
//     chunk pair s, lane t holds dims 32s + 8t .. + 7 -- one 16-byte load of the query row.
//   * V (A operand of O^T += V^T P^T, dims x tokens): a lane reads 4 consecutive bytes (dims
//     32jj + 4g .. + 3) of token rows 2t, 2t+1, 2t+8, 2t+9; a byte permute pairs the tokens of
//     one dim. Rows g / g+8 of output tile 2jj + cc are then dims 32jj + 4g + 2cc / + 1: the
//     output's dim order is permuted, which `end` undoes when it writes the partial.
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h2) : "h"((uint16_t)two_bytes));
  return h2;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}

template <int D, int NT, int NST, int CTAS>
struct WalkMMAF8 {
  static constexpr int MIN_CTAS = CTAS;   // CTAs an SM the kernel is compiled and launched for
  static_assert(D % 32 == 0, "dims are taken 32 at a time");
  static constexpr int ES = 1;
  static constexpr int ROWB = D;
  using Loader = TileLoader<ROWB, true>;
  static constexpr int STAGE_BYTES = 2 * Loader::TILE_BYTES;
  static constexpr int KD = D / 16;
  static constexpr int SPANS = D / 32;
  static constexpr int HEADS = NT * 8;
  static constexpr int RING_SMEM = NST * STAGE_BYTES;
  static constexpr int WPR = 1;
  static constexpr int PASS_HEADS = HEADS;
  static constexpr int STAGES = NST;
  static constexpr int HEAD_DIM = D;
  static constexpr float F16_MAX = 65504.f;
  static constexpr float RESCALE_LOG2 = 8.f;   // how far a tile's maximum may exceed the reference (P <= 2^8 fits f16)
  __host__ __device__ static constexpr int passes(int) { return 1; }

  struct State {
    uint32_t qb[NT][KD][2];
    float m[NT][2], l[NT][2], o[NT][KD][4];
    uint32_t koff[SPANS], voff[SPANS][2];   // this lane's byte offsets inside a K tile / a V tile
  };

  __device__ static __forceinline__ void begin(State& st, const DecodeArgs& a, int row, int hq0, int nh, int lane,
                                               float /*qs*/) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int s = 0; s < SPANS; ++s) {
      st.koff[s] = tile_off_f8<ROWB>(g, 2 * s + (t >> 1)) + (t & 1) * 8;
      st.voff[s][0] = tile_off_f8<ROWB>(2 * t, 2 * s + (g >> 2)) + (g & 3) * 4;
      st.voff[s][1] = tile_off_f8<ROWB>(2 * t + 1, 2 * s + (g >> 2)) + (g & 3) * 4;
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int h = nt * 8 + g;
      const uint4* qp = reinterpret_cast<const uint4*>(a.q + (int64_t)row * a.q_stride_tok + (int64_t)(hq0 + h) * a.q_stride_head);
#pragma unroll
      for (int s = 0; s < SPANS; ++s) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (h < nh) v = __ldg(qp + s * 4 + t);            // dims 32s + 8t .. + 7
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t f[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          f[i] = pack_f16x2(fminf(fmaxf(bf16lo(w[i]), -F16_MAX), F16_MAX), fminf(fmaxf(bf16hi(w[i]), -F16_MAX), F16_MAX));
        st.qb[nt][2 * s][0] = f[0]; st.qb[nt][2 * s][1] = f[1];
        st.qb[nt][2 * s + 1][0] = f[2]; st.qb[nt][2 * s + 1][1] = f[3];
      }
#pragma unroll
      for (int kc = 0; kc < KD; ++kc)
#pragma unroll
        for (int i = 0; i < 4; ++i) st.o[nt][kc][i] = 0.f;
      st.m[nt][0] = st.m[nt][1] = -INFINITY;
      st.l[nt][0] = st.l[nt][1] = 0.f;
    }
  }

  template <bool LAST>
  __device__ static __forceinline__ void tile(State& st, uint32_t ktile, uint32_t vtile, int tok0, int seq_len, int lane,
                                              float qs) {
    // two accumulators a column tile (even and odd chunks), so the chain of dependent mma is half as long
    float sc[NT][4], sd[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[nt][i] = sd[nt][i] = 0.f;
#pragma unroll
    for (int s = 0; s < SPANS; ++s) {
      const uint2 lo = lds64(ktile + st.koff[s]);                    // row g
      const uint2 hi = lds64(ktile + st.koff[s] + 8 * ROWB);         // row g + 8: the same swizzle
      const uint32_t a0[4] = {e4m3x2_to_f16x2(lo.x), e4m3x2_to_f16x2(hi.x), e4m3x2_to_f16x2(lo.x >> 16), e4m3x2_to_f16x2(hi.x >> 16)};
      const uint32_t a1[4] = {e4m3x2_to_f16x2(lo.y), e4m3x2_to_f16x2(hi.y), e4m3x2_to_f16x2(lo.y >> 16), e4m3x2_to_f16x2(hi.y >> 16)};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma_f16(sc[nt], a0, st.qb[nt][2 * s]);
        mma_f16(sd[nt], a1, st.qb[nt][2 * s + 1]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[nt][i] += sd[nt][i];
    const int tA = tok0 + (lane >> 2), tB = tA + 8;  // the two tokens this lane holds scores of
    uint32_t pb[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      // scores stay unscaled: the exponent is exp2(s * qs - m) in one fma, m kept in scaled units
      if (LAST) {
        if (tA >= seq_len) { sc[nt][0] = -INFINITY; sc[nt][1] = -INFINITY; }
        if (tB >= seq_len) { sc[nt][2] = -INFINITY; sc[nt][3] = -INFINITY; }
      }
      float mx[2] = {fmaxf(sc[nt][0], sc[nt][2]), fmaxf(sc[nt][1], sc[nt][3])};
#pragma unroll
      for (int x = 4; x < 32; x <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], x));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], x));
      }
      mx[0] *= qs; mx[1] *= qs;   // qs > 0
      // lazy reference: the running maximum moves (and the accumulators are rescaled) only when a
      // tile's maximum exceeds it by 2^RESCALE_LOG2 -- one warp-uniform branch, rarely taken
      if (__any_sync(0xffffffffu, mx[0] > st.m[nt][0] + RESCALE_LOG2 || mx[1] > st.m[nt][1] + RESCALE_LOG2)) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float m_new = fmaxf(st.m[nt][c], mx[c]);
          const float alpha = fast_exp2(st.m[nt][c] - ((m_new == -INFINITY) ? 0.f : m_new));
          st.l[nt][c] *= alpha;
#pragma unroll
          for (int dt = 0; dt < KD; ++dt) { st.o[nt][dt][c] *= alpha; st.o[nt][dt][c + 2] *= alpha; }
          st.m[nt][c] = m_new;
        }
      }
      const float mu0 = (st.m[nt][0] == -INFINITY) ? 0.f : -st.m[nt][0], mu1 = (st.m[nt][1] == -INFINITY) ? 0.f : -st.m[nt][1];
      const float p0 = fast_exp2(fmaf(sc[nt][0], qs, mu0)), p1 = fast_exp2(fmaf(sc[nt][1], qs, mu1));
      const float p2 = fast_exp2(fmaf(sc[nt][2], qs, mu0)), p3 = fast_exp2(fmaf(sc[nt][3], qs, mu1));
      st.l[nt][0] += p0 + p2;
      st.l[nt][1] += p1 + p3;
      // [token, head] fragments -> [head, token] = the B operand of the second product
      pb[nt][0] = movmatrix_trans(pack_f16x2(p0, p1));
      pb[nt][1] = movmatrix_trans(pack_f16x2(p2, p3));
    }
#pragma unroll
    for (int jj = 0; jj < SPANS; ++jj) {
      const uint32_t w0 = lds32(vtile + st.voff[jj][0]), w1 = lds32(vtile + st.voff[jj][1]);                      // tokens 2t, 2t+1
      const uint32_t w2 = lds32(vtile + st.voff[jj][0] + 8 * ROWB), w3 = lds32(vtile + st.voff[jj][1] + 8 * ROWB);  // 2t+8, 2t+9
      const uint32_t x01 = __byte_perm(w0, w1, 0x5140), y01 = __byte_perm(w0, w1, 0x7362);   // (dim, token pair) byte pairs
      const uint32_t x23 = __byte_perm(w2, w3, 0x5140), y23 = __byte_perm(w2, w3, 0x7362);
      const uint32_t a0[4] = {e4m3x2_to_f16x2(x01), e4m3x2_to_f16x2(x01 >> 16), e4m3x2_to_f16x2(x23), e4m3x2_to_f16x2(x23 >> 16)};
      const uint32_t a1[4] = {e4m3x2_to_f16x2(y01), e4m3x2_to_f16x2(y01 >> 16), e4m3x2_to_f16x2(y23), e4m3x2_to_f16x2(y23 >> 16)};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma_f16(st.o[nt][2 * jj], a0, pb[nt]);
        mma_f16(st.o[nt][2 * jj + 1], a1, pb[nt]);
      }
    }
  }

  // Zero the V rows of a tail tile that lie past seq_len (0x00 is +0 in e4m3): P is 0 there, but 0 * NaN is NaN.
  __device__ static __forceinline__ void scrub_tail(uint32_t vtile, int tok0, int seq_len, int lane) {
    constexpr int CPR = ROWB / 16;
    for (int x = lane; x < TILE_TOKENS * CPR; x += 32) {
      const int r = x / CPR, c = x % CPR;
      if (tok0 + r >= seq_len)
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(vtile + tile_off_f8<ROWB>(r, c)), "r"(0u) : "memory");
    }
  }

  __device__ static __forceinline__ void step(State& st, uint32_t warp_smem, int stage_idx, int tok0, int seq_len,
                                              bool last, int lane, float qs) {
    const uint32_t ktile = warp_smem + stage_idx * STAGE_BYTES, vtile = ktile + Loader::TILE_BYTES;
    if (last) {
      scrub_tail(vtile, tok0, seq_len, lane);
      __syncwarp();
      tile<true>(st, ktile, vtile, tok0, seq_len, lane, qs);
    } else {
      tile<false>(st, ktile, vtile, tok0, seq_len, lane, qs);
    }
  }

  // As WalkMMA::end, with the output's dim order undone: rows g / g+8 of output tile dt hold
  // dims 32 (dt / 2) + 4 g + 2 (dt % 2) and the next one.
  __device__ static __forceinline__ void end(const State& st, int lane, int nh, float vs, float* po, float* pl) {
    const int g = lane >> 2;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float lt = st.l[nt][c];
#pragma unroll
        for (int x = 4; x < 32; x <<= 1) lt += __shfl_xor_sync(0xffffffffu, lt, x);
        const int h = nt * 8 + 2 * (lane & 3) + c;
        const float inv = lt > 0.f ? vs / lt : 0.f;
        if (h < nh) {
#pragma unroll
          for (int dt = 0; dt < KD; ++dt)
            *reinterpret_cast<float2*>(po + h * D + 32 * (dt >> 1) + 4 * g + 2 * (dt & 1)) =
                make_float2(st.o[nt][dt][c] * inv, st.o[nt][dt][c + 2] * inv);
          if (g == 0) pl[h] = lt > 0.f ? (st.m[nt][c] + log2f(lt)) * LN2 : -INFINITY;
        }
      }
  }
};

template <int D, bool FP8, int NT, int WARPS, int NST, bool F16 = false>
__global__ void __launch_bounds__(WARPS * 32) walk_mma_kernel(const DecodeArgs a) {
  extern __shared__ __align__(128) uint8_t hkb_smem[];
  WalkMMA<D, FP8, NT, WARPS, NST, F16>::run(a, hkb_smem);
}

}  // namespace hkb
