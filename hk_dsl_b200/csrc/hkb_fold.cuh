// The LSE merge folded into the walk: the last ring to finish a piece of a sequence folds
// the sequence's partials itself, so the decode step needs no merge launch.
//
// hk-dsl names this as what is left of its decode step -- "a merge folded into the
// last-arriving split" (docs/history/17-the-decode-step-captured-whole.md:181-188). Nobody
// waits here: a ring that finishes a piece publishes its partial, counts itself in, and goes
// on; only the ring that counts last does more work. With the stream's slot layout the live
// slots of a sequence are the prefix [0, pieces), so the fold needs no -inf marks.
//
// A warp folds at most FOLD_ROWS partials at a time. A sequence in more pieces is folded as
// a two-level tree: its slots form groups of FOLD_ROWS, the last ring of a group folds the
// group in place into the group's first slot (a normalised partial + lse again), and the
// last group to finish folds the group results into the output. Each counter is set back to
// zero by the ring that saw it full, so the array is left as it was found.
//
// Counting in happens when a piece is closed; the folds a ring owes are run after its last
// tile, when the walk's registers are free (a ring can owe at most two: for the sequence it
// began inside of, and for the one it ends on -- every sequence between lies wholly inside the
// ring, is one piece, and is only converted to bf16 on the spot).
#pragma once

#include "hkb_decode.cuh"

namespace hkb {

constexpr int FOLD_ROWS = 16;
// counters a (plane, sequence): [0] counts finished groups, [1 + g] the finished pieces of group g
constexpr int ARRIVAL_INTS = 1 + HKB_MAX_SPLITS / FOLD_ROWS;

__host__ __device__ constexpr int pow2_at_least(int x) { return x <= 1 ? 1 : x <= 2 ? 2 : x <= 4 ? 4 : x <= 8 ? 8 : 16; }

template <int D, int HEADS>
struct Fold {
  static constexpr int HP = HEADS > 8 ? 8 : pow2_at_least(HEADS);   // the warp's lanes are dealt to HP heads at a time
  static constexpr int LPH = 32 / HP;               // lanes a head
  static constexpr int FPL = D / LPH;               // output floats a lane
  static constexpr int VW = FPL >= 4 ? 4 : 2;       // floats a load
  static constexpr int LR = (FOLD_ROWS + LPH - 1) / LPH;   // lse values a lane holds
  static constexpr int RB = FPL >= 64 ? 2 : FPL >= 32 ? 4 : 8;      // rows requested at a time (128 registers: the walk's own are free by then)

  // Folds `count` <= FOLD_ROWS partials of sequence `seq` -- slots s0, s0 + step, ... -- for the
  // warp's nh heads from hq0. final_: the result goes to the output row as bf16; otherwise
  // it replaces slot s0 (normalised fp32 + lse). All loads bypass L1: other SMs wrote the data.
  __device__ static __forceinline__ void rows(const DecodeArgs& a, int seq, int s0, int step, int count, int hq0, int nh,
                                              int lane, bool final_) {
#pragma unroll 1
    for (int h0 = 0; h0 < nh; h0 += HP) some_heads(a, seq, s0, step, count, hq0 + h0, min(HP, nh - h0), lane, final_);
  }

  __device__ static __forceinline__ void some_heads(const DecodeArgs& a, int seq, int s0, int step, int count, int hq0,
                                                    int nh, int lane, bool final_) {
    const int hl = lane / LPH, j = lane % LPH;
    const bool on = hl < nh;
    const int hc = min(hl, nh - 1);   // lanes without a head read another's rows, so that no load is conditional
    const int64_t slot0 = (int64_t)seq * a.num_splits + s0;
    float* lse = a.part_lse + slot0 * a.num_q_heads + hq0 + hc;
    float* po = a.part_out + (slot0 * a.num_q_heads + hq0 + hc) * D + j * FPL;
    const int64_t lse_step = (int64_t)step * a.num_q_heads, po_step = lse_step * D;

    // The lse values and the first batch of rows are requested together: a row's address does
    // not depend on its weight, so a fold of up to RB rows costs one trip to L2, not two.
    float wgt[LR];
#pragma unroll
    for (int i = 0; i < LR; ++i) {
      const int r = j + i * LPH;
      wgt[i] = r < count ? __ldcg(lse + r * lse_step) : -INFINITY;
    }
    float acc[FPL];
#pragma unroll
    for (int v = 0; v < FPL; ++v) acc[v] = 0.f;
    float den = 0.f, mx = -INFINITY;
#pragma unroll
    for (int r0 = 0; r0 < FOLD_ROWS; r0 += RB) {
      if (r0 >= count) break;
      float x[RB][FPL];
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        const float* xp = po + min(r0 + u, count - 1) * po_step;   // past the end: a live row again, weight 0
#pragma unroll
        for (int v = 0; v < FPL; v += VW) {
          if (VW == 4) {
            const float4 t = __ldcg(reinterpret_cast<const float4*>(xp + v));
            x[u][v] = t.x; x[u][v + 1] = t.y; x[u][v + 2] = t.z; x[u][v + 3] = t.w;
          } else {
            const float2 t = __ldcg(reinterpret_cast<const float2*>(xp + v));
            x[u][v] = t.x; x[u][v + 1] = t.y;
          }
        }
      }
      if (r0 == 0) {   // the weights, once the lse values are here
#pragma unroll
        for (int i = 0; i < LR; ++i) mx = fmaxf(mx, wgt[i]);
#pragma unroll
        for (int x2 = LPH / 2; x2 > 0; x2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, x2));
#pragma unroll
        for (int i = 0; i < LR; ++i) wgt[i] = wgt[i] == -INFINITY ? 0.f : __expf(wgt[i] - mx);
      }
#pragma unroll
      for (int u = 0; u < RB; ++u) {   // ascending slot order, as the merge kernel folds
        const float w = __shfl_sync(0xffffffffu, wgt[(r0 + u) / LPH], (lane & ~(LPH - 1)) + (r0 + u) % LPH);
#pragma unroll
        for (int v = 0; v < FPL; ++v) acc[v] = fmaf(w, x[u][v], acc[v]);
        den += w;
      }
    }
    if (!on) return;
    const float inv = den > 0.f ? 1.f / den : 0.f;
    if (final_) {
      const int row = a.q_start ? __ldg(a.q_start + seq) : seq;
      __nv_bfloat16* o = a.out + (int64_t)row * a.out_stride_tok + (int64_t)(hq0 + hl) * a.out_stride_head + j * FPL;
#pragma unroll
      for (int v = 0; v < FPL; v += 2)
        *reinterpret_cast<__nv_bfloat162*>(o + v) = __floats2bfloat162_rn(acc[v] * inv, acc[v + 1] * inv);
    } else {
#pragma unroll
      for (int v = 0; v < FPL; v += VW) {
        if (VW == 4) *reinterpret_cast<float4*>(po + v) = make_float4(acc[v] * inv, acc[v + 1] * inv, acc[v + 2] * inv, acc[v + 3] * inv);
        else *reinterpret_cast<float2*>(po + v) = make_float2(acc[v] * inv, acc[v + 1] * inv);
      }
      if (j == 0) *lse = den > 0.f ? mx + __logf(den) : -INFINITY;
    }
  }

  // The warp has just written the only piece of `seq`: the normalised partial in slot 0 is the
  // answer, converted here (the lanes that wrote it are not the lanes that convert it).
  __device__ static __forceinline__ void single(const DecodeArgs& a, int seq, int hq0, int nh, int lane) {
    __threadfence_block();
    __syncwarp();
    const int row = a.q_start ? __ldg(a.q_start + seq) : seq;
    const float* po = a.part_out + ((int64_t)seq * a.num_splits * a.num_q_heads + hq0) * D;
    for (int h = 0; h < nh; ++h) {
      __nv_bfloat16* o = a.out + (int64_t)row * a.out_stride_tok + (int64_t)(hq0 + h) * a.out_stride_head;
      for (int d = lane * 2; d < D; d += 64) {
        const float2 t = __ldcg(reinterpret_cast<const float2*>(po + h * D + d));
        *reinterpret_cast<__nv_bfloat162*>(o + d) = __floats2bfloat162_rn(t.x, t.y);
      }
    }
  }

  // The warp has just written piece `p` of the `np` > 1 pieces of `seq`; `ctr`: the ARRIVAL_INTS
  // counters of this (plane, sequence). True if the piece's group is now complete -- the warp
  // then owes `finish` for it.
  __device__ static __forceinline__ bool count_in(int* ctr, int p, int np, int lane) {
    const int g = p / FOLD_ROWS;
    const int gsize = min(FOLD_ROWS, np - g * FOLD_ROWS);
    __threadfence();            // the partial is visible device-wide before it is counted
    __syncwarp();
    if (gsize == 1) return true;
    int old = 0;
    if (lane == 0) old = atomicAdd(ctr + 1 + g, 1);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != gsize - 1) return false;
    if (lane == 0) ctr[1 + g] = 0;
    return true;
  }

  // What a warp owes after count_in returned true.
  __device__ static __forceinline__ void finish(const DecodeArgs& a, int* ctr, int seq, int p, int np, int hq0, int nh,
                                                int lane) {
    const int g = p / FOLD_ROWS, ng = (np + FOLD_ROWS - 1) / FOLD_ROWS;
    const int gsize = min(FOLD_ROWS, np - g * FOLD_ROWS);
    __threadfence();
    if (ng == 1) {
      rows(a, seq, 0, 1, np, hq0, nh, lane, true);
      return;
    }
    if (gsize > 1) rows(a, seq, g * FOLD_ROWS, 1, gsize, hq0, nh, lane, false);
    __threadfence();
    __syncwarp();
    int old = 0;
    if (lane == 0) old = atomicAdd(ctr, 1);
    old = __shfl_sync(0xffffffffu, old, 0);
    if (old != ng - 1) return;
    if (lane == 0) ctr[0] = 0;
    __threadfence();
    rows(a, seq, 0, FOLD_ROWS, ng, hq0, nh, lane, true);
  }
};

}  // namespace hkb
