// The LSE fold of many parts by one CTA: used where a (sequence, head) has up to HKB_MAX_SPLITS
// partial slots of which a few dozen are live (a long sequence cut into pieces by the stream walk).
//
// A fold that reads "lse of part p, then, if it is live, its row" pays two dependent trips to L2
// a part; with sixteen parts a warp that is tens of microseconds for a kernel that moves 100 KB.
// Here the trips are three in all: (1) every thread fetches one lse into shared memory; (2) the
// live parts are listed (ascending, so the order of the sums is fixed); (3) the warps take the live
// rows round-robin, FLIGHT rows in flight a warp. The warps' sums are added through shared memory in
// warp order: the same bits every call.
#pragma once

#include "hkb_common.cuh"

namespace hkb {

template <int VEC, int WARPS>
struct WideFold {
  static constexpr int FLIGHT = 8;   // rows a warp requests before it uses any (a sequence in 64 live pieces: one round)
  struct Smem {
    float lse[HKB_MAX_SPLITS];
    int live[HKB_MAX_SPLITS];
    int count;
    float mx[WARPS];
    float acc[WARPS][32 * VEC + 1];
  };

  // `lse` -> the (sequence, head)'s first lse, parts `lse_stride` apart; `po` -> this LANE's first float
  // of part 0's row, parts `part_stride` apart. On return warp 0 holds the sums (`acc`, `den`) under the
  // maximum `mx` (-inf: nothing live, or `empty`). All threads of the CTA must call.
  __device__ static __forceinline__ void run(Smem& sm, const float* lse, int64_t lse_stride, const float* po,
                                             int64_t part_stride, int num_parts, bool empty, float (&acc)[VEC],
                                             float& den, float& mx) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    mx = -INFINITY;
    for (int p = threadIdx.x; p < num_parts; p += WARPS * 32) {
      const float v = __ldg(lse + (int64_t)p * lse_stride);
      sm.lse[p] = v;
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int x = 16; x > 0; x >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, x));
    if (lane == 0) sm.mx[warp] = mx;
    __syncthreads();
    mx = sm.mx[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, sm.mx[w]);
    if (empty) mx = -INFINITY;
    if (warp == 0) {                       // the live parts, ascending
      int count = 0;
      for (int base = 0; base < num_parts; base += 32) {
        const int p = base + lane;
        const bool live = p < num_parts && sm.lse[p] != -INFINITY;
        const unsigned m = __ballot_sync(0xffffffffu, live);
        if (live) sm.live[count + __popc(m & ((1u << lane) - 1u))] = p;
        count += __popc(m);
      }
      if (lane == 0) sm.count = count;
    }
    __syncthreads();
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
    den = 0.f;
    if (mx != -INFINITY) {
      const int count = sm.count;
      for (int i = warp; i < count; i += FLIGHT * WARPS) {
        float w[FLIGHT];
        float2 x[FLIGHT][VEC / 2];
#pragma unroll
        for (int u = 0; u < FLIGHT; ++u) {       // all requested before any is used
          const int ii = i + u * WARPS;
          w[u] = 0.f;
#pragma unroll
          for (int v = 0; v < VEC / 2; ++v) x[u][v] = make_float2(0.f, 0.f);
          if (ii < count) {
            const int p = sm.live[ii];
            w[u] = __expf(sm.lse[p] - mx);
            if (w[u] != 0.f) {              // a weight that underflowed: its row is not read
#pragma unroll
              for (int v = 0; v < VEC / 2; ++v) x[u][v] = __ldg(reinterpret_cast<const float2*>(po + (int64_t)p * part_stride) + v);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < FLIGHT; ++u) {
#pragma unroll
          for (int v = 0; v < VEC / 2; ++v) {
            acc[2 * v] = fmaf(w[u], x[u][v].x, acc[2 * v]);
            acc[2 * v + 1] = fmaf(w[u], x[u][v].y, acc[2 * v + 1]);
          }
          den += w[u];
        }
      }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) sm.acc[warp][lane * VEC + v] = acc[v];
    if (lane == 0) sm.acc[warp][32 * VEC] = den;
    __syncthreads();
    if (warp == 0) {
      den = sm.acc[0][32 * VEC];
      for (int w = 1; w < WARPS; ++w) {     // fixed order
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] += sm.acc[w][lane * VEC + v];
        den += sm.acc[w][32 * VEC];
      }
    }
  }
};

}  // namespace hkb
