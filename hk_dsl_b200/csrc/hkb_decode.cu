// Host entry points of the paged decode (walk + LSE merge), the merge kernel, and
// the dispatch from (head_dim, kv dtype, GQA group) to a walk instantiation.
#include "hkb_walk_cc.cuh"
#include "hkb_walk_mma.cuh"
#include "hkb_walk_stream.cuh"
#include "hkb_fold_wide.cuh"

#include <cstdlib>
#include <mutex>

extern thread_local int hkb_tls_cuda_error;

namespace hkb {

// ---------------------------------------------------------------------------------
// LSE merge. grid = (q heads, sequences). Latency-bound at decode sizes (a few microseconds).
// Weights follow the normalised-partial convention (python/hk/ops/paged.py:394-458):
// w_p = exp(lse_p - max lse); the numerator takes w_p * out_p, the denominator w_p.
// ---------------------------------------------------------------------------------
struct MergeArgs {
  void* out;
  int64_t out_stride_tok, out_stride_head;
  int out_is_f32;   // 0: bf16, 1: fp32, 2: fp16
  float* out_lse;
  const float* part_out;
  int64_t part_stride_p, part_stride_seq;
  const float* part_lse;
  int64_t lse_stride_p, lse_stride_seq;
  int num_parts, num_q_heads, head_dim;
  const int* seq_lens;
  const int* q_start;
};

// One warp a (sequence, q head), 8 heads a CTA. A lane first loads the lse of one part (32 parts
// a round), the warp votes which parts are live, and only those are read: with the stream's
// slot layout most of a sequence's `num_parts` slots are marked -inf, so a merge reads two or
// three partials however many slots there are. Each lane owns head_dim / 32 output columns.
constexpr int MERGE_WARPS = 8;
constexpr int MERGE_ROUND = 8;   // partials a warp of merge_kernel requests at a time

template <int VEC>   // floats a lane: head_dim / 32
__global__ void __launch_bounds__(MERGE_WARPS * 32) merge_kernel(const MergeArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * MERGE_WARPS + warp, seq = blockIdx.y;
  if (h >= a.num_q_heads) return;
  int row = seq;
  if (a.q_start) {
    row = __ldg(a.q_start + seq);
    if (__ldg(a.q_start + seq + 1) <= row) return;
  }
  const bool empty = a.seq_lens && __ldg(a.seq_lens + seq) <= 0;
  const float* lse = a.part_lse + (int64_t)seq * a.lse_stride_seq + h;
  const float* po = a.part_out + (int64_t)seq * a.part_stride_seq + (int64_t)h * a.head_dim + lane * VEC;

  // pass 1: the maximum lse over the parts. The lse values are requested whether or not the
  // sequence is empty, so that they fly together with seq_lens instead of after it.
  float mx = -INFINITY;
  for (int p = lane; p < a.num_parts; p += 32) mx = fmaxf(mx, __ldg(lse + (int64_t)p * a.lse_stride_p));
#pragma unroll
  for (int x = 16; x > 0; x >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, x));
  if (empty) mx = -INFINITY;

  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
  float den = 0.f;
  if (mx != -INFINITY) {
    for (int p0 = 0; p0 < a.num_parts; p0 += 32) {
      const int p = p0 + lane;
      const float lp = p < a.num_parts ? __ldg(lse + (int64_t)p * a.lse_stride_p) : -INFINITY;
      const float w = lp == -INFINITY ? 0.f : __expf(lp - mx);
      unsigned live = __ballot_sync(0xffffffffu, lp != -INFINITY);   // an empty part's memory is never read
      while (live) {   // ascending part order, MERGE_ROUND parts a round so that their loads overlap (a row costs a trip to L2:
                       // a sequence in 16 pieces is two rounds, not four)
        int src[MERGE_ROUND];
        float ws[MERGE_ROUND];
#pragma unroll
        for (int u = 0; u < MERGE_ROUND; ++u) {
          src[u] = live ? __ffs(live) - 1 : 0;
          ws[u] = live ? __shfl_sync(0xffffffffu, w, src[u]) : 0.f;
          live &= live - 1;   // 0 stays 0
        }
        float x[MERGE_ROUND][VEC];
#pragma unroll
        for (int u = 0; u < MERGE_ROUND; ++u) {
          if (ws[u] == 0.f) {   // no part (or a live part whose weight underflowed): nothing to read
#pragma unroll
            for (int v = 0; v < VEC; ++v) x[u][v] = 0.f;
            continue;
          }
          const float* xp = po + (int64_t)(p0 + src[u]) * a.part_stride_p;
#pragma unroll
          for (int v = 0; v < VEC; v += 2) {
            const float2 t = __ldg(reinterpret_cast<const float2*>(xp + v));
            x[u][v] = t.x; x[u][v + 1] = t.y;
          }
        }
#pragma unroll
        for (int u = 0; u < MERGE_ROUND; ++u) {
#pragma unroll
          for (int v = 0; v < VEC; ++v) acc[v] = fmaf(ws[u], x[u][v], acc[v]);
          den += ws[u];
        }
      }
    }
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  const int64_t off = (int64_t)row * a.out_stride_tok + (int64_t)h * a.out_stride_head + lane * VEC;
  if (a.out_is_f32 == 1) {
    float* o = reinterpret_cast<float*>(a.out) + off;
#pragma unroll
    for (int v = 0; v < VEC; v += 2) *reinterpret_cast<float2*>(o + v) = make_float2(acc[v] * inv, acc[v + 1] * inv);
  } else if (a.out_is_f32 == 2) {   // fp16 activations
    __half* o = reinterpret_cast<__half*>(a.out) + off;
#pragma unroll
    for (int v = 0; v < VEC; v += 2) *reinterpret_cast<__half2*>(o + v) = __floats2half2_rn(acc[v] * inv, acc[v + 1] * inv);
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + off;
#pragma unroll
    for (int v = 0; v < VEC; v += 2)
      *reinterpret_cast<__nv_bfloat162*>(o + v) = __floats2bfloat162_rn(acc[v] * inv, acc[v + 1] * inv);
  }
  if (a.out_lse && lane == 0)
    a.out_lse[(int64_t)row * a.num_q_heads + h] = den > 0.f ? mx + __logf(den) : -INFINITY;
}

// The same fold for many parts a (sequence, head) -- a long sequence cut into a hundred pieces: one
// CTA a (sequence, q head), three trips to memory in all (WideFold).
template <int VEC>
__global__ void __launch_bounds__(MERGE_WARPS * 32) merge_wide_kernel(const MergeArgs a) {
  __shared__ typename WideFold<VEC, MERGE_WARPS>::Smem sm;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, seq = blockIdx.y;
  int row = seq;
  if (a.q_start) {
    row = __ldg(a.q_start + seq);
    if (__ldg(a.q_start + seq + 1) <= row) return;
  }
  const bool empty = a.seq_lens && __ldg(a.seq_lens + seq) <= 0;
  const float* lse = a.part_lse + (int64_t)seq * a.lse_stride_seq + h;
  const float* po = a.part_out + (int64_t)seq * a.part_stride_seq + (int64_t)h * a.head_dim + lane * VEC;
  float acc[VEC], den, mx;
  WideFold<VEC, MERGE_WARPS>::run(sm, lse, a.lse_stride_p, po, a.part_stride_p, a.num_parts, empty, acc, den, mx);
  if (warp != 0) return;
  const float inv = den > 0.f ? 1.f / den : 0.f;
  const int64_t off = (int64_t)row * a.out_stride_tok + (int64_t)h * a.out_stride_head + lane * VEC;
  if (a.out_is_f32 == 1) {
    float* o = reinterpret_cast<float*>(a.out) + off;
#pragma unroll
    for (int v = 0; v < VEC; v += 2) *reinterpret_cast<float2*>(o + v) = make_float2(acc[v] * inv, acc[v + 1] * inv);
  } else if (a.out_is_f32 == 2) {   // fp16 activations
    __half* o = reinterpret_cast<__half*>(a.out) + off;
#pragma unroll
    for (int v = 0; v < VEC; v += 2) *reinterpret_cast<__half2*>(o + v) = __floats2half2_rn(acc[v] * inv, acc[v + 1] * inv);
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + off;
#pragma unroll
    for (int v = 0; v < VEC; v += 2)
      *reinterpret_cast<__nv_bfloat162*>(o + v) = __floats2bfloat162_rn(acc[v] * inv, acc[v + 1] * inv);
  }
  if (a.out_lse && lane == 0)
    a.out_lse[(int64_t)row * a.num_q_heads + h] = den > 0.f ? mx + __logf(den) : -INFINITY;
}

// ---------------------------------------------------------------------------------
// Launch helpers
// ---------------------------------------------------------------------------------
template <void (*kernel)(const DecodeArgs)>
static int launch_walk(int smem_bytes, int threads, dim3 grid, const DecodeArgs& a, cudaStream_t st) {
  // Opt in to more than 48 KB of dynamic shared memory once per device for this kernel
  // (one flag array per kernel: the kernel is a template argument).
  static bool armed[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess && dev >= 0 && dev < 64 && !armed[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e == cudaSuccess) armed[dev] = true;
  }
  if (e == cudaSuccess) {
    kernel<<<grid, threads, smem_bytes, st>>>(a);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}

// What the last stream walk of this thread looked like, for the merge that follows it: a sequence is cut
// where the rings' equal shares fall, so it arrives in about (rings of a plane) / (sequences) pieces,
// whatever its length. Only a hint -- it picks between two kernels that compute the same thing.
struct MergeHint { int num_seqs = -1, num_parts = -1, pieces = 0; };
static thread_local MergeHint g_merge_hint;

template <void (*kernel)(const DecodeArgs, int)>
static int launch_stream(int smem_bytes, int threads, dim3 grid, const DecodeArgs& a, int num_seqs, cudaStream_t st) {
  g_merge_hint.num_seqs = num_seqs; g_merge_hint.num_parts = a.num_splits;
  g_merge_hint.pieces = (int)(grid.x * (threads / 32)) / (num_seqs > 0 ? num_seqs : 1) + 2;
  static bool armed[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess && dev >= 0 && dev < 64 && !armed[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e == cudaSuccess) armed[dev] = true;
  }
  if (e == cudaSuccess) {
    kernel<<<grid, threads, smem_bytes, st>>>(a, num_seqs);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}

// An on/off switch of the environment, read at every call (a getenv is a fraction of a
// microsecond), so a process can flip it between calls.
static bool env_on(const char* name) {
  const char* v = std::getenv(name);
  return v && v[0] == '1';
}

// More than one part and a prefix table that fits shared memory: the persistent balanced
// stream. One part, or HKB_FIXED_SPLITS=1 in the environment (the reference's grid, kept as
// the comparison arm): the fixed-split grid, one CTA a (sequence, kv head, split).
static bool use_stream(const DecodeArgs& a, int num_seqs) {
  return a.num_splits > 1 && num_seqs <= STREAM_MAX_SEQS && !env_on("HKB_FIXED_SPLITS");
}

static dim3 stream_grid(int planes, int ctas_per_sm = 2) {
  int sms = hkb_sm_count(-1);
  if (sms <= 0) sms = 148;
  int per = (sms * ctas_per_sm) / planes;
  if (per < 1) per = 1;
  return dim3(per, planes, 1);
}

// CUDA-core walk. Fixed splits: GH query heads a CTA pass, ceil(group / GH) passes a kv head.
// Stream: one warp a ring, holding up to four heads.
template <int D, bool FP8>
static int dispatch_cc(const DecodeArgs& a, int num_seqs, cudaStream_t st) {
  constexpr int NST = FP8 ? 4 : 3;
  if (use_stream(a, num_seqs)) {
    constexpr int RINGS = 4;
    if (a.group == 1) {
      using P = StreamCC<D, FP8, 1, 1, NST>;
      return launch_stream<walk_stream_kernel<P, RINGS>>(WalkStream<P, RINGS>::SMEM_BYTES, WalkStream<P, RINGS>::THREADS,
                                                         stream_grid(a.num_kv_heads * P::passes(a.group)), a, num_seqs, st);
    }
    if (a.group == 2) {
      using P = StreamCC<D, FP8, 2, 1, NST>;
      return launch_stream<walk_stream_kernel<P, RINGS>>(WalkStream<P, RINGS>::SMEM_BYTES, WalkStream<P, RINGS>::THREADS,
                                                         stream_grid(a.num_kv_heads * P::passes(a.group)), a, num_seqs, st);
    }
    if (a.group == 3) {
      using P = StreamCC<D, FP8, 3, 1, NST>;
      return launch_stream<walk_stream_kernel<P, RINGS>>(WalkStream<P, RINGS>::SMEM_BYTES, WalkStream<P, RINGS>::THREADS,
                                                         stream_grid(a.num_kv_heads * P::passes(a.group)), a, num_seqs, st);
    }
    // a group of 4 or more: one warp a ring holding four heads (rings of two warps with two heads
    // each measured slower, 4.6 against 5.4 TB/s on the Llama-3-8B shape: every K/V element is
    // unpacked twice)
    using P = StreamCC4<D, FP8, NST>;
    return launch_stream<walk_stream_kernel<P, RINGS>>(WalkStream<P, RINGS>::SMEM_BYTES, WalkStream<P, RINGS>::THREADS,
                                                       stream_grid(a.num_kv_heads * P::passes(a.group)), a, num_seqs, st);
  }
  constexpr int WARPS = 4;
  int gh;
  switch (a.group) {
    case 1: gh = 1; break;
    case 2: gh = 2; break;
    case 3: case 5: case 6: gh = 3; break;
    default: gh = 4; break;
  }
  const int chunks = (a.group + gh - 1) / gh;
  dim3 grid(a.num_splits, a.num_kv_heads * chunks, num_seqs);
#define HKB_CC(GH_)                                                                               \
  case GH_:                                                                                       \
    return launch_walk<walk_cc_kernel<D, FP8, GH_, WARPS, NST>>(WalkCC<D, FP8, GH_, WARPS, NST>::SMEM_BYTES, \
                                                                 WARPS * 32, grid, a, st);
  switch (gh) {
    HKB_CC(1) HKB_CC(2) HKB_CC(3) HKB_CC(4)
  }
#undef HKB_CC
  return HKB_ERR_UNSUPPORTED;
}

// Tensor-core walk for groups of 8 to 16: NT 8-head column tiles a CTA.
template <int D, bool FP8, bool F16 = false>
static int dispatch_mma(const DecodeArgs& a, int num_seqs, cudaStream_t st) {
  constexpr int WARPS = 4;
  // a 16-token K+V tile of head_dim 256 is 16 KB: two stages a ring, six rings in the one CTA an SM has room for
  constexpr int NST = FP8 ? 4 : (D == 256 ? 2 : 3);
  dim3 grid(a.num_splits, a.num_kv_heads, num_seqs);
  if (use_stream(a, num_seqs)) {
    if constexpr (FP8 && D != 128) {
      // fp8 rows of 64 and 256 bytes: the same worker on the layout tile_off_f8 gives them. Head size 256:
      // a tile is as many bytes as a bf16 tile of head size 128, and the accumulators take as many registers
      // as the bf16 walk's at 256 -- one CTA an SM, six rings; head size 64: 1 KB tiles, three CTAs an SM.
      if constexpr (D == 256) {
        constexpr int RINGS = 6;
        grid = stream_grid(a.num_kv_heads, 1);
        if (a.group <= 8) {
          using P = WalkMMAF8<D, 1, 3, 1>;
          return launch_stream<walk_stream_kernel<P, RINGS>>(WalkStream<P, RINGS>::SMEM_BYTES, RINGS * 32, grid, a, num_seqs, st);
        }
        using P2 = WalkMMAF8<D, 2, 3, 1>;
        return launch_stream<walk_stream_kernel<P2, RINGS>>(WalkStream<P2, RINGS>::SMEM_BYTES, RINGS * 32, grid, a, num_seqs, st);
      } else {
        if (a.group <= 8) {
          using P = WalkMMAF8<D, 1, 4, 3>;
          return launch_stream<walk_stream_kernel<P, WARPS>>(WalkStream<P, WARPS>::SMEM_BYTES, WARPS * 32,
                                                             stream_grid(a.num_kv_heads, 3), a, num_seqs, st);
        }
        using P2 = WalkMMAF8<D, 2, 4, 2>;
        return launch_stream<walk_stream_kernel<P2, WARPS>>(WalkStream<P2, WARPS>::SMEM_BYTES, WARPS * 32,
                                                            stream_grid(a.num_kv_heads), a, num_seqs, st);
      }
    } else if constexpr (D == 256) {
      constexpr int RINGS = 6;
      grid = stream_grid(a.num_kv_heads, 1);
      if (a.group <= 8) {
        using P = WalkMMA<D, FP8, 1, WARPS, NST, F16>;
        return launch_stream<walk_stream_kernel<P, RINGS>>(WalkStream<P, RINGS>::SMEM_BYTES, RINGS * 32, grid, a, num_seqs, st);
      }
      using P2 = WalkMMA<D, FP8, 2, WARPS, NST, F16>;
      return launch_stream<walk_stream_kernel<P2, RINGS>>(WalkStream<P2, RINGS>::SMEM_BYTES, RINGS * 32, grid, a, num_seqs, st);
    } else {
      grid = stream_grid(a.num_kv_heads);
      if constexpr (FP8) {
        // The fp8 stream builds its mma fragments straight from the fp8 tile (WalkMMAF8). Twelve warps
        // an SM (168 registers a thread) for a group of up to 8: the walk of an fp8 tile is a chain of
        // dependent shared-memory loads, converts, mma and shuffles, and with half the bytes a tile it
        // needs more warps in flight than the bf16 walk to keep HBM busy (6.2 against 4.9 TB/s at eight
        // warps; sixteen at 128 registers spill and fall to 4.3; widening tiles to bf16 in shared memory
        // first reads 2.8). Twelve warps as two CTAs of six rings with three stages each: measured with
        // the libraries run in turn on one B200, batch 64 x 2k-8k tokens: 5856-5895 GB/s, against 5703-5761
        // for three CTAs of four rings and four stages, 5753 for one CTA of twelve rings, 5366-5430 with
        // two stages a ring.
        if (a.group <= 8) {
          constexpr int RINGS = 6;
          using P = WalkMMAF8<D, 1, 3, 2>;
          return launch_stream<walk_stream_kernel<P, RINGS>>(WalkStream<P, RINGS>::SMEM_BYTES, RINGS * 32,
                                                             stream_grid(a.num_kv_heads, 2), a, num_seqs, st);
        }
        using P2 = WalkMMAF8<D, 2, NST, 2>;
        return launch_stream<walk_stream_kernel<P2, WARPS>>(WalkStream<P2, WARPS>::SMEM_BYTES, WARPS * 32, grid, a, num_seqs, st);
      } else {
        if (a.group <= 8) {
          // Eight warps an SM as ONE CTA of eight rings (three stages a ring, 192 KB): the same rings a plane as
          // two CTAs of four, half the CTAs to start and to finish. Measured with the two libraries run in turn
          // on one B200, us a layer: 16 x 1024 tokens 19.1 against 20.1, 16 x 8192 90.7 against 92.4, 32 x 8192
          // 170.7 against 174.4, 128 x 8192 644.6 against 655.1, every other shape of the grid within 0.5 %;
          // batch 64 x 2k-8k 6444 against 6382 GB/s. (Six rings of four stages: 6145 GB/s.)
          constexpr int RINGS = 8;
          using P8 = WalkMMA<D, FP8, 1, RINGS, NST, F16>;
          return launch_stream<walk_stream_kernel<P8, RINGS>>(WalkStream<P8, RINGS>::SMEM_BYTES, RINGS * 32,
                                                              stream_grid(a.num_kv_heads, 1), a, num_seqs, st);
        }
        return launch_stream<walk_stream_kernel<WalkMMA<D, FP8, 2, WARPS, NST, F16>, WARPS>>(
            WalkStream<WalkMMA<D, FP8, 2, WARPS, NST, F16>, WARPS>::SMEM_BYTES, WARPS * 32, grid, a, num_seqs, st);
      }
    }
  }
  if (a.group <= 8)
    return launch_walk<walk_mma_kernel<D, FP8, 1, WARPS, NST, F16>>(WalkMMA<D, FP8, 1, WARPS, NST, F16>::SMEM_BYTES,
                                                               WARPS * 32, grid, a, st);
  return launch_walk<walk_mma_kernel<D, FP8, 2, WARPS, NST, F16>>(WalkMMA<D, FP8, 2, WARPS, NST, F16>::SMEM_BYTES,
                                                             WARPS * 32, grid, a, st);
}

}  // namespace hkb

namespace hkb {

// What the one-launch decode step adds to a walk: the step's new K/V rows and the fold counters.
struct StepExtra {
  const void* key = nullptr;
  const void* value = nullptr;
  int64_t key_stride_tok = 0, key_stride_head = 0, val_stride_tok = 0, val_stride_head = 0;
  const void* slots = nullptr;
  int slot_is_i64 = 0;
  int32_t* arrivals = nullptr;
  bool wrote = false;    // out: the walk wrote the new rows into the cache itself
  bool folded = false;   // out: the walk folded the partials itself
  int ablate = 0;        // ABL_* mask: an attribution run (hkb_paged_decode_ablate)
  bool xsplit = false;   // the caches are in the x-split layout (hkb_paged_decode_xsplit)
};

// The stream walk over x-split caches: head_dim 128, 16-bit caches, the tensor-core worker at
// every group (a group below 8 leaves columns of its one tile empty, as at a group of 4).
template <bool F16>
static int dispatch_xsplit(const DecodeArgs& a, int num_seqs, cudaStream_t st) {
  const dim3 grid = stream_grid(a.num_kv_heads);
  if (a.group <= 8) {
    using P = WalkMMA<128, false, 1, 4, 3, F16, true>;
    return launch_stream<walk_stream_kernel<P, 4>>(WalkStream<P, 4>::SMEM_BYTES, 4 * 32, grid, a, num_seqs, st);
  }
  using P2 = WalkMMA<128, false, 2, 4, 3, F16, true>;
  return launch_stream<walk_stream_kernel<P2, 4>>(WalkStream<P2, 4>::SMEM_BYTES, 4 * 32, grid, a, num_seqs, st);
}

// The stream walk with stages left out. Built for the headline shape only -- head_dim 128, a bf16
// cache, a GQA group of 4 to 8 on the tensor-core worker, more than one split -- and for the masks
// an attribution table needs: each stage alone, both copies, all the math.
static int dispatch_ablated(const DecodeArgs& a, int num_seqs, int ablate, cudaStream_t st) {
  using P = WalkMMA<128, false, 1, 8, 3, false>;          // the shape dispatch_mma launches: one CTA of eight rings an SM
  const dim3 grid = stream_grid(a.num_kv_heads, 1);
#define HKB_ABL(MASK)                                                                                               \
  case MASK:                                                                                                        \
    return launch_stream<walk_stream_ablated_kernel<P, 8, MASK>>(WalkStream<P, 8>::SMEM_BYTES, 8 * 32, grid, a, num_seqs, st);
  switch (ablate) {
    HKB_ABL(ABL_PAGE) HKB_ABL(ABL_KLOAD) HKB_ABL(ABL_VLOAD) HKB_ABL(ABL_QK) HKB_ABL(ABL_SOFTMAX) HKB_ABL(ABL_PV)
    HKB_ABL(ABL_KLOAD | ABL_VLOAD) HKB_ABL(ABL_QK | ABL_SOFTMAX | ABL_PV)
  }
#undef HKB_ABL
  return HKB_ERR_UNSUPPORTED;
}

// The stream kernel takes the whole step (every ring is a single warp). HKB_STEP_UNFUSED=1 keeps
// the three separate launches, the arm the joined step is compared with.
static bool step_fusable(int num_splits, int num_seqs) {
  return num_splits > 1 && num_seqs <= STREAM_MAX_SEQS && !env_on("HKB_FIXED_SPLITS") && !env_on("HKB_STEP_UNFUSED");
}

// Everything a decode call can be refused for, checked before anything is launched.
static int decode_check(const void* out, const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                        const hkb_cache_t& kc, const hkb_cache_t& vc, const int32_t* block_table, int max_pages,
                        const int32_t* seq_lens, int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                        int block_size, int kv_dtype, const float* k_scale, const float* v_scale,
                        int num_splits, const float* part_out, const float* part_lse) {
  if (num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || max_pages < 0) return HKB_ERR_SIZE;
  if (num_seqs == 0) return HKB_OK;
  if (num_seqs > 65535 * 16 || num_splits > 0x7fffffff) return HKB_ERR_SIZE;
  if (!out || !q || !kc.ptr || !vc.ptr || !block_table || !seq_lens) return HKB_ERR_NULL;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return HKB_ERR_HEAD_DIM;
  if (block_size <= 0 || block_size % TILE_TOKENS) return HKB_ERR_BLOCK_SIZE;
  if (num_q_heads % num_kv_heads) return HKB_ERR_GROUP;
  if (num_q_heads / num_kv_heads > HKB_MAX_GROUP) return HKB_ERR_GROUP;
  if (kv_dtype != HKB_KV_BF16 && kv_dtype != HKB_KV_FP8_E4M3 && kv_dtype != HKB_KV_F16) return HKB_ERR_DTYPE;
  const bool fp8 = kv_dtype == HKB_KV_FP8_E4M3;
  if (fp8 && (!k_scale || !v_scale)) return HKB_ERR_SCALE;
  if (num_splits < 1 || num_splits > HKB_MAX_SPLITS) return HKB_ERR_SPLITS;
  if (num_splits > 1 && (!part_out || !part_lse)) return HKB_ERR_SPLITS;
  if (max_pages < 1 || kc.num_blocks < 1 || vc.num_blocks < 1) return HKB_ERR_SIZE;
  if (num_seqs > 65535 || num_kv_heads * 2 > 65535) return HKB_ERR_SIZE;
  const int es = fp8 ? 1 : 2;
  // every 16-byte chunk of a KV row, a q row and an out row must be 16-byte aligned
  const int64_t kv_strides = kc.stride_block | kc.stride_token | kc.stride_head | vc.stride_block |
                             vc.stride_token | vc.stride_head;
  if ((kv_strides * es) % 16) return HKB_ERR_STRIDE;
  if ((q_stride_tok | q_stride_head) % 8) return HKB_ERR_STRIDE;
  if (((uintptr_t)kc.ptr | (uintptr_t)vc.ptr | (uintptr_t)q) % 16) return HKB_ERR_ALIGN;
  if ((uintptr_t)out % 2 || (part_out && (uintptr_t)part_out % 16)) return HKB_ERR_ALIGN;
  return HKB_OK;
}

// What hkb_merge refuses, for a caller that wants to know before it launches the walk.
static int merge_check(const void* out, int64_t out_stride_tok, int64_t out_stride_head, int out_kind,
                       const float* part_out, int64_t part_stride_p, int64_t part_stride_seq, const float* part_lse,
                       int num_parts, int num_seqs, int num_q_heads, int head_dim) {
  if (num_seqs < 0 || num_q_heads <= 0 || num_parts < 1) return HKB_ERR_SIZE;
  if (num_parts > HKB_MAX_SPLITS) return HKB_ERR_SPLITS;
  if (num_seqs == 0) return HKB_OK;
  if (!out || !part_out || !part_lse) return HKB_ERR_NULL;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return HKB_ERR_HEAD_DIM;
  if (num_seqs > 65535) return HKB_ERR_SIZE;
  if ((part_stride_p | part_stride_seq) % 4 || (out_stride_tok | out_stride_head) % 4) return HKB_ERR_STRIDE;
  if ((uintptr_t)part_out % 16 || (uintptr_t)out % (out_kind == 1 ? 16 : 8)) return HKB_ERR_ALIGN;
  return HKB_OK;
}

static int decode_impl(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                       const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                       hkb_cache_t kc, hkb_cache_t vc,
                       const int32_t* block_table, int64_t table_stride, int max_pages,
                       const int32_t* seq_lens, const int32_t* q_start,
                       int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                       int block_size, float scale, int kv_dtype,
                       const float* k_scale, const float* v_scale,
                       int num_splits, float* part_out, float* part_lse, void* stream, StepExtra* extra) {
  const int rc = decode_check(out, q, q_stride_tok, q_stride_head, kc, vc, block_table, max_pages, seq_lens, num_seqs,
                              num_q_heads, num_kv_heads, head_dim, block_size, kv_dtype, k_scale, v_scale, num_splits,
                              part_out, part_lse);
  if (rc != HKB_OK || num_seqs == 0) return rc;
  const int group = num_q_heads / num_kv_heads;
  const bool fp8 = kv_dtype == HKB_KV_FP8_E4M3, f16 = kv_dtype == HKB_KV_F16;
  const int es = fp8 ? 1 : 2;

  DecodeArgs a;
  a.out = (__nv_bfloat16*)out; a.out_stride_tok = out_stride_tok; a.out_stride_head = out_stride_head;
  a.q = (const __nv_bfloat16*)q; a.q_stride_tok = q_stride_tok; a.q_stride_head = q_stride_head;
  a.k = (const uint8_t*)kc.ptr; a.v = (const uint8_t*)vc.ptr;
  a.k_stride_block = kc.stride_block * es; a.k_stride_token = kc.stride_token * es; a.k_stride_head = kc.stride_head * es;
  a.v_stride_block = vc.stride_block * es; a.v_stride_token = vc.stride_token * es; a.v_stride_head = vc.stride_head * es;
  const int64_t nb = kc.num_blocks < vc.num_blocks ? kc.num_blocks : vc.num_blocks;
  a.num_blocks = nb > 0x7fffffff ? 0x7fffffff : (int)nb;
  a.block_table = block_table; a.table_stride = table_stride; a.max_pages = max_pages;
  a.seq_lens = seq_lens; a.q_start = q_start;
  a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads; a.group = group;
  a.tiles_per_page = block_size / TILE_TOKENS;
  a.scale = scale;
  a.k_scale = fp8 ? k_scale : nullptr;   // scales apply to fp8 caches only
  a.v_scale = fp8 ? v_scale : nullptr;
  a.num_splits = num_splits; a.part_out = part_out; a.part_lse = part_lse;
  a.arrivals = nullptr; a.new_k = nullptr; a.new_v = nullptr;
  a.new_k_stride_tok = a.new_k_stride_head = a.new_v_stride_tok = a.new_v_stride_head = 0;
  a.slots = nullptr; a.slot_is_i64 = 0; a.block_size = block_size;
  a.xsplit = extra && extra->xsplit;
  if (a.xsplit) {
    if (head_dim != 128 || fp8 || num_splits < 2 || num_seqs > STREAM_MAX_SEQS) return HKB_ERR_UNSUPPORTED;
    return f16 ? dispatch_xsplit<true>(a, num_seqs, (cudaStream_t)stream) : dispatch_xsplit<false>(a, num_seqs, (cudaStream_t)stream);
  }
  if (extra && step_fusable(num_splits, num_seqs)) {
    if (extra->arrivals && !f16) {   // the fold on arrival writes bf16; fp16 steps keep the merge launch
      a.arrivals = extra->arrivals;
      extra->folded = true;
    }
    if (extra->key) {
      a.new_k = (const __nv_bfloat16*)extra->key; a.new_v = (const __nv_bfloat16*)extra->value;
      a.new_k_stride_tok = extra->key_stride_tok; a.new_k_stride_head = extra->key_stride_head;
      a.new_v_stride_tok = extra->val_stride_tok; a.new_v_stride_head = extra->val_stride_head;
      a.slots = extra->slots; a.slot_is_i64 = extra->slot_is_i64;
      extra->wrote = true;
    }
  }
  cudaStream_t st = (cudaStream_t)stream;

  if (extra && extra->ablate) {
    if (head_dim != 128 || fp8 || f16 || group < 4 || group > 8 || !use_stream(a, num_seqs) || !hkb_walk_uses_mma(group, kv_dtype))
      return HKB_ERR_UNSUPPORTED;
    return dispatch_ablated(a, num_seqs, extra->ablate, st);
  }
  if (f16) {   // fp16: the tensor-core worker at every group (the CUDA-core workers unpack bf16)
    if (head_dim == 128) return dispatch_mma<128, false, true>(a, num_seqs, st);
    if (head_dim == 256) return dispatch_mma<256, false, true>(a, num_seqs, st);
    return dispatch_mma<64, false, true>(a, num_seqs, st);
  }
  const bool mma = hkb_walk_uses_mma(group, kv_dtype) != 0;
  if (head_dim == 128) {
    if (fp8) return mma ? dispatch_mma<128, true>(a, num_seqs, st) : dispatch_cc<128, true>(a, num_seqs, st);
    return mma ? dispatch_mma<128, false>(a, num_seqs, st) : dispatch_cc<128, false>(a, num_seqs, st);
  }
  if (head_dim == 256)   // 512-byte rows (256 in fp8): tensor-core tiles at every group
    return fp8 ? dispatch_mma<256, true>(a, num_seqs, st) : dispatch_mma<256, false>(a, num_seqs, st);
  if (fp8) return dispatch_mma<64, true>(a, num_seqs, st);   // fp8: the tensor-core worker at every group
  return mma ? dispatch_mma<64, false>(a, num_seqs, st) : dispatch_cc<64, false>(a, num_seqs, st);
}

}  // namespace hkb

// Which worker walks a GQA group. The usual rule puts tensor-core tiles at groups of 8 and more
// (a full 8-column mma tile) and CUDA cores below. Measured on B200 that bound is too high: a CUDA-core walk of a
// group of 5 to 7 takes its heads in two passes and reads the KV twice (3.4 against 6.5 TB/s for
// bf16), and at a group of 4 the bf16 CUDA-core walk -- 692 instructions a tile against ~300 --
// draws enough power to run at 1.62 GHz under the 1 kW cap, where the mma walk with half its
// columns empty holds 6.4 TB/s (5.7-5.8 for CUDA cores; equal in short bursts). For fp8 caches
// the mma walk builds its fragments straight from the fp8 tile (WalkMMAF8) and reads 4.9-5.0 TB/s
// at every group, against 4.9 / 4.0 / 3.1 TB/s for CUDA cores at groups of 1 / 2 / 4.
// So: bf16 from 4, fp8 always. HKB_MMA_MIN_GROUP=8 restores the bound of 8; 1..8 is taken.
extern "C" int hkb_walk_uses_mma(int group, int kv_dtype) {
  const char* v = std::getenv("HKB_MMA_MIN_GROUP");
  const int x = v ? std::atoi(v) : 0;
  const int forced = x >= 1 && x <= 8 ? x : 0;
  if (kv_dtype == HKB_KV_F16) return 1;
  const int bound = forced ? forced : (kv_dtype == HKB_KV_FP8_E4M3 ? 1 : 4);
  return group >= bound ? 1 : 0;
}

extern "C" int hkb_paged_decode(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                                const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                                hkb_cache_t kc, hkb_cache_t vc,
                                const int32_t* block_table, int64_t table_stride, int max_pages,
                                const int32_t* seq_lens, const int32_t* q_start,
                                int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                int block_size, float scale, int kv_dtype,
                                const float* k_scale, const float* v_scale,
                                int num_splits, float* part_out, float* part_lse, void* stream) {
  return hkb::decode_impl(out, out_stride_tok, out_stride_head, q, q_stride_tok, q_stride_head, kc, vc, block_table,
                          table_stride, max_pages, seq_lens, q_start, num_seqs, num_q_heads, num_kv_heads, head_dim,
                          block_size, scale, kv_dtype, k_scale, v_scale, num_splits, part_out, part_lse, stream, nullptr);
}

// The walk of hkb_paged_decode over caches in vLLM's x-split layout, read in place: K is
// (blocks, kv_heads, head_dim / 8, block_size, 8) and V is (blocks, kv_heads, head_dim, block_size),
// 16-bit elements, heads and everything inside them contiguous; `*_stride_block` is elements between
// blocks. Replaces python/hk/ops/paged_prefill.py:768-772 (`rocm_views`, strided views that the
// reference's kernels read) and the decode over them (`_rocm_decode`,
// python/hk/integration/vllm_prefill.py:1332-1356). Always split (num_splits >= 2): partials go to
// `part_out` / `part_lse` as in hkb_paged_decode and hkb_merge folds them.
extern "C" int hkb_paged_decode_xsplit(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                                       const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                                       const void* k_cache, int64_t k_stride_block,
                                       const void* v_cache, int64_t v_stride_block, int64_t num_blocks,
                                       const int32_t* block_table, int64_t table_stride, int max_pages,
                                       const int32_t* seq_lens, const int32_t* q_start,
                                       int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                       int block_size, float scale, int kv_dtype,
                                       int num_splits, float* part_out, float* part_lse, void* stream) {
  if (block_size <= 0) return HKB_ERR_BLOCK_SIZE;
  if (head_dim != 128 || (kv_dtype != HKB_KV_BF16 && kv_dtype != HKB_KV_F16)) return HKB_ERR_UNSUPPORTED;
  if (num_splits < 2) return HKB_ERR_SPLITS;
  if (num_seqs > hkb::STREAM_MAX_SEQS) return HKB_ERR_SIZE;
  const int64_t head = (int64_t)head_dim * block_size;
  if (num_kv_heads > 0 && (k_stride_block < head * num_kv_heads || v_stride_block < head * num_kv_heads)) return HKB_ERR_STRIDE;
  hkb_cache_t kc{const_cast<void*>(k_cache), k_stride_block, 8, head, num_blocks};
  hkb_cache_t vc{const_cast<void*>(v_cache), v_stride_block, 8, head, num_blocks};
  hkb::StepExtra extra;
  extra.xsplit = true;
  return hkb::decode_impl(out, out_stride_tok, out_stride_head, q, q_stride_tok, q_stride_head, kc, vc, block_table,
                          table_stride, max_pages, seq_lens, q_start, num_seqs, num_q_heads, num_kv_heads, head_dim,
                          block_size, scale, kv_dtype, nullptr, nullptr, num_splits, part_out, part_lse, stream, &extra);
}

namespace hkb {

// One decode step: cache write, walk, merge. `out_kind` 0 / 2: the bf16 / fp16 answer in `out`;
// 1: the step's normalised fp32 answer in `out` and its natural-log lse in `out_lse` -- one rank's
// record of a KV axis cut across GPUs. Every refusal happens before the first launch.
static int step_impl(void* out, int64_t out_stride_tok, int64_t out_stride_head, int out_kind, float* out_lse,
                     const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                     const void* key, const void* value,
                     int64_t key_stride_tok, int64_t key_stride_head,
                     int64_t val_stride_tok, int64_t val_stride_head,
                     const void* slot_mapping, int slot_is_i64,
                     hkb_cache_t kc, hkb_cache_t vc,
                     const int32_t* block_table, int64_t table_stride, int max_pages,
                     const int32_t* seq_lens, const int32_t* q_start,
                     int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                     int block_size, float scale, int kv_dtype,
                     const float* k_scale, const float* v_scale,
                     int num_splits, float* part_out, float* part_lse, int32_t* arrivals, void* stream) {
  if (num_seqs < 0) return HKB_ERR_SIZE;
  if (num_seqs == 0) return HKB_OK;
  if ((key == nullptr) != (value == nullptr)) return HKB_ERR_NULL;
  if (key && !slot_mapping) return HKB_ERR_NULL;
  if (out_kind == 1 && (out == nullptr) != (out_lse == nullptr)) return HKB_ERR_NULL;   // a record is both halves, or neither
  const bool out_record_is_null = out_kind == 1 && out == nullptr;
  if (out_record_is_null) out = const_cast<void*>(q);   // never written: a split walk without a fold touches no output row
  if (key) {
    // the new rows are read as 16-byte chunks, whichever launch writes them
    if ((key_stride_tok | key_stride_head | val_stride_tok | val_stride_head) % 8) return HKB_ERR_STRIDE;
    if (((uintptr_t)key | (uintptr_t)value) % 16) return HKB_ERR_ALIGN;
  }
  // the walk's and the merge's refusals, before the cache write (or anything else) is launched
  int rc = decode_check(out, q, q_stride_tok, q_stride_head, kc, vc, block_table, max_pages, seq_lens, num_seqs,
                        num_q_heads, num_kv_heads, head_dim, block_size, kv_dtype, k_scale, v_scale, num_splits,
                        part_out, part_lse);
  if (rc != HKB_OK) return rc;
  // a record is written by the merge of at least two splits; with no record to write (out_kind 1, out NULL)
  // the step is the walk alone and the partials stay in the scratch for the caller to fold
  const bool walk_only = out_kind == 1 && out_record_is_null;
  if (out_kind == 1 && (num_splits < 2 || (!walk_only && !out_lse))) return HKB_ERR_SPLITS;
  const bool fusable = step_fusable(num_splits, num_seqs);
  const bool fold = arrivals && fusable && kv_dtype != HKB_KV_F16 && out_kind == 0;
  if (num_splits > 1 && !fold && !walk_only) {
    rc = merge_check(out, out_stride_tok, out_stride_head, out_kind, part_out, (int64_t)num_q_heads * head_dim,
                     (int64_t)num_splits * num_q_heads * head_dim, part_lse, num_splits, num_seqs, num_q_heads, head_dim);
    if (rc != HKB_OK) return rc;
  }
  // the fold on arrival and the walk's zero rows store two 16-bit elements at a time
  if (fold && ((uintptr_t)out % 4 || (out_stride_tok | out_stride_head) % 2)) return HKB_ERR_STRIDE;
  if (key && !fusable) {
    const int64_t dmask = kc.stride_block | kc.stride_token | kc.stride_head | vc.stride_block | vc.stride_token | vc.stride_head;
    if (dmask % 8) return HKB_ERR_STRIDE;   // the separate cache write's own bound
  }

  StepExtra x;
  x.key = key; x.value = value;
  x.key_stride_tok = key_stride_tok; x.key_stride_head = key_stride_head;
  x.val_stride_tok = val_stride_tok; x.val_stride_head = val_stride_head;
  x.slots = slot_mapping; x.slot_is_i64 = slot_is_i64; x.arrivals = fold ? arrivals : nullptr;
  if (key && !fusable) {   // the separate cache write: one row a sequence
    rc = hkb_reshape_and_cache(key, value, key_stride_tok, key_stride_head, val_stride_tok, val_stride_head, kc,
                               vc, slot_mapping, slot_is_i64, num_seqs, num_kv_heads, head_dim, block_size,
                               kv_dtype, k_scale, v_scale, stream);
    if (rc != HKB_OK) return rc;
  }
  rc = decode_impl(out, out_stride_tok, out_stride_head, q, q_stride_tok, q_stride_head, kc, vc, block_table,
                   table_stride, max_pages, seq_lens, q_start, num_seqs, num_q_heads, num_kv_heads, head_dim,
                   block_size, scale, kv_dtype, k_scale, v_scale, num_splits, part_out, part_lse, stream, &x);
  if (rc != HKB_OK || x.folded || num_splits <= 1 || walk_only) return rc;
  const int kind = out_kind == 1 ? 1 : (kv_dtype == HKB_KV_F16 ? 2 : 0);
  return hkb_merge(out, out_stride_tok, out_stride_head, kind, out_kind == 1 ? out_lse : nullptr, part_out,
                   (int64_t)num_q_heads * head_dim, (int64_t)num_splits * num_q_heads * head_dim, part_lse, num_q_heads,
                   (int64_t)num_splits * num_q_heads, num_splits, num_seqs, num_q_heads, head_dim, seq_lens, q_start,
                   stream);
}

}  // namespace hkb

extern "C" int hkb_paged_decode_ablate(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                                       const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                                       hkb_cache_t kc, hkb_cache_t vc,
                                       const int32_t* block_table, int64_t table_stride, int max_pages,
                                       const int32_t* seq_lens, const int32_t* q_start,
                                       int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                       int block_size, float scale, int kv_dtype,
                                       const float* k_scale, const float* v_scale,
                                       int num_splits, float* part_out, float* part_lse, int ablate, void* stream) {
  if (ablate == 0)
    return hkb_paged_decode(out, out_stride_tok, out_stride_head, q, q_stride_tok, q_stride_head, kc, vc, block_table,
                            table_stride, max_pages, seq_lens, q_start, num_seqs, num_q_heads, num_kv_heads, head_dim,
                            block_size, scale, kv_dtype, k_scale, v_scale, num_splits, part_out, part_lse, stream);
  hkb::StepExtra x;
  x.ablate = ablate;
  return hkb::decode_impl(out, out_stride_tok, out_stride_head, q, q_stride_tok, q_stride_head, kc, vc, block_table,
                          table_stride, max_pages, seq_lens, q_start, num_seqs, num_q_heads, num_kv_heads, head_dim,
                          block_size, scale, kv_dtype, k_scale, v_scale, num_splits, part_out, part_lse, stream, &x);
}

extern "C" int hkb_decode_step(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                               const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                               const void* key, const void* value,
                               int64_t key_stride_tok, int64_t key_stride_head,
                               int64_t val_stride_tok, int64_t val_stride_head,
                               const void* slot_mapping, int slot_is_i64,
                               hkb_cache_t kc, hkb_cache_t vc,
                               const int32_t* block_table, int64_t table_stride, int max_pages,
                               const int32_t* seq_lens, const int32_t* q_start,
                               int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                               int block_size, float scale, int kv_dtype,
                               const float* k_scale, const float* v_scale,
                               int num_splits, float* part_out, float* part_lse, int32_t* arrivals, void* stream) {
  return hkb::step_impl(out, out_stride_tok, out_stride_head, 0, nullptr, q, q_stride_tok, q_stride_head, key, value,
                        key_stride_tok, key_stride_head, val_stride_tok, val_stride_head, slot_mapping, slot_is_i64, kc,
                        vc, block_table, table_stride, max_pages, seq_lens, q_start, num_seqs, num_q_heads, num_kv_heads,
                        head_dim, block_size, scale, kv_dtype, k_scale, v_scale, num_splits, part_out, part_lse, arrivals,
                        stream);
}

extern "C" int hkb_decode_step_record(float* rec_out, float* rec_lse,
                                      const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                                      const void* key, const void* value,
                                      int64_t key_stride_tok, int64_t key_stride_head,
                                      int64_t val_stride_tok, int64_t val_stride_head,
                                      const void* slot_mapping, int slot_is_i64,
                                      hkb_cache_t kc, hkb_cache_t vc,
                                      const int32_t* block_table, int64_t table_stride, int max_pages,
                                      const int32_t* seq_lens, const int32_t* q_start,
                                      int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                      int block_size, float scale, int kv_dtype,
                                      const float* k_scale, const float* v_scale,
                                      int num_splits, float* part_out, float* part_lse, void* stream) {
  return hkb::step_impl(rec_out, (int64_t)num_q_heads * head_dim, head_dim, 1, rec_lse, q, q_stride_tok, q_stride_head,
                        key, value, key_stride_tok, key_stride_head, val_stride_tok, val_stride_head, slot_mapping,
                        slot_is_i64, kc, vc, block_table, table_stride, max_pages, seq_lens, q_start, num_seqs,
                        num_q_heads, num_kv_heads, head_dim, block_size, scale, kv_dtype, k_scale, v_scale, num_splits,
                        part_out, part_lse, nullptr, stream);
}

extern "C" int hkb_merge(void* out, int64_t out_stride_tok, int64_t out_stride_head, int out_is_f32,
                         float* out_lse,
                         const float* part_out, int64_t part_stride_p, int64_t part_stride_seq,
                         const float* part_lse, int64_t lse_stride_p, int64_t lse_stride_seq,
                         int num_parts, int num_seqs, int num_q_heads, int head_dim,
                         const int32_t* seq_lens, const int32_t* q_start, void* stream) {
  using namespace hkb;
  const int rc = merge_check(out, out_stride_tok, out_stride_head, out_is_f32, part_out, part_stride_p, part_stride_seq,
                             part_lse, num_parts, num_seqs, num_q_heads, head_dim);
  if (rc != HKB_OK || num_seqs == 0) return rc;
  MergeArgs a;
  a.out = out; a.out_stride_tok = out_stride_tok; a.out_stride_head = out_stride_head;
  a.out_is_f32 = out_is_f32; a.out_lse = out_lse;
  a.part_out = part_out; a.part_stride_p = part_stride_p; a.part_stride_seq = part_stride_seq;
  a.part_lse = part_lse; a.lse_stride_p = lse_stride_p; a.lse_stride_seq = lse_stride_seq;
  a.num_parts = num_parts; a.num_q_heads = num_q_heads; a.head_dim = head_dim;
  a.seq_lens = seq_lens; a.q_start = q_start;
  // Few slots a sequence: a warp a (sequence, head). Many (a long sequence in a hundred pieces):
  // a CTA a (sequence, head), the parts spread over its warps -- unless the walk before it cut every
  // sequence into a handful of pieces only (many sequences share the rings): then most of the slots
  // are marked empty, a warp folds the few live ones in one round, and 8 heads share a CTA (measured
  // at 32 sequences x 1024 tokens, 64 slots: 3.8 against 5.9 us).
  const bool few_live = g_merge_hint.num_seqs == num_seqs && g_merge_hint.num_parts == num_parts && g_merge_hint.pieces <= MERGE_ROUND;
  if (num_parts > 32 && !few_live) {
    const dim3 grid(num_q_heads, num_seqs);
    if (head_dim == 128) merge_wide_kernel<4><<<grid, MERGE_WARPS * 32, 0, (cudaStream_t)stream>>>(a);
    else if (head_dim == 64) merge_wide_kernel<2><<<grid, MERGE_WARPS * 32, 0, (cudaStream_t)stream>>>(a);
    else merge_wide_kernel<8><<<grid, MERGE_WARPS * 32, 0, (cudaStream_t)stream>>>(a);
  } else {
    const dim3 grid((num_q_heads + MERGE_WARPS - 1) / MERGE_WARPS, num_seqs);
    if (head_dim == 128) merge_kernel<4><<<grid, MERGE_WARPS * 32, 0, (cudaStream_t)stream>>>(a);
    else if (head_dim == 64) merge_kernel<2><<<grid, MERGE_WARPS * 32, 0, (cudaStream_t)stream>>>(a);
    else merge_kernel<8><<<grid, MERGE_WARPS * 32, 0, (cudaStream_t)stream>>>(a);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}

// ---------------------------------------------------------------------------------
// The split decode on scratch built into the library, for callers that cannot allocate.
// ---------------------------------------------------------------------------------
// A fixed file-scope device array holds the split partials. The name below is only a
// host-side handle for the symbol: host code must not pass it to a kernel; the device
// address comes from cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) unsigned char hkb_static_scratch[HKB_STATIC_SCRATCH_BYTES];

namespace {

std::mutex g_static_mu;
void* g_static_ptr[64] = {};

// Device address of the built-in scratch on the current device; nullptr (and the CUDA error
// recorded) if the lookup fails. No allocation happens here: the array is part of the module.
void* static_scratch_address() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    hkb_tls_cuda_error = (int)(e != cudaSuccess ? e : cudaErrorInvalidDevice);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, hkb_static_scratch);
    if (e != cudaSuccess || !p) {
      hkb_tls_cuda_error = (int)e;
      (void)cudaGetLastError();
      return nullptr;
    }
    g_static_ptr[dev] = p;
  }
  return g_static_ptr[dev];
}

}  // namespace

extern "C" int hkb_paged_decode_static(void* out, int64_t out_stride_tok, int64_t out_stride_head,
                                       const void* q, int64_t q_stride_tok, int64_t q_stride_head,
                                       hkb_cache_t kc, hkb_cache_t vc,
                                       const int32_t* block_table, int64_t table_stride, int max_pages,
                                       const int32_t* seq_lens, const int32_t* q_start,
                                       int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                       int block_size, float scale, int kv_dtype,
                                       const float* k_scale, const float* v_scale,
                                       int num_splits, void* stream) {
  if (num_splits <= 1)   // one split writes the answer itself: no partials, nothing to hold
    return hkb_paged_decode(out, out_stride_tok, out_stride_head, q, q_stride_tok, q_stride_head, kc, vc, block_table,
                            table_stride, max_pages, seq_lens, q_start, num_seqs, num_q_heads, num_kv_heads, head_dim,
                            block_size, scale, kv_dtype, k_scale, v_scale, num_splits, nullptr, nullptr, stream);
  if (num_seqs < 0 || num_q_heads <= 0 || head_dim <= 0) return HKB_ERR_SIZE;
  if (num_seqs == 0) return HKB_OK;
  if (num_splits > HKB_MAX_SPLITS) return HKB_ERR_SPLITS;
  const size_t need = hkb_scratch_bytes(num_seqs, num_q_heads, head_dim, num_splits);
  if (need == 0 || need > (size_t)HKB_STATIC_SCRATCH_BYTES) return HKB_ERR_STATIC_SCRATCH;
  unsigned char* base = static_cast<unsigned char*>(static_scratch_address());
  if (!base) return HKB_ERR_CUDA;
  float* part_out = reinterpret_cast<float*>(base);
  float* part_lse = reinterpret_cast<float*>(base + hkb_scratch_lse_offset(num_seqs, num_q_heads, head_dim, num_splits));
  // The walk rewrites the lse of every (sequence, slot, head) before the merge reads any of
  // them -- a value, or -inf for a slot without tokens -- so what the last call left behind
  // in the array is never read and nothing needs clearing first.
  int rc = hkb_paged_decode(out, out_stride_tok, out_stride_head, q, q_stride_tok, q_stride_head, kc, vc, block_table,
                            table_stride, max_pages, seq_lens, q_start, num_seqs, num_q_heads, num_kv_heads, head_dim,
                            block_size, scale, kv_dtype, k_scale, v_scale, num_splits, part_out, part_lse, stream);
  if (rc != HKB_OK) return rc;
  return hkb_merge(out, out_stride_tok, out_stride_head, kv_dtype == HKB_KV_F16 ? 2 : 0, nullptr, part_out, (int64_t)num_q_heads * head_dim,
                   (int64_t)num_splits * num_q_heads * head_dim, part_lse, num_q_heads,
                   (int64_t)num_splits * num_q_heads, num_splits, num_seqs, num_q_heads, head_dim, seq_lens, q_start,
                   stream);
}
