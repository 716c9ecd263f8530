// The split decode as a persistent, balanced tile stream.
//
// hk-dsl cuts every sequence into the same number of splits and launches one workgroup a
// (request, kv head, split) (python/hk/ops/paged.py:171-194, 552-559): short sequences get
// tiny splits, long ones long splits, and every workgroup pays its own start-up. On B200 that
// costs a few microseconds a CTA wave and leaves a tail. Here the grid is sized to the
// machine instead -- eight to twelve warps an SM, as one to three CTAs -- and the work is dealt in equal shares:
//
//   * each kv head (x head chunk) is a plane with its own CTAs; inside a plane all sequences'
//     16-token tiles form ONE line, total = sum_i ceil(seq_len_i / 16) tiles, computed by every
//     CTA in its prologue with a warp scan over seq_lens (device values: graph-safe);
//   * a ring is one cp.async pipeline in shared memory with the warp(s) that consume it: one
//     warp on the tensor-core path; on the CUDA-core path two warps that each hold two of the
//     four query heads (half the registers a thread, twice the warps an SM) and fill the K and
//     the V tiles respectively;
//   * ring w of the plane's W rings owns tiles [w R, (w+1) R) of that line,
//     R = max(ceil(total / W), ceil(longest / (parts - 1)), 1): equal shares, cut where they
//     fall -- a share may end one sequence and begin the next;
//   * the warp's cp.async ring runs on across sequence boundaries (the loader has its own
//     cursor, NST-1 tiles ahead of the compute), so only the first tiles of a warp wait for memory;
//   * for every (sequence, piece) a ring writes one normalised partial + lse into slot
//     p = w - floor(base_i / R) of the sequence's `parts` slots; R's second term guarantees
//     p < parts. Slots no warp will write are marked lse = -inf by the plane's first CTA.
//     The LSE-merge kernel then folds a sequence's slots as it folds fixed splits.
//
// The whole decode step in this one launch (DecodeArgs::arrivals / new_k set; rings of one
// warp): the ring that owns a sequence's last tile first writes the step's new K/V row of
// that sequence into the cache -- its own later fetch of the tile then reads it back, no
// other ring of the plane touches that tile -- and the ring that finishes a sequence's last
// outstanding piece folds the partials (hkb_fold.cuh). This is hk-dsl's "cache write + walk +
// merge as <= 2 launches" (docs/history/17-the-decode-step-captured-whole.md:181-188), as one.
//
// `num_splits` of the C ABI is `parts` here: still a host-known power of two, still the row
// count of the caller's scratch, so plans and CUDA graphs behave as with fixed splits.
#pragma once

#include "hkb_decode.cuh"
#include "hkb_fold.cuh"

namespace hkb {

constexpr int STREAM_MIN_RANGE = 1;      // tiles: a small batch is spread over as many rings as it has tiles (latency, not bandwidth)
constexpr int STREAM_MAX_SEQS = 2048;    // rows of the prefix table kept in shared memory

// Barrier among the WPR warps that share a ring (a named barrier a ring; __syncwarp for one).
template <int WPR>
__device__ __forceinline__ void ring_sync(int ring) {
  if (WPR == 1) __syncwarp();
  else asm volatile("bar.sync %0, %1;\n" ::"r"(ring + 1), "n"(WPR * 32) : "memory");
}

template <class P, int RINGS>
struct WalkStream {
  static constexpr int WPR = P::WPR;
  static constexpr int THREADS = RINGS * WPR * 32;
  static constexpr int BASE_BYTES = (STREAM_MAX_SEQS + 2) * 4;
  static constexpr int SMEM_BYTES = RINGS * P::RING_SMEM + BASE_BYTES;

  template <int ABL = 0>
  __device__ static __forceinline__ void run(const DecodeArgs& a, uint8_t* smem, int num_seqs) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ring_id = warp / WPR, sub = warp % WPR;     // which ring, and which of its warps
    const int passes = P::passes(a.group);
    const int kvh = blockIdx.y / passes;
    const int h0 = (blockIdx.y % passes) * P::PASS_HEADS + sub * P::HEADS;   // this warp's first head in the group
    const int nh = max(0, min(P::HEADS, a.group - h0));
    const int hq0 = kvh * a.group + h0;
    const int parts = a.num_splits;
    int* base = reinterpret_cast<int*>(smem + RINGS * P::RING_SMEM);   // [num_seqs + 1] exclusive tile counts, then the max

    // ---- prologue: the line of tiles ----
    // Every thread fetches the lengths of its share of the sequences at once (one trip to memory for the
    // CTA, however many sequences: a warp that fetched them 32 at a time inside its scan paid a trip a
    // round, 8 of them -- 5 us -- at 256 sequences); then one warp scans the tile counts in shared memory.
#pragma unroll 4
    for (int i = threadIdx.x; i < num_seqs; i += THREADS) {
      int len = max(__ldg(a.seq_lens + i), 0);
      if (a.q_start && __ldg(a.q_start + i + 1) <= __ldg(a.q_start + i)) len = 0;   // no query: nothing to walk
      base[i] = (len + TILE_TOKENS - 1) / TILE_TOKENS;
    }
    __syncthreads();
    if (warp == 0) {
      int running = 0, longest = 0;
      for (int s0 = 0; s0 < num_seqs; s0 += 32) {
        const int i = s0 + lane;
        const int nt = i < num_seqs ? base[i] : 0;
        int incl = nt;
#pragma unroll
        for (int x = 1; x < 32; x <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, incl, x);
          if (lane >= x) incl += y;
        }
        if (i < num_seqs) base[i] = running + incl - nt;
        running += __shfl_sync(0xffffffffu, incl, 31);
        longest = max(longest, nt);
      }
#pragma unroll
      for (int x = 16; x > 0; x >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, x));
      if (lane == 0) { base[num_seqs] = running; base[num_seqs + 1] = longest; }
    }
    __syncthreads();
    const int total = base[num_seqs], longest = base[num_seqs + 1];
    const int plane_rings = gridDim.x * RINGS;
    int range = max((total + plane_rings - 1) / plane_rings, STREAM_MIN_RANGE);
    range = max(range, (longest + parts - 2) / max(parts - 1, 1));

    const bool fold = WPR == 1 && a.arrivals != nullptr;
    // Housekeeping every ring owes the plane, run once its first tiles are on their way (an idle ring
    // runs it before it leaves): it only writes, so it costs the stream no latency.
    auto housekeeping = [&]() {
      if (!fold) {
        // slots that no ring of this plane will write: marked by all the plane's CTAs, a slice each
        // (every warp marks the heads it owns)
        for (int x = blockIdx.x * (RINGS * 32) + ring_id * 32 + lane; x < num_seqs * parts; x += gridDim.x * RINGS * 32) {
          const int i = x / parts, p = x % parts;
          const int nt = base[i + 1] - base[i];
          const int np = nt > 0 ? (base[i] + nt - 1) / range - base[i] / range + 1 : 0;
          if (p >= np) {
            float* pl = a.part_lse + (int64_t)(i * parts + p) * a.num_q_heads + hq0;
            for (int h = 0; h < nh; ++h) pl[h] = -INFINITY;
          }
        }
      } else {
        // folding in this launch: no marks are read, but a sequence without tokens has no ring to
        // write its output row -- zeros, as the merge kernel gives it
        for (int i = blockIdx.x * (RINGS * 32) + ring_id * 32 + lane; i < num_seqs; i += gridDim.x * RINGS * 32) {
          if (base[i + 1] != base[i]) continue;
          int row = i;
          if (a.q_start) {
            row = __ldg(a.q_start + i);
            if (__ldg(a.q_start + i + 1) <= row) continue;   // no query row either
          }
          for (int h = 0; h < nh; ++h) {
            __nv_bfloat16* o = a.out + (int64_t)row * a.out_stride_tok + (int64_t)(hq0 + h) * a.out_stride_head;
            for (int d = 0; d < P::HEAD_DIM; d += 2) *reinterpret_cast<__nv_bfloat162*>(o + d) = __floats2bfloat162_rn(0.f, 0.f);
          }
        }
      }
    };

    const int w = blockIdx.x * RINGS + ring_id;
    const int64_t g_lo64 = (int64_t)w * range;
    if (g_lo64 >= total) {                                // both warps of a ring leave together
      housekeeping();
      return;
    }
    const int g_lo = (int)g_lo64;
    const int g_hi = min(total, g_lo + range);
    const int n = g_hi - g_lo;

    // the sequence that holds tile g_lo: the last i with base[i] <= g_lo
    int lo = 0, hi = num_seqs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (base[mid] <= g_lo) lo = mid; else hi = mid - 1;
    }

    float qs = a.scale * LOG2E;
    float vs = 1.f;
    if (a.k_scale) qs *= __ldg(a.k_scale);
    if (a.v_scale) vs = __ldg(a.v_scale);

    typename P::Loader ld;
    ld.kbase = a.k + (int64_t)kvh * a.k_stride_head;
    ld.vbase = a.v + (int64_t)kvh * a.v_stride_head;
    ld.ksb = a.k_stride_block; ld.kst = a.k_stride_token;
    ld.vsb = a.v_stride_block; ld.vst = a.v_stride_token;
    ld.tiles_per_page = a.tiles_per_page; ld.num_blocks = a.num_blocks;
    ld.prepare(lane);
    PageIds ids;
    ids.max_pages = a.max_pages; ids.tiles_per_page = a.tiles_per_page;

    const uint32_t ring = smem_u32(smem) + ring_id * P::RING_SMEM;

    // loader cursor (each warp of the ring keeps its own and issues its share of every tile)
    int seq_l = lo, gl = g_lo;
    bool fresh = true;
    auto issue = [&](int stage_idx) {
      while (gl >= base[seq_l + 1]) { ++seq_l; fresh = true; }
      const int t = gl - base[seq_l];
      if (fresh) {
        ids.row = a.block_table + (int64_t)seq_l * a.table_stride;
        ids.t_hi = min(base[seq_l + 1], g_hi) - base[seq_l];
        if (!(ABL & ABL_PAGE)) ids.init(t, lane);
        fresh = false;
      }
      if (WPR == 1 && a.new_k && t == base[seq_l + 1] - base[seq_l] - 1) {
        // the sequence's last tile: the step's new token goes into the cache first (this kv head's
        // K row and V row, one 16-byte chunk a lane), then the tile is fetched with it inside
        const int row = a.q_start ? __ldg(a.q_start + seq_l) : seq_l;
        const int64_t slot = a.slot_is_i64 ? (int64_t)__ldg(reinterpret_cast<const long long*>(a.slots) + row)
                                           : (int64_t)__ldg(reinterpret_cast<const int*>(a.slots) + row);
        if (slot >= 0 && slot < (int64_t)a.num_blocks * a.block_size) {
          constexpr int CH = P::HEAD_DIM / 8;
          const int64_t blk = slot / a.block_size, off = slot - blk * a.block_size;
          for (int c = lane; c < 2 * CH; c += 32) {
            const bool is_v = c >= CH;
            const int cc = is_v ? c - CH : c;
            const __nv_bfloat16* src = is_v ? a.new_v + (int64_t)row * a.new_v_stride_tok + (int64_t)kvh * a.new_v_stride_head
                                            : a.new_k + (int64_t)row * a.new_k_stride_tok + (int64_t)kvh * a.new_k_stride_head;
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + cc * 8));
            uint8_t* dst = const_cast<uint8_t*>(is_v ? ld.vbase + blk * ld.vsb + off * ld.vst : ld.kbase + blk * ld.ksb + off * ld.kst);
            if (P::ES == 2) *reinterpret_cast<uint4*>(dst + cc * 16) = v;
            else *reinterpret_cast<uint2*>(dst + cc * 8) = quantize_chunk_e4m3(v, __ldg(is_v ? a.v_scale : a.k_scale));
          }
        }
        __threadfence_block();
        __syncwarp();
      }
      const uint32_t stage = ring + stage_idx * P::STAGE_BYTES;
      if (ABL & (ABL_PAGE | ABL_KLOAD | ABL_VLOAD)) {      // attribution builds: no table read, or one of the copies left out
        const int id = (ABL & ABL_PAGE) ? gl % a.num_blocks : ids.get(t, lane);
        if (!(ABL & ABL_KLOAD)) ld.issue_one(stage, t, id, lane, 0);
        if (!(ABL & ABL_VLOAD)) ld.issue_one(stage, t, id, lane, 1);
      } else if (WPR == 1) ld.issue(stage, t, ids.get(t, lane), lane);
      else ld.issue_one(stage, t, ids.get(t, lane), lane, sub);
      ++gl;
    };

#pragma unroll
    for (int k = 0; k < P::STAGES - 1; ++k) {
      if (k < n) issue(k);
      cp_async_commit();
    }

    // compute cursor
    // The ring's first sequence is entered here, before the first tile is waited for, so that the
    // loads of its query rows fly together with the tiles just requested.
    typename P::State st;
    int seq_c = lo, seq_base = base[lo], seq_end = base[lo + 1];
    int n_tiles = seq_end - seq_base, seq_len = max(__ldg(a.seq_lens + lo), 0);
    if (nh > 0) P::begin(st, a, a.q_start ? __ldg(a.q_start + lo) : lo, hq0, nh, lane, qs);
    housekeeping();
    int sc = 0, sl = P::STAGES - 1;   // ring stages of the compute and of the loader
    int owe_seq[2] = {-1, -1}, owe_p[2] = {0, 0}, owe_np[2] = {0, 0};   // folds to run after the last tile
    auto close_piece = [&]() {
      const int p = min(w - seq_base / range, parts - 1);   // < parts by the choice of `range`
      P::end(st, lane, nh, vs, a.part_out + ((int64_t)(seq_c * parts + p) * a.num_q_heads + hq0) * P::HEAD_DIM,
             a.part_lse + (int64_t)(seq_c * parts + p) * a.num_q_heads + hq0);
      if (fold) {
        const int np = (seq_end - 1) / range - seq_base / range + 1;   // pieces of this sequence
        if (np == 1) {
          Fold<P::HEAD_DIM, P::HEADS>::single(a, seq_c, hq0, nh, lane);
        } else if (Fold<P::HEAD_DIM, P::HEADS>::count_in(
                       a.arrivals + ((int64_t)blockIdx.y * num_seqs + seq_c) * ARRIVAL_INTS, p, np, lane)) {
          if (owe_seq[0] < 0) { owe_seq[0] = seq_c; owe_p[0] = p; owe_np[0] = np; }
          else { owe_seq[1] = seq_c; owe_p[1] = p; owe_np[1] = np; }
        }
      }
    };
    for (int k = 0; k < n; ++k) {
      cp_async_wait<P::STAGES - 2>();
      ring_sync<WPR>(ring_id);
      if (k + P::STAGES - 1 < n) issue(sl);
      cp_async_commit();
      const int g = g_lo + k;
      if (g >= seq_end) {
        if (nh > 0) close_piece();   // the piece of the sequence just finished
        ++seq_c;
        while (g >= base[seq_c + 1]) ++seq_c;
        seq_base = base[seq_c];
        seq_end = base[seq_c + 1];
        n_tiles = seq_end - seq_base;
        seq_len = max(__ldg(a.seq_lens + seq_c), 0);
        const int row = a.q_start ? __ldg(a.q_start + seq_c) : seq_c;
        if (nh > 0) P::begin(st, a, row, hq0, nh, lane, qs);
      }
      const int t = g - seq_base;
      if (nh > 0) {
        if constexpr (ABL != 0) P::template step<ABL>(st, ring, sc, t * TILE_TOKENS, seq_len, t == n_tiles - 1, lane, qs);
        else P::step(st, ring, sc, t * TILE_TOKENS, seq_len, t == n_tiles - 1, lane, qs);
      }
      sc = sc + 1 == P::STAGES ? 0 : sc + 1;
      sl = sl + 1 == P::STAGES ? 0 : sl + 1;
    }
    cp_async_wait<0>();
    if (nh > 0) close_piece();
    if (fold) {
#pragma unroll 1
      for (int k = 0; k < 2; ++k) {
        const int s = k ? owe_seq[1] : owe_seq[0];
        if (s < 0) break;
        Fold<P::HEAD_DIM, P::HEADS>::finish(a, a.arrivals + ((int64_t)blockIdx.y * num_seqs + s) * ARRIVAL_INTS, s,
                                            k ? owe_p[1] : owe_p[0], k ? owe_np[1] : owe_np[0], hq0, nh, lane);
      }
    }
  }
};

template <class P, int RINGS>
__global__ void __launch_bounds__(RINGS * P::WPR * 32, P::MIN_CTAS) walk_stream_kernel(const DecodeArgs a, int num_seqs) {
  extern __shared__ __align__(128) uint8_t hkb_smem[];
  WalkStream<P, RINGS>::run(a, hkb_smem, num_seqs);
}

// The same kernel with stages left out (ABL_* mask), for attribution measurements only.
template <class P, int RINGS, int ABL>
__global__ void __launch_bounds__(RINGS * P::WPR * 32, P::MIN_CTAS) walk_stream_ablated_kernel(const DecodeArgs a, int num_seqs) {
  extern __shared__ __align__(128) uint8_t hkb_smem[];
  WalkStream<P, RINGS>::template run<ABL>(a, hkb_smem, num_seqs);
}

}  // namespace hkb
