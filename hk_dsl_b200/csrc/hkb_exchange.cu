// The exchange step of a KV axis cut across GPUs, without a library collective: the fold of a
// rank's splits writes its record straight into every peer's gather buffer over NVLink (plain peer
// stores into memory the ranks mapped into each other), and the final merge waits -- boundedly --
// for every rank's record before it folds them.
//
// (hkb_kvsplit_exchange does both in ONE launch, with a flag a row instead of a flag a rank; the two
// separate kernels stay as its comparison arm and for callers that want work between the two.)
//
// A step on every rank, on one stream: walk (hkb_paged_decode, partials into local scratch) ->
// hkb_kvsplit_push (fold of the local splits; the record goes to all peers, then one flag a peer)
// -> hkb_kvsplit_merge (wait for all ranks' flags of this step, fold the records). Against an
// all-gather between two launches this saves the collective's launch and protocol latency: the
// record is 66 KB at the long-context shape, far below what a ring or tree is built to move.
//
// Protocol. Every rank keeps a step counter `epoch` in its own memory (zero before the first
// step; the merge kernel's last CTA increments it), so nothing on the host changes between steps
// and a captured graph replays. Gather buffers and flags are double-buffered by the step's parity:
// a rank that is one step ahead writes the other half. A push CTA stores its part of the record to
// every peer, fences at system scope and counts itself done; the CTA that counts last stores
// epoch + 1 into this rank's flag on every peer. The merge kernel's CTAs poll the flags of all
// ranks (volatile loads, at most `spin_limit` polls a flag); if one does not arrive in time the
// CTA sets the rank's error word, skips the fold and returns -- the context stays usable, and the
// host reads the word. No multimem, no multicast: peer pointers only.
//
// hk-dsl has no counterpart: it cuts the KV axis inside one GPU (python/hk/ops/paged.py:171-194)
// and leaves tensor parallelism to the engine.
#include "hkb_fold_wide.cuh"

extern thread_local int hkb_tls_cuda_error;

namespace hkb {

constexpr int XCH_WARPS = 8;

struct PushArgs {
  const float* part_out;   // (seqs, splits, heads, d) normalised partials of this rank
  const float* part_lse;   // (seqs, splits, heads)
  int num_splits, num_q_heads, head_dim, num_seqs;
  int world, rank;
  float* gather[8];        // peer r's gather buffer as mapped here
  uint32_t* flags[8];      // peer r's flag block as mapped here
  uint32_t* epoch;         // this rank's step counter
  uint32_t* done;          // this rank's CTA counter (zero between launches)
  int64_t rec_floats;      // floats of one record (out then lse, padded to 4)
};

// One CTA a (sequence, head): the fold of the rank's live splits (WideFold: lse = -inf marks a split
// without tokens; its memory is never read), then warp 0 stores the normalised fp32 row and its lse
// into slot `rank` of the step's half of every peer's gather buffer.
template <int VEC>
__global__ void __launch_bounds__(XCH_WARPS * 32) kvsplit_push_kernel(const PushArgs a) {
  __shared__ typename WideFold<VEC, XCH_WARPS>::Smem sm;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, seq = blockIdx.y;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch);
  const int64_t half_off = (int64_t)(epoch & 1u) * a.world * a.rec_floats + (int64_t)a.rank * a.rec_floats;
  const float* lse = a.part_lse + (int64_t)seq * a.num_splits * a.num_q_heads + h;
  const float* po = a.part_out + ((int64_t)seq * a.num_splits * a.num_q_heads + h) * a.head_dim + lane * VEC;
  float acc[VEC], den, mx;
  WideFold<VEC, XCH_WARPS>::run(sm, lse, a.num_q_heads, po, (int64_t)a.num_q_heads * a.head_dim, a.num_splits, false, acc, den, mx);
  if (warp == 0) {
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const float out_lse = den > 0.f ? mx + __logf(den) : -INFINITY;
    const int64_t row = ((int64_t)seq * a.num_q_heads + h) * a.head_dim + lane * VEC;
    const int64_t lse_at = (int64_t)a.num_seqs * a.num_q_heads * a.head_dim + (int64_t)seq * a.num_q_heads + h;
    for (int r = 0; r < a.world; ++r) {
      float* g = a.gather[r] + half_off;
#pragma unroll
      for (int v = 0; v < VEC; v += 2) *reinterpret_cast<float2*>(g + row + v) = make_float2(acc[v] * inv, acc[v + 1] * inv);
      if (lane == 0) g[lse_at] = out_lse;
    }
    // every store of this CTA is visible system-wide before it counts itself done; the last CTA raises the flags
    __threadfence_system();
    __syncwarp();
    if (lane == 0) {
      const uint32_t total = gridDim.x * gridDim.y;
      if (atomicAdd(a.done, 1u) == total - 1) {
        *a.done = 0u;
        __threadfence_system();
        for (int r = 0; r < a.world; ++r)
          *reinterpret_cast<volatile uint32_t*>(a.flags[r] + (epoch & 1u) * 8 + a.rank) = epoch + 1u;
        __threadfence_system();
      }
    }
  }
}

struct XMergeArgs {
  void* out;
  int64_t out_stride_tok, out_stride_head;
  int out_kind;            // 0 bf16, 2 fp16
  const float* gather;     // this rank's gather buffer (own memory)
  uint32_t* flags;         // this rank's flag block (own memory)
  uint32_t* epoch;
  uint32_t* done;          // CTA counter of this kernel (zero between launches)
  int32_t* error;          // set to 1 + the rank whose record did not arrive in time
  int world, num_q_heads, head_dim, num_seqs;
  int64_t rec_floats;
  int spin_limit;
};

template <int VEC>
__global__ void __launch_bounds__(XCH_WARPS * 32) kvsplit_merge_kernel(const XMergeArgs a) {
  __shared__ int s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * XCH_WARPS + warp, seq = blockIdx.y;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch);
  // one thread a rank polls that rank's flag of this step: bounded, and a miss is reported, not waited out
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world) {
    const volatile uint32_t* f = reinterpret_cast<const volatile uint32_t*>(a.flags + (epoch & 1u) * 8 + threadIdx.x);
    int polls = 0;
    while (*f != epoch + 1u) {
      if (++polls > a.spin_limit) {
        s_ok = 0;
        atomicCAS(a.error, 0, 1 + (int)threadIdx.x);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  __threadfence_system();          // the records were written before the flags: order this CTA's reads after the flags
  if (s_ok && h < a.num_q_heads) {
    const float* base = a.gather + (int64_t)(epoch & 1u) * a.world * a.rec_floats;
    const int64_t row = ((int64_t)seq * a.num_q_heads + h) * a.head_dim + lane * VEC;
    const int64_t lse_at = (int64_t)a.num_seqs * a.num_q_heads * a.head_dim + (int64_t)seq * a.num_q_heads + h;
    float lp[8];
    float mx = -INFINITY;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      lp[r] = r < a.world ? *reinterpret_cast<const volatile float*>(base + r * a.rec_floats + lse_at) : -INFINITY;
      mx = fmaxf(mx, lp[r]);
    }
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
    float den = 0.f;
    if (mx != -INFINITY) {
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (lp[r] == -INFINITY) continue;
        const float w = __expf(lp[r] - mx);
        const float* xp = base + r * a.rec_floats + row;
#pragma unroll
        for (int v = 0; v < VEC; v += 2) {
          const float2 t = __ldcv(reinterpret_cast<const float2*>(xp + v));   // written by a peer: not through a stale cache line
          acc[v] = fmaf(w, t.x, acc[v]);
          acc[v + 1] = fmaf(w, t.y, acc[v + 1]);
        }
        den += w;
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const int64_t off = (int64_t)seq * a.out_stride_tok + (int64_t)h * a.out_stride_head + lane * VEC;
    if (a.out_kind == 2) {
      __half* o = reinterpret_cast<__half*>(a.out) + off;
#pragma unroll
      for (int v = 0; v < VEC; v += 2) *reinterpret_cast<__half2*>(o + v) = __floats2half2_rn(acc[v] * inv, acc[v + 1] * inv);
    } else {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out) + off;
#pragma unroll
      for (int v = 0; v < VEC; v += 2)
        *reinterpret_cast<__nv_bfloat162*>(o + v) = __floats2bfloat162_rn(acc[v] * inv, acc[v + 1] * inv);
    }
  }
  // the step is over on this rank when its last CTA is: the counter moves on for the next step
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t total = gridDim.x * gridDim.y;
    if (atomicAdd(a.done, 1u) == total - 1) {
      *a.done = 0u;
      *reinterpret_cast<volatile uint32_t*>(a.epoch) = epoch + 1u;
    }
  }
}

// Both steps in one launch. A CTA a (sequence, head): it folds the rank's splits, stores its row of the
// record into every peer, fences, raises ITS OWN flag on every peer -- a flag a (rank, row), not one a
// rank, so no CTA waits for the slowest CTA of its grid -- then waits (boundedly) for the same row's flag
// of every rank and folds the eight rows. Against push + merge this saves a launch, the count to the last
// CTA before any flag goes up, and the second kernel's start. CTAs are dispatched in index order on every
// rank and wait only for the CTA of their own index, so the lowest unfinished CTA of every rank always has
// its partners resident or done: the wait cannot starve a grid larger than the GPUs hold at once.
struct XchgArgs {
  PushArgs p;              // flags[] unused
  uint32_t* row_flags[8];  // peer r's per-row flags as mapped here: [parity][rank][row]
  uint32_t* my_row_flags;
  void* out;
  int64_t out_stride_tok, out_stride_head;
  int out_kind;            // 0 bf16, 2 fp16
  const float* my_gather;  // this rank's gather buffer (own memory)
  int32_t* error;
  int spin_limit;
};

template <int VEC>
__global__ void __launch_bounds__(XCH_WARPS * 32) kvsplit_exchange_kernel(const XchgArgs x) {
  __shared__ typename WideFold<VEC, XCH_WARPS>::Smem sm;
  const PushArgs& a = x.p;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, seq = blockIdx.y;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch);
  const int64_t rows = (int64_t)a.num_seqs * a.num_q_heads, row_id = (int64_t)seq * a.num_q_heads + h;
  const int64_t half = (int64_t)(epoch & 1u) * a.world * a.rec_floats;
  const float* lse = a.part_lse + (int64_t)seq * a.num_splits * a.num_q_heads + h;
  const float* po = a.part_out + ((int64_t)seq * a.num_splits * a.num_q_heads + h) * a.head_dim + lane * VEC;
  float acc[VEC], den, mx;
  WideFold<VEC, XCH_WARPS>::run(sm, lse, a.num_q_heads, po, (int64_t)a.num_q_heads * a.head_dim, a.num_splits, false, acc, den, mx);
  if (warp != 0) return;
  const int64_t row = row_id * a.head_dim + lane * VEC;
  const int64_t lse_at = rows * a.head_dim + row_id;
  {
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const float out_lse = den > 0.f ? mx + __logf(den) : -INFINITY;
    for (int r = 0; r < a.world; ++r) {
      float* g = a.gather[r] + half + (int64_t)a.rank * a.rec_floats;
#pragma unroll
      for (int v = 0; v < VEC; v += 2) *reinterpret_cast<float2*>(g + row + v) = make_float2(acc[v] * inv, acc[v + 1] * inv);
      if (lane == 0) g[lse_at] = out_lse;
    }
  }
  // the row is visible system-wide before its flag: every lane fences its own stores, then a lane a peer raises the flag
  __threadfence_system();
  __syncwarp();
  const int64_t flag_at = ((int64_t)(epoch & 1u) * 8 + a.rank) * rows + row_id;
  if (lane < a.world) *reinterpret_cast<volatile uint32_t*>(x.row_flags[lane] + flag_at) = epoch + 1u;
  // a lane a rank polls that rank's flag of this row and step: bounded, and a miss is reported, not waited out
  // (an acquire load at system scope: the rows' reads below cannot move ahead of it -- the other lanes' reads
  // follow the warp vote -- which is what a second system-scope fence was here for, at a few microseconds)
  bool ok = true;
  if (lane < a.world) {
    const uint32_t* f = x.my_row_flags + ((int64_t)(epoch & 1u) * 8 + lane) * rows + row_id;
    int polls = 0;
    while (true) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(f) : "memory");
      if (seen == epoch + 1u) break;
      if (++polls > x.spin_limit) {
        ok = false;
        atomicCAS(x.error, 0, 1 + lane);
        break;
      }
      __nanosleep(64);
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    const float* base = x.my_gather + half;
    float lp[8];
    float m2 = -INFINITY;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      lp[r] = r < a.world ? *reinterpret_cast<const volatile float*>(base + r * a.rec_floats + lse_at) : -INFINITY;
      m2 = fmaxf(m2, lp[r]);
    }
    float o[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) o[v] = 0.f;
    float d2 = 0.f;
    if (m2 != -INFINITY) {
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (lp[r] == -INFINITY) continue;
        const float w = __expf(lp[r] - m2);
        const float* xp = base + r * a.rec_floats + row;
#pragma unroll
        for (int v = 0; v < VEC; v += 2) {
          const float2 t = __ldcv(reinterpret_cast<const float2*>(xp + v));   // written by a peer: not through a stale cache line
          o[v] = fmaf(w, t.x, o[v]);
          o[v + 1] = fmaf(w, t.y, o[v + 1]);
        }
        d2 += w;
      }
    }
    const float inv = d2 > 0.f ? 1.f / d2 : 0.f;
    const int64_t off = (int64_t)seq * x.out_stride_tok + (int64_t)h * x.out_stride_head + lane * VEC;
    if (x.out_kind == 2) {
      __half* op = reinterpret_cast<__half*>(x.out) + off;
#pragma unroll
      for (int v = 0; v < VEC; v += 2) *reinterpret_cast<__half2*>(op + v) = __floats2half2_rn(o[v] * inv, o[v + 1] * inv);
    } else {
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(x.out) + off;
#pragma unroll
      for (int v = 0; v < VEC; v += 2)
        *reinterpret_cast<__nv_bfloat162*>(op + v) = __floats2bfloat162_rn(o[v] * inv, o[v + 1] * inv);
    }
  }
  // the step is over on this rank when its last CTA is: the counter moves on for the next step
  if (lane == 0) {
    const uint32_t total = gridDim.x * gridDim.y;
    if (atomicAdd(a.done, 1u) == total - 1) {
      *a.done = 0u;
      *reinterpret_cast<volatile uint32_t*>(a.epoch) = epoch + 1u;
    }
  }
}

static int64_t record_floats(int num_seqs, int num_q_heads, int head_dim) {
  const int64_t n = (int64_t)num_seqs * num_q_heads * (head_dim + 1);
  return (n + 3) / 4 * 4;
}

}  // namespace hkb

extern "C" size_t hkb_exchange_gather_bytes(int world, int num_seqs, int num_q_heads, int head_dim) {
  if (world < 1 || world > 8 || num_seqs <= 0 || num_q_heads <= 0 || head_dim <= 0) return 0;
  return (size_t)(2 * world * hkb::record_floats(num_seqs, num_q_heads, head_dim)) * sizeof(float);
}

// two parity halves of eight flags, then the step counter, the two CTA counters and the error word
extern "C" size_t hkb_exchange_state_bytes(void) { return (16 + 4) * sizeof(uint32_t); }

// the state block of hkb_kvsplit_exchange: the 20 words above, then a flag a (parity, rank, row)
extern "C" size_t hkb_exchange_state_bytes_rows(int num_seqs, int num_q_heads) {
  if (num_seqs <= 0 || num_q_heads <= 0) return 0;
  return (size_t)(20 + 2 * 8 * (int64_t)num_seqs * num_q_heads) * sizeof(uint32_t);
}

extern "C" int hkb_kvsplit_exchange(hkb_exchange_t x, const float* part_out, const float* part_lse, int num_splits,
                                    void* out, int64_t out_stride_tok, int64_t out_stride_head, int out_kind,
                                    int num_seqs, int num_q_heads, int head_dim, int spin_limit, void* stream) {
  using namespace hkb;
  if (x.world < 1 || x.world > 8 || x.rank < 0 || x.rank >= x.world) return HKB_ERR_SIZE;
  if (num_seqs < 0 || num_q_heads <= 0 || num_splits < 1 || num_splits > HKB_MAX_SPLITS || spin_limit < 1) return HKB_ERR_SIZE;
  if (num_seqs == 0) return HKB_OK;
  if (num_seqs > 65535) return HKB_ERR_SIZE;
  if (!part_out || !part_lse || !out || !x.state[x.rank] || !x.gather[x.rank]) return HKB_ERR_NULL;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return HKB_ERR_HEAD_DIM;
  if (out_kind != 0 && out_kind != 2) return HKB_ERR_DTYPE;
  if ((out_stride_tok | out_stride_head) % 4) return HKB_ERR_STRIDE;
  if ((uintptr_t)part_out % 16 || (uintptr_t)out % 8) return HKB_ERR_ALIGN;
  XchgArgs a;
  a.p.part_out = part_out; a.p.part_lse = part_lse;
  a.p.num_splits = num_splits; a.p.num_q_heads = num_q_heads; a.p.head_dim = head_dim; a.p.num_seqs = num_seqs;
  a.p.world = x.world; a.p.rank = x.rank;
  for (int r = 0; r < 8; ++r) {
    a.p.gather[r] = r < x.world ? static_cast<float*>(x.gather[r]) : nullptr;
    a.p.flags[r] = nullptr;
    a.row_flags[r] = r < x.world && x.state[r] ? static_cast<uint32_t*>(x.state[r]) + 20 : nullptr;
    if (r < x.world && (!a.p.gather[r] || !a.row_flags[r] || (uintptr_t)a.p.gather[r] % 16)) return HKB_ERR_NULL;
  }
  uint32_t* mine = static_cast<uint32_t*>(x.state[x.rank]);
  a.p.epoch = mine + 16; a.p.done = mine + 17;
  a.p.rec_floats = record_floats(num_seqs, num_q_heads, head_dim);
  a.my_row_flags = mine + 20;
  a.out = out; a.out_stride_tok = out_stride_tok; a.out_stride_head = out_stride_head; a.out_kind = out_kind;
  a.my_gather = static_cast<const float*>(x.gather[x.rank]);
  a.error = reinterpret_cast<int32_t*>(mine + 19);
  a.spin_limit = spin_limit;
  const dim3 grid(num_q_heads, num_seqs);
  cudaStream_t st = (cudaStream_t)stream;
  if (head_dim == 128) kvsplit_exchange_kernel<4><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  else if (head_dim == 64) kvsplit_exchange_kernel<2><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  else kvsplit_exchange_kernel<8><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}

extern "C" int hkb_kvsplit_push(hkb_exchange_t x, const float* part_out, const float* part_lse, int num_splits,
                                int num_seqs, int num_q_heads, int head_dim, void* stream) {
  using namespace hkb;
  if (x.world < 1 || x.world > 8 || x.rank < 0 || x.rank >= x.world) return HKB_ERR_SIZE;
  if (num_seqs < 0 || num_q_heads <= 0 || num_splits < 1 || num_splits > HKB_MAX_SPLITS) return HKB_ERR_SIZE;
  if (num_seqs == 0) return HKB_OK;
  if (num_seqs > 65535) return HKB_ERR_SIZE;
  if (!part_out || !part_lse || !x.state[x.rank]) return HKB_ERR_NULL;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return HKB_ERR_HEAD_DIM;
  if ((uintptr_t)part_out % 16) return HKB_ERR_ALIGN;
  PushArgs a;
  a.part_out = part_out; a.part_lse = part_lse;
  a.num_splits = num_splits; a.num_q_heads = num_q_heads; a.head_dim = head_dim; a.num_seqs = num_seqs;
  a.world = x.world; a.rank = x.rank;
  for (int r = 0; r < 8; ++r) {
    a.gather[r] = r < x.world ? static_cast<float*>(x.gather[r]) : nullptr;
    a.flags[r] = r < x.world ? static_cast<uint32_t*>(x.state[r]) : nullptr;
    if (r < x.world && (!a.gather[r] || !a.flags[r] || (uintptr_t)a.gather[r] % 16)) return HKB_ERR_NULL;
  }
  uint32_t* mine = static_cast<uint32_t*>(x.state[x.rank]);
  a.epoch = mine + 16; a.done = mine + 17;
  a.rec_floats = record_floats(num_seqs, num_q_heads, head_dim);
  const dim3 grid(num_q_heads, num_seqs);
  cudaStream_t st = (cudaStream_t)stream;
  if (head_dim == 128) kvsplit_push_kernel<4><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  else if (head_dim == 64) kvsplit_push_kernel<2><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  else kvsplit_push_kernel<8><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}

extern "C" int hkb_kvsplit_merge(hkb_exchange_t x, void* out, int64_t out_stride_tok, int64_t out_stride_head, int out_kind,
                                 int num_seqs, int num_q_heads, int head_dim, int spin_limit, void* stream) {
  using namespace hkb;
  if (x.world < 1 || x.world > 8 || x.rank < 0 || x.rank >= x.world) return HKB_ERR_SIZE;
  if (num_seqs < 0 || num_q_heads <= 0 || spin_limit < 1) return HKB_ERR_SIZE;
  if (num_seqs == 0) return HKB_OK;
  if (num_seqs > 65535) return HKB_ERR_SIZE;
  if (!out || !x.gather[x.rank] || !x.state[x.rank]) return HKB_ERR_NULL;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return HKB_ERR_HEAD_DIM;
  if (out_kind != 0 && out_kind != 2) return HKB_ERR_DTYPE;
  if ((out_stride_tok | out_stride_head) % 4) return HKB_ERR_STRIDE;
  if ((uintptr_t)out % 8) return HKB_ERR_ALIGN;
  XMergeArgs a;
  a.out = out; a.out_stride_tok = out_stride_tok; a.out_stride_head = out_stride_head; a.out_kind = out_kind;
  a.gather = static_cast<const float*>(x.gather[x.rank]);
  uint32_t* mine = static_cast<uint32_t*>(x.state[x.rank]);
  a.flags = mine; a.epoch = mine + 16; a.done = mine + 18; a.error = reinterpret_cast<int32_t*>(mine + 19);
  a.world = x.world; a.num_q_heads = num_q_heads; a.head_dim = head_dim; a.num_seqs = num_seqs;
  a.rec_floats = record_floats(num_seqs, num_q_heads, head_dim);
  a.spin_limit = spin_limit;
  const dim3 grid((num_q_heads + XCH_WARPS - 1) / XCH_WARPS, num_seqs);
  cudaStream_t st = (cudaStream_t)stream;
  if (head_dim == 128) kvsplit_merge_kernel<4><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  else if (head_dim == 64) kvsplit_merge_kernel<2><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  else kvsplit_merge_kernel<8><<<grid, XCH_WARPS * 32, 0, st>>>(a);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}
