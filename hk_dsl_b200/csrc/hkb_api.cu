// Host-only entry points: the split planner, scratch sizing, device facts, status text.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/hkb.h"

thread_local int hkb_tls_cuda_error = 0;

namespace {

struct DeviceFacts {
  std::once_flag once;
  int sm_count = 0;
};
DeviceFacts g_facts[64];

}  // namespace

extern "C" int hkb_sm_count(int device) {
  if (device < 0) {
    if (cudaGetDevice(&device) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
  }
  if (device >= 64) return 0;
  DeviceFacts& f = g_facts[device];
  std::call_once(f.once, [&] {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
      (void)cudaGetLastError();
      n = 0;
    }
    f.sm_count = n;
  });
  return f.sm_count;
}

// How many partial slots a sequence gets (`num_splits`). The split decode deals the tiles of
// all sequences of a kv head in equal shares to the W warps that serve the head (two four-warp
// CTAs an SM, divided among the heads); a share may not be shorter than longest / (parts - 1),
// so that no sequence needs more than `parts` slots. With n sequences whose longest is up to
// 8x the mean, parts = 1 + 8 W / n keeps that bound from limiting the shares. Capped by the
// pieces the longest allowed sequence can usefully have (2 tiles a piece) and HKB_MAX_SPLITS,
// rounded up to a power of two: a function of host values only, so a captured graph's plan is
// right for every replay. hk-dsl's rule has the same shape -- ceil(target / (requests * kv
// heads)), capped by pages and a maximum (python/hk/ops/paged.py:838-914) -- with AMD's target.
extern "C" int hkb_plan_splits(int num_seqs, int num_kv_heads, int max_tiles, int sm_count) {
  if (sm_count <= 0) sm_count = 148;
  const long long n = num_seqs > 0 ? num_seqs : 1;
  const long long heads = num_kv_heads > 0 ? num_kv_heads : 1;
  long long per = ((long long)sm_count * 2) / heads;
  if (per < 1) per = 1;
  const long long w = per * 4;
  long long want = 1 + (8 * w + n - 1) / n;
  const long long cap = max_tiles > 0 ? (max_tiles + 1) / 2 + 1 : 2;
  if (want > cap) want = cap;
  if (want < 2) want = 2;
  long long p = 2;
  while (p < want) p *= 2;
  if (p > HKB_MAX_SPLITS) p = HKB_MAX_SPLITS;
  return (int)p;
}

// 1 + HKB_MAX_SPLITS / 16 counters (finished groups, then finished pieces of each 16-slot group) a
// (plane, sequence); a kv head has at most two planes (a CUDA-core walk of a group of 5 to 7
// takes its heads in two passes).
extern "C" size_t hkb_arrivals_bytes(int num_seqs, int num_kv_heads) {
  if (num_seqs <= 0 || num_kv_heads <= 0) return 0;
  return (size_t)num_seqs * num_kv_heads * 2 * (1 + HKB_MAX_SPLITS / 16) * sizeof(int32_t);
}

extern "C" size_t hkb_scratch_lse_offset(int num_seqs, int num_q_heads, int head_dim, int num_splits) {
  if (num_seqs <= 0 || num_q_heads <= 0 || head_dim <= 0 || num_splits <= 0) return 0;
  size_t b = (size_t)num_seqs * num_splits * num_q_heads * head_dim * sizeof(float);
  return (b + 255) & ~(size_t)255;
}

extern "C" size_t hkb_scratch_bytes(int num_seqs, int num_q_heads, int head_dim, int num_splits) {
  if (num_seqs <= 0 || num_q_heads <= 0 || head_dim <= 0 || num_splits <= 0) return 0;
  size_t lse = (size_t)num_seqs * num_splits * num_q_heads * sizeof(float);
  return hkb_scratch_lse_offset(num_seqs, num_q_heads, head_dim, num_splits) + ((lse + 255) & ~(size_t)255);
}

extern "C" const char* hkb_strerror(int code) {
  switch (code) {
    case HKB_OK: return "ok";
    case HKB_ERR_NULL: return "a required pointer is NULL";
    case HKB_ERR_HEAD_DIM: return "head_dim is not one this build has a kernel for (64, 128, 256)";
    case HKB_ERR_BLOCK_SIZE: return "block_size is not a positive multiple of 16";
    case HKB_ERR_GROUP: return "query heads are not a multiple of kv heads, or more than 16 a kv head";
    case HKB_ERR_DTYPE: return "kv_dtype is not bf16 (0), fp8-e4m3 (1) or fp16 throughout (2)";
    case HKB_ERR_STRIDE: return "a stride breaks the 16-byte alignment of a row";
    case HKB_ERR_ALIGN: return "a base pointer is not aligned as the kernels read it";
    case HKB_ERR_SPLITS: return "num_splits out of range, or split scratch missing";
    case HKB_ERR_SIZE: return "a count is negative or past a launch limit";
    case HKB_ERR_SCALE: return "an fp8 cache needs k_scale and v_scale";
    case HKB_ERR_UNSUPPORTED: return "no kernel for this combination of head_dim, dtype and group";
    case HKB_ERR_STATIC_SCRATCH:
      return "the split partials need more than the library's built-in scratch (HKB_STATIC_SCRATCH_BYTES): use fewer "
             "splits or the caller-scratch entry points";
    case HKB_ERR_CUDA: return "CUDA reported an error at launch (hkb_last_cuda_error)";
    default: return "unknown hkb status";
  }
}

extern "C" int hkb_last_cuda_error(void) { return hkb_tls_cuda_error; }

extern "C" int hkb_version(void) { return HKB_VERSION; }
