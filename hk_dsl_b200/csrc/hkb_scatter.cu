// The KV-cache write (reshape_and_cache): new K/V rows scattered into a block-paged
// cache by slot, bf16 passthrough or fused fp8-e4m3 quantisation.
//
// Semantics follow the torch scatter hk-dsl's own test holds vLLM's op to
// (tests/hk/gpu/test_vllm_backend_decode.py:44-49): cache[s / bs, :, s % bs] = key[live],
// live = slots >= 0; slot -1 is skipped (examples/09_kv_scatter.py:53-65).
//
// HBM-bound byte mover: every thread moves one 16-byte chunk of a source row, so a
// warp reads 512 contiguous bytes; the destination row of a (token, head) pair is
// contiguous too, whatever the cache's block / token / head strides are.
#include "hkb_common.cuh"

namespace hkb {

struct ScatterArgs {
  const __nv_bfloat16* src[2];  // key, value
  int64_t src_stride_tok[2], src_stride_head[2];
  void* dst[2];                 // k_cache, v_cache
  int64_t dst_stride_block[2], dst_stride_token[2], dst_stride_head[2];
  int64_t num_slots[2];         // num_blocks * block_size of each cache
  const float* scale[2];
  const void* slots;
  int slot_is_i64;
  int num_tokens, num_kv_heads, head_dim, block_size;
};

// grid = (ceil(tokens / TOK_PER_CTA), 2 [K, V]); a warp takes a token at a time -- its slot is
// read and split into (block, offset) once -- and its lanes the token's 16-byte chunks (8 bf16
// elements of a (head, chunk) each), so the per-chunk work is one load, one store and a shift.
template <bool FP8>
__global__ void __launch_bounds__(256) scatter_kernel(const ScatterArgs a, int tok_per_cta) {
  const int which = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks_per_head = a.head_dim >> 3;
  const int chunks_per_tok = a.num_kv_heads * chunks_per_head;
  const int shift = (chunks_per_head & (chunks_per_head - 1)) == 0 ? __ffs(chunks_per_head) - 1 : -1;
  const int t0 = blockIdx.x * tok_per_cta;
  const int t1 = min(a.num_tokens, t0 + tok_per_cta);
  float inv_scale_den = 1.0f;
  if (FP8) inv_scale_den = __ldg(a.scale[which]);

  // a token with fewer than 32 chunks (one kv head of 128 on a GPU of a head-sharded job): the warp
  // takes 32 / chunks of them at once, so that no lane idles
  const int tpw = chunks_per_tok < 32 && 32 % chunks_per_tok == 0 ? 32 / chunks_per_tok : 1;
  const int sub = tpw > 1 ? lane / chunks_per_tok : 0;
  const int x0 = tpw > 1 ? lane - sub * chunks_per_tok : lane;
  const int xstep = tpw > 1 ? chunks_per_tok : 32;
  for (int tw = t0 + warp * tpw; tw < t1; tw += 8 * tpw) {
    const int t = tw + sub;
    if (t >= t1) continue;
    int64_t slot;
    if (a.slot_is_i64) slot = __ldg(reinterpret_cast<const long long*>(a.slots) + t);
    else slot = __ldg(reinterpret_cast<const int*>(a.slots) + t);
    if (slot < 0 || slot >= a.num_slots[which]) continue;  // padding token, or out of the pool
    const int64_t blk = slot / a.block_size;
    const int64_t off = slot - blk * a.block_size;
    const __nv_bfloat16* src = a.src[which] + (int64_t)t * a.src_stride_tok[which];
    const int64_t dst = blk * a.dst_stride_block[which] + off * a.dst_stride_token[which];
    for (int x = x0; x < chunks_per_tok; x += xstep) {
      const int h = shift >= 0 ? x >> shift : x / chunks_per_head;
      const int c = x - h * chunks_per_head;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)h * a.src_stride_head[which] + c * 8));
      const int64_t d = dst + (int64_t)h * a.dst_stride_head[which] + c * 8;
      if (!FP8) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.dst[which]) + d) = v;
      } else {
        *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(a.dst[which]) + d) = quantize_chunk_e4m3(v, inv_scale_den);
      }
    }
  }
}

}  // namespace hkb

extern thread_local int hkb_tls_cuda_error;

extern "C" int hkb_reshape_and_cache(const void* key, const void* value,
                                     int64_t key_stride_tok, int64_t key_stride_head,
                                     int64_t val_stride_tok, int64_t val_stride_head,
                                     hkb_cache_t kc, hkb_cache_t vc,
                                     const void* slot_mapping, int slot_is_i64,
                                     int num_tokens, int num_kv_heads, int head_dim, int block_size,
                                     int kv_dtype, const float* k_scale, const float* v_scale,
                                     void* stream) {
  using namespace hkb;
  if (num_tokens < 0 || num_kv_heads <= 0 || kc.num_blocks < 0 || vc.num_blocks < 0) return HKB_ERR_SIZE;
  if (num_tokens == 0) return HKB_OK;
  if (!key || !value || !kc.ptr || !vc.ptr || !slot_mapping) return HKB_ERR_NULL;
  if (head_dim <= 0 || head_dim % 8 != 0 || head_dim > 1024) return HKB_ERR_HEAD_DIM;
  if (block_size <= 0) return HKB_ERR_BLOCK_SIZE;
  // fp16 rows are copied like bf16 rows: 16-bit elements, no conversion
  if (kv_dtype != HKB_KV_BF16 && kv_dtype != HKB_KV_FP8_E4M3 && kv_dtype != HKB_KV_F16) return HKB_ERR_DTYPE;
  const bool fp8 = kv_dtype == HKB_KV_FP8_E4M3;
  if (fp8 && (!k_scale || !v_scale)) return HKB_ERR_SCALE;
  // 16-byte source chunks; destination chunks are 16 bytes (bf16) or 8 bytes (fp8).
  if ((key_stride_tok | key_stride_head | val_stride_tok | val_stride_head) % 8) return HKB_ERR_STRIDE;
  const int64_t dmask =
      kc.stride_block | kc.stride_token | kc.stride_head | vc.stride_block | vc.stride_token | vc.stride_head;
  if (dmask % 8) return HKB_ERR_STRIDE;
  if (((uintptr_t)key | (uintptr_t)value) % 16) return HKB_ERR_ALIGN;
  if (((uintptr_t)kc.ptr | (uintptr_t)vc.ptr) % (fp8 ? 8 : 16)) return HKB_ERR_ALIGN;

  ScatterArgs a;
  a.src[0] = (const __nv_bfloat16*)key; a.src[1] = (const __nv_bfloat16*)value;
  a.src_stride_tok[0] = key_stride_tok; a.src_stride_tok[1] = val_stride_tok;
  a.src_stride_head[0] = key_stride_head; a.src_stride_head[1] = val_stride_head;
  a.dst[0] = kc.ptr; a.dst[1] = vc.ptr;
  a.dst_stride_block[0] = kc.stride_block; a.dst_stride_block[1] = vc.stride_block;
  a.dst_stride_token[0] = kc.stride_token; a.dst_stride_token[1] = vc.stride_token;
  a.dst_stride_head[0] = kc.stride_head; a.dst_stride_head[1] = vc.stride_head;
  a.num_slots[0] = kc.num_blocks * block_size; a.num_slots[1] = vc.num_blocks * block_size;
  a.scale[0] = k_scale; a.scale[1] = v_scale;
  a.slots = slot_mapping; a.slot_is_i64 = slot_is_i64;
  a.num_tokens = num_tokens; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.block_size = block_size;

  // One CTA of 256 threads moves ~16 KB: enough CTAs to cover the SMs at decode
  // sizes (64 tokens) and few enough items per thread at prefill sizes.
  const int chunks_per_tok = num_kv_heads * (head_dim / 8);
  int tok_per_cta = (1024 + chunks_per_tok - 1) / chunks_per_tok;
  if (tok_per_cta < 1) tok_per_cta = 1;
  const int64_t ctas = ((int64_t)num_tokens + tok_per_cta - 1) / tok_per_cta;
  if (ctas > 0x7fffffffLL) return HKB_ERR_SIZE;
  dim3 grid((unsigned)ctas, 2);
  cudaStream_t st = (cudaStream_t)stream;
  if (fp8) scatter_kernel<true><<<grid, 256, 0, st>>>(a, tok_per_cta);
  else scatter_kernel<false><<<grid, 256, 0, st>>>(a, tok_per_cta);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}
