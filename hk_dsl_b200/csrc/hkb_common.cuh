// Device helpers shared by the hkb kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hkb.h"

namespace hkb {

constexpr int TILE_TOKENS = 16;  // tokens per KV tile: one 16-token page, or a 16-token slice of a larger one
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global->shared copy that bypasses L1 (KV is read once).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Two bf16 packed in 32 bits -> two floats (exact: bf16 is the top half of an fp32).
__device__ __forceinline__ float bf16lo(uint32_t x) { return __uint_as_float(x << 16); }
__device__ __forceinline__ float bf16hi(uint32_t x) { return __uint_as_float(x & 0xffff0000u); }

// Two e4m3 in the low 16 bits -> two floats (exact), through the f16x2 convert.
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t x) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h2) : "h"(x));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half22float2(h);
}

// Eight bf16 (one 16-byte chunk) -> eight e4m3 bytes of a cache with scale `den`:
// float(x) / den in IEEE fp32 division, then round-to-nearest-even, saturating at +-448.
__device__ __forceinline__ uint2 quantize_chunk_e4m3(const uint4& v, float den) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f;
    f.x = __fdiv_rn(bf16lo(w[i]), den);
    f.y = __fdiv_rn(bf16hi(w[i]), den);
    const uint32_t p = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
    if (i & 1) o[i >> 1] |= p << 16; else o[i >> 1] = p;
  }
  return make_uint2(o[0], o[1]);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Packed fp32 pairs (sm_100 f32x2 arithmetic: one issue slot for two FMAs).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Position of 16-byte chunk `c` of row `r` inside a shared-memory tile whose rows
// are ROW_BYTES long: chunks are XOR-swizzled by the row so that eight rows read
// at the same column (ldmatrix) and eight columns of one row are both conflict-free.
// (A 64-byte row -- an fp8 row of head size 64 -- has four chunks: the XOR is then with r & 3, which
// keeps a chunk inside its row.)
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
  constexpr int MASK = ROW_BYTES / 16 - 1 < 7 ? ROW_BYTES / 16 - 1 : 7;
  return static_cast<uint32_t>(r * ROW_BYTES + ((c ^ (r & MASK)) << 4));
}

// The same tile in the layout the fp8 fragment loads want: rows of 128 bytes whose 32-byte
// units are XOR-ed with f(r) = (r & 3) ^ ((r >> 2) & 1). A lane of those loads reads 8 or 4
// bytes of a row and 8 lanes cover 32 bytes, so a warp-wide request touches rows {0..3} or {4..7}
// (K: 64-bit loads, two phases) or {0,2,4,6} / {1,3,5,7} (V: 32-bit loads): f is one-to-one on
// each of those sets, which the 16-byte swizzle above is not, so no two rows share a bank.
__device__ __forceinline__ uint32_t tile_off_u32(int r, int c) {
  const int f = (r & 3) ^ ((r >> 2) & 1);
  return r * 128 + (((((c >> 1) ^ f) << 1) | (c & 1)) << 4);
}

// The same idea for fp8 rows of any head size (ROWB = head_dim bytes). Rows of 128 bytes and more
// keep the form above (f touches the low two bits of the unit index, so a 256-byte row's eight units
// stay inside the row). A 64-byte row is two units, too few to tell four rows apart by a XOR inside
// the row, so rows are placed in pairs: units are dealt to 32 slots of 32 bytes, slot
// 4 (r / 2) + m with m = (r + ((r >> 2) & 1) + 2 u) & 3 -- the rows {0..3}, {4..7}, {0,2,4,6} and
// {1,3,5,7} of one unit index u each fall on four different m, i.e. on different banks. Both forms
// repeat every 8 rows (8 ROWB bytes on), which the loaders and the row + 8 loads rely on.
template <int ROWB>
__device__ __forceinline__ uint32_t tile_off_f8(int r, int c) {
  static_assert(ROWB == 64 || ROWB == 128 || ROWB == 256, "fp8 rows of head sizes 64, 128, 256");
  if (ROWB == 64) return (uint32_t)((4 * (r >> 1) + ((r + ((r >> 2) & 1) + 2 * (c >> 1)) & 3)) * 32 + (c & 1) * 16);
  const int f = (r & 3) ^ ((r >> 2) & 1);
  return r * ROWB + (((((c >> 1) ^ f) << 1) | (c & 1)) << 4);
}

}  // namespace hkb
