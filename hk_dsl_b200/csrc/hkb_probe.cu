// A read-only streaming probe: how fast can a kernel read bytes it touches exactly once.
//
// The decode walk is ~100 % reads, while the usual "HBM peak" is a copy (half reads, half
// writes, with the bus turnarounds that costs). This kernel is the ceiling the walk should be
// held to: every thread keeps INFLIGHT independent 16-byte loads in the air, a warp reads 512
// contiguous bytes a load, the grid is persistent (a multiple of the SM count) and walks the
// buffer in CTA-sized slabs. The host rotates it over buffers larger than L2 so that nothing is
// served from cache, and sweeps CTAs an SM x loads in flight, keeping the best.
//
// hk-dsl has the same tool for its cards (tools/hk-bench/hbm_probe.hip:1-134); this is the
// sm_100a counterpart, behind the C ABI so that the benchmark needs no second build.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hkb.h"

extern thread_local int hkb_tls_cuda_error;

namespace hkb {

__device__ __forceinline__ uint4 ld_stream16(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int INFLIGHT>
__global__ void __launch_bounds__(256) hbm_read_kernel(const uint4* __restrict__ buf, size_t n16, uint32_t* sink) {
  // a CTA's slab: 256 threads x INFLIGHT chunks, consecutive threads on consecutive chunks
  const size_t slab = (size_t)blockDim.x * INFLIGHT;
  uint32_t acc = 0;
  for (size_t base = (size_t)blockIdx.x * slab; base < n16; base += (size_t)gridDim.x * slab) {
    uint4 v[INFLIGHT];
#pragma unroll
    for (int u = 0; u < INFLIGHT; ++u) {
      const size_t i = base + (size_t)u * blockDim.x + threadIdx.x;
      v[u] = i < n16 ? ld_stream16(buf + i) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < INFLIGHT; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
  }
  // keeps the loads alive; the fill pattern the host writes never produces this value
  if (acc == 0x9e3779b9u) sink[0] = acc;
}

}  // namespace hkb

extern "C" int hkb_hbm_read_probe(const void* buf, size_t bytes, int ctas_per_sm, int loads_in_flight, void* sink,
                                  void* stream) {
  using namespace hkb;
  if (!buf || !sink) return HKB_ERR_NULL;
  if ((uintptr_t)buf % 16 || (uintptr_t)sink % 4) return HKB_ERR_ALIGN;
  if (bytes < 16 || ctas_per_sm < 1 || ctas_per_sm > 32) return HKB_ERR_SIZE;
  int sms = hkb_sm_count(-1);
  if (sms <= 0) sms = 148;
  const size_t n16 = bytes / 16;
  const dim3 grid(sms * ctas_per_sm);
  cudaStream_t st = (cudaStream_t)stream;
  const uint4* p = static_cast<const uint4*>(buf);
  uint32_t* s = static_cast<uint32_t*>(sink);
  switch (loads_in_flight) {
    case 1: hbm_read_kernel<1><<<grid, 256, 0, st>>>(p, n16, s); break;
    case 2: hbm_read_kernel<2><<<grid, 256, 0, st>>>(p, n16, s); break;
    case 4: hbm_read_kernel<4><<<grid, 256, 0, st>>>(p, n16, s); break;
    case 8: hbm_read_kernel<8><<<grid, 256, 0, st>>>(p, n16, s); break;
    case 16: hbm_read_kernel<16><<<grid, 256, 0, st>>>(p, n16, s); break;
    default: return HKB_ERR_SIZE;
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { hkb_tls_cuda_error = (int)e; return HKB_ERR_CUDA; }
  return HKB_OK;
}
