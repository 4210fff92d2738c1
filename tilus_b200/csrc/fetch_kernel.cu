// Copy-in of b200q_gemm_host for small activation blocks: a kernel instead of a copy-engine
// operation.  The rows A[M, K] live in pinned host memory that the GPU can address; every thread
// loads up to four 16-byte pieces of them over PCIe into registers FIRST, then waits for the
// previous kernel of the stream (griddepcontrol.wait) and only then stores them to the device
// staging buffer.  Launched with programmatic stream serialization, the kernel is resident while
// the previous GEMM still runs, so the PCIe round trips of call i lie under the GEMM of call
// i - 1; what stays on the critical path is a few KB of device stores.  The GEMM that follows is
// itself a programmatic dependent of this kernel and starts its weight pipeline under it.
// (The reference operator takes device tensors only; this path has no counterpart there.)
#include "common.cuh"

namespace b200q {

constexpr int FETCH_THREADS = 256;
constexpr int FETCH_PIECES = 4;  // 16-byte pieces per thread

__global__ void __launch_bounds__(FETCH_THREADS) host_fetch_kernel(const unsigned short* __restrict__ src, int lds,
                                                                   unsigned short* __restrict__ dst, int M, int K) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int vec_per_row = K / 8;
  const int total = M * vec_per_row;
  const int base = (blockIdx.x * FETCH_THREADS + threadIdx.x) * FETCH_PIECES;
  uint4 v[FETCH_PIECES];
#pragma unroll
  for (int u = 0; u < FETCH_PIECES; ++u) {
    const int idx = base + u;
    if (idx < total) {
      const int m = idx / vec_per_row, c = idx - m * vec_per_row;
      // host memory: read past the caches (the host may rewrite the rows between calls)
      v[u] = __ldcv(reinterpret_cast<const uint4*>(src + (size_t)m * lds + (size_t)c * 8));
    }
  }
  // the staging buffer may still be read by the previous GEMM of the stream
  asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
  for (int u = 0; u < FETCH_PIECES; ++u) {
    const int idx = base + u;
    if (idx < total) *reinterpret_cast<uint4*>(dst + (size_t)idx * 8) = v[u];
  }
}

// src: device-side address of the pinned host rows (row stride lds elements); dst: [M, K] dense
cudaError_t host_fetch_launch(const void* src, int lds, void* dst, int M, int K, cudaStream_t stream) {
  const int total = M * (K / 8);
  const int per_cta = FETCH_THREADS * FETCH_PIECES;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((total + per_cta - 1) / per_cta), 1, 1);
  cfg.blockDim = dim3(FETCH_THREADS, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, host_fetch_kernel, reinterpret_cast<const unsigned short*>(src), lds,
                            reinterpret_cast<unsigned short*>(dst), M, K);
}

}  // namespace b200q
