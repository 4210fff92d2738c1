// All-gather of column shards over peer-mapped memory for batches the fused decode kernel does not
// take (M > 16): two small kernels behind one call.
//
//   push    : copies this rank's shard C[M, N_loc] (the GEMM's output) into its column range of the
//             full output row [M, ldc] in row buffer (E + 1) % 2 of every rank (16-byte stores over
//             NVLink; stores only, no loads from peers), then - last CTA, one system-scope fence -
//             raises this rank's flag to E + 1 on every rank and moves the call counter on.
//   collect : waits (bounded, 0.25 s, else the status word) until every rank's flag has reached the
//             call counter, i.e. all shards of this call have landed here, and copies the complete
//             rows from the row buffer to a fixed local buffer that the next operator reads.
//
// Same regions, flags, call counter and buffer alternation as the fused gather of the decode kernel
// (stream_kernel.cu, GatherArgs), so both kinds of call can be mixed in one sequence and a captured
// sequence replays from a CUDA graph.  The second kernel only waits for flags raised by earlier
// launches (this rank's push, complete by stream order) and by other GPUs: no CTA waits for a CTA of
// its own launch.  The reference is single-GPU and has no counterpart.
#include "common.cuh"

namespace b200q {

struct PushParams {
  const unsigned short* src;  // [M, N_loc], row stride lds
  unsigned short* dst_local;  // [M, ldc] fixed local copy of the gathered rows (collect), row stride ld_local
  int lds, ld_local;
  int M, N_loc, ldc;
  int* status;
  GatherArgs ga;
};

__device__ __forceinline__ bool wait_flags(const PushParams& p, unsigned target, int where) {
  // one thread per source rank
  bool ok = true;
  if ((int)threadIdx.x < p.ga.G) {
    uint64_t t0 = 0;
    for (int spin = 0;; ++spin) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.ga.flags + threadIdx.x) : "memory");
      if ((int)(v - target) >= 0) break;
      uint64_t now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (spin == 0) t0 = now;
      else if (now - t0 > 250000000ull) {  // give up: report, carry on with what is there
        atomicExch(p.status, ST_DEVICE_TIMEOUT);
        p.status[1] = where;
        p.status[2] = blockIdx.x;
        p.status[3] = threadIdx.x;
        ok = false;
        break;
      }
    }
  }
  __syncthreads();
  return ok;
}

__global__ void __launch_bounds__(256) gather_push_kernel(const PushParams p) {
  // launched with programmatic stream serialization: resident early, waits here for the GEMM whose
  // output it copies
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const unsigned epoch = *reinterpret_cast<volatile const unsigned*>(p.ga.epoch);
  if (p.ga.mode == 1) {
    // Tagged words: every pair of values leaves with the call number in one 64-bit store, into buffer
    // (E + 1) % 3 of every rank.  Nothing to wait for and nothing to fence: the collect kernels poll the
    // words, and the buffer written here was last read two calls ago (every rank has since pushed twice,
    // each time after collecting).  The last CTA only moves this rank's call counter on.
    const size_t buf = (size_t)((epoch + 1) % GATHER_TAG_BUFFERS) * (size_t)p.ga.buf_elems;
    const int vec_per_row = p.N_loc / 8;
    const int total = p.M * vec_per_row;
    const unsigned long long tag = (unsigned long long)(epoch + 1) << 32;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
      const int m = idx / vec_per_row, v = idx - m * vec_per_row;
      const uint4 x = *reinterpret_cast<const uint4*>(p.src + (size_t)m * p.lds + v * 8);
      const size_t word = buf + (((size_t)m * p.ldc + p.ga.col_off + v * 8) >> 1);
      const unsigned long long w0 = tag | x.x, w1 = tag | x.y, w2 = tag | x.z, w3 = tag | x.w;
      for (int g = 0; g < p.ga.G; ++g) {
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.ga.out[g]) + word;
        asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(w0), "l"(w1) : "memory");
        asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(dst + 2), "l"(w2), "l"(w3) : "memory");
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned* done = p.ga.epoch + 8;
      if (atomicAdd(done, 1u) == gridDim.x - 1) {
        atomicExch(done, 0u);
        *p.ga.epoch = epoch + 1;
      }
    }
    return;
  }
  // nobody may still be reading the buffer about to be overwritten: every rank has finished call E
  if (epoch != 0) wait_flags(p, epoch, 7);
  const size_t buf = ((epoch + 1) & 1u) ? (size_t)p.ga.buf_elems : 0;
  const int vec_per_row = p.N_loc / 8;
  const int total = p.M * vec_per_row;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int m = idx / vec_per_row, v = idx - m * vec_per_row;
    const uint4 x = *reinterpret_cast<const uint4*>(p.src + (size_t)m * p.lds + v * 8);
    const size_t off = buf + (size_t)m * p.ldc + p.ga.col_off + v * 8;
    for (int g = 0; g < p.ga.G; ++g) *reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(p.ga.out[g]) + off) = x;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned arrived;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(p.ga.done) : "memory");
    if (arrived == gridDim.x - 1) {
      atomicExch(p.ga.done, 0u);
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      for (int g = 0; g < p.ga.G; ++g)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.ga.flag_slot[g]), "r"(epoch + 1) : "memory");
      *p.ga.epoch = epoch + 1;
    }
  }
}

// Tagged rows (GatherArgs mode 1) -> dense rows: every 8-byte word {two values, call number} of the latest
// call's row buffer is read until it carries that call's number (bounded), then its values are written
// to the local copy.  dst_local == nullptr: wait only.
__device__ __forceinline__ void collect_tagged(const PushParams& p, unsigned epoch) {
  const unsigned long long* row = reinterpret_cast<const unsigned long long*>(p.ga.out[p.ga.rank]) +
                                  (size_t)(epoch % GATHER_TAG_BUFFERS) * (size_t)p.ga.buf_elems;
  const int vec_per_row = p.ldc / 4;  // two words = four values per step
  const int total = p.M * vec_per_row;
  bool waiting = true;  // cleared once a wait has run out
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int m = idx / vec_per_row, v = idx - m * vec_per_row;
    const unsigned long long* src = row + (((size_t)m * p.ldc) >> 1) + v * 2;
    ulonglong2 w;
    uint64_t t0 = 0;
    for (int spin = 0;; ++spin) {
      asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w.x), "=l"(w.y) : "l"(src) : "memory");
      if (!waiting || ((unsigned)(w.x >> 32) == epoch && (unsigned)(w.y >> 32) == epoch)) break;
      uint64_t now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (spin == 0) t0 = now;
      else if (now - t0 > 250000000ull) {  // give up for good: report, carry on with what is there
        atomicExch(p.status, ST_DEVICE_TIMEOUT);
        p.status[1] = 8;
        p.status[2] = blockIdx.x;
        p.status[3] = threadIdx.x;
        waiting = false;
        break;
      }
    }
    if (p.dst_local)
      *reinterpret_cast<uint2*>(p.dst_local + (size_t)m * p.ld_local + v * 4) = make_uint2((uint32_t)w.x, (uint32_t)w.y);
  }
}

__global__ void __launch_bounds__(256) gather_collect_kernel(const PushParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // this rank's push has completed: the call counter is final
  const unsigned epoch = *reinterpret_cast<volatile const unsigned*>(p.ga.epoch);  // includes this call's push
  if (p.ga.mode == 1) {
    if (epoch != 0) collect_tagged(p, epoch);
    return;
  }
  wait_flags(p, epoch, 8);
  if (!p.dst_local) return;
  const unsigned short* row = reinterpret_cast<const unsigned short*>(p.ga.out[p.ga.rank]) +
                              ((epoch & 1u) ? (size_t)p.ga.buf_elems : 0);
  const int vec_per_row = p.ldc / 8;
  const int total = p.M * vec_per_row;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
    const int m = idx / vec_per_row, v = idx - m * vec_per_row;
    // the rows were written through L2 by other GPUs: read them past L1
    const uint4 x = __ldcg(reinterpret_cast<const uint4*>(row + (size_t)m * p.ldc + v * 8));
    *reinterpret_cast<uint4*>(p.dst_local + (size_t)m * p.ld_local + v * 8) = x;
  }
}

static cudaError_t launch_pdl(void (*kern)(const PushParams), int grid, const PushParams& p, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

static PushParams make_params(const void* src, int lds, void* dst_local, int ld_local, int M, int N_loc, int ldc,
                              int* status, const GatherArgs& ga) {
  PushParams p;
  p.src = reinterpret_cast<const unsigned short*>(src);
  p.dst_local = reinterpret_cast<unsigned short*>(dst_local);
  p.lds = lds; p.ld_local = ld_local;
  p.M = M; p.N_loc = N_loc; p.ldc = ldc;
  p.status = status;
  p.ga = ga;
  return p;
}

cudaError_t gather_push_launch(const void* src, int lds, int M, int N_loc, int ldc, int* status, const GatherArgs& ga,
                               cudaStream_t stream) {
  const PushParams p = make_params(src, lds, nullptr, 0, M, N_loc, ldc, status, ga);
  int grid = (M * (N_loc / 8) + 255) / 256;
  if (grid > 64) grid = 64;
  if (grid < 1) grid = 1;
  return launch_pdl(gather_push_kernel, grid, p, stream);
}

cudaError_t gather_collect_launch(void* dst_local, int ld_local, int M, int ldc, int* status, const GatherArgs& ga,
                                  cudaStream_t stream) {
  const PushParams p = make_params(nullptr, 0, dst_local, ld_local, M, 0, ldc, status, ga);
  int grid = (M * (ldc / (ga.mode == 1 ? 4 : 8)) + 255) / 256;
  if (grid > 296) grid = 296;
  if (grid < 1) grid = 1;
  return launch_pdl(gather_collect_kernel, grid, p, stream);
}

}  // namespace b200q
