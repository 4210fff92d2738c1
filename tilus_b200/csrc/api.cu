// C ABI of libb200q (declared in include/b200q.h): argument validation, the static
// shape -> tile table, and kernel dispatch.  No torch types, no allocation.
#include <cstdio>
#include <cstring>

#include "../../include/b200q.h"
#include "common.cuh"

#ifndef B200Q_NPARTS
#define B200Q_NPARTS 8
#endif

namespace b200q {

#define B200Q_DECL_PART(i) \
  cudaError_t skinny_launch_part##i(int, const SkinnyParams&, int, int, cudaStream_t);
B200Q_DECL_PART(0) B200Q_DECL_PART(1) B200Q_DECL_PART(2) B200Q_DECL_PART(3)
B200Q_DECL_PART(4) B200Q_DECL_PART(5) B200Q_DECL_PART(6) B200Q_DECL_PART(7)
cudaError_t dequant_launch(int var, const DequantParams& p, cudaStream_t stream);

static thread_local int g_last_cuda_error = 0;

static cudaError_t skinny_launch(int var, const SkinnyParams& p, int mt, int smem, cudaStream_t s) {
  switch (var % B200Q_NPARTS) {
    case 0: return skinny_launch_part0(var, p, mt, smem, s);
    case 1: return skinny_launch_part1(var, p, mt, smem, s);
    case 2: return skinny_launch_part2(var, p, mt, smem, s);
    case 3: return skinny_launch_part3(var, p, mt, smem, s);
    case 4: return skinny_launch_part4(var, p, mt, smem, s);
    case 5: return skinny_launch_part5(var, p, mt, smem, s);
    case 6: return skinny_launch_part6(var, p, mt, smem, s);
    default: return skinny_launch_part7(var, p, mt, smem, s);
  }
}

// wtype tag + zero point -> kernel variant (decode.cuh), or -1
static int variant_of(int wtype, int zero_point) {
  const int kind = (wtype >> 16) & 0xff, nbits = (wtype >> 8) & 0xff, e = (wtype >> 4) & 0xf, m = wtype & 0xf;
  if (nbits < 1 || nbits > 8) return -1;
  if (kind == 0) {
    if (zero_point == 0) return (nbits - 1) * 2;
    if (zero_point == (1 << (nbits - 1))) return (nbits - 1) * 2 + 1;
    return -1;
  }
  if (kind == 1) return zero_point == 0 ? (nbits - 1) * 2 + 1 : -1;
  if (kind == 2 && zero_point == 0 && nbits == 1 + e + m) {
    for (int v = 16; v < VAR_COUNT; ++v)
      if (var_float_bits(v) == nbits && var_float_ebits(v) == e) return v;
  }
  return -1;
}

struct DeviceInfo {
  int sm_count = 0;
  int max_smem = 0;
};
static DeviceInfo device_info() {
  static DeviceInfo cache[16];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 16 && cache[dev].sm_count) return cache[dev];
  DeviceInfo d;
  cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (d.sm_count <= 0) d.sm_count = 148;
  if (d.max_smem <= 0) d.max_smem = 227 * 1024;
  if (dev >= 0 && dev < 16) cache[dev] = d;
  return d;
}

// shared-memory row pitch (halfs) of an activation chunk of kc columns: 16 bytes of padding
// per 128 columns, and pitch bytes = 64 (mod 128) so that 8 lanes reading 16 bytes each from
// two rows x four 128-column segments touch 8 different 16-byte bank groups
static int skinny_pitch(int kc) {
  int bytes = kc * 2 + (kc / 128) * 16;
  if (bytes % 128 != 64) bytes += (64 - bytes % 128 + 128) % 128;
  return bytes / 2;
}

// ---- static shape -> tile table ------------------------------------------------------------
// Exact entries for the shapes this library is benchmarked on come first; anything else
// goes through the balance rule below.
struct TableEntry {
  int bits, m_lo, m_hi, N, K;
  int splits;
};
static const TableEntry kSkinnyTable[] = {
    // bits  M range   N      K     S
    {4, 1, 16, 8192, 8192, 2},
};

static int plan_skinny(int m_pass, int N, int K, int bits, const DeviceInfo& di, b200q_plan_t* pl) {
  const int KB = K / BLOCK_K, NT = N / BLOCK_N;
  const int occ_regs = bits <= 4 ? 2 : 1;  // register budget of the kernel (launch bounds)
  int forced = 0;
  for (const TableEntry& t : kSkinnyTable)
    if (t.bits == bits && m_pass >= t.m_lo && m_pass <= t.m_hi && t.N == N && t.K == K) forced = t.splits;
  double best_cost = 1e30;
  int best_s = 0, best_p = 0;
  for (int pass = 0; pass < 2 && !best_s; ++pass) {  // pass 0 honours the table, pass 1 ignores it
    for (int s = 1; s <= KB; ++s) {
      if (KB % s) continue;
      if (pass == 0 && forced && s != forced) continue;
      const int kbc = KB / s;
      const int smem = m_pass * skinny_pitch(kbc * 512) * 2;
      if (smem + 1024 > di.max_smem) continue;
      for (int occ = 1; occ <= occ_regs; ++occ) {
        if ((smem + 1024) * occ > di.max_smem) continue;
        const int slots = di.sm_count * occ;
        if (s > slots) continue;
        int P = slots / s;
        if (P > NT) P = NT;
        const int tiles_max = (NT + P - 1) / P;
        const int warp_items = (tiles_max * kbc + 7) / 8;
        // time ~ items the busiest SM streams + staging the activation chunk + reduction traffic
        const double cost = warp_items * 8.0 * occ + 0.05 * m_pass * kbc * occ + 0.2 * s;
        if (cost < best_cost) { best_cost = cost; best_s = s; best_p = P; }
      }
    }
  }
  if (!best_s) return ST_UNSUPPORTED;
  const int kbc = KB / best_s;
  pl->kernel = 0;
  pl->m_tiles = (m_pass + 7) / 8;
  pl->splits = best_s;
  pl->ctas_per_split = best_p;
  pl->smem_bytes = m_pass * skinny_pitch(kbc * 512) * 2;
  pl->tile_m = 0;
  pl->stages = 0;
  return ST_OK;
}

static int check_problem(int M, int N, int K, int wtype, int zero_point, int group, int* var) {
  if (M < 1 || N < 1 || K < 1 || group < 1) return ST_INVALID_ARG;
  *var = variant_of(wtype, zero_point);
  if (*var < 0) return ST_UNSUPPORTED;
  if (K % BLOCK_K != 0 || N % BLOCK_N != 0) return ST_UNSUPPORTED;
  if (group % 32 != 0 || K % group != 0) return ST_UNSUPPORTED;
  return ST_OK;
}

static int make_plan(int M, int N, int K, int var, b200q_plan_t* pl) {
  const DeviceInfo di = device_info();
  std::memset(pl, 0, sizeof(*pl));
  const int bits = var_bits(var);
  const int m_pass = M < 16 ? M : 16;
  int st = plan_skinny(m_pass, N, K, bits, di, pl);
  if (st != ST_OK) return st;
  pl->passes = (M + 15) / 16;
  pl->workspace_bytes = WS_HEADER_BYTES + ws_counter_bytes(N) + (size_t)m_pass * N * sizeof(float);
  return ST_OK;
}

static int run_gemm(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
                    int var, int group, void* workspace, size_t ws_bytes, cudaStream_t stream,
                    const b200q_plan_t& pl) {
  if (!a || !bq || !scales || !c) return ST_INVALID_ARG;
  if (((uintptr_t)a | (uintptr_t)bq | (uintptr_t)c) & 15) return ST_INVALID_ARG;
  if (((uintptr_t)scales) & 1) return ST_INVALID_ARG;
  if (lda < K || ldc < N || (lda % 8) != 0) return ST_INVALID_ARG;
  if (pl.kernel != 0) return ST_UNSUPPORTED;
  if (pl.splits < 1 || (K / BLOCK_K) % pl.splits != 0 || pl.ctas_per_split < 1) return ST_INVALID_ARG;
  const int m_pass = M < 16 ? M : 16;
  const size_t need = WS_HEADER_BYTES + ws_counter_bytes(N) + (size_t)m_pass * N * sizeof(float);
  if (!workspace || ws_bytes < need || ((uintptr_t)workspace & 255)) return ST_WORKSPACE;

  SkinnyParams p;
  p.bq = reinterpret_cast<const uint4*>(bq);
  p.scales = reinterpret_cast<const __half*>(scales);
  p.counters = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES + ws_counter_bytes(N));
  p.N = N; p.K = K; p.group = group; p.lda = lda; p.ldc = ldc;
  p.KB = K / BLOCK_K; p.NT = N / BLOCK_N;
  p.S = pl.splits; p.P = pl.ctas_per_split; p.KBc = p.KB / p.S;
  p.pitch = skinny_pitch(p.KBc * 512);
  for (int m0 = 0; m0 < M; m0 += 16) {
    const int mc = (M - m0) < 16 ? (M - m0) : 16;
    p.a = reinterpret_cast<const __half*>(a) + (size_t)m0 * lda;
    p.c = reinterpret_cast<__half*>(c) + (size_t)m0 * ldc;
    p.M = mc;
    const int smem = mc * p.pitch * 2;
    cudaError_t e = skinny_launch(var, p, (mc + 7) / 8, smem, stream);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  }
  return ST_OK;
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_version(void) { return 100; }
int b200q_layout_version(void) { return 1; }

const char* b200q_status_string(int status) {
  switch (status) {
    case ST_OK: return "ok";
    case ST_INVALID_ARG: return "invalid argument (null or misaligned pointer, bad size or stride)";
    case ST_UNSUPPORTED: return "unsupported weight dtype, zero point, shape or group size";
    case ST_WORKSPACE: return "workspace missing, misaligned or too small";
    case ST_CUDA: return "CUDA runtime error";
    case ST_DEVICE_TIMEOUT: return "a bounded device-side wait timed out";
    default: return "unknown status";
  }
}

int b200q_last_cuda_error(void) { return g_last_cuda_error; }

int b200q_plan(int M, int N, int K, int wtype, int zero_point, int group, b200q_plan_t* plan) {
  if (!plan) return ST_INVALID_ARG;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, &var);
  if (st != ST_OK) return st;
  return make_plan(M, N, K, var, plan);
}

size_t b200q_workspace_bytes(int M, int N, int K, int wtype, int zero_point, int group) {
  b200q_plan_t pl;
  if (b200q_plan(M, N, K, wtype, zero_point, group, &pl) != ST_OK) return 0;
  return (size_t)pl.workspace_bytes;
}

int b200q_gemm_planned(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N,
                       int K, int wtype, int zero_point, int group, int act_dtype, void* workspace,
                       size_t workspace_bytes, void* stream, const b200q_plan_t* plan) {
  if (!plan) return ST_INVALID_ARG;
  if (act_dtype != B200Q_F16) return ST_UNSUPPORTED;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, &var);
  if (st != ST_OK) return st;
  return run_gemm(a, lda, bq, scales, c, ldc, M, N, K, var, group, workspace, workspace_bytes,
                  reinterpret_cast<cudaStream_t>(stream), *plan);
}

int b200q_gemm(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
               int wtype, int zero_point, int group, int act_dtype, void* workspace, size_t workspace_bytes,
               void* stream) {
  if (act_dtype != B200Q_F16) return ST_UNSUPPORTED;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, &var);
  if (st != ST_OK) return st;
  b200q_plan_t pl;
  st = make_plan(M, N, K, var, &pl);
  if (st != ST_OK) return st;
  return run_gemm(a, lda, bq, scales, c, ldc, M, N, K, var, group, workspace, workspace_bytes,
                  reinterpret_cast<cudaStream_t>(stream), pl);
}

int b200q_dequantize(const void* bq, const void* scales, void* w, int N, int K, int wtype, int zero_point, int group,
                     void* stream) {
  int var;
  int st = check_problem(1, N, K, wtype, zero_point, group, &var);
  if (st != ST_OK) return st;
  if (!bq || !scales || !w) return ST_INVALID_ARG;
  if (((uintptr_t)bq | (uintptr_t)w) & 15) return ST_INVALID_ARG;
  DequantParams p;
  p.bq = reinterpret_cast<const uint4*>(bq);
  p.scales = reinterpret_cast<const __half*>(scales);
  p.w = reinterpret_cast<__half*>(w);
  p.N = N; p.K = K; p.group = group; p.KB = K / BLOCK_K; p.NT = N / BLOCK_N;
  cudaError_t e = dequant_launch(var, p, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

int b200q_device_status(void* workspace, int32_t status[4], void* stream) {
  if (!workspace || !status) return ST_INVALID_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(status, workspace, 16, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && status[0] != 0) {
    e = cudaMemsetAsync(workspace, 0, 16, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  }
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return status[0] == 0 ? ST_OK : ST_DEVICE_TIMEOUT;
}

}  // extern "C"
