// C ABI of libb200q (declared in include/b200q.h): argument validation, the static
// shape -> tile table, and kernel dispatch.  No torch types, no allocation.
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda.h>

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
#define B200Q_DECL_UPART(i) \
  cudaError_t umma_launch_part##i(int, const UmmaParams&, const void*, int, cudaStream_t);
B200Q_DECL_UPART(0) B200Q_DECL_UPART(1) B200Q_DECL_UPART(2) B200Q_DECL_UPART(3)
B200Q_DECL_UPART(4) B200Q_DECL_UPART(5) B200Q_DECL_UPART(6) B200Q_DECL_UPART(7)
int umma_smem_bytes(int tm);

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

static cudaError_t umma_launch(int var, const UmmaParams& p, const void* tmap, int smem, cudaStream_t s) {
  switch (var % B200Q_NPARTS) {
    case 0: return umma_launch_part0(var, p, tmap, smem, s);
    case 1: return umma_launch_part1(var, p, tmap, smem, s);
    case 2: return umma_launch_part2(var, p, tmap, smem, s);
    case 3: return umma_launch_part3(var, p, tmap, smem, s);
    case 4: return umma_launch_part4(var, p, tmap, smem, s);
    case 5: return umma_launch_part5(var, p, tmap, smem, s);
    case 6: return umma_launch_part6(var, p, tmap, smem, s);
    default: return umma_launch_part7(var, p, tmap, smem, s);
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link to libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
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
// per 32 columns, and pitch bytes = 64 (mod 128), so that 8 lanes reading 16 bytes each from
// two rows x four 32-column units touch 8 different 16-byte bank groups
static int skinny_pitch(int kc) {
  int bytes = kc * 2 + (kc / 32) * 16;
  if (bytes % 128 != 64) bytes += (64 - bytes % 128 + 128) % 128;
  return bytes / 2;
}
// warps per CTA of the skinny kernel (fixed by its launch bounds)
// mirrors of skinny_kernel.cu: 8 warps per CTA, one weight ring per warp, items of GI groups
static const int kSkinnyWarps = 8;
static int skinny_item_bytes(int bits) { return (bits <= 2 ? 4 : 2) * 256 * bits; }
// dynamic shared memory of the skinny kernel: barriers + per-warp weight rings + output tile
// sums + activation chunk + per-group activation sums
static int skinny_smem(int m_pass, int kc, int bits, int stages, int tiles_max) {
  const int mt = (m_pass + 7) / 8;
  return 512 + kSkinnyWarps * stages * skinny_item_bytes(bits) + tiles_max * 16 * 8 * mt * 4 +
         m_pass * skinny_pitch(kc) * 2 + (kc / 128) * 8 * mt * 4;
}
// k splits inside a cluster (reduced through distributed shared memory): pairs of CTAs
// (clusters of four 200 KB CTAs measured twice as slow: fewer of them fit a GPC at once)
static int skinny_cluster(int splits) { return splits % 2 == 0 ? 2 : 1; }

// ---- static shape -> tile table ------------------------------------------------------------
// Exact entries for the shapes this library is benchmarked on come first; anything else
// goes through the balance rule below.
struct TableEntry {
  int bits, m_lo, m_hi, N, K;
  int splits;
};
static const TableEntry kSkinnyTable[] = {
    // bits  M range   N      K     S
    {4, 1, 8, 8192, 8192, 1},
};

static int plan_skinny(int m_pass, int N, int K, int bits, const DeviceInfo& di, b200q_plan_t* pl) {
  const int KB = K / BLOCK_K, NT = N / BLOCK_N;
  const int mt = (m_pass + 7) / 8;
  const int ipb = bits <= 2 ? 1 : 2;  // items per block
  int forced = 0;
  for (const TableEntry& t : kSkinnyTable)
    if (t.bits == bits && m_pass >= t.m_lo && m_pass <= t.m_hi && t.N == N && t.K == K) forced = t.splits;
  double best_cost = 1e30;
  int best_s = 0, best_p = 0, best_st = 0;
  for (int pass = 0; pass < 2 && !best_s; ++pass) {  // pass 0 honours the table, pass 1 ignores it
    for (int s = 1; s <= KB && s <= di.sm_count; ++s) {
      if (KB % s) continue;
      if (pass == 0 && forced && s != forced) continue;
      const int kbc = KB / s;
      for (int occ = 2; occ >= 1; --occ) {  // CTAs per SM
        int P = di.sm_count * occ / s;
        if (P < 1) continue;
        if (P > NT) P = NT;
        const int tiles_max = (NT + P - 1) / P;
        const int fixed = skinny_smem(m_pass, kbc * 512, bits, 0, tiles_max);
        const int cap = (di.max_smem + 1024) / occ - 1024 - (occ == 2 ? 1024 : 0);
        int stages = (cap - fixed) / (kSkinnyWarps * skinny_item_bytes(bits));
        if (stages > 8) stages = 8;
        if (stages < 2) continue;
        const int cta_items = tiles_max * kbc * ipb;
        const int warp_items = (cta_items + kSkinnyWarps - 1) / kSkinnyWarps;
        const int gs = s / skinny_cluster(s);
        // time ~ the busiest SM's longest warp, staging the activation chunk, reduction traffic
        const double cost = (double)warp_items * kSkinnyWarps * occ / ipb + 0.05 * m_pass * kbc * occ + 0.3 * s +
                            2.0 * (s > 1) + 3.0 * (gs > 1) + (stages < 3 ? 2.0 : 0.0) + (occ == 1 ? 1.0 : 0.0);
        if (cost < best_cost) { best_cost = cost; best_s = s; best_p = P; best_st = stages; }
      }
    }
  }
  if (!best_s) return ST_UNSUPPORTED;
  const int kbc = KB / best_s;
  // enough bytes in flight per CTA to cover the memory latency; more only costs shared memory
  while (best_st > 3 && kSkinnyWarps * (best_st - 1) * skinny_item_bytes(bits) >= 64 * 1024) --best_st;
  pl->kernel = 0;
  pl->m_tiles = mt;
  pl->splits = best_s;
  pl->cluster = skinny_cluster(best_s);
  pl->ctas_per_split = best_p;
  pl->warps = kSkinnyWarps;
  pl->stages = best_st;
  pl->smem_bytes = skinny_smem(m_pass, kbc * 512, bits, best_st, (NT + best_p - 1) / best_p);
  pl->tile_m = 0;
  pl->pdl = 1;
  pl->debug = 0;
  return ST_OK;
}

// group_mult: 128 for the GEMM kernels (one scale per 128-row group and column), 32 for
// the dequantize kernel
static int check_problem(int M, int N, int K, int wtype, int zero_point, int group, int group_mult, int* var) {
  if (M < 1 || N < 1 || K < 1 || group < 1) return ST_INVALID_ARG;
  *var = variant_of(wtype, zero_point);
  if (*var < 0) return ST_UNSUPPORTED;
  if (K % BLOCK_K != 0 || N % BLOCK_N != 0) return ST_UNSUPPORTED;
  if (group % group_mult != 0 || K % group != 0) return ST_UNSUPPORTED;
  // the GEMM kernels index scale rows with a shift: group = 128 * 2^s, or one group per column
  if (group_mult == 128 && group != K && ((group / 128) & (group / 128 - 1)) != 0) return ST_UNSUPPORTED;
  return ST_OK;
}
static int gshift_of(int group, int K) {
  if (group == K) return -1;
  int s = 0;
  while ((128 << s) < group) ++s;
  return s;
}

// tcgen05 kernel: tile rows, tiles and split-K so that the grid fills the SMs
static void plan_umma(int M, int N, int K, const DeviceInfo& di, b200q_plan_t* pl) {
  const int tm = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const int m_tiles = (M + tm - 1) / tm, n_tiles = (N + 127) / 128;
  const int ctas = m_tiles * n_tiles;
  const int kblocks = K / 64;
  int splits = 1;
  if (ctas * 2 <= di.sm_count && ctas <= N / BLOCK_N) {
    for (int s = 2; s <= 16; ++s)
      if (kblocks % s == 0 && kblocks / s >= 8 && ctas * s <= di.sm_count + di.sm_count / 8) splits = s;
  }
  pl->kernel = 1;
  pl->m_tiles = m_tiles;
  pl->splits = splits;
  pl->cluster = 1;
  pl->ctas_per_split = ctas;
  pl->smem_bytes = umma_smem_bytes(tm);
  pl->tile_m = tm;
  pl->stages = 4;
  pl->warps = 10;
  pl->passes = 1;
  pl->pdl = 0;
  pl->debug = 0;
}

static int make_plan(int M, int N, int K, int var, b200q_plan_t* pl) {
  const DeviceInfo di = device_info();
  std::memset(pl, 0, sizeof(*pl));
  const int bits = var_bits(var);
  if (M > 16) {
    plan_umma(M, N, K, di, pl);
    const size_t part = pl->splits > 1 ? (size_t)M * N * sizeof(float) : 0;
    pl->workspace_bytes = WS_HEADER_BYTES + ws_counter_bytes(N) + part;
    return ST_OK;
  }
  const int m_pass = M < 16 ? M : 16;
  int st = plan_skinny(m_pass, N, K, bits, di, pl);
  if (st != ST_OK) return st;
  pl->passes = (M + 15) / 16;
  pl->workspace_bytes = WS_HEADER_BYTES + ws_counter_bytes(N) + (size_t)m_pass * N * sizeof(float);
  return ST_OK;
}

static int run_umma(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
                    int var, int group, void* workspace, size_t ws_bytes, cudaStream_t stream,
                    const b200q_plan_t& pl) {
  const int tm = pl.tile_m;
  if (tm != 32 && tm != 64 && tm != 128 && tm != 256) return ST_INVALID_ARG;
  const int m_tiles = (M + tm - 1) / tm, n_tiles = (N + 127) / 128;
  const int kblocks = K / 64;
  if (pl.splits < 1 || kblocks % pl.splits != 0) return ST_INVALID_ARG;
  if (pl.splits > 1 && m_tiles * n_tiles > N / BLOCK_N) return ST_INVALID_ARG;  // counters region
  const size_t need = WS_HEADER_BYTES + ws_counter_bytes(N) + (pl.splits > 1 ? (size_t)M * N * sizeof(float) : 0);
  if (!workspace || ws_bytes < need || ((uintptr_t)workspace & 255)) return ST_WORKSPACE;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return ST_CUDA;
  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t gstride[1] = {(cuuint64_t)lda * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)tm};
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(a), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = (int)r; return ST_CUDA; }
  UmmaParams p;
  p.bq = reinterpret_cast<const uint4*>(bq);
  p.scales = reinterpret_cast<const __half*>(scales);
  p.c = reinterpret_cast<__half*>(c);
  p.status = reinterpret_cast<int*>(workspace);
  p.counters = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES + ws_counter_bytes(N));
  p.M = M; p.N = N; p.K = K; p.KB = K / BLOCK_K; p.ldc = ldc;
  p.gshift = gshift_of(group, K);
  p.tm = tm; p.m_tiles = m_tiles; p.n_tiles = n_tiles;
  p.splits = pl.splits; p.kblocks_per_split = kblocks / pl.splits;
  const int smem = umma_smem_bytes(tm);
  if (smem > device_info().max_smem) return ST_UNSUPPORTED;
  cudaError_t e = umma_launch(var, p, &tmap, smem, stream);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

static int run_gemm(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
                    int var, int group, void* workspace, size_t ws_bytes, cudaStream_t stream,
                    const b200q_plan_t& pl) {
  if (!a || !bq || !scales || !c) return ST_INVALID_ARG;
  if (((uintptr_t)a | (uintptr_t)bq | (uintptr_t)c) & 15) return ST_INVALID_ARG;
  if (((uintptr_t)scales) & 1) return ST_INVALID_ARG;
  if (lda < K || ldc < N || (lda % 8) != 0) return ST_INVALID_ARG;
  if (pl.kernel == 1)
    return run_umma(a, lda, bq, scales, c, ldc, M, N, K, var, group, workspace, ws_bytes, stream, pl);
  if (pl.kernel != 0) return ST_UNSUPPORTED;
  if (pl.splits < 1 || (K / BLOCK_K) % pl.splits != 0 || pl.ctas_per_split < 1) return ST_INVALID_ARG;
  const int bits = var_bits(var);
  if (pl.stages < 1 || pl.stages > 8) return ST_INVALID_ARG;
  if (pl.cluster < 1 || pl.cluster > 8 || pl.splits % pl.cluster != 0) return ST_INVALID_ARG;
  if (pl.ctas_per_split > N / BLOCK_N) return ST_INVALID_ARG;
  const int m_pass = M < 16 ? M : 16;
  const size_t need = WS_HEADER_BYTES + ws_counter_bytes(N) + (size_t)m_pass * N * sizeof(float);
  if (!workspace || ws_bytes < need || ((uintptr_t)workspace & 255)) return ST_WORKSPACE;

  SkinnyParams p;
  p.bq = reinterpret_cast<const uint4*>(bq);
  p.scales = reinterpret_cast<const __half*>(scales);
  p.counters = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES + ws_counter_bytes(N));
  p.N = N; p.K = K; p.group = group; p.gshift = gshift_of(group, K); p.lda = lda; p.ldc = ldc;
  p.KB = K / BLOCK_K; p.NT = N / BLOCK_N;
  p.CS = pl.cluster; p.GS = pl.splits / pl.cluster; p.P = pl.ctas_per_split; p.KBc = p.KB / pl.splits;
  p.tiles_max = (p.NT + p.P - 1) / p.P;
  p.pitch = skinny_pitch(p.KBc * 512);
  p.stages = pl.stages;
  p.status = reinterpret_cast<int*>(workspace);
  p.debug_skip = pl.debug;
  p.pdl = pl.pdl;
  for (int m0 = 0; m0 < M; m0 += 16) {
    const int mc = (M - m0) < 16 ? (M - m0) : 16;
    p.a = reinterpret_cast<const __half*>(a) + (size_t)m0 * lda;
    p.c = reinterpret_cast<__half*>(c) + (size_t)m0 * ldc;
    p.M = mc;
    const int smem = skinny_smem(mc, p.KBc * 512, bits, pl.stages, p.tiles_max);
    if (smem > device_info().max_smem) return ST_UNSUPPORTED;
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
  int st = check_problem(M, N, K, wtype, zero_point, group, 128, &var);
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
  int st = check_problem(M, N, K, wtype, zero_point, group, 128, &var);
  if (st != ST_OK) return st;
  return run_gemm(a, lda, bq, scales, c, ldc, M, N, K, var, group, workspace, workspace_bytes,
                  reinterpret_cast<cudaStream_t>(stream), *plan);
}

int b200q_gemm(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
               int wtype, int zero_point, int group, int act_dtype, void* workspace, size_t workspace_bytes,
               void* stream) {
  if (act_dtype != B200Q_F16) return ST_UNSUPPORTED;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, 128, &var);
  if (st != ST_OK) return st;
  b200q_plan_t pl;
  st = make_plan(M, N, K, var, &pl);
  if (st != ST_OK) return st;
  return run_gemm(a, lda, bq, scales, c, ldc, M, N, K, var, group, workspace, workspace_bytes,
                  reinterpret_cast<cudaStream_t>(stream), pl);
}

// ---- GEMM without a caller-supplied workspace and without any allocation ----------------------
// The split-K scratch (status header, arrival counters, fp32 partial sums) lives in this
// file-scope device array instead of a caller buffer.  Every GPU that loads the library holds
// these bytes until the process exits.  In host code `g_static_ws` is only a handle for the
// symbol, not a device address: the address each device uses is looked up once with
// cudaGetSymbolAddress while that device is current.
#define B200Q_STATIC_WS_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_static_ws[B200Q_STATIC_WS_BYTES];

static int static_ws_pointer(void** out, cudaStream_t stream) {
  static std::mutex mu;
  static void* ptrs[16] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  if (dev < 0 || dev >= 16) return ST_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_ws);  // device `dev` is current
    if (e != cudaSuccess || !ptr) { g_last_cuda_error = (int)e; return ST_CUDA; }
    // the kernels expect zeros and leave zeros; start from a known state all the same
    e = cudaMemsetAsync(ptr, 0, B200Q_STATIC_WS_BYTES, stream);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
    ptrs[dev] = ptr;
  }
  *out = ptrs[dev];
  return ST_OK;
}

size_t b200q_static_workspace_limit(void) { return (size_t)B200Q_STATIC_WS_BYTES; }

int b200q_gemm_static_ws(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N,
                         int K, int wtype, int zero_point, int group, int act_dtype, void* stream) {
  if (act_dtype != B200Q_F16) return ST_UNSUPPORTED;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, 128, &var);
  if (st != ST_OK) return st;
  b200q_plan_t pl;
  st = make_plan(M, N, K, var, &pl);
  if (st != ST_OK) return st;
  if (pl.workspace_bytes > (uint64_t)B200Q_STATIC_WS_BYTES) return ST_WORKSPACE;  // beyond the built-in scratch
  void* ws = nullptr;
  st = static_ws_pointer(&ws, reinterpret_cast<cudaStream_t>(stream));
  if (st != ST_OK) return st;
  return run_gemm(a, lda, bq, scales, c, ldc, M, N, K, var, group, ws, (size_t)B200Q_STATIC_WS_BYTES,
                  reinterpret_cast<cudaStream_t>(stream), pl);
}

int b200q_dequantize(const void* bq, const void* scales, void* w, int N, int K, int wtype, int zero_point, int group,
                     void* stream) {
  int var;
  int st = check_problem(1, N, K, wtype, zero_point, group, 32, &var);
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
