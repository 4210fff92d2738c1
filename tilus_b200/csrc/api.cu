// C ABI of libb200q (declared in include/b200q.h): argument validation, the static
// shape -> tile table, and kernel dispatch.  No torch types, no allocation.
#include <cmath>
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

#define B200Q_DECL_SPART(i) \
  cudaError_t stream_launch_part##i(int, const StreamParams&, int, int, cudaStream_t);
B200Q_DECL_SPART(0) B200Q_DECL_SPART(1) B200Q_DECL_SPART(2) B200Q_DECL_SPART(3)
B200Q_DECL_SPART(4) B200Q_DECL_SPART(5) B200Q_DECL_SPART(6) B200Q_DECL_SPART(7)
cudaError_t dequant_launch(int var, const DequantParams& p, cudaStream_t stream);
cudaError_t cast_launch(const CastParams& p, int act, bool swiglu, cudaStream_t stream);
cudaError_t host_fetch_launch(const void* src, int lds, void* dst, int M, int K, cudaStream_t stream);
cudaError_t gather_push_launch(const void* src, int lds, int M, int N_loc, int ldc, int* status, const GatherArgs& ga,
                               cudaStream_t stream);
cudaError_t gather_collect_launch(void* dst_local, int ld_local, int M, int ldc, int* status, const GatherArgs& ga,
                                  cudaStream_t stream);
cudaError_t quantize_launch(const void* w, int w_dtype, int ldw, void* bq, void* scales, int N, int K, int group,
                            int kind, int nbits, int ebits, int mbits, float minv, float maxv, int act,
                            cudaStream_t stream);
#define B200Q_DECL_UPART(i) \
  cudaError_t umma_launch_part##i(int, const UmmaParams&, const void*, int, cudaStream_t);
B200Q_DECL_UPART(0) B200Q_DECL_UPART(1) B200Q_DECL_UPART(2) B200Q_DECL_UPART(3)
B200Q_DECL_UPART(4) B200Q_DECL_UPART(5) B200Q_DECL_UPART(6) B200Q_DECL_UPART(7)
#define B200Q_DECL_WPART(i) \
  cudaError_t wide_launch_part##i(int, const WideParams&, const void*, int, cudaStream_t);
B200Q_DECL_WPART(0) B200Q_DECL_WPART(1) B200Q_DECL_WPART(2) B200Q_DECL_WPART(3)
B200Q_DECL_WPART(4) B200Q_DECL_WPART(5) B200Q_DECL_WPART(6) B200Q_DECL_WPART(7)
int wide_smem_bytes(int bits, int wg_stages, int a_rows, int rpg);
int wide_wg_stages(int bits, int max_smem, int a_rows, int rpg);
int wide_a_rows(int M);
int umma_smem_bytes(int tm, int bits, int a_stages, int rpg);
int umma_a_stages(int tm, int bits, int max_smem, int rpg);

static thread_local int g_last_cuda_error = 0;

static cudaError_t stream_launch(int var, const StreamParams& p, int mt, int smem, cudaStream_t s) {
  switch (var % B200Q_NPARTS) {
    case 0: return stream_launch_part0(var, p, mt, smem, s);
    case 1: return stream_launch_part1(var, p, mt, smem, s);
    case 2: return stream_launch_part2(var, p, mt, smem, s);
    case 3: return stream_launch_part3(var, p, mt, smem, s);
    case 4: return stream_launch_part4(var, p, mt, smem, s);
    case 5: return stream_launch_part5(var, p, mt, smem, s);
    case 6: return stream_launch_part6(var, p, mt, smem, s);
    default: return stream_launch_part7(var, p, mt, smem, s);
  }
}

static cudaError_t wide_launch(int var, const WideParams& p, const void* tmap, int smem, cudaStream_t s) {
  switch (var % B200Q_NPARTS) {
    case 0: return wide_launch_part0(var, p, tmap, smem, s);
    case 1: return wide_launch_part1(var, p, tmap, smem, s);
    case 2: return wide_launch_part2(var, p, tmap, smem, s);
    case 3: return wide_launch_part3(var, p, tmap, smem, s);
    case 4: return wide_launch_part4(var, p, tmap, smem, s);
    case 5: return wide_launch_part5(var, p, tmap, smem, s);
    case 6: return wide_launch_part6(var, p, tmap, smem, s);
    default: return wide_launch_part7(var, p, tmap, smem, s);
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
static int stream_pitch(int kc) {
  int bytes = kc * 2 + (kc / 32) * 16;
  if (bytes % 128 != 64) bytes += (64 - bytes % 128 + 128) % 128;
  return bytes / 2;
}
// ---- stream kernel (kernel 2) ---------------------------------------------------------------------
// Up to 8 rows: a CTA takes at most half an SM, so that two consecutive launches share an SM (the
// second prefetches while the first computes) or two CTAs of one launch do: (228 KB - 2 x 1 KB
// reserved) / 2 of shared memory.  9..16 rows: one CTA per SM with all of its shared memory, so
// that a long K chunk of the 16 activation rows fits next to the rings.
static const int kStreamSmemCap = 113 * 1024;
static int stream_slot_bytes(int bits) { return stream_gi(bits) * 256 * bits; }
// 8-row activation tiles per launch: 1 or 2 (the kernel's MT)
static int stream_mt(int m_pass) { return m_pass <= 8 ? 1 : 2; }
// CTAs of one launch per SM
static int stream_per_sm(int m_pass) { return m_pass <= 8 ? 2 : 1; }
// most activation rows one launch of the stream kernel takes
static int stream_rows_per_pass(int M) { (void)M; return 16; }
static int stream_smem_cap(int m_pass, const DeviceInfo& di) {
  return m_pass <= 8 ? kStreamSmemCap : di.max_smem;
}
// whole column tiles a CTA owns (their sums live in at most 16 KB of shared memory)
static int stream_tiles_owned(int m_pass, int NT, int cpc) {
  const int mt = stream_mt(m_pass), cap = 32 / mt;
  const int t = NT / cpc;
  return t < cap ? t : cap;
}
static int stream_fixed_smem(int m_pass, int kc, int t_own) {
  const int mt = stream_mt(m_pass);
  // barriers, scale caches, own-tile sums, activation chunk (+ 64 zero bytes), group sums as accumulator quads
  return stream_header_bytes(mt) + stream_warps(mt) * STREAM_SC_GROUPS * 32 + t_own * 16 * 8 * mt * 4 +
         m_pass * stream_pitch(kc) * 2 + 64 +
         (kc / 128) * 16 * mt * 4;
}
static int stream_smem(int m_pass, int kc, int bits, int stages, int t_own) {
  return stream_fixed_smem(m_pass, kc, t_own) + stream_warps(stream_mt(m_pass)) * stages * stream_slot_bytes(bits);
}
static int stream_stages_for(int m_pass, int kc, int bits, int t_own, const DeviceInfo& di) {
  int st = (stream_smem_cap(m_pass, di) - stream_fixed_smem(m_pass, kc, t_own)) /
           (stream_warps(stream_mt(m_pass)) * stream_slot_bytes(bits));
  return st > 8 ? 8 : st;
}
// CTAs per k chunk.  First choice (up to 8 rows): two CTAs per SM (32 warps hide the latency of the
// decode / mma chains best) with a count that divides the column tiles evenly, so that no tile is
// shared between CTAs and nothing goes through the global scratch; then one CTA per SM with
// such a count; else one CTA per SM with the left-over tiles shared item-wise.
static int stream_ctas_per_chunk(int NT, int s, int per_sm, const DeviceInfo& di) {
  const int full = di.sm_count / s;
  if (full < 1) return 0;
  for (int c = 2 * full; per_sm == 2 && c >= 1 && c * 5 >= full * 8; --c)
    if (NT % c == 0) return c;
  for (int c = full; c >= 1 && c * 5 >= full * 4; --c)
    if (NT % c == 0) return c;
  return full > NT ? NT : full;
}
static const int kStreamMaxRows = 16;
static size_t stream_workspace_bytes(int N) { return WS_HEADER_BYTES + ws_counter_bytes(N) + (size_t)16 * N * sizeof(float); }
// K is cut into S chunks (a divisor of K/512, at most one per SM) so that the activation chunk
// [M, K/S] fits next to the rings; the grid is S * CPC.  Measured preferences, in this order: all of
// K in one chunk with two ring slots per warp (the CTAs then write their own tiles without meeting
// anybody in the global scratch); the fewest chunks with three slots and no column tiles left over
// (left-over tiles are shared item-wise through the scratch, 40 % slower on the 28672-column layer
// at M = 8); the fewest chunks with two slots and none left over; then whatever fits.
static int plan_stream(int m_pass, int N, int K, int bits, const DeviceInfo& di, b200q_plan_t* pl) {
  const int KB = K / BLOCK_K, NT = N / BLOCK_N;
  int best_s = 0, best_st = 0, best_c = 0;
  auto consider = [&](int s, int want, bool no_leftover) {
    if (best_s || KB % s) return;
    const int cpc = stream_ctas_per_chunk(NT, s, stream_per_sm(m_pass), di);
    if (cpc < 1) return;
    const int t_own = stream_tiles_owned(m_pass, NT, cpc);
    if (no_leftover && cpc * t_own != NT) return;
    const int st = stream_stages_for(m_pass, (KB / s) * 512, bits, t_own, di);
    if (st >= want) { best_s = s; best_st = st; best_c = cpc; }
  };
  const int s_max = KB < di.sm_count ? KB : di.sm_count;
  consider(1, 2, true);
  for (int s = 1; s <= s_max; ++s) consider(s, 3, true);
  for (int s = 1; s <= s_max; ++s) consider(s, 2, true);
  for (int want = 3; want >= 1; --want)
    for (int s = 1; s <= s_max; ++s) consider(s, want, false);
  if (!best_s) return ST_UNSUPPORTED;
  pl->kernel = 2;
  pl->m_tiles = stream_mt(m_pass);
  pl->splits = best_s;
  pl->cluster = 1;
  pl->ctas_per_split = best_c;
  pl->warps = stream_warps(stream_mt(m_pass));
  pl->stages = best_st;
  pl->smem_bytes = stream_smem(m_pass, (KB / best_s) * 512, bits, best_st, stream_tiles_owned(m_pass, NT, best_c));
  pl->tile_m = 0;
  pl->pdl = 1;
  return ST_OK;
}

// Shapes every kernel takes: K a multiple of 128 (the packed layout's row group), N a multiple of 16,
// one scale per `group` rows with group = 32, 64 or a multiple of 128 that divides K.  The reference
// asks for K % 16 == 0, N % 16 == 0 and group % block_k == 0 with block_k = 32 as shipped
// (examples/quantization/matmul_a16wx.py:66-71, :207).  for_gemm = false: the dequantize kernel, which
// takes any multiple of 32.
static int check_problem(int M, int N, int K, int wtype, int zero_point, int group, bool for_gemm, int* var) {
  if (M < 1 || N < 1 || K < 1 || group < 1) return ST_INVALID_ARG;
  *var = variant_of(wtype, zero_point);
  if (*var < 0) return ST_UNSUPPORTED;
  if (K % 128 != 0 || N % BLOCK_N != 0) return ST_UNSUPPORTED;
  if (group % 32 != 0 || K % group != 0) return ST_UNSUPPORTED;
  if (for_gemm && group != 32 && group != 64 && group % 128 != 0) return ST_UNSUPPORTED;
  return ST_OK;
}
// the decode kernel works in whole 512-row blocks and applies one scale per 128-row group
static bool stream_takes(int K, int group) { return K % BLOCK_K == 0 && group % 128 == 0; }
static int gshift_of(int group) {  // log2(group / 128) when that is a power of two, else -1
  const int d = group / 128;
  if (d < 1 || (d & (d - 1)) != 0) return -1;
  int s = 0;
  while ((1 << s) < d) ++s;
  return s;
}

// tcgen05 kernel: tile rows, tiles and split-K so that the grid fills the SMs
static int rpg_of(int group) { return group < 128 ? 128 / group : 1; }

static void plan_umma(int M, int N, int K, int bits, int group, const DeviceInfo& di, b200q_plan_t* pl) {
  const int tm = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const int m_tiles = (M + tm - 1) / tm, n_tiles = (N + 127) / 128;
  const int ctas = m_tiles * n_tiles;
  const int kblocks = K / 64;
  int splits = 1;
  if (ctas * 2 <= di.sm_count && ctas <= N / BLOCK_N) {
    for (int s = 2; s <= 16; ++s)
      if (kblocks % (2 * s) == 0 && kblocks / s >= 8 && ctas * s <= di.sm_count + di.sm_count / 8) splits = s;
  }
  pl->kernel = 1;
  pl->m_tiles = m_tiles;
  pl->splits = splits;
  pl->cluster = 1;
  pl->ctas_per_split = ctas;
  pl->stages = umma_a_stages(tm, bits, di.max_smem, rpg_of(group));
  pl->smem_bytes = umma_smem_bytes(tm, bits, pl->stages, rpg_of(group));
  pl->tile_m = tm;
  pl->warps = 19;
  pl->passes = 1;
  pl->pdl = 0;
}

// wide tcgen05 kernel (kernel 3): 128-row x 256-column tiles, split-K while the tiles do not fill the SMs
static const int kWideMaxRows = 128;
static void plan_wide(int M, int N, int K, int bits, int group, const DeviceInfo& di, b200q_plan_t* pl) {
  const int m_tiles = (M + 127) / 128, n_tiles = (N + 255) / 256;
  const int tiles = m_tiles * n_tiles, G = K / 128;
  int splits = 1;
  for (int s = 2; s <= 32; ++s)
    if (G % s == 0 && G / s >= 2 && tiles * s <= di.sm_count + di.sm_count / 8) splits = s;
  pl->kernel = 3;
  pl->m_tiles = m_tiles;
  pl->splits = splits;
  pl->cluster = 1;
  pl->ctas_per_split = tiles;
  pl->stages = wide_wg_stages(bits, di.max_smem, wide_a_rows(M), rpg_of(group));
  pl->smem_bytes = wide_smem_bytes(bits, pl->stages, wide_a_rows(M), rpg_of(group));
  pl->tile_m = 128;
  pl->warps = 23;
  pl->passes = 1;
  pl->pdl = 1;  // always launched as a programmatic dependent
}

// The persistent CTAs of the transposed tcgen05 kernel take tiles round by round.  When the last round
// would be less than half full, its tiles are cut into `splits` K ranges (whole 128-row groups, at
// least 8 64-row blocks each) so that the round costs a fraction of a tile's time.  Returns the number
// of such tail tiles (0: none).
static int umma_tail(int tiles, int grid, int kblocks, int uniform_splits, int N, int* splits) {
  *splits = 1;
  if (uniform_splits != 1 || tiles <= grid) return 0;
  const int rem = tiles % grid;
  if (rem == 0 || rem * 2 > grid || rem > N / BLOCK_N) return 0;
  int best = 1;
  for (int s = 2; s <= 16; s *= 2)
    if (s * rem <= grid && kblocks % (2 * s) == 0 && kblocks / s >= 8) best = s;
  if (best == 1) return 0;
  *splits = best;
  return rem;
}
// fp32 scratch of the transposed tcgen05 kernel: one [tm][128] slab per tile slot
static size_t umma_partial_bytes(int slots, int tm) { return (size_t)slots * tm * 128 * sizeof(float); }

static int make_plan_uncached(int M, int N, int K, int var, int group, b200q_plan_t* pl) {
  const DeviceInfo di = device_info();
  std::memset(pl, 0, sizeof(*pl));
  const int bits = var_bits(var);
  // up to 16 rows: the mma.sync stream kernel (one weight decode per 16 x 128 tile feeds one or two
  // 8-row activation tiles); above, the tcgen05 kernels
  if (M <= kStreamMaxRows && stream_takes(K, group)) {
    if (plan_stream(M, N, K, bits, di, pl) == ST_OK) {
      pl->passes = 1;
      pl->workspace_bytes = stream_workspace_bytes(N);  // fp32 scratch [N][8 or 16]
      return ST_OK;
    }
  }
  // a few dozen rows: weights on the wide side of the MMA; beyond, the transposed prefill kernel
  if (M <= kWideMaxRows) {
    plan_wide(M, N, K, bits, group, di, pl);
  } else {
    // A last row tile of at most 16 rows (M = 4097: one row) would cost a whole 256-row tile per
    // column tile; those rows go to the decode kernel in a second launch instead (passes = 2).
    const int tail = M % 256;
    b200q_plan_t tail_plan;
    if (M > 256 && tail >= 1 && tail <= kStreamMaxRows && stream_takes(K, group) &&
        plan_stream(tail, N, K, bits, di, &tail_plan) == ST_OK) {
      plan_umma(M - tail, N, K, bits, group, di, pl);
      pl->passes = 2;
    } else {
      plan_umma(M, N, K, bits, group, di, pl);
    }
  }
  size_t part = pl->splits > 1 ? (size_t)M * N * sizeof(float) : 0;
  if (pl->kernel == 1) {  // fp32 slabs per tile slot: every tile of a split-K launch, or the cut tiles of the last round
    const int Mu = pl->passes == 2 ? M - M % 256 : M;
    const int tiles = ((Mu + pl->tile_m - 1) / pl->tile_m) * ((N + 127) / 128);
    const int grid = tiles * pl->splits < di.sm_count ? tiles * pl->splits : di.sm_count;
    int tail_splits;
    const int tail = umma_tail(tiles, grid, K / 64, pl->splits, N, &tail_splits);
    part = umma_partial_bytes(pl->splits > 1 ? tiles : tail, pl->tile_m);
  }
  size_t need = WS_HEADER_BYTES + ws_counter_bytes(N) + part;
  if (pl->passes == 2 && need < stream_workspace_bytes(N)) need = stream_workspace_bytes(N);
  pl->workspace_bytes = need;
  return ST_OK;
}

// The table is a pure function of the shape (and of the device's SM count and shared memory, which
// device_info caches for the current device), and a serving loop asks for the same few shapes over
// and over: the latest results are kept per thread.
static int make_plan(int M, int N, int K, int var, int group, b200q_plan_t* pl) {
  struct Entry { int dev, M, N, K, var, group, status; b200q_plan_t plan; };
  static thread_local Entry cache[16];
  static thread_local int used = 0, next = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  for (int i = 0; i < used; ++i) {
    const Entry& e = cache[i];
    if (e.M == M && e.N == N && e.K == K && e.var == var && e.group == group && e.dev == dev) {
      *pl = e.plan;
      return e.status;
    }
  }
  const int status = make_plan_uncached(M, N, K, var, group, pl);
  Entry& e = cache[next];
  e.dev = dev; e.M = M; e.N = N; e.K = K; e.var = var; e.group = group; e.status = status; e.plan = *pl;
  next = (next + 1) % 16;
  if (used < 16) ++used;
  return status;
}

// row tiles per raster group of the transposed tcgen05 kernel: as many as keep one group's
// activation rows (tm x K 16-bit values per tile) within 32 MB, a quarter of L2
static int umma_m_group(int tm, int K, int m_tiles) {
  const long long per_tile = (long long)tm * K * 2;
  long long g = (32ll << 20) / (per_tile > 0 ? per_tile : 1);
  if (g < 1) g = 1;
  if (g > m_tiles) g = m_tiles;
  return (int)g;
}

static int run_umma(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
                    int var, int group, int act, void* workspace, size_t ws_bytes, cudaStream_t stream,
                    const b200q_plan_t& pl) {
  const int tm = pl.tile_m;
  if (tm != 32 && tm != 64 && tm != 128 && tm != 256) return ST_INVALID_ARG;
  const int m_tiles = (M + tm - 1) / tm, n_tiles = (N + 127) / 128;
  const int kblocks = K / 64;
  if (pl.splits < 1 || kblocks % (2 * pl.splits) != 0) return ST_INVALID_ARG;  // whole 128-row groups per split
  if (pl.splits > 1 && m_tiles * n_tiles > N / BLOCK_N) return ST_INVALID_ARG;  // counters region
  if ((ldc % 8) != 0 || (((uintptr_t)scales) & 15)) return ST_INVALID_ARG;  // 16-byte stores, bulk-copied scale rows
  const int bits = var_bits(var);
  const int a_stages = umma_a_stages(tm, bits, device_info().max_smem, rpg_of(group));
  const int all_tiles = m_tiles * n_tiles;
  const int grid = pl.splits * all_tiles < device_info().sm_count ? pl.splits * all_tiles : device_info().sm_count;
  int tail_splits = 1;
  int tail_tiles = umma_tail(all_tiles, grid, kblocks, pl.splits, N, &tail_splits);
  size_t need = WS_HEADER_BYTES + ws_counter_bytes(N) + umma_partial_bytes(pl.splits > 1 ? all_tiles : tail_tiles, tm);
  if (tail_tiles > 0 && workspace && ws_bytes < need) {  // a caller with a smaller workspace: whole tiles only
    tail_tiles = 0;
    tail_splits = 1;
    need = WS_HEADER_BYTES + ws_counter_bytes(N);
  }
  if (!workspace || ws_bytes < need || ((uintptr_t)workspace & 255)) return ST_WORKSPACE;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return ST_CUDA;
  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t gstride[1] = {(cuuint64_t)lda * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)tm};
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(&tmap, act == B200Q_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(a), gdim, gstride, box, estr,
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
  p.M = M; p.N = N; p.K = K; p.G = K / 128; p.ldc = ldc;
  p.group = group;
  p.rpg = rpg_of(group);
  p.tm = tm; p.m_tiles = m_tiles; p.n_tiles = n_tiles;
  p.splits = pl.splits; p.kblocks_per_split = kblocks / pl.splits;
  p.tail_tiles = tail_tiles; p.tail_splits = tail_tiles > 0 ? tail_splits : 0;
  p.tail_kblocks = tail_tiles > 0 ? kblocks / tail_splits : 0;
  p.a_stages = a_stages;
  p.m_group = umma_m_group(tm, K, m_tiles);
  p.act = act;
  p.grid = grid;
  const int smem = umma_smem_bytes(tm, bits, a_stages, rpg_of(group));
  if (smem > device_info().max_smem) return ST_UNSUPPORTED;
  cudaError_t e = umma_launch(var, p, &tmap, smem, stream);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

static int run_wide(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
                    int var, int group, int act, void* workspace, size_t ws_bytes, cudaStream_t stream,
                    const b200q_plan_t& pl) {
  const int bits = var_bits(var);
  const int m_tiles = (M + 127) / 128, n_tiles = (N + 255) / 256, G = K / 128;
  if (pl.splits < 1 || G % pl.splits != 0) return ST_INVALID_ARG;  // whole 128-row groups per split
  if ((ldc % 8) != 0 || (((uintptr_t)scales) & 15)) return ST_INVALID_ARG;  // 16-byte stores, bulk-copied scale rows
  const size_t need = WS_HEADER_BYTES + ws_counter_bytes(N) + (pl.splits > 1 ? (size_t)M * N * sizeof(float) : 0);
  if (!workspace || ws_bytes < need || ((uintptr_t)workspace & 255)) return ST_WORKSPACE;
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return ST_CUDA;
  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t gstride[1] = {(cuuint64_t)lda * 2};
  const int a_rows = wide_a_rows(M);
  const cuuint32_t box[2] = {64u, (cuuint32_t)a_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(&tmap, act == B200Q_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(a), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = (int)r; return ST_CUDA; }
  WideParams p;
  p.bq = bq;
  p.scales = reinterpret_cast<const __half*>(scales);
  p.c = reinterpret_cast<__half*>(c);
  p.status = reinterpret_cast<int*>(workspace);
  p.counters = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES + ws_counter_bytes(N));
  p.M = M; p.N = N; p.K = K; p.G = K / 128; p.ldc = ldc;
  p.group = group;
  p.rpg = rpg_of(group);
  p.m_tiles = m_tiles; p.n_tiles = n_tiles;
  p.splits = pl.splits; p.kblocks_per_split = 2 * G / pl.splits;
  p.a_rows = a_rows;
  p.act = act;
  p.wg_stages = wide_wg_stages(bits, device_info().max_smem, a_rows, rpg_of(group));
  const int items = pl.splits * m_tiles * n_tiles;
  p.grid = items < device_info().sm_count ? items : device_info().sm_count;
  const int smem = wide_smem_bytes(bits, p.wg_stages, a_rows, rpg_of(group));
  if (smem > device_info().max_smem) return ST_UNSUPPORTED;
  cudaError_t e = wide_launch(var, p, &tmap, smem, stream);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

// b200q_gather_t of the C ABI -> the kernels' GatherArgs (checked)
static int fill_gather_args(const b200q_gather_t* gather, int M, int N, void* workspace, GatherArgs* ga) {
  std::memset(ga, 0, sizeof(*ga));
  if (gather->world < 1 || gather->world > 8 || gather->rank < 0 || gather->rank >= gather->world) return ST_INVALID_ARG;
  if (gather->mode != B200Q_GATHER_FLAGS && gather->mode != B200Q_GATHER_TAGGED) return ST_INVALID_ARG;
  const bool tagged = gather->mode == B200Q_GATHER_TAGGED;
  if (gather->ldc < gather->col_offset + N || gather->col_offset < 0 || !gather->epoch_local) return ST_INVALID_ARG;
  if ((gather->ldc & 1) || (gather->col_offset & 1)) return ST_INVALID_ARG;  // outputs leave in column pairs
  // dense rows: buffer_elems 16-bit elements between the two buffers; tagged: 64-bit words between the three
  if (gather->buffer_elems < (int64_t)M * gather->ldc / (tagged ? 2 : 1)) return ST_INVALID_ARG;
  if (!tagged && !gather->flags_local) return ST_INVALID_ARG;
  if (gather->a_prev_offset >= 0 && (gather->a_prev_offset & 7)) return ST_INVALID_ARG;
  ga->G = gather->world;
  ga->rank = gather->rank;
  ga->col_off = gather->col_offset;
  ga->mode = gather->mode;
  for (int g = 0; g < gather->world; ++g) {
    if (!gather->out[g] || (!tagged && !gather->flag_slot[g])) return ST_INVALID_ARG;
    ga->out[g] = reinterpret_cast<__half*>(gather->out[g]);
    ga->flag_slot[g] = reinterpret_cast<unsigned*>(gather->flag_slot[g]);
  }
  ga->flags = reinterpret_cast<const unsigned*>(gather->flags_local);
  ga->epoch = reinterpret_cast<unsigned*>(gather->epoch_local);
  ga->buf_elems = gather->buffer_elems;
  ga->a_prev_off = gather->a_prev_offset;
  ga->done = reinterpret_cast<unsigned*>(workspace) + 8;  // word 8 of the status header
  return ST_OK;
}

static int run_stream(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N,
                      int K, int var, int group, int act, void* workspace, size_t ws_bytes, cudaStream_t stream,
                      const b200q_plan_t& pl, const b200q_gather_t* gather = nullptr, const void* a_host = nullptr,
                      int lda_host = 0, bool staging_released = false) {
  // a_host: device-side address of activations in pinned host memory (row stride lda_host); `a` is then
  // the dense [M, K] device staging the kernel's first CTAs fill (see StreamParams)
  const int bits = var_bits(var);
  const int KB = K / BLOCK_K;
  if (!stream_takes(K, group)) return ST_UNSUPPORTED;
  if (pl.splits < 1 || KB % pl.splits != 0 || pl.ctas_per_split < 1) return ST_INVALID_ARG;
  if (pl.stages < 1 || pl.stages > 8) return ST_INVALID_ARG;
  if (((uintptr_t)scales) & 15) return ST_INVALID_ARG;  // scale rows are fetched with 32-byte bulk copies
  const size_t need = stream_workspace_bytes(N);
  if (!workspace || ws_bytes < need || ((uintptr_t)workspace & 255)) return ST_WORKSPACE;
  StreamParams p;
  p.bq = bq;
  p.scales = reinterpret_cast<const __half*>(scales);
  p.status = reinterpret_cast<int*>(workspace);
  p.counters = reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + WS_HEADER_BYTES + ws_counter_bytes(N));
  p.N = N; p.K = K; p.lda = lda; p.ldc = ldc; p.KB = KB; p.NT = N / BLOCK_N;
  p.gshift = gshift_of(group);
  // Launches that hand rows over between GPUs release the launch of their successor late: measured on two
  // GPUs, a successor that becomes resident while this launch still waits for its peers costs 0.3 - 0.5 ms
  // per 128-layer step; launches that wait for nobody lose nothing either way.
  p.trig = gather ? 1 : 0;
  p.gdiv = group / 128;
  p.S = pl.splits; p.KBc = KB / pl.splits; p.CPC = pl.ctas_per_split;
  if (p.S * p.CPC > 4 * device_info().sm_count) return ST_INVALID_ARG;
  p.pitch = stream_pitch(p.KBc * 512);
  p.stages = pl.stages;
  p.pdl = pl.pdl;
  p.act = act;
  {
    const int ipt = p.KBc * (4 / stream_gi(bits));  // items per column tile inside a k chunk
    p.ipt_shift = -1;
    if ((ipt & (ipt - 1)) == 0)
      for (int sh = 0; sh < 31; ++sh)
        if ((1 << sh) == ipt) p.ipt_shift = sh;
  }
  std::memset(&p.ga, 0, sizeof(p.ga));
  p.a_host = nullptr; p.fetch_flag = nullptr; p.fetch_ctas = 0; p.nowait = 0;
  if (a_host) {
    if (gather || M > stream_rows_per_pass(M)) return ST_INVALID_ARG;
    const int per_cta = stream_warps(stream_mt(M)) * 32 * 4;  // 16-byte pieces one CTA fetches
    p.a_host = reinterpret_cast<const __half*>(a_host);
    p.lda = lda_host;
    p.fetch_flag = reinterpret_cast<unsigned*>(workspace) + 16;  // words 16, 17 of the status header
    p.fetch_ctas = (M * (K / 8) + per_cta - 1) / per_cta;
    if (p.fetch_ctas > p.S * p.CPC) return ST_INVALID_ARG;
  }
  if (gather) {
    if (M > 16) return ST_INVALID_ARG;
    const int gst = fill_gather_args(gather, M, N, workspace, &p.ga);
    if (gst != ST_OK) return gst;
    p.ldc = gather->ldc;
  }
  const int rows = stream_rows_per_pass(M);
  for (int m0 = 0; m0 < M; m0 += rows) {
    const int mc = (M - m0) < rows ? (M - m0) : rows;
    p.a = reinterpret_cast<const __half*>(a) + (size_t)m0 * lda;  // (a_host: one pass, lda unused)
    p.c = reinterpret_cast<__half*>(c) + (size_t)m0 * ldc;
    p.M = mc;
    p.T_own = stream_tiles_owned(mc, p.NT, p.CPC);
    // (staging_released: the previous user of the staging buffer on this stream lets go of it before it
    // releases its successor - only then may this launch write it without waiting)
    p.nowait = (a_host && staging_released && p.S == 1 && p.T_own * p.CPC == p.NT) ? 1 : 0;
    const int smem = stream_smem(mc, p.KBc * 512, bits, pl.stages, p.T_own);
    if (smem > device_info().max_smem) return ST_UNSUPPORTED;
    cudaError_t e = stream_launch(var, p, stream_mt(mc), smem, stream);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  }
  return ST_OK;
}

static int run_gemm(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
                    int var, int group, int act, void* workspace, size_t ws_bytes, cudaStream_t stream,
                    const b200q_plan_t& pl) {
  if (!a || !bq || !scales || !c) return ST_INVALID_ARG;
  if (((uintptr_t)a | (uintptr_t)bq | (uintptr_t)c) & 15) return ST_INVALID_ARG;
  if (((uintptr_t)scales) & 1) return ST_INVALID_ARG;
  if (lda < K || ldc < N || (lda % 8) != 0) return ST_INVALID_ARG;
  if (pl.kernel == 1 && pl.passes == 2) {
    // the full 256-row tiles on the tcgen05 kernel, the short last tile on the decode kernel
    const int tail = M % 256;
    if (M <= 256 || tail < 1 || tail > kStreamMaxRows) return ST_INVALID_ARG;
    b200q_plan_t tail_plan;
    std::memset(&tail_plan, 0, sizeof(tail_plan));
    if (plan_stream(tail, N, K, var_bits(var), device_info(), &tail_plan) != ST_OK) return ST_UNSUPPORTED;
    b200q_plan_t head = pl;
    head.passes = 1;
    const int st = run_umma(a, lda, bq, scales, c, ldc, M - tail, N, K, var, group, act, workspace, ws_bytes, stream, head);
    if (st != ST_OK) return st;
    const size_t row0 = (size_t)(M - tail);
    return run_stream(reinterpret_cast<const unsigned short*>(a) + row0 * lda, lda, bq, scales,
                      reinterpret_cast<unsigned short*>(c) + row0 * ldc, ldc, tail, N, K, var, group, act, workspace,
                      ws_bytes, stream, tail_plan);
  }
  if (pl.kernel == 1)
    return run_umma(a, lda, bq, scales, c, ldc, M, N, K, var, group, act, workspace, ws_bytes, stream, pl);
  if (pl.kernel == 2)
    return run_stream(a, lda, bq, scales, c, ldc, M, N, K, var, group, act, workspace, ws_bytes, stream, pl);
  if (pl.kernel == 3)
    return run_wide(a, lda, bq, scales, c, ldc, M, N, K, var, group, act, workspace, ws_bytes, stream, pl);
  return ST_UNSUPPORTED;
}

static bool act_ok(int act) { return act == B200Q_F16 || act == B200Q_BF16; }

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
  int st = check_problem(M, N, K, wtype, zero_point, group, true, &var);
  if (st != ST_OK) return st;
  return make_plan(M, N, K, var, group, plan);
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
  if (!act_ok(act_dtype)) return ST_UNSUPPORTED;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, true, &var);
  if (st != ST_OK) return st;
  return run_gemm(a, lda, bq, scales, c, ldc, M, N, K, var, group, act_dtype, workspace, workspace_bytes,
                  reinterpret_cast<cudaStream_t>(stream), *plan);
}

int b200q_gemm_gather(const void* a, int lda, const void* bq, const void* scales, int M, int N, int K, int wtype,
                      int zero_point, int group, int act_dtype, void* workspace, size_t workspace_bytes, void* stream,
                      const b200q_gather_t* gather) {
  if (!act_ok(act_dtype)) return ST_UNSUPPORTED;
  if (!gather || !bq || !scales) return ST_INVALID_ARG;
  if (M > 16) return ST_UNSUPPORTED;  // the tcgen05 kernel has no fused gather: use b200q_gemm + a collective
  if (gather->a_prev_offset < 0 && (!a || ((uintptr_t)a & 15))) return ST_INVALID_ARG;
  if (gather->a_prev_offset >= 0 && (gather->a_prev_offset % 8) != 0) return ST_INVALID_ARG;
  if (((uintptr_t)bq) & 15) return ST_INVALID_ARG;
  if (lda < K || (lda % 8) != 0) return ST_INVALID_ARG;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, true, &var);
  if (st != ST_OK) return st;
  b200q_plan_t pl;
  st = make_plan(M, N, K, var, group, &pl);  // the fused gather lives in the stream kernel only
  if (st != ST_OK) return st;
  if (pl.kernel != 2) return ST_UNSUPPORTED;
  return run_stream(a, lda, bq, scales, nullptr, gather->ldc, M, N, K, var, group, act_dtype, workspace,
                    workspace_bytes, reinterpret_cast<cudaStream_t>(stream), pl, gather);
}

int b200q_gather_push(const void* shard, int lds, int M, int N_loc, void* workspace, size_t workspace_bytes,
                      void* stream, const b200q_gather_t* gather) {
  if (!shard || !gather || M < 1 || N_loc < 8) return ST_INVALID_ARG;
  if ((N_loc % 8) != 0 || (lds % 8) != 0 || lds < N_loc || (((uintptr_t)shard) & 15)) return ST_INVALID_ARG;
  if ((gather->ldc % 8) != 0 || (gather->col_offset % 8) != 0) return ST_INVALID_ARG;
  if (!workspace || workspace_bytes < WS_HEADER_BYTES || ((uintptr_t)workspace & 255)) return ST_WORKSPACE;
  GatherArgs ga;
  const int st = fill_gather_args(gather, M, N_loc, workspace, &ga);
  if (st != ST_OK) return st;
  cudaError_t e = gather_push_launch(shard, lds, M, N_loc, gather->ldc, reinterpret_cast<int*>(workspace), ga,
                                     reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

int b200q_gather_collect(void* full_local, int ld_local, int M, void* workspace, size_t workspace_bytes, void* stream,
                         const b200q_gather_t* gather) {
  if (!gather || M < 1) return ST_INVALID_ARG;
  if ((gather->ldc % 8) != 0) return ST_INVALID_ARG;
  if (full_local && ((ld_local % 8) != 0 || ld_local < gather->ldc || (((uintptr_t)full_local) & 15))) return ST_INVALID_ARG;
  if (!workspace || workspace_bytes < WS_HEADER_BYTES || ((uintptr_t)workspace & 255)) return ST_WORKSPACE;
  GatherArgs ga;
  const int st = fill_gather_args(gather, M, 0, workspace, &ga);
  if (st != ST_OK) return st;
  cudaError_t e = gather_collect_launch(full_local, ld_local, M, gather->ldc, reinterpret_cast<int*>(workspace), ga,
                                        reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

int b200q_peer_alloc(size_t bytes, void** ptr) {
  if (!ptr || bytes == 0) return ST_INVALID_ARG;
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}
int b200q_peer_export(void* ptr, unsigned char handle[64]) {
  if (!ptr || !handle) return ST_INVALID_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  std::memcpy(handle, &h, 64);
  return ST_OK;
}
int b200q_peer_open(const unsigned char handle[64], void** ptr) {
  if (!ptr || !handle) return ST_INVALID_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}
int b200q_peer_close(void* ptr) {
  if (!ptr) return ST_INVALID_ARG;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}
int b200q_peer_free(void* ptr) {
  if (!ptr) return ST_INVALID_ARG;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

int b200q_gemm(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
               int wtype, int zero_point, int group, int act_dtype, void* workspace, size_t workspace_bytes,
               void* stream) {
  if (!act_ok(act_dtype)) return ST_UNSUPPORTED;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, true, &var);
  if (st != ST_OK) return st;
  b200q_plan_t pl;
  st = make_plan(M, N, K, var, group, &pl);
  if (st != ST_OK) return st;
  return run_gemm(a, lda, bq, scales, c, ldc, M, N, K, var, group, act_dtype, workspace, workspace_bytes,
                  reinterpret_cast<cudaStream_t>(stream), pl);
}

// ---- GEMM on host buffers ------------------------------------------------------------------------
// Activations in (pinned) host memory, result back in host memory, queued on the stream by one
// call.  The activations are copied into a staging buffer the caller owns (every CTA reads all
// of them, which must not cross the host link each time).  The result, which every element of
// is written exactly once, goes straight to the host buffer when that is pinned memory the GPU
// can address (the kernel's stores are the transfer); otherwise through the second staging
// buffer and a copy.
// Who used a staging buffer last on a stream, as far as this thread's b200q_gemm_host calls know: a
// decode launch that fetches its own activations has finished reading the buffer by the time its
// successor can start; every other kernel reads it until it ends.  (Within a captured graph the order
// of launches is the order of capture; the first launch of a graph follows everything before it.)
struct StagingUse { cudaStream_t stream; const void* buf; bool released; };
static bool staging_released_by_last_use(cudaStream_t st, const void* buf, bool now_released) {
  static thread_local StagingUse uses[8];
  static thread_local int next = 0;
  for (StagingUse& u : uses)
    if (u.stream == st && u.buf == buf && u.buf != nullptr) {
      const bool was = u.released;
      u.released = now_released;
      return was;
    }
  uses[next] = {st, buf, now_released};
  next = (next + 1) % 8;
  return false;  // unknown history: wait
}

int b200q_gemm_host(const void* a_host, int lda, const void* bq, const void* scales, void* c_host, int ldc, int M,
                    int N, int K, int wtype, int zero_point, int group, int act_dtype, void* a_staging,
                    void* c_staging, void* workspace, size_t workspace_bytes, void* stream) {
  if (!a_host || !c_host || !a_staging || !c_staging) return ST_INVALID_ARG;
  if (M < 1 || N < 1 || K < 1 || lda < K || ldc < N) return ST_INVALID_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e;
  // Small activation blocks in pinned memory the GPU can address are fetched by a kernel whose PCIe
  // reads lie under the previous GEMM of the stream (fetch_kernel.cu); the rest goes through the copy engine.
  const void* a_mapped = nullptr;
  if ((size_t)M * K * 2 <= (256u << 10) && (K % 8) == 0 && (lda % 8) == 0 && (((uintptr_t)a_staging) & 15) == 0) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, a_host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer && (((uintptr_t)attr.devicePointer) & 15) == 0)
      a_mapped = attr.devicePointer;
    else
      (void)cudaGetLastError();  // an unregistered host pointer is not an error here
  }
  // Decode batches: the GEMV kernel's own first CTAs fetch the rows (one kernel, no copy operation at
  // all) when the result can also go straight to the host buffer.
  if (a_mapped && act_ok(act_dtype) && (ldc % 8) == 0 && (size_t)M * N * 2 <= (1u << 20)) {
    int var;
    b200q_plan_t pl;
    cudaPointerAttributes cattr;
    if (check_problem(M, N, K, wtype, zero_point, group, true, &var) == ST_OK &&
        make_plan(M, N, K, var, group, &pl) == ST_OK && pl.kernel == 2 && pl.passes == 1 &&
        M <= stream_rows_per_pass(M) && pl.splits * pl.ctas_per_split <= 2 * device_info().sm_count / stream_mt(M)) {
      if (cudaPointerGetAttributes(&cattr, c_host) == cudaSuccess && cattr.type == cudaMemoryTypeHost &&
          cattr.devicePointer && (((uintptr_t)cattr.devicePointer) & 15) == 0) {
        if (!bq || !scales) return ST_INVALID_ARG;
        if ((((uintptr_t)bq) & 15) || lda < K) return ST_INVALID_ARG;
        const bool released = staging_released_by_last_use(st, a_staging, true);
        return run_stream(a_staging, K, bq, scales, cattr.devicePointer, ldc, M, N, K, var, group, act_dtype, workspace,
                          workspace_bytes, st, pl, nullptr, a_mapped, lda, released);
      }
      (void)cudaGetLastError();
    }
  }
  (void)staging_released_by_last_use(st, a_staging, false);  // what follows reads the buffer until it ends
  if (a_mapped)
    e = host_fetch_launch(a_mapped, lda, a_staging, M, K, st);
  else
    e = lda == K ? cudaMemcpyAsync(a_staging, a_host, (size_t)M * K * 2, cudaMemcpyHostToDevice, st)
                 : cudaMemcpy2DAsync(a_staging, (size_t)K * 2, a_host, (size_t)lda * 2, (size_t)K * 2, M,
                                     cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  // small results into mapped pinned memory: no copy-out operation on the stream
  void* c_direct = nullptr;
  if ((size_t)M * N * 2 <= (1u << 20) && (ldc % 8) == 0) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, c_host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer && (((uintptr_t)attr.devicePointer) & 15) == 0)
      c_direct = attr.devicePointer;
    else
      (void)cudaGetLastError();  // an unregistered host pointer is not an error here
  }
  if (c_direct)
    return b200q_gemm(a_staging, K, bq, scales, c_direct, ldc, M, N, K, wtype, zero_point, group, act_dtype, workspace,
                      workspace_bytes, stream);
  const int status = b200q_gemm(a_staging, K, bq, scales, c_staging, N, M, N, K, wtype, zero_point, group, act_dtype,
                                workspace, workspace_bytes, stream);
  if (status != ST_OK) return status;
  e = ldc == N ? cudaMemcpyAsync(c_host, c_staging, (size_t)M * N * 2, cudaMemcpyDeviceToHost, st)
               : cudaMemcpy2DAsync(c_host, (size_t)ldc * 2, c_staging, (size_t)N * 2, (size_t)N * 2, M,
                                   cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

// ---- GEMM without a caller-supplied workspace and without any allocation ----------------------
// The split-K scratch (status header, arrival counters, fp32 partial sums) lives in this
// file-scope device array instead of a caller buffer.  Every GPU on which the array's module has
// been loaded holds these bytes until the process exits.  In host code `g_static_ws` is only a
// handle for the symbol, not a device address: the address each device uses is looked up once with
// cudaGetSymbolAddress while that device is current.  Device arrays start zeroed and the kernels
// leave their scratch zeroed, so nothing is cleared here.
#define B200Q_STATIC_WS_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_static_ws[B200Q_STATIC_WS_BYTES];

static int static_ws_pointer(void** out) {
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
    ptrs[dev] = ptr;
  }
  *out = ptrs[dev];
  return ST_OK;
}

size_t b200q_static_workspace_limit(void) { return (size_t)B200Q_STATIC_WS_BYTES; }

int b200q_static_ws_init(void) {
  void* ws = nullptr;
  return static_ws_pointer(&ws);
}

int b200q_gemm_static_ws(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N,
                         int K, int wtype, int zero_point, int group, int act_dtype, void* stream) {
  if (!act_ok(act_dtype)) return ST_UNSUPPORTED;
  int var;
  int st = check_problem(M, N, K, wtype, zero_point, group, true, &var);
  if (st != ST_OK) return st;
  b200q_plan_t pl;
  st = make_plan(M, N, K, var, group, &pl);
  if (st != ST_OK) return st;
  if (pl.workspace_bytes > (uint64_t)B200Q_STATIC_WS_BYTES) {
    // beyond the built-in scratch - unless all that asks for the room is the optional K split of the
    // prefill kernel's last round, which the kernel does without when the scratch is too small
    const uint64_t without_tail = pl.passes == 2 ? stream_workspace_bytes(N) : WS_HEADER_BYTES + ws_counter_bytes(N);
    if (!(pl.kernel == 1 && pl.splits == 1 && without_tail <= (uint64_t)B200Q_STATIC_WS_BYTES)) return ST_WORKSPACE;
  }
  void* ws = nullptr;
  st = static_ws_pointer(&ws);
  if (st != ST_OK) return st;
  return run_gemm(a, lda, bq, scales, c, ldc, M, N, K, var, group, act_dtype, ws, (size_t)B200Q_STATIC_WS_BYTES,
                  reinterpret_cast<cudaStream_t>(stream), pl);
}

int b200q_dequantize(const void* bq, const void* scales, void* w, int N, int K, int wtype, int zero_point, int group,
                     int act_dtype, void* stream) {
  if (!act_ok(act_dtype)) return ST_UNSUPPORTED;
  int var;
  int st = check_problem(1, N, K, wtype, zero_point, group, false, &var);
  if (st != ST_OK) return st;
  if (!bq || !scales || !w) return ST_INVALID_ARG;
  if (((uintptr_t)bq | (uintptr_t)w) & 15) return ST_INVALID_ARG;
  DequantParams p;
  p.bq = reinterpret_cast<const uint4*>(bq);
  p.scales = reinterpret_cast<const __half*>(scales);
  p.w = reinterpret_cast<__half*>(w);
  p.N = N; p.K = K; p.group = group; p.G = K / 128; p.NT = N / BLOCK_N;
  p.act = act_dtype;
  cudaError_t e = dequant_launch(var, p, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

int b200q_quantize(const void* weight, int weight_dtype, int ldw, void* bq, void* scales, int N, int K, int wtype,
                   int group, int act_dtype, void* stream) {
  if (!act_ok(act_dtype)) return ST_UNSUPPORTED;
  if (!weight || !bq || !scales) return ST_INVALID_ARG;
  if (N < 1 || K < 1 || group < 1 || ldw < K) return ST_INVALID_ARG;
  if (weight_dtype < 0 || weight_dtype > 2) return ST_UNSUPPORTED;
  const int kind = (wtype >> 16) & 0xff, nbits = (wtype >> 8) & 0xff, e = (wtype >> 4) & 0xf, m = wtype & 0xf;
  if (kind > 2 || nbits < 1 || nbits > 8) return ST_UNSUPPORTED;
  if (kind == 2 && (nbits != 1 + e + m || e < 1 || m < 1)) return ST_UNSUPPORTED;
  if (K % 128 != 0 || N % BLOCK_N != 0 || group % 32 != 0 || K % group != 0) return ST_UNSUPPORTED;
  if (((uintptr_t)bq & 15) || ((uintptr_t)scales & 1) || ((uintptr_t)weight & 3)) return ST_INVALID_ARG;
  float minv, maxv;
  if (kind == 0) { minv = 0.f; maxv = (float)((1 << nbits) - 1); }
  else if (kind == 1) { minv = -(float)(1 << (nbits - 1)); maxv = (float)((1 << (nbits - 1)) - 1); }
  else {
    const int bias = (1 << (e - 1)) - 1, top = (1 << e) - 1 - (e == 5 ? 1 : 0);
    maxv = ldexpf(2.0f - ldexpf(1.0f, -m), top - bias);
    minv = -maxv;
  }
  cudaError_t err = quantize_launch(weight, weight_dtype, ldw, bq, scales, N, K, group, kind, nbits, e, m, minv, maxv,
                                    act_dtype, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) { g_last_cuda_error = (int)err; return ST_CUDA; }
  return ST_OK;
}

static int run_cast(const void* x, int ldx, void* out, int ldo, float* out_sf, int tokens, int hidden, int group,
                    int act_dtype, bool swiglu, const int32_t* pos_to_token_topk, const float* topk_weights,
                    const int32_t* pos_to_expert, int use_clamp, float clamp_value, void* stream) {
  if (!act_ok(act_dtype)) return ST_UNSUPPORTED;
  if (!x || !out || !out_sf) return ST_INVALID_ARG;
  if (tokens < 1 || hidden < 1 || group < 1) return ST_INVALID_ARG;
  if (group % 128 != 0 || group > 512 || hidden % group != 0) return ST_UNSUPPORTED;
  if (ldx < (swiglu ? 2 * hidden : hidden) || ldo < hidden || (ldx % 8) != 0 || (ldo % 8) != 0) return ST_INVALID_ARG;
  if ((((uintptr_t)x) & 15) || (((uintptr_t)out) & 7) || (((uintptr_t)out_sf) & 3)) return ST_INVALID_ARG;
  CastParams p;
  p.x = reinterpret_cast<const unsigned short*>(x);
  p.out = reinterpret_cast<unsigned char*>(out);
  p.out_sf = out_sf;
  p.T = tokens; p.H = hidden; p.ldx = ldx; p.ldo = ldo; p.group = group;
  p.pos_to_token_topk = pos_to_token_topk;
  p.topk_weights = topk_weights;
  p.pos_to_expert = pos_to_expert;
  p.clamp = clamp_value;
  p.use_clamp = use_clamp ? 1 : 0;
  cudaError_t e = cast_launch(p, act_dtype, swiglu, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return ST_OK;
}

int b200q_per_token_cast(const void* x, int ldx, void* out, int ldo, float* out_sf, int tokens, int hidden, int group,
                         int act_dtype, void* stream) {
  return run_cast(x, ldx, out, ldo, out_sf, tokens, hidden, group, act_dtype, false, nullptr, nullptr, nullptr, 0, 0.f,
                  stream);
}

int b200q_swiglu_per_token_cast(const void* x, int ldx, void* out, int ldo, float* out_sf, int tokens, int hidden,
                                int group, int act_dtype, const int32_t* pos_to_token_topk, const float* topk_weights,
                                const int32_t* pos_to_expert, int use_clamp, float clamp_value, void* stream) {
  return run_cast(x, ldx, out, ldo, out_sf, tokens, hidden, group, act_dtype, true, pos_to_token_topk, topk_weights,
                  pos_to_expert, use_clamp, clamp_value, stream);
}

int b200q_gemm_swiglu_cast(const void* a, int lda, const void* bq, const void* scales, void* gate_up, int ldg,
                           void* out, int ldo, float* out_sf, int M, int N, int K, int wtype, int zero_point, int group,
                           int act_dtype, int cast_group, int use_clamp, float clamp_value, void* workspace,
                           size_t workspace_bytes, void* stream) {
  if ((N & 1) != 0) return ST_INVALID_ARG;
  const int st = b200q_gemm(a, lda, bq, scales, gate_up, ldg, M, N, K, wtype, zero_point, group, act_dtype, workspace,
                            workspace_bytes, stream);
  if (st != ST_OK) return st;
  return run_cast(gate_up, ldg, out, ldo, out_sf, M, N / 2, cast_group, act_dtype, true, nullptr, nullptr, nullptr,
                  use_clamp, clamp_value, stream);
}

int b200q_device_status(void* workspace, int32_t status[4], void* stream) {
  if (!status) return ST_INVALID_ARG;
  const bool builtin = workspace == nullptr;  // the scratch of b200q_gemm_static_ws
  if (builtin) {
    const int st = static_ws_pointer(&workspace);
    if (st != ST_OK) return st;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(status, workspace, 16, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && status[0] != 0) {
    // a launch that gave up may have left partial sums and arrival counters behind: the built-in
    // scratch is put back to zero as a whole (its owner cannot do it), a caller's workspace only
    // loses the report (the caller clears the rest, whose size only it knows)
    e = cudaMemsetAsync(workspace, 0, builtin ? (size_t)B200Q_STATIC_WS_BYTES : 16, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  }
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return ST_CUDA; }
  return status[0] == 0 ? ST_OK : ST_DEVICE_TIMEOUT;
}

}  // extern "C"
