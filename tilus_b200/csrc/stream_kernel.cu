// Decode path: C[M<=16, N] = A[M, K] x dequant(Bq[K, N]) - the memory-bound GEMV / skinny GEMM.
//
// Data movement.  The (column tile, k block) items of the weight matrix - GI consecutive
// 128-row groups of a 16-column x 512-row block, 1..2 KB contiguous - are cut into equal
// contiguous runs, one per warp, and every CTA gets the same number of items whatever the
// shape.  Lane 0 of a warp keeps the warp's own shared-memory ring full with TMA bulk copies
// (cp.async.bulk, completion on an mbarrier per slot).  Weights and scales are constants, so
// the ring is filled and the warp's scales are cached in shared memory before the kernel
// waits for its predecessor in the stream (programmatic dependent launch): the memory
// system always has the next layer's requests queued behind the current layer's.  A CTA
// takes at most half of an SM (16 warps at <= 64 registers, <= 113 KB of shared memory): two
// CTAs of one launch share an SM, or - when a launch has one CTA per SM - the next launch
// of the stream becomes resident beside it and prefetches while it computes.  K is cut into S
// chunks when the activation chunk [M, K/S] would not fit next to the rings; a CTA works
// inside one chunk.
//
// Compute.  One 128-row group at a time.  A lane reads its two units (columns r and r+8, 32
// rows each) with one vector load per unit, turns them into tensor-core operands with the
// unit decoder's "linear" patterns (decode.cuh, pair_lin: one mask per pair of codes, no
// floating-point work per weight) and issues mma.sync.m16n8k16 with the weight tile as the
// 16-row operand and the (up to 8-row) activation slice as the 8-column operand.  An integer
// code q lands in the mantissa of an fp16 subnormal (value q * 2^(T-24)), a float code in
// its own exponent / mantissa bits; the tensor core multiplies these exactly by activations
// that were pre-multiplied by 2^-T when the CTA staged them into shared memory.  The
// accumulator of a group starts from the zero-point term -zero_point * sum_k(a_k) / F (group
// sums computed during staging, stored in accumulator-fragment order), and once per group
// and column it is scaled:   C += (s * F) * acc_group,   F = 2^24 (integers) or 2^(15 - bias).
// Products are exact, sums fp32; the weights are never rounded to fp16 here, so the result
// is at least as close to the real-valued product as the reference's cast-scale-dot; the
// bit-exact weight values are what the dequantize kernel returns.  The k index of the mma is
// a private permutation (a dot product does not care about the order of its terms): lane
// (r, j) owns rows j*32 .. j*32+31 of the group, so its weights are one contiguous unit per
// column and its activations contiguous 16-byte pieces.
//
// Output.  Every CTA owns T_own whole column tiles, whose partial 16 x M sums its warps add
// into a tile buffer in shared memory (red.shared) and which the CTA writes to C at the end
// without any traffic to other CTAs.  The tiles that do not divide among the CTAs are cut
// into equal item runs, one per CTA, which are worked through first: such a partial tile is
// added into an fp32 scratch array [N][8*MT] with vector red.global, then the warp adds its
// item count to the tile's arrival counter; whoever completes the count converts the sums
// to fp16, writes C and puts scratch and counter back to zero - long before the CTA's own
// tiles are done, so these round trips stay off the tail.  When K is cut in chunks the own
// tiles meet in the same scratch at the end of the kernel.  Nobody waits for anybody: the only
// waits are on the mbarriers of the warp's own bulk copies (bounded).
//
// Reference: QuantizedMatmul.__call__, examples/quantization/matmul_a16wx.py:231-405 (cast,
// scale multiply, fp32 dot, fp16 store; its serial fp16 split-K, :375-398, is replaced by the
// fp32 reduction).
#include "common.cuh"

#ifndef B200Q_PART
#define B200Q_PART 0
#endif
#ifndef B200Q_NPARTS
#define B200Q_NPARTS 1
#endif

namespace b200q {


// the B words of one unit, from shared memory (plain loads: the compiler may predicate and schedule them)
template <int B>
__device__ __forceinline__ void ld_unit_words(const unsigned char* ptr, uint32_t (&w)[B]) {
  if constexpr (B % 4 == 0) {
#pragma unroll
    for (int q = 0; q < B / 4; ++q) {
      const uint4 v = reinterpret_cast<const uint4*>(ptr)[q];
      w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
    }
  } else if constexpr (B % 2 == 0) {
#pragma unroll
    for (int q = 0; q < B / 2; ++q) {
      const uint2 v = reinterpret_cast<const uint2*>(ptr)[q];
      w[2 * q] = v.x; w[2 * q + 1] = v.y;
    }
  } else {
#pragma unroll
    for (int q = 0; q < B; ++q) w[q] = reinterpret_cast<const uint32_t*>(ptr)[q];
  }
}

// 16-bit pattern of an output value in the activation dtype (ACT 0: fp16, 1: bf16)
template <int ACT>
__device__ __forceinline__ unsigned short out_bits(float v) {
  if constexpr (ACT == 0) return __half_as_ushort(__float2half_rn(v));
  else return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
// Two adjacent output values (columns n and n + 1 of row m, n even) of a launch with a fused
// all-gather, written into the full output row of every rank (peer-mapped pointers, stores only): a
// 4-byte store into the dense row buffer, or - tagged mode - one 64-bit store of the two values with
// the call number `tag` in the upper half.
template <int GATHER, int ACT>
__device__ __forceinline__ void store_pair(const StreamParams& p, size_t gather_buf, unsigned tag, int m, int n,
                                           float v0, float v1) {
  const uint32_t h2 = (uint32_t)out_bits<ACT>(v0) | ((uint32_t)out_bits<ACT>(v1) << 16);
  if constexpr (GATHER == 1) {
    const size_t off = gather_buf + (size_t)m * p.ldc + p.ga.col_off + n;
    for (int g = 0; g < p.ga.G; ++g)
      *reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned short*>(p.ga.out[g]) + off) = h2;
  } else {
    const size_t word = gather_buf + (((size_t)m * p.ldc + p.ga.col_off + n) >> 1);
    const unsigned long long v = (unsigned long long)h2 | ((unsigned long long)tag << 32);
    for (int g = 0; g < p.ga.G; ++g)
      asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long*>(p.ga.out[g]) + word),
                   "l"(v)
                   : "memory");
  }
}
// One output value of a launch without gather: a 2-byte store into C.
template <int ACT>
__device__ __forceinline__ void store_one(const StreamParams& p, int m, int n, float v) {
  reinterpret_cast<unsigned short*>(p.c)[(size_t)m * p.ldc + n] = out_bits<ACT>(v);
}
constexpr bool gather_pairs(int gather) { return gather == 1 || gather == 2; }
// two tagged words (16 bytes) as they are now in memory; each 64-bit half is read atomically
__device__ __forceinline__ ulonglong2 ld_tagged2(const unsigned long long* src) {
  ulonglong2 v;
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(src) : "memory");
  return v;
}
// a scale of the activation dtype (raw 16 bits in the shared-memory cache) as fp32
template <int ACT>
__device__ __forceinline__ float scale_f32(unsigned short bits) {
  if constexpr (ACT == 0) return __half2float(__ushort_as_half(bits));
  else return __uint_as_float((uint32_t)bits << 16);
}
// Two bf16 activations (one 32-bit word) as fp16: exact for every bf16 value whose magnitude lies in
// fp16's range (bf16 carries 8 significant bits, fp16 11); larger magnitudes saturate at +-65504,
// magnitudes below 2^-24 round to zero.  The mma.sync path multiplies in fp16.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w) {
  const float lo = fminf(fmaxf(__uint_as_float(w << 16), -65504.f), 65504.f);
  const float hi = fminf(fmaxf(__uint_as_float(w & 0xffff0000u), -65504.f), 65504.f);
  return bits_from_h2(__floats2half2_rn(lo, hi));
}

// one non-blocking look at an mbarrier phase
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Shared-memory layout (byte offsets from the dynamic smem base):
//   [0, HDR)     mbarriers [warp][stage]   (up to 8 stages of 8 bytes per warp, HDR a multiple of 1 KB)
//   [HDR, ...)   rings [warp][stage][ITEM_BYTES] of packed weights
//   then         scale caches [warp][STREAM_SC_GROUPS][16] 16-bit scales: those of the warp's next groups
//   then         tile sums of the CTA's own column tiles [T_own][16 columns][8*MT rows] floats
//   then         activation chunk [M][pitch] halfs, then group sums [groups][8*MT] floats
//
// MT = 1 (up to 8 rows): at most half an SM per CTA, so that two CTAs - of this launch or of the next
// one in the stream - share an SM.  MT = 2 (up to 16 rows): one CTA per SM with all of its registers
// and shared memory, which keeps the two 8-row accumulator sets in registers and a K chunk of the
// 16 activation rows next to the rings.
template <int VAR, int MT, int GATHER, int ACT>
__global__ void __launch_bounds__(stream_warps(MT) * 32, MT == 1 ? 2 : 1) stream_kernel(const StreamParams p) {
  constexpr int B = var_bits(VAR);
  constexpr int MP = 8 * MT;
  constexpr int BIAS = var_bias(VAR);
  constexpr int GI = stream_gi(B);
  constexpr int NI = 4 / GI;  // items per block
  constexpr int ITEM_BYTES = GI * 256 * B;
  constexpr int SLOT_BYTES = ITEM_BYTES;
  constexpr int NWARPS = stream_warps(MT);
  constexpr int HDR = stream_header_bytes(MT);
  constexpr int SCG = STREAM_SC_GROUPS;
  constexpr float F = (float)(1u << lin_factor_log2(VAR));
  // Where the linear pattern of a pair sits in the fp16 mantissa (bit T, decode.cuh int_target) sets a
  // factor 2^T on its products; the activations are pre-multiplied by 2^-T when they are staged.
  // 8-bit integers and the float types have T = 0 for every pair and need no such pass.
  constexpr bool PRESCALE = !var_is_float(VAR) && B != 8;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int NST = p.stages;
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem_raw);
  unsigned char* sScale = smem_raw + HDR + (size_t)NWARPS * NST * SLOT_BYTES;
  float* sAcc = reinterpret_cast<float*>(sScale + (size_t)NWARPS * SCG * 32);
  __half* sA = reinterpret_cast<__half*>(sAcc + (size_t)p.T_own * 16 * MP);
  // 64 zero bytes after the activation chunk: what the lanes of rows that do not exist read
  // -zero_point * sum of the activations of each 128-row group, divided by F, laid out as the
  // accumulator fragment of the first MMA of a group: [group][MT][j = 0..3] x {row 2j, row 2j+1, row 2j, row 2j+1}
  float* sNb = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(sA) + (size_t)p.M * p.pitch * 2 + 64);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, j = lane & 3;
  const int chunk = blockIdx.x % p.S, ci = blockIdx.x / p.S;
  const int kb_base = chunk * p.KBc;
  const int IPT = p.KBc * NI;  // items per column tile inside a k chunk
  // x / IPT and x % IPT: a shift when IPT is a power of two (the host says so), which keeps integer
  // divisions out of the start of every warp
  const int ipt_shift = p.ipt_shift;
  auto div_ipt = [&](int x, int& rem) -> int {
    if (ipt_shift >= 0) { rem = x & (IPT - 1); return x >> ipt_shift; }
    const int qd = x / IPT;
    rem = x - qd * IPT;
    return qd;
  };
  // The CTA owns T_own whole column tiles; the NT - CPC * T_own tiles left over are cut into
  // equal item runs, one per CTA.  A CTA works through its left-over run first.
  const int own_tile0 = ci * p.T_own;
  const int left_tile0 = p.CPC * p.T_own;
  int l0 = 0, l1 = 0;
  if (left_tile0 < p.NT) {  // 32-bit division where the products fit (64-bit division costs ~100 instructions)
    const long long left_items = (long long)(p.NT - left_tile0) * IPT;
    if (left_items <= 0x7fffffffLL / p.CPC) {
      l0 = (int)((unsigned)left_items * (unsigned)ci / (unsigned)p.CPC);
      l1 = (int)((unsigned)left_items * (unsigned)(ci + 1) / (unsigned)p.CPC);
    } else {
      l0 = (int)(left_items * ci / p.CPC);
      l1 = (int)(left_items * (ci + 1) / p.CPC);
    }
  }
  const int n_left = l1 - l0, n_total = n_left + p.T_own * IPT;
  // n_total < 2^26 (column tiles x k blocks x 4 of one CTA), NWARPS <= 32: the products fit in 32 bits
  const int v0 = (int)((unsigned)n_total * (unsigned)warp / NWARPS), v1 = (int)((unsigned)n_total * (unsigned)(warp + 1) / NWARPS);
  // this warp's two item runs: cA items of left-over tiles, then cB items of the CTA's own tiles
  const int cA = v0 < n_left ? min(v1, n_left) - v0 : 0;
  int qA = 0, qB = 0;
  const int tileA = cA > 0 ? left_tile0 + div_ipt(l0 + v0, qA) : 0;
  const int oB = max(v0, n_left) - n_left;
  const int cB = max(v1 - max(v0, n_left), 0);
  const int tileB = own_tile0 + div_ipt(oB, qB);
  const int n_items = cA + cB;
  // The next kernel of the stream may become resident as soon as there is room for it - once every
  // CTA of this launch has said so.  p.trig == 1: CTA 0 says so only after its own wait for the
  // previous kernel, which keeps the next kernel's CTAs off the SMs until the previous one has gone.
  // Launches that fetch their activations from the host (GATHER == 3) say so after staging them: their
  // successor may then overwrite the staging buffer at once.
  const bool late_trigger = p.trig == 1 && blockIdx.x == 0;
  if (GATHER != 3 && !late_trigger) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const uint32_t bar0 = smem_base + warp * 64;
  const uint32_t ring_s = smem_base + HDR + warp * NST * SLOT_BYTES;

  // ---- producer: lane 0 requests the items of the warp, in order, into the warp's ring ----
  int pc_q, issued = 0;
  const unsigned char* pc_src;
  const size_t tile_skip = (size_t)(p.KB - p.KBc) * (1024 * B);  // from the end of a chunk to the next tile's
  auto cursor_set = [&](int tile, int q) {
    pc_q = q;
    pc_src = reinterpret_cast<const unsigned char*>(p.bq) + ((size_t)tile * p.KB + kb_base) * (size_t)(1024 * B) +
             (size_t)q * ITEM_BYTES;
  };
  if (cA > 0) cursor_set(tileA, qA); else cursor_set(tileB, qB);
  auto issue_next = [&](uint32_t bar, uint32_t dst) {  // lane 0
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(ITEM_BYTES) : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(pc_src), "r"(ITEM_BYTES), "r"(bar)
        : "memory");
    if (++issued == cA) {
      cursor_set(tileB, qB);
    } else {
      pc_src += ITEM_BYTES;
      if (++pc_q == IPT) { pc_q = 0; pc_src += tile_skip; }
    }
  };
  // ---- scale cache: entry i % SCG holds the 16 scales of the warp's i-th group; a lane fetches
  // half a row (16 bytes) of one of 16 consecutive groups.  Scales are constants: the first
  // fill runs ahead of the wait on the previous kernel. ----
  unsigned char* sc_warp = sScale + (size_t)warp * SCG * 32;
  auto scale_src = [&](int gidx) -> const uint4* {
    const int itx = gidx / GI, gi = gidx - itx * GI;
    int tile, q;
    if (itx < cA) {
      tile = left_tile0 + div_ipt(l0 + v0 + itx, q);
    } else {
      tile = own_tile0 + div_ipt(oB + itx - cA, q);
    }
    const int gidx128 = kb_base * 4 + q * GI + gi;  // 128-row group of K
    const int row = p.gshift >= 0 ? (gidx128 >> p.gshift) : gidx128 / p.gdiv;
    return reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.scales) + (size_t)row * p.N + tile * 16) + (lane & 1);
  };
  auto fill_scales = [&](int first) {
    const int gidx = first + (lane >> 1);
    if (gidx < n_items * GI)
      *reinterpret_cast<uint4*>(sc_warp + (gidx % SCG) * 32 + (lane & 1) * 16) = __ldg(scale_src(gidx));
  };
  if (lane == 0) {
    for (int s = 0; s < NST; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + s * 8) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  if (lane == 0)
    for (int s = 0; s < NST && issued < n_items; ++s) issue_next(bar0 + s * 8, ring_s + s * SLOT_BYTES);
  // the first fill of the scale cache: requested now, stored after the activations have been
  // requested as well (a CTA that starts after its predecessor has finished then waits for the
  // two round trips at the same time, not one after the other)
  uint4 sc_first = make_uint4(0u, 0u, 0u, 0u);
  const bool sc_first_valid = (lane >> 1) < n_items * GI;
  if (sc_first_valid) sc_first = __ldg(scale_src(lane >> 1));
  for (int idx = tid; idx < p.T_own * 16 * MP; idx += NWARPS * 32) sAcc[idx] = 0.f;
  // Activations in host memory (GATHER == 3): the first CTAs bring them over PCIe now, under the
  // previous kernel of the stream, and hold them in registers until that kernel has finished with the
  // staging buffer.
  constexpr int FETCH_PIECES = 4;
  uint4 fetched[GATHER == 3 ? FETCH_PIECES : 1];
  if (GATHER == 3 && (int)blockIdx.x < p.fetch_ctas) {
    const int vec_per_row = p.K / 8, total = p.M * vec_per_row;
#pragma unroll
    for (int u = 0; u < FETCH_PIECES; ++u) {
      const int idx = ((int)blockIdx.x * FETCH_PIECES + u) * NWARPS * 32 + tid;
      if (idx < total) {
        const int m = idx / vec_per_row, c = idx - m * vec_per_row;
        fetched[GATHER == 3 ? u : 0] =
            __ldcv(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.a_host) + (size_t)m * p.lda + (size_t)c * 8));
      }
    }
  }
  // everything below may read what the previous kernel of the stream wrote (a launch with host
  // activations, one K chunk and only own tiles reads nothing of it: it waits before its output instead)
  const bool nowait = GATHER == 3 && p.nowait;
  if (!nowait) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (late_trigger) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- fused all-gather: this launch is fused call number E + 1 of the rank (E is kept on the
  // device, so that the same launch can be replayed from a CUDA graph).  It may start once every
  // rank has finished call E: then the activations - if they are call E's gathered output - are
  // complete and nobody still reads the row buffer this call overwrites (bounded wait on this
  // rank's flags, one thread per source rank). ----
  const unsigned short* a_base = reinterpret_cast<const unsigned short*>(p.a);
  size_t gather_buf = 0;  // element offset of the row buffer this call writes, inside every rank's region
  unsigned epoch = 0;
  const unsigned long long* a_tagged = nullptr;  // tagged mode: the activations as {two values, tag} words
  if constexpr (GATHER == 2) {
    // Tagged words: the call number was stored by the last CTA of this rank's previous fused launch,
    // which has completed (stream order).  Nothing to wait for here: the staging loop polls the words
    // it reads, and the buffer written below was last read two calls ago (see GatherArgs).
    epoch = *reinterpret_cast<volatile const unsigned*>(p.ga.epoch);
    gather_buf = (size_t)((epoch + 1) % GATHER_TAG_BUFFERS) * (size_t)p.ga.buf_elems;
    if (p.ga.a_prev_off >= 0)
      a_tagged = reinterpret_cast<const unsigned long long*>(p.ga.out[p.ga.rank]) +
                 (size_t)(epoch % GATHER_TAG_BUFFERS) * (size_t)p.ga.buf_elems + (size_t)(p.ga.a_prev_off >> 1);
  } else if constexpr (GATHER == 1) {
    // The rank's own flag slot holds the number of its completed fused calls (its last CTA raises it
    // with the others), so one round of loads brings both the epoch and the peers' progress.
    __shared__ unsigned s_epoch_word;
    unsigned* s_epoch = &s_epoch_word;
    unsigned mine = 0;
    if (tid < p.ga.G) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(mine) : "l"(p.ga.flags + tid) : "memory");
      if (tid == p.ga.rank) *s_epoch = mine;
    }
    __syncthreads();
    epoch = *s_epoch;
    gather_buf = ((epoch + 1) & 1u) ? p.ga.buf_elems : 0;
    if (p.ga.a_prev_off >= 0)
      a_base = reinterpret_cast<const unsigned short*>(p.ga.out[p.ga.rank]) + ((epoch & 1u) ? p.ga.buf_elems : 0) + p.ga.a_prev_off;
    if (epoch != 0) {
      if (tid < p.ga.G && (int)(mine - epoch) < 0) {  // a peer has not finished call `epoch` yet: bounded wait
        uint64_t t0 = 0;
        for (int spin = 0;; ++spin) {
          unsigned v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.ga.flags + tid) : "memory");
          if ((int)(v - epoch) >= 0) break;
          uint64_t now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (spin == 0) t0 = now;
          else if (now - t0 > 250000000ull) {  // give up: report, carry on with what is there
            atomicExch(p.status, ST_DEVICE_TIMEOUT);
            p.status[1] = 5;  // where: wait for a peer's columns
            p.status[2] = blockIdx.x;
            p.status[3] = tid;
            break;
          }
        }
      }
      __syncthreads();
    }
  }
  const unsigned out_tag = epoch + 1;  // tagged mode: what this call's output words carry
  int a_ld = p.lda;  // row stride of what the staging loop reads
  if constexpr (GATHER == 3) {
    // fetching CTAs: registers -> dense device rows, then count in; everybody: wait for the count (bounded)
    const int vec_per_row = p.K / 8, total = p.M * vec_per_row;
    if ((int)blockIdx.x < p.fetch_ctas) {
#pragma unroll
      for (int u = 0; u < FETCH_PIECES; ++u) {
        const int idx = ((int)blockIdx.x * FETCH_PIECES + u) * NWARPS * 32 + tid;
        if (idx < total)
          __stcg(reinterpret_cast<uint4*>(const_cast<unsigned short*>(a_base) + (size_t)idx * 8), fetched[u]);
      }
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.fetch_flag) : "memory");
      }
    }
    if (tid == 0) {
      uint64_t t0 = 0;
      for (int spin = 0;; ++spin) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.fetch_flag) : "memory");
        if (v >= (unsigned)p.fetch_ctas) break;
        uint64_t now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (spin == 0) t0 = now;
        else if (now - t0 > 250000000ull) {  // give up: report, carry on with what is there
          atomicExch(p.status, ST_DEVICE_TIMEOUT);
          p.status[1] = 9;  // where: wait for the CTAs that fetch the activations
          p.status[2] = blockIdx.x;
          break;
        }
      }
      // the last CTA to get here puts the two words back to zero for the next launch
      if (atomicAdd(p.fetch_flag + 1, 1u) == gridDim.x - 1) {
        atomicExch(p.fetch_flag, 0u);
        atomicExch(p.fetch_flag + 1, 0u);
      }
    }
    __syncthreads();
    a_ld = p.K;
  }

  // ---- stage the activation chunk A[0:M, kb_base*512 : +KBc*512] as fp16 (pre-scaled where the
  // weight type needs it), and the zero-point term of every 128-row group ----
  {
    const int kc = p.KBc * 512;
    const int vec_per_row = kc / 8;  // multiple of 64
    const int total = p.M * vec_per_row;
    if constexpr (BIAS != 0) {  // rows that do not exist contribute exact zeros
      for (int idx = tid; idx < p.KBc * 4 * MP * 2; idx += NWARPS * 32) {
        const int m = ((idx >> 4) % MT) * 8 + ((idx >> 2) & 3) * 2 + (idx & 1);
        if (m >= p.M) sNb[idx] = 0.f;
      }
    }
    if (tid < 16) reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(sA) + (size_t)p.M * p.pitch * 2)[tid] = 0u;
    // a thread always lands on the same 8-column slot of a 32-column unit: pairs h0 .. h0+3
    const int h0 = (tid & 3) * 4;
    __half2 mult[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = lin_prescale_shift(VAR, h0 + q);
      mult[q] = h2_from_bits(dup16((uint32_t)(15 - e) << 10));  // 2^-e
    }
    // four loads in flight per thread: the staging pass costs one memory round trip per four
    // 16-byte pieces instead of one per piece
    constexpr int SB = 4;
    bool tag_wait = true;  // tagged mode: cleared once a wait has run out
    int m = 0, vv = tid;  // idx = m * vec_per_row + vv
    for (int idx0 = tid; idx0 < total; idx0 += SB * NWARPS * 32) {
      uint4 vq[SB];
      int mq[SB], kq[SB];
      ulonglong2 tlo[GATHER == 2 ? SB : 1], thi[GATHER == 2 ? SB : 1];  // tagged mode: the words as loaded
#pragma unroll
      for (int u = 0; u < SB; ++u) {
        const int idx = idx0 + u * NWARPS * 32;
        while (vv >= vec_per_row) { vv -= vec_per_row; ++m; }
        mq[u] = m; kq[u] = vv * 8;
        vv += NWARPS * 32;
        if (idx < total) {
          if (GATHER == 2 && a_tagged != nullptr) {
            // eight activations = four tagged words, checked once all loads of the batch are in flight
            const unsigned long long* src = a_tagged + (((size_t)mq[u] * p.lda + (size_t)kb_base * 512 + kq[u]) >> 1);
            tlo[GATHER == 2 ? u : 0] = ld_tagged2(src);
            thi[GATHER == 2 ? u : 0] = ld_tagged2(src + 2);
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(a_base + (size_t)mq[u] * a_ld + (size_t)kb_base * 512 + kq[u]);
            vq[u] = GATHER ? __ldcg(src) : __ldg(src);  // gathered rows were written through L2 by other GPUs
          }
        }
      }
      if (GATHER == 2 && a_tagged != nullptr) {
        // every word must carry the previous call's number; a word that does not yet is read again (bounded)
#pragma unroll
        for (int u = 0; u < SB; ++u) {
          if (idx0 + u * NWARPS * 32 >= total) continue;
          ulonglong2 lo = tlo[GATHER == 2 ? u : 0], hi = thi[GATHER == 2 ? u : 0];
          const unsigned long long* src = a_tagged + (((size_t)mq[u] * p.lda + (size_t)kb_base * 512 + kq[u]) >> 1);
          uint64_t t0 = 0;
          for (int spin = 0; tag_wait && ((unsigned)(lo.x >> 32) != epoch || (unsigned)(lo.y >> 32) != epoch ||
                                          (unsigned)(hi.x >> 32) != epoch || (unsigned)(hi.y >> 32) != epoch); ++spin) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (spin == 0) t0 = now;
            else if (now - t0 > 250000000ull) {  // give up for good: report, carry on with what is there
              atomicExch(p.status, ST_DEVICE_TIMEOUT);
              p.status[1] = 5;  // where: wait for a peer's columns
              p.status[2] = blockIdx.x;
              p.status[3] = tid;
              tag_wait = false;
              break;
            }
            lo = ld_tagged2(src); hi = ld_tagged2(src + 2);
          }
          vq[u] = make_uint4((uint32_t)lo.x, (uint32_t)lo.y, (uint32_t)hi.x, (uint32_t)hi.y);
        }
      }
#pragma unroll
      for (int u = 0; u < SB; ++u) {
        const int idx = idx0 + u * NWARPS * 32;
        if (idx >= total) continue;  // uniform over each half-warp: 16 consecutive pieces lie in one row
        uint4 v = vq[u];
        const int mm = mq[u], kk = kq[u];
        if constexpr (ACT == 1) {
          v.x = bf16x2_to_f16x2(v.x); v.y = bf16x2_to_f16x2(v.y);
          v.z = bf16x2_to_f16x2(v.z); v.w = bf16x2_to_f16x2(v.w);
        }
        __half2 x0 = h2_from_bits(v.x), x1 = h2_from_bits(v.y), x2 = h2_from_bits(v.z), x3 = h2_from_bits(v.w);
        if constexpr (BIAS != 0) {
          const float2 f0 = __half22float2(x0), f1 = __half22float2(x1), f2 = __half22float2(x2),
                       f3 = __half22float2(x3);
          float sum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
          const unsigned hm = 0xffffu << (lane & 16);  // the 16 lanes that share this 128-column group
          sum += __shfl_xor_sync(hm, sum, 1);
          sum += __shfl_xor_sync(hm, sum, 2);
          sum += __shfl_xor_sync(hm, sum, 4);
          sum += __shfl_xor_sync(hm, sum, 8);
          if ((lane & 15) == 0) {
            const float nbv = -(float)BIAS * sum * (1.0f / F);
            float* q4 = sNb + (((kk >> 7) * MT + (mm >> 3)) * 4 + ((mm & 7) >> 1)) * 4 + (mm & 1);
            q4[0] = nbv;
            q4[2] = nbv;
          }
        }
        if constexpr (PRESCALE) {
          x0 = __hmul2(x0, mult[0]); x1 = __hmul2(x1, mult[1]);
          x2 = __hmul2(x2, mult[2]); x3 = __hmul2(x3, mult[3]);
        }
        v.x = bits_from_h2(x0); v.y = bits_from_h2(x1); v.z = bits_from_h2(x2); v.w = bits_from_h2(x3);
        *reinterpret_cast<uint4*>(sA + (size_t)mm * p.pitch + kk + (kk >> 5) * 8) = v;
      }
    }
  }
  if (sc_first_valid) *reinterpret_cast<uint4*>(sc_warp + ((lane >> 1) % SCG) * 32 + (lane & 1) * 16) = sc_first;
  __syncthreads();  // activations staged, tile sums cleared, first scales cached
  if (GATHER == 3) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int items_per_tile_total = p.KB * NI;
  bool ok = true;
  if (n_items > 0) {
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[mt][q] = 0.f;

    // Activation fragments: lane (r, j) reads row mt*8 + r, columns j*32 .. of each group (32
    // columns + 8 of padding per unit, 4 units per group).  Lanes whose row does not exist
    // read the 64 zero bytes behind the chunk instead (kmask clears their group offset).
    const unsigned char* a_ptr[MT];
    uint32_t kmask[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int m = mt * 8 + r;
      const bool valid = m < p.M;
      a_ptr[mt] = reinterpret_cast<const unsigned char*>(sA) +
                  (valid ? 2u * (uint32_t)(m * p.pitch + j * 40) : 2u * (uint32_t)(p.M * p.pitch));
      kmask[mt] = valid ? 0xffffffffu : 0u;
    }
    const float4* nb4 = reinterpret_cast<const float4*>(sNb) + j;
    const unsigned char* ring_g = smem_raw + (ring_s - smem_base);  // this warp's ring, generic pointer
    const uint32_t w_lane = (uint32_t)(lane * B * 4);

    int seg = cA > 0 ? 0 : 1;          // 0: left-over tiles (shared with other CTAs), 1: own tiles
    int seg_left = cA > 0 ? cA : cB;
    int cur_tile = cA > 0 ? tileA : tileB;
    int q = cA > 0 ? qA : qB;  // item index inside the tile chunk: k block q / NI, groups (q % NI) * GI ...
    uint32_t slot_off = 0, bar = bar0;
    uint32_t parity = 0;
    int it = 0;
    while (it < n_items && ok) {
      const int run = min(IPT - q, seg_left);  // items of this column tile
      for (int e = 0; e < run; ++e, ++it, ++q) {
        const int g0 = q * GI;  // first 128-row group of the item, counted inside the chunk
        if (!__all_sync(0xffffffffu, mbar_test(bar, parity) ? 1 : 0)) {  // not there yet: bounded wait
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar, parity) ? 1 : 0)) { ok = false; break; }
        }
        const unsigned char* slot = ring_g + slot_off;
        if (it != 0 && (it * GI) % SCG == 0) {  // the cache has been used up: next SCG groups
          __syncwarp();
          fill_scales(it * GI);
          __syncwarp();
        }
        // this item's scales: columns r and r+8 of each group
        float sf0[GI], sf1[GI];
#pragma unroll
        for (int gi = 0; gi < GI; ++gi) {
          const unsigned short* sp = reinterpret_cast<const unsigned short*>(sc_warp + ((it * GI + gi) % SCG) * 32) + r;
          sf0[gi] = scale_f32<ACT>(sp[0]);
          sf1[gi] = scale_f32<ACT>(sp[8]);
        }
#pragma unroll
        for (int gi = 0; gi < GI; ++gi) {
          uint32_t w0[B], w1[B];
          ld_unit_words<B>(slot + w_lane + gi * (256 * B), w0);
          ld_unit_words<B>(slot + w_lane + gi * (256 * B) + 128 * B, w1);
          uint32_t W0[16], W1[16];
          unit_decode_linear<VAR>(w0, W0);
          unit_decode_linear<VAR>(w1, W1);
          if (gi == GI - 1) {
            // every lane has turned its copy of the item's last group into operands (the loads have
            // returned: their values were used), so lane 0 may ask for the next item into this slot
            __syncwarp();
            if (lane == 0 && issued < n_items) issue_next(bar, ring_s + slot_off);
          }
          const uint32_t koff = (uint32_t)((g0 + gi) * 320);  // bytes: 128 columns + 4 x 8 of padding per group
          // two accumulation chains per 8-row tile; the first starts from the zero-point term of the group
          float d[MT][2][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            float4 nb = make_float4(0.f, 0.f, 0.f, 0.f);
            if constexpr (BIAS != 0) nb = nb4[((g0 + gi) * MT + mt) * 4];
            d[mt][0][0] = nb.x; d[mt][0][1] = nb.y; d[mt][0][2] = nb.z; d[mt][0][3] = nb.w;
          }
          // pairs h = 4*sp .. 4*sp+3 of both units against the same four pairs of activations
#pragma unroll
          for (int sp = 0; sp < 4; ++sp) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4 av = *reinterpret_cast<const uint4*>(a_ptr[mt] + (koff & kmask[mt]) + sp * 16);
              mma_m16n8k16(d[mt][0], W0[4 * sp], W1[4 * sp], W0[4 * sp + 1], W1[4 * sp + 1], av.x, av.y);
              if (sp == 0)
                mma_m16n8k16_init(d[mt][1], W0[2], W1[2], W0[3], W1[3], av.z, av.w);
              else
                mma_m16n8k16(d[mt][1], W0[4 * sp + 2], W1[4 * sp + 2], W0[4 * sp + 3], W1[4 * sp + 3], av.z, av.w);
            }
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            acc[mt][0] = fmaf(sf0[gi], d[mt][0][0] + d[mt][1][0], acc[mt][0]);
            acc[mt][1] = fmaf(sf0[gi], d[mt][0][1] + d[mt][1][1], acc[mt][1]);
            acc[mt][2] = fmaf(sf1[gi], d[mt][0][2] + d[mt][1][2], acc[mt][2]);
            acc[mt][3] = fmaf(sf1[gi], d[mt][0][3] + d[mt][1][3], acc[mt][3]);
          }
        }
        slot_off += SLOT_BYTES; bar += 8;
        if (slot_off == (uint32_t)NST * SLOT_BYTES) { slot_off = 0; bar = bar0; parity ^= 1u; }
      }
      if (!ok) break;
      // ---- this warp's share of column tile cur_tile is complete: hand it over ----
      // lane (r, j) holds rows 2j, 2j+1 (of each 8-row tile) of columns r and r+8
      if (seg == 1) {
        // one of the CTA's own tiles: add into its tile sums in shared memory
        float* dst = sAcc + (size_t)(cur_tile - own_tile0) * 16 * MP;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) {
            const int m = mt * 8 + 2 * j + (qq & 1);
            if (m < p.M) atomicAdd(dst + (r + (qq >> 1) * 8) * MP + m, acc[mt][qq] * F);
            acc[mt][qq] = 0.f;
          }
      } else {
        // a tile shared with other CTAs: add into the global scratch, count the items in
        float* dst = p.partial + (size_t)cur_tile * 16 * MP;  // [column][MP]
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int m0 = mt * 8 + 2 * j;
          if (m0 < p.M) {
            red_add_v2(dst + r * MP + m0, acc[mt][0] * F, acc[mt][1] * F);
            red_add_v2(dst + (r + 8) * MP + m0, acc[mt][2] * F, acc[mt][3] * F);
          }
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) acc[mt][qq] = 0.f;
        }
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          __threadfence();  // cumulative over the warp's additions (ordered by the barrier above)
          const int old = atomicAdd(p.counters + cur_tile, run);
          last = (old + run == items_per_tile_total) ? 1 : 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {  // every share has arrived: convert, write C, put the scratch back to zero
          __threadfence();
          if constexpr (!gather_pairs(GATHER)) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const int m0 = mt * 8 + 2 * j;
              if (m0 < p.M) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  float2* src = reinterpret_cast<float2*>(dst + (r + h * 8) * MP + m0);
                  const float2 v = __ldcg(src);
                  __stcg(src, make_float2(0.f, 0.f));
                  const int n = cur_tile * 16 + r + h * 8;
                  store_one<ACT>(p, m0, n, v.x);
                  if (m0 + 1 < p.M) store_one<ACT>(p, m0 + 1, n, v.y);
                }
              }
            }
          } else {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const int m0 = mt * 8 + 2 * j;
              const bool rows = m0 < p.M;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                float2* src = reinterpret_cast<float2*>(dst + (r + h * 8) * MP + m0);
                float2 v = make_float2(0.f, 0.f);
                if (rows) {
                  v = __ldcg(src);
                  __stcg(src, make_float2(0.f, 0.f));
                }
                // columns r and r ^ 1 sit four lanes apart (same rows): the even one writes row m0 of
                // both columns, the odd one row m0 + 1
                const float ox = __shfl_xor_sync(0xffffffffu, v.x, 4), oy = __shfl_xor_sync(0xffffffffu, v.y, 4);
                const int nb = cur_tile * 16 + (r & ~1) + h * 8;
                if (rows) {
                  if (!(r & 1)) store_pair<GATHER, ACT>(p, gather_buf, out_tag, m0, nb, v.x, ox);
                  else if (m0 + 1 < p.M) store_pair<GATHER, ACT>(p, gather_buf, out_tag, m0 + 1, nb, oy, v.y);
                }
              }
            }
          }
          if (lane == 0) p.counters[cur_tile] = 0;
        }
      }
      seg_left -= run;
      if (seg == 0 && seg_left == 0) {
        seg = 1; seg_left = cB; cur_tile = tileB; q = qB;
      } else {
        q = 0;
        ++cur_tile;
      }
    }
  }
  if (!ok) {
    // a bulk copy never completed: report it and give the copies still in flight a bounded
    // chance to land (the CTA must not retire under them)
    if (lane == 0) {
      atomicExch(p.status, ST_DEVICE_TIMEOUT);
      p.status[1] = 3;  // where: stream kernel weight ring
      p.status[2] = blockIdx.x;
      p.status[3] = warp;
    }
    for (int s = 0; s < NST; ++s) mbar_wait_bounded(bar0 + s * 8, 0);
  }

  // ---- the CTA's own tiles ----
  if (nowait) asm volatile("griddepcontrol.wait;" ::: "memory");  // outputs of consecutive calls land in order
  if (p.T_own > 0) {
    __syncthreads();
    const int n0 = own_tile0 * 16, ncols = p.T_own * 16;
    if (p.S == 1) {  // all of K was here: write C
      if constexpr (!gather_pairs(GATHER)) {
        for (int m = 0; m < p.M; ++m)
          for (int n = tid; n < ncols; n += NWARPS * 32) store_one<ACT>(p, m, n0 + n, sAcc[n * MP + m]);
      } else {
        for (int m = 0; m < p.M; ++m)
          for (int n = 2 * tid; n < ncols; n += 2 * NWARPS * 32)
            store_pair<GATHER, ACT>(p, gather_buf, out_tag, m, n0 + n, sAcc[n * MP + m], sAcc[(n + 1) * MP + m]);
      }
    } else {
      // other k chunks hold the rest: meet in the global scratch; the last chunk to arrive converts
      for (int idx = tid * 4; idx < ncols * MP; idx += NWARPS * 32 * 4)
        if ((idx % MP) < p.M) {  // four rows of one column at a time; rows past M hold exact zeros
          const float4 v = *reinterpret_cast<const float4*>(sAcc + idx);
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p.partial + (size_t)n0 * MP + idx),
                       "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                       : "memory");
        }
      __syncthreads();
      int* s_last = reinterpret_cast<int*>(sAcc);  // the tile sums are no longer needed
      if (tid == 0) __threadfence();  // cumulative over the CTA's additions (ordered by the barrier above)
      __syncthreads();
      for (int t = tid; t < p.T_own; t += NWARPS * 32) {
        const int old = atomicAdd(p.counters + own_tile0 + t, IPT);
        s_last[t] = (old + IPT == items_per_tile_total) ? 1 : 0;
      }
      __syncthreads();
      // four rows of one column per thread and step; one fence per thread, not per element
      bool fenced = false;
      for (int idx = tid * 4; idx < ncols * MP; idx += NWARPS * 32 * 4) {
        const int t = idx / (16 * MP);
        if (!s_last[t]) continue;
        if (!fenced) { __threadfence(); fenced = true; }
        if constexpr (!gather_pairs(GATHER)) {
          const int m = idx % MP, n = n0 + idx / MP;
          if (m < p.M) {
            float4* src = reinterpret_cast<float4*>(p.partial + (size_t)n0 * MP + idx);
            const float4 v = __ldcg(src);
            __stcg(src, make_float4(0.f, 0.f, 0.f, 0.f));
            store_one<ACT>(p, m, n, v.x);
            if (m + 1 < p.M) store_one<ACT>(p, m + 1, n, v.y);
            if (m + 2 < p.M) store_one<ACT>(p, m + 2, n, v.z);
            if (m + 3 < p.M) store_one<ACT>(p, m + 3, n, v.w);
          }
        } else {
        const int m = idx % MP, col = idx / MP;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < p.M) {
          float4* src = reinterpret_cast<float4*>(p.partial + (size_t)n0 * MP + idx);
          v = __ldcg(src);
          __stcg(src, make_float4(0.f, 0.f, 0.f, 0.f));
        }
        // the same four rows of column col ^ 1 are held MP / 4 threads away (a warp lies inside one tile
        // and takes this branch as a whole): the even column's thread writes rows m and m + 2 of both
        // columns, the odd one's rows m + 1 and m + 3
        float4 o;
        o.x = __shfl_xor_sync(0xffffffffu, v.x, MP / 4); o.y = __shfl_xor_sync(0xffffffffu, v.y, MP / 4);
        o.z = __shfl_xor_sync(0xffffffffu, v.z, MP / 4); o.w = __shfl_xor_sync(0xffffffffu, v.w, MP / 4);
        if (m < p.M) {
          const int nb = n0 + (col & ~1);
          if (!(col & 1)) {
            store_pair<GATHER, ACT>(p, gather_buf, out_tag, m, nb, v.x, o.x);
            if (m + 2 < p.M) store_pair<GATHER, ACT>(p, gather_buf, out_tag, m + 2, nb, v.z, o.z);
          } else {
            if (m + 1 < p.M) store_pair<GATHER, ACT>(p, gather_buf, out_tag, m + 1, nb, o.y, v.y);
            if (m + 3 < p.M) store_pair<GATHER, ACT>(p, gather_buf, out_tag, m + 3, nb, o.w, v.w);
          }
        }
        }
        if ((idx % (16 * MP)) == 0) p.counters[own_tile0 + t] = 0;
      }
    }
  }

  // ---- fused all-gather: the last CTA of the launch tells every rank that this rank's columns
  // of the output row are in place.  Every CTA orders its stores before its arrival at GPU scope;
  // the last arriver, which has observed all arrivals, releases at system scope: by cumulativity
  // every CTA's stores are visible to whoever acquires the flag. ----
  if (GATHER == 1 || GATHER == 2) {
    __syncthreads();
    if (tid == 0 && GATHER == 2) {
      // tagged words need no release: every word announces itself.  The last CTA only moves the call
      // counter on for this rank's next launch, which starts after this one has completed.
      unsigned* done = p.ga.epoch + 8;  // arrival counter in the rank's region
      if (atomicAdd(done, 1u) == gridDim.x - 1) {
        atomicExch(done, 0u);
        *p.ga.epoch = epoch + 1;
      }
    } else if (tid == 0) {
      // release at GPU scope what this CTA's threads stored (ordered before by the barrier), acquire
      // what the CTAs that arrived earlier released
      unsigned arrived;
      asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(p.ga.done) : "memory");
      if (arrived == gridDim.x - 1) {
        atomicExch(p.ga.done, 0u);
        asm volatile("fence.acq_rel.sys;" ::: "memory");  // one system-scope fence, then plain flag stores
        for (int g = 0; g < p.ga.G; ++g)
          asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.ga.flag_slot[g]), "r"(epoch + 1) : "memory");
        *p.ga.epoch = epoch + 1;  // for the host (PeerGather.calls_completed)
      }
    }
  }
}

template <int VAR, int MT, int GATHER, int ACT>
static cudaError_t launch_one(const StreamParams& p, int smem_bytes, cudaStream_t stream) {
  auto kern = stream_kernel<VAR, MT, GATHER, ACT>;
  static int configured_smem[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem_bytes > 48 * 1024 && (dev < 0 || dev >= 16 || configured_smem[dev] < smem_bytes)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 16) configured_smem[dev] = smem_bytes;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.S * p.CPC), 1, 1);
  cfg.blockDim = dim3(stream_warps(MT) * 32, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  // programmatic dependent launch: this kernel may become resident while the previous kernel
  // of the stream still runs; it waits (griddepcontrol.wait) before it reads anything but
  // the weights and scales
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = p.pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int VAR, int MT, int GATHER>
static cudaError_t launch_act(const StreamParams& p, int smem_bytes, cudaStream_t stream) {
  return p.act == 0 ? launch_one<VAR, MT, GATHER, 0>(p, smem_bytes, stream)
                    : launch_one<VAR, MT, GATHER, 1>(p, smem_bytes, stream);
}

template <int VAR>
static cudaError_t launch_var(int var, const StreamParams& p, int mt, int smem_bytes, cudaStream_t stream) {
  if constexpr (VAR % B200Q_NPARTS == B200Q_PART) {
    if (var == VAR) {
      if (p.a_host != nullptr)
        return mt == 1 ? launch_act<VAR, 1, 3>(p, smem_bytes, stream) : launch_act<VAR, 2, 3>(p, smem_bytes, stream);
      if (p.ga.G > 0 && p.ga.mode == 1)
        return mt == 1 ? launch_act<VAR, 1, 2>(p, smem_bytes, stream) : launch_act<VAR, 2, 2>(p, smem_bytes, stream);
      if (p.ga.G > 0)
        return mt == 1 ? launch_act<VAR, 1, 1>(p, smem_bytes, stream) : launch_act<VAR, 2, 1>(p, smem_bytes, stream);
      return mt == 1 ? launch_act<VAR, 1, 0>(p, smem_bytes, stream) : launch_act<VAR, 2, 0>(p, smem_bytes, stream);
    }
  }
  if constexpr (VAR + 1 < VAR_COUNT) return launch_var<VAR + 1>(var, p, mt, smem_bytes, stream);
  else return cudaErrorInvalidValue;
}

#define B200Q_CAT2(a, b) a##b
#define B200Q_CAT(a, b) B200Q_CAT2(a, b)

// One of these per compiled part; api.cu picks the part as var % B200Q_NPARTS.
cudaError_t B200Q_CAT(stream_launch_part, B200Q_PART)(int var, const StreamParams& p, int mt, int smem_bytes,
                                                       cudaStream_t stream) {
  return launch_var<0>(var, p, mt, smem_bytes, stream);
}

}  // namespace b200q
