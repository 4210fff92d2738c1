/* b200q - B200 (sm_100a) weight-only quantized matmul, C ABI.
 *
 *   C[M, N] (fp16) = A[M, K] (fp16) x dequant(Bq[K, N]),   W[k, n] = fp16_rn(value(q[k, n]) * s[k / group, n])
 *
 * This library replaces, for that one operator, the launch entry the reference JIT
 * generates per kernel: `tilus_launch(int32 m_size, void_p a_ptr, void_p b_ptr,
 * void_p scale_ptr, void_p c_ptr)` exported through tvm_ffi as "launch"
 * (python/tilus/hidet/backend/codegen.py:650-660, :1021-1025 of the reference; called from
 * python/tilus/lang/instantiated_script.py:824-858 and, for this operator, from
 * examples/quantization/matmul_a16wx.py:535-548).  N, K, the weight dtype and the group
 * size, which the reference bakes into each generated kernel, are explicit arguments
 * here.  All pointers are device pointers; `stream` is a cudaStream_t passed as void*
 * (NULL = the default stream) and replaces the reference's implicit environment stream
 * (python/tilus/hidet/include/tilus/stream.h:12-16).  Nothing here allocates device memory except
 * where a function says so; the caller owns every buffer, including the workspace that
 * replaces the reference's process-global zero-restored pool
 * (python/tilus/hidet/include/tilus/context.h:30-42, :97-131).
 *
 * Every function returns a status code (0 = ok); no exception crosses this boundary.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200Q_OK = 0,
  B200Q_ERR_INVALID_ARG = 1,    /* null / misaligned pointer, non-positive size */
  B200Q_ERR_UNSUPPORTED = 2,    /* dtype, zero point, shape or group size not covered */
  B200Q_ERR_WORKSPACE = 3,      /* workspace missing or smaller than b200q_workspace_bytes */
  B200Q_ERR_CUDA = 4,           /* a CUDA runtime call failed; see b200q_last_cuda_error */
  B200Q_ERR_DEVICE_TIMEOUT = 5  /* a bounded device-side wait gave up; see b200q_device_status */
};

/* Weight dtype tag: kind << 16 | nbits << 8 | exponent_bits << 4 | mantissa_bits,
 * kind 0 = unsigned integer, 1 = two's-complement integer, 2 = float (sign/exponent/mantissa,
 * bias 2^(e-1)-1, all exponent codes finite when e < 5).  These are the reference's
 * uintNb / intNb / floatN_eXmY types (python/tilus/hidet/ir/dtypes/integer_subbyte.py:66-98,
 * floats_subbyte.py:89-109). */
#define B200Q_WTYPE(kind, nbits, e, m) (((kind) << 16) | ((nbits) << 8) | ((e) << 4) | (m))

/* Activation dtype tags: the type of A, of the scales and of C, as the reference's a_dtype
 * (float16 or bfloat16, examples/quantization/matmul_a16wx.py:35-41, :418-419). */
enum { B200Q_F16 = 0, B200Q_BF16 = 1 };

/* Kernel selection made by the static shape table (replaces the reference's autotuner,
 * python/tilus/lang/instantiated_script.py:700-801).  Filled by b200q_plan; may be edited
 * and passed to b200q_gemm_planned for experiments. */
typedef struct b200q_plan {
  int32_t kernel;        /* 2 = mma.sync stream kernel (M <= 16), 3 = tcgen05 kernel with the weights on the
                            256-column side (M <= 128), 1 = tcgen05 kernel for larger M */
  int32_t m_tiles;       /* kernel 2: 8-row activation tiles per pass (1 or 2); kernels 1, 3: tiles along M */
  int32_t splits;        /* k chunks (kernel 2) / split-K factor (kernels 1, 3) */
  int32_t cluster;       /* 1 (no kernel launches clusters) */
  int32_t ctas_per_split;/* kernel 2: CTAs per k chunk, grid = splits * ctas_per_split; kernels 1, 3: output tiles */
  int32_t smem_bytes;    /* dynamic shared memory per CTA */
  int32_t tile_m;        /* kernel 1: activation rows per CTA tile (32, 64, 128 or 256); kernel 3: 128 */
  int32_t stages;        /* pipeline depth (kernel 2: ring slots per warp; kernel 1: activation stages;
                            kernel 3: 128-row weight groups in the packed ring) */
  int32_t warps;         /* warps per CTA (output only) */
  int32_t passes;        /* launches: 2 when kernel 1 takes the full 256-row tiles and kernel 2 a last tile of <= 16 rows */
  int32_t pdl;           /* 1: launch with programmatic stream serialization (overlap with the previous kernel);
                            kernel 3 always is, kernel 1 never */
  int32_t reserved;      /* 0 */
  uint64_t workspace_bytes;
} b200q_plan_t;

/* Library / weight-layout versions.  The layout version tags the private interleaved
 * weight format produced by the host re-packer (tilus_b200/packing.py). */
int b200q_version(void);
int b200q_layout_version(void);
const char* b200q_status_string(int status);
/* Last CUDA runtime error code seen by this thread inside the library (cudaError_t). */
int b200q_last_cuda_error(void);

/* Static shape -> tile table for the current device.  Replaces the reference's per-shape
 * autotuning and dispatch table (python/tilus/lang/instantiated_script.py:327-358, :700-801). */
int b200q_plan(int M, int N, int K, int wtype, int zero_point, int group, b200q_plan_t* plan);

/* Bytes of workspace b200q_gemm needs for this problem.  The workspace must be zeroed
 * once by the caller; every call leaves it zeroed again (as the reference's
 * `requires_clean` global tensors do, python/tilus/lang/instantiated_script.py +
 * python/tilus/hidet/include/tilus/context.h:97-117).  One workspace per stream. */
size_t b200q_workspace_bytes(int M, int N, int K, int wtype, int zero_point, int group);

/* C = A x dequant(Bq).  a: [M, K] (row stride lda elements), bq: b200-packed weights,
 * scales: [K/group, N], c: [M, N] (row stride ldc), all three of dtype act_dtype.  Replaces
 * tilus_launch for QuantizedMatmul (examples/quantization/matmul_a16wx.py:231-405).  With bf16
 * and M <= 16 the activations are converted to fp16 for the tensor core: exactly, except that
 * magnitudes above 65504 saturate there and magnitudes below 2^-24 become zero. */
int b200q_gemm(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
               int wtype, int zero_point, int group, int act_dtype, void* workspace, size_t workspace_bytes,
               void* stream);

/* The same GEMM for a host that keeps activations and results in host memory (no counterpart in
 * the reference, whose operator takes device tensors): brings A[M, K] from `a_host` (row stride
 * lda) into `a_staging` (device, M*K 16-bit elements, 16-byte aligned) and runs b200q_gemm.  A result
 * of at most 1 MiB whose `c_host` (row stride ldc) is pinned memory the GPU can address is written
 * there by the kernel itself; otherwise the GEMM writes `c_staging` (device, M*N elements) and a
 * copy to `c_host` follows.  All of it is queued on `stream` by this one call; the caller
 * synchronises before it reads c_host.
 *
 * How A travels depends on where it lies.  Pageable memory, or more than 256 KB: a copy operation
 * on the stream.  Pinned memory the GPU can address: a small kernel whose PCIe reads run under the
 * previous kernel of the stream.  Pinned memory and a decode batch (M <= 16 on the stream kernel, result
 * written straight to pinned c_host): no separate operation at all - the first CTAs of the GEMV kernel
 * fetch the rows, the others wait for them (bounded, status[1] = 9), and consecutive such calls overlap on
 * the GPU: a call does not wait for the kernel before it until it writes its outputs, which therefore
 * still land in call order (a call only starts early when the previous b200q_gemm_host call of this
 * thread with the same `stream` and `a_staging` was such a call too).  `a_staging` must belong to the
 * b200q_gemm_host calls of one thread and stream, `workspace` to this stream's calls of this library. */
int b200q_gemm_host(const void* a_host, int lda, const void* bq, const void* scales, void* c_host, int ldc, int M,
                    int N, int K, int wtype, int zero_point, int group, int act_dtype, void* a_staging,
                    void* c_staging, void* workspace, size_t workspace_bytes, void* stream);

/* Same as b200q_gemm, with the kernel selection supplied by the caller. */
int b200q_gemm_planned(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N,
                       int K, int wtype, int zero_point, int group, int act_dtype, void* workspace,
                       size_t workspace_bytes, void* stream, const b200q_plan_t* plan);

/* C = A x dequant(Bq) for callers that cannot hand over a workspace because they must not
 * allocate device memory: a plugin inside a serving runtime that owns the whole GPU heap, a
 * step that runs after the framework has frozen its memory plan, code on a path where
 * cudaMalloc's implicit synchronisation is not acceptable.  (No counterpart in the
 * reference, whose launcher always draws from its own growing pool,
 * python/tilus/hidet/include/tilus/context.h:97-131.)
 *
 * Same arguments and results as b200q_gemm without `workspace`: the split-K scratch is a
 * fixed array inside the library, b200q_static_workspace_limit() bytes (8 MiB) per GPU.  Problems
 * whose b200q_workspace_bytes exceeds that limit return B200Q_ERR_WORKSPACE and launch nothing.
 * The function allocates nothing and frees nothing.  The array belongs to the library's device
 * code: the CUDA runtime reserves its 8 MiB on a GPU when it loads that code there, which with
 * lazy module loading (the default) is the first call of b200q_static_ws_init or of this
 * function on that GPU.  Call b200q_static_ws_init once per GPU at set-up time, outside any stream
 * capture and before the memory plan is frozen; it looks the array's address up (the first call of
 * this function does the same if it was skipped).  All calls on a device share the one array:
 * calls that may overlap on the GPU (different streams) race on it and must be serialised by the
 * caller; back-to-back calls on one stream are fine, each leaves the scratch zeroed.  A bounded
 * device-side wait that gave up is reported by b200q_device_status(NULL, ...), which also puts
 * the array back to zero. */
int b200q_gemm_static_ws(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N,
                         int K, int wtype, int zero_point, int group, int act_dtype, void* stream);
int b200q_static_ws_init(void);
size_t b200q_static_workspace_limit(void);

/* ---- column-sharded GEMV with the all-gather fused into the kernel -------------------------------
 * The reference is single-GPU (no collective anywhere in its tree), so these have no counterpart
 * there; they serve the N-sharded decode stack: rank r holds columns [col_offset, col_offset + N)
 * of a layer and every rank needs the full output row as the next layer's activations.
 *
 * b200q_gemm_gather computes this rank's columns like b200q_gemm (M <= 16; workspace of
 * b200q_workspace_bytes for the same problem) and stores them straight
 * into the full output row [M, ldc] of every rank (peer-mapped device pointers; stores only, no
 * loads from peers), then raises this rank's flag on every rank.  Every rank owns two row
 * buffers used alternately (`out[g]` = buffer 0 of rank g, buffer 1 is `buffer_elems` elements
 * further), `world` 32-bit flags and a call counter `epoch_local`, all zero at the start.  A
 * launch is fused call number E + 1 of its rank, with E read from `epoch_local` on the device:
 * it waits - bounded, 0.25 s, else B200Q_ERR_DEVICE_TIMEOUT in the status word - until all
 * `world` slots of `flags_local` have reached E (every rank has finished call E, so the
 * activations are complete and nobody still reads the buffer about to be overwritten), writes
 * buffer (E + 1) % 2 of every rank, sets `flag_slot[g]` (= this rank's slot in rank g's flags) to
 * E + 1 and stores E + 1 to `epoch_local`.  With `a_prev_offset >= 0` the activations are this
 * rank's previous gathered output (buffer E % 2, from that element on, row stride lda) and `a`
 * is ignored.  No per-call state is passed from the host, so the same call sequence can be
 * captured once and replayed from a CUDA graph.  All ranks must make the same sequence of calls.
 * Word 8 of the workspace header counts the CTAs of the launch.
 *
 * mode = B200Q_GATHER_TAGGED replaces flags by tags inside the data: for these batches the hand-over
 * between GPUs is most of a layer's time.  The row buffers then hold 64-bit words
 * {two 16-bit outputs, 32-bit call number}: `out[g]` = word buffer 0 of rank g ([M, ldc / 2] words),
 * THREE buffers per rank used in turn, `buffer_elems` = words between consecutive buffers,
 * `epoch_local` = 16 consecutive 32-bit words of this mode's own (word 0 the call counter, word 8 an
 * arrival counter, the rest spare; zero at the start), `flag_slot` / `flags_local` unused.  Fused call E + 1
 * stores each pair of its outputs with the tag E + 1 in one 64-bit store into buffer (E + 1) % 3 of
 * every rank; with `a_prev_offset >= 0` it reads buffer E % 3 word by word and repeats a load -
 * bounded as above - until the word carries tag E.  No launch waits for a whole grid of another
 * GPU and nothing is fenced; the previous call's data is safe because whoever overwrites a buffer
 * has read words that were written after its last reader finished.  Two rules follow: a call with
 * activations from outside (`a_prev_offset < 0`) must not follow another such call directly unless a
 * b200q_gather_collect (wait only is enough) lies between them, and every rank issues its calls on
 * one stream.  b200q_gather_collect turns the latest call's tagged rows into dense rows;
 * b200q_gather_push stores a shard as tagged words and counts as a call of this mode.  Tagged and flag
 * calls use separate buffers and counters and do not see each other. */
#define B200Q_GATHER_FLAGS 0
#define B200Q_GATHER_TAGGED 1
typedef struct b200q_gather {
  int32_t world, rank;
  int32_t ldc;            /* elements per full output row */
  int32_t col_offset;     /* first column of this rank's shard */
  void* out[8];           /* row buffer 0 of every rank, fp16 [M, ldc] */
  void* flag_slot[8];     /* this rank's slot in every rank's flag array */
  const void* flags_local;/* this rank's flag array, uint32[world] */
  void* epoch_local;      /* this rank's call counter, uint32 */
  int64_t buffer_elems;   /* elements between a rank's two row buffers */
  int64_t a_prev_offset;  /* >= 0: activations = this rank's previous gathered output from this element on */
  int32_t mode;           /* B200Q_GATHER_FLAGS or B200Q_GATHER_TAGGED */
  int32_t reserved;       /* 0 */
} b200q_gather_t;

int b200q_gemm_gather(const void* a, int lda, const void* bq, const void* scales, int M, int N, int K, int wtype,
                      int zero_point, int group, int act_dtype, void* workspace, size_t workspace_bytes, void* stream,
                      const b200q_gather_t* gather);

/* The same all-gather for an output that some other kernel produced (batches of more than 16 rows run
 * b200q_gemm on the local shard first), as two calls made one after the other on one stream:
 * b200q_gather_push copies shard[M, N_loc] (row stride lds) into this rank's column range of row
 * buffer (E + 1) % 2 of every rank and raises the flags like a fused call; b200q_gather_collect waits
 * (bounded) until all ranks' shards of that call have landed here and copies the complete rows to
 * full_local [M, ldc] (row stride ld_local; NULL: wait only).  Same regions, counters and rules as
 * b200q_gemm_gather, with which they can be mixed; `workspace` holds the status header (256 bytes are
 * enough).  status[1] = 7 / 8 names a wait of push / collect that gave up.  In tagged mode collect
 * waits for the tags of the latest fused call and writes the values of its words as dense rows. */
int b200q_gather_push(const void* shard, int lds, int M, int N_loc, void* workspace, size_t workspace_bytes,
                      void* stream, const b200q_gather_t* gather);
int b200q_gather_collect(void* full_local, int ld_local, int M, void* workspace, size_t workspace_bytes, void* stream,
                         const b200q_gather_t* gather);

/* Device memory that other processes of the node can map (cudaMalloc + CUDA IPC): allocate,
 * export a 64-byte handle, open a peer's handle (enables peer access), close, free.  These five
 * are the only functions of the library that allocate or free device memory. */
int b200q_peer_alloc(size_t bytes, void** ptr);
int b200q_peer_export(void* ptr, unsigned char handle[64]);
int b200q_peer_open(const unsigned char handle[64], void** ptr);
int b200q_peer_close(void* ptr);
int b200q_peer_free(void* ptr);

/* W[K, N] (row-major, dtype act_dtype like the scales) = dequantized weights, bit-exact with the
 * reference's cast-then-scale (examples/quantization/matmul_a16wx.py:316-320; cast kernel
 * python/tilus/kernels/cast.py:27-55). */
int b200q_dequantize(const void* bq, const void* scales, void* w, int N, int K, int wtype, int zero_point, int group,
                     int act_dtype, void* stream);

/* QuantizedLinear.load_and_quantize on the GPU (examples/quantization/matmul_a16wx.py:470-528):
 * weight [N, K] (row = output feature; weight_dtype 0 = fp16, 1 = fp32, 2 = bf16; row stride ldw
 * elements) -> scales [K/group, N] of dtype act_dtype = max(absmax / max_value, 1e-6) per (group, column) and the packed
 * weights bq (b200 layout, K*N*nbits/8 bytes): q = clamp(w / scale, min, max), integers rounded
 * half to even, floats encoded as python/tilus/hidet/ir/primitives/cuda/cast.py:44-100.  The
 * reference does this with PyTorch ops followed by its change-layout kernel (:520-525). */
int b200q_quantize(const void* weight, int weight_dtype, int ldw, void* bq, void* scales, int N, int K, int wtype,
                   int group, int act_dtype, void* stream);

/* ---- the step behind the gate_up projection: SwiGLU and the per-token FP8 cast -----------------------
 * Per token and group of `group` channels (a multiple of 128, at most 512): scale = absmax / 448
 * (1 if the group is all zero), out = e4m3(value * (448 / absmax)) rounded to nearest even and
 * saturated, out_sf = scale (fp32 [tokens, hidden / group]).  x is fp16 or bf16 (act_dtype), row
 * stride ldx elements; out is e4m3 bytes, row stride ldo.
 *
 * b200q_per_token_cast: value = x[tokens, hidden].  Replaces the reference's PerTokenCast script
 * (examples/quantization/per_token_cast.py:22-97).
 *
 * b200q_swiglu_per_token_cast: x is [tokens, 2 * hidden]; value = silu(x[:, :hidden]) * x[:, hidden:]
 * in fp32 with silu(l) = l / (exp(-l) + 1); with use_clamp l is clamped from above and r on both
 * sides to clamp_value; a row whose pos_to_token_topk entry p is >= 0 is multiplied by
 * topk_weights[p]; a row whose pos_to_expert entry is negative is skipped (nothing is written for
 * it).  Each of the three index arrays may be NULL (no weights / no skipping).  Replaces
 * SwiGLUForwardAndPerTokenCast (examples/quantization/swiglu_forward_and_per_token_cast.py:28-166).
 *
 * b200q_gemm_swiglu_cast: the gate_up projection followed by the SwiGLU cast in one call:
 * gate_up[M, N] = A x dequant(Bq) as b200q_gemm (N = 2 * hidden, gate columns first), then the
 * cast kernel - launched with programmatic stream serialization, so that it is resident and
 * waiting when the GEMM retires - reads gate_up and writes out / out_sf.  The two kernels are
 * not merged: the decode kernel spreads one token's 128-channel group over several CTAs and the
 * tcgen05 kernels keep a channel's gate and up columns in different warps, so the group maximum
 * is taken in a kernel of its own. */
int b200q_per_token_cast(const void* x, int ldx, void* out, int ldo, float* out_sf, int tokens, int hidden, int group,
                         int act_dtype, void* stream);
int b200q_swiglu_per_token_cast(const void* x, int ldx, void* out, int ldo, float* out_sf, int tokens, int hidden,
                                int group, int act_dtype, const int32_t* pos_to_token_topk, const float* topk_weights,
                                const int32_t* pos_to_expert, int use_clamp, float clamp_value, void* stream);
int b200q_gemm_swiglu_cast(const void* a, int lda, const void* bq, const void* scales, void* gate_up, int ldg,
                           void* out, int ldo, float* out_sf, int M, int N, int K, int wtype, int zero_point, int group,
                           int act_dtype, int cast_group, int use_clamp, float clamp_value, void* workspace,
                           size_t workspace_bytes, void* stream);

/* Reads the device status header of a workspace (synchronises `stream`): status[0] is 0 or
 * B200Q_ERR_DEVICE_TIMEOUT, status[1..3] say which wait gave up (1: 2 = tcgen05 prefill pipeline,
 * 3 = decode kernel's weight ring, 5 = wait for a peer's columns, 6 = tcgen05 small-batch pipeline,
 * 7 / 8 = gather push / collect, 9 = wait for the CTAs that fetch host activations; 2: CTA; 3: warp or
 * thread).  Clears the header.  A launch that gave up may leave partial sums
 * behind: zero the workspace before it is used again.  workspace == NULL names the built-in
 * scratch of b200q_gemm_static_ws, which this call then puts back to zero itself. */
int b200q_device_status(void* workspace, int32_t status[4], void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
