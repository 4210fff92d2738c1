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

/* Activation / output dtype tags. */
enum { B200Q_F16 = 0 };

/* Kernel selection made by the static shape table (replaces the reference's autotuner,
 * python/tilus/lang/instantiated_script.py:700-801).  Filled by b200q_plan; may be edited
 * and passed to b200q_gemm_planned for experiments. */
typedef struct b200q_plan {
  int32_t kernel;        /* 2 = mma.sync stream kernel (M <= 16 per pass), 1 = tcgen05 kernel */
  int32_t m_tiles;       /* kernel 2: 8-row activation tiles per pass (1 or 2); kernel 1: tiles along M */
  int32_t splits;        /* k chunks (kernel 2) / split-K factor (kernel 1) */
  int32_t cluster;       /* 1 (no kernel launches clusters) */
  int32_t ctas_per_split;/* kernel 2: CTAs per k chunk, grid = splits * ctas_per_split; kernel 1: output tiles */
  int32_t smem_bytes;    /* dynamic shared memory per CTA */
  int32_t tile_m;        /* kernel 1: activation rows per CTA tile (32, 64, 128 or 256) */
  int32_t stages;        /* pipeline depth (kernel 2: ring slots per warp; kernel 1: activation stages) */
  int32_t warps;         /* warps per CTA (output only) */
  int32_t passes;        /* launches needed to cover M */
  int32_t pdl;           /* 1: launch with programmatic stream serialization (overlap with the previous kernel) */
  int32_t debug;         /* 0; non-zero values switch parts of the kernels off for timing experiments */
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

/* C = A x dequant(Bq).  a: fp16 [M, K] (row stride lda elements), bq: b200-packed weights,
 * scales: fp16 [K/group, N], c: fp16 [M, N] (row stride ldc).  Replaces tilus_launch for
 * QuantizedMatmul (examples/quantization/matmul_a16wx.py:231-405). */
int b200q_gemm(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N, int K,
               int wtype, int zero_point, int group, int act_dtype, void* workspace, size_t workspace_bytes,
               void* stream);

/* Same, with the kernel selection supplied by the caller. */
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
 * fixed array inside the library, b200q_static_workspace_limit() bytes (8 MiB) per GPU, held
 * from library load to process exit.  Problems whose b200q_workspace_bytes exceeds that limit
 * return B200Q_ERR_WORKSPACE and launch nothing.  The function allocates nothing and frees
 * nothing.  The first call on each device looks the array's address up and clears it, so make
 * that call outside any stream capture.  All calls on a device share the one array: calls
 * that may overlap on the GPU (different streams) race on it and must be serialised by the
 * caller; back-to-back calls on one stream are fine, each leaves the scratch zeroed. */
int b200q_gemm_static_ws(const void* a, int lda, const void* bq, const void* scales, void* c, int ldc, int M, int N,
                         int K, int wtype, int zero_point, int group, int act_dtype, void* stream);
size_t b200q_static_workspace_limit(void);

/* W[K, N] (fp16, row-major) = dequantized weights, bit-exact with the reference's
 * cast-then-scale (examples/quantization/matmul_a16wx.py:316-320; cast kernel
 * python/tilus/kernels/cast.py:27-55). */
int b200q_dequantize(const void* bq, const void* scales, void* w, int N, int K, int wtype, int zero_point, int group,
                     void* stream);

/* QuantizedLinear.load_and_quantize on the GPU (examples/quantization/matmul_a16wx.py:470-528):
 * weight [N, K] (row = output feature; weight_dtype 0 = fp16, 1 = fp32; row stride ldw elements) ->
 * scales fp16 [K/group, N] = max(absmax / max_value, 1e-6) per (group, column) and the packed
 * weights bq (b200 layout, K*N*nbits/8 bytes): q = clamp(w / scale, min, max), integers rounded
 * half to even, floats encoded as python/tilus/hidet/ir/primitives/cuda/cast.py:44-100.  The
 * reference does this with PyTorch ops followed by its change-layout kernel (:520-525). */
int b200q_quantize(const void* weight, int weight_dtype, int ldw, void* bq, void* scales, int N, int K, int wtype,
                   int group, void* stream);

/* Reads the device status header of a workspace (synchronises `stream`): status[0] is 0 or
 * B200Q_ERR_DEVICE_TIMEOUT, status[1..3] say which wait gave up.  Clears the header. */
int b200q_device_status(void* workspace, int32_t status[4], void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
