/* tracea_b200.h -- C ABI of the B200-native Conv2d library (libtracea_b200.so).
 *
 * The library is a drop-in for the Conv2d entry of Tracea's FFI: every type below has the layout of
 * the reference's `#[repr(C)]` / C declaration of the same name, and `tracea_conv2d` has the
 * reference's six-argument signature, so a caller built against the reference's own
 * `include/tracea.hpp` links against this library unchanged. Each declaration cites the reference
 * interface it replaces (paths are relative to the reference project's root).
 *
 * Plain C: pointers and sizes only, no C++ or torch types.
 */
#ifndef TRACEA_B200_H_
#define TRACEA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: include/tracea.hpp:16-23, tracea-ffi/src/lib.rs:23-30. */
typedef enum {
  TRACEA_SUCCESS = 0,
  TRACEA_INVALID_PARAMS = 1,
  TRACEA_UNSUPPORTED_CONFIG = 2,
  TRACEA_CUDA_ERROR = 3,
  TRACEA_CPU_ERROR = 4,
  TRACEA_UNKNOWN_ERROR = 99
} TraceaStatus;

/* Element types: include/tracea.hpp:29-35, tracea-ffi/src/lib.rs:34-40.
 * This library computes FLOAT32 (as TF32 on the tensor cores), FLOAT16 and BFLOAT16, all with
 * fp32 accumulation. INT32 / INT8 are rejected with TRACEA_UNSUPPORTED_CONFIG. */
typedef enum {
  TRACEA_DTYPE_FLOAT32 = 0,
  TRACEA_DTYPE_FLOAT16 = 1,
  TRACEA_DTYPE_BFLOAT16 = 2,
  TRACEA_DTYPE_INT32 = 3,
  TRACEA_DTYPE_INT8 = 4
} TraceaDType;

/* Fused epilogue selector: include/tracea.hpp:37-47; op lists per kind follow
 * src/interface/c_bindings.rs:144-197 (bias is added only under the BIAS_* kinds and only if `b`
 * is non-NULL; residual only under the RESIDUAL* kinds and only if non-NULL).
 * Values 9 and 10 extend the enum: the reference's runtime entry accepts the op string
 * "bias+residual+relu" (src/interface/python.rs:41-87) but its C enum has no value for it.
 * Order is always bias -> residual -> activation. */
typedef enum {
  TRACEA_EPILOGUE_IDENTITY = 0,
  TRACEA_EPILOGUE_BIAS_ADD = 1,
  TRACEA_EPILOGUE_RELU = 2,
  TRACEA_EPILOGUE_GELU = 3,
  TRACEA_EPILOGUE_SILU = 4,
  TRACEA_EPILOGUE_BIAS_RELU = 5,
  TRACEA_EPILOGUE_BIAS_SILU = 6,
  TRACEA_EPILOGUE_RESIDUAL = 7,
  TRACEA_EPILOGUE_RESIDUAL_RELU = 8,
  TRACEA_EPILOGUE_BIAS_RESIDUAL_RELU = 9,
  TRACEA_EPILOGUE_BIAS_RESIDUAL = 10
} TraceaEpilogueKind;

/* Borrowed tensor view: include/tracea.hpp:59-66, tracea-ffi/src/lib.rs:42-57.
 * `shape` is always the logical shape (x: N,C,H,W; w: K,C,R,S; out: N,K,Ho,Wo; bias: K);
 * `stride` is in elements and decides the physical layout. Channels-last memory
 * (stride[1] == 1) is consumed and produced directly; NCHW-contiguous x / OIHW-contiguous w go
 * through a transpose into library scratch first. `device_id` -1 means host memory: the
 * library stages such tensors through the current CUDA device and synchronises before returning. */
typedef struct {
  void *ptr;
  uint32_t rank;
  const uint64_t *shape;
  const int64_t *stride;
  TraceaDType dtype;
  int32_t device_id;
} TraceaTensorView;

/* Conv2d parameters: include/tracea.hpp:72-82 (the tracea-ffi crate's struct,
 * tracea-ffi/src/lib.rs:61-71, is the same minus `epilogue`). */
typedef struct {
  uint32_t stride_h;
  uint32_t stride_w;
  uint32_t padding_h;
  uint32_t padding_w;
  uint32_t dilation_h;
  uint32_t dilation_w;
  uint32_t groups;
  TraceaEpilogueKind epilogue;
  void *stream; /* cudaStream_t; NULL = default stream. Work is enqueued, not synchronised. */
} TraceaConv2dParams;

/* The older parameter block without `epilogue` (tracea-ffi/src/lib.rs:61-71). */
typedef struct {
  uint32_t stride_h;
  uint32_t stride_w;
  uint32_t padding_h;
  uint32_t padding_w;
  uint32_t dilation_h;
  uint32_t dilation_w;
  uint32_t groups;
  void *stream;
} TraceaConv2dParamsV0;

/* out = epilogue(conv2d(x, w)). Replaces include/tracea.hpp:107-110 (the tracea-ffi entry,
 * tracea-ffi/src/lib.rs:121-207). Validation mirrors tracea-ffi/src/lib.rs:150-207:
 * NULL x.ptr / w.ptr / out -> INVALID_PARAMS; rank != 4 -> INVALID_PARAMS; groups != 1 ->
 * UNSUPPORTED_CONFIG; zero stride or an `out` shape that is not [N,K,Ho,Wo] -> INVALID_PARAMS.
 *
 * Shape order: `shape` is logical [N,C,H,W] for x / out / residual and [K,C,R,S] for w, as tracea.hpp
 * documents and tracea-ffi reads them; the strides say how that sits in memory. The reference's OTHER conv2d
 * entry of the same name, the in-crate src/interface/c_bindings.rs:205-290, reads x.shape as [N,H,W,C] and
 * w.shape as [K,R,S,C]: a caller of that entry must permute its shape (and stride) arrays to [N,C,H,W] /
 * [K,C,R,S] when it moves to this library -- the call still links unchanged, and a shape check cannot tell
 * the two orders apart when the extents happen to agree. tracea_conv_transpose2d below does take the
 * [N,H,W,C] / [K,R,S,C] order, because the in-crate entry is the only one the reference has for it. */
TraceaStatus tracea_conv2d(TraceaTensorView x, TraceaTensorView w, const TraceaTensorView *b,
                           const TraceaTensorView *residual, TraceaTensorView *out,
                           TraceaConv2dParams params);

/* Five-argument form of the tracea-ffi crate (tracea-ffi/src/lib.rs:121-128): no residual, no
 * epilogue field; bias is added when `b` is non-NULL. Same symbol name as the six-argument form
 * in the reference, so it is exported here under a suffix. */
TraceaStatus tracea_conv2d_v0(TraceaTensorView x, TraceaTensorView w, const TraceaTensorView *b,
                              TraceaTensorView *out, TraceaConv2dParamsV0 params);

/* tracea_conv2d for callers that must not touch the CUDA allocator. No counterpart in the reference.
 *
 * tracea_conv2d borrows staging memory from a stream-ordered pool whenever x arrives NCHW-contiguous
 * or w OIHW-contiguous (they are rearranged to channels-last before the conv kernel runs). Some
 * callers cannot afford that: a serving process that handed every free byte of the GPU to its own
 * arena at start-up (a later allocation fails, or makes the arena give memory back), or a
 * latency-critical loop where an allocation's implicit synchronisation and driver locks are not
 * acceptable. This entry point does the same work with the staging area taken from a fixed
 * 16 MiB array that is part of the library's device image; it never calls cudaMalloc / cudaFree,
 * the pool allocator, or any library routine that allocates.
 *
 * Limits and rules:
 *   - x, w, b, residual and out must be device tensors (device_id >= 0); host views are rejected
 *     with INVALID_PARAMS, because staging them would need an allocation.
 *   - The channels-last copy of x plus the repacked w (each rounded up to 256 bytes) must fit in
 *     16 MiB; otherwise the call returns UNSUPPORTED_CONFIG and the message states the sizes.
 *     Channels-last x and w need no staging at all and are accepted at any size.
 *   - The first call on each device looks up the array's device address (with that device made
 *     current); issue that first call before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's bytes. The adapters rewrite
 *     every byte they later read, so nothing depends on old contents, but two calls whose kernels
 *     can overlap on the GPU (different streams, no ordering between them) race on it. Order such
 *     calls with events or keep them on one stream.
 *   - The array is resident on every GPU that loads the library, until the process exits.
 *   - A kernel that gives up a bounded wait records its code in status words that also live in the device
 *     image (not in pinned host memory, which would have to be allocated). Unlike tracea_conv2d, this entry
 *     therefore does not look at them on the way in; tracea_b200_device_status copies them back and clears them.
 * Arguments, epilogue rules, validation and status codes are those of tracea_conv2d. */
TraceaStatus tracea_conv2d_noalloc(TraceaTensorView x, TraceaTensorView w, const TraceaTensorView *b,
                                   const TraceaTensorView *residual, TraceaTensorView *out,
                                   TraceaConv2dParams params);

/* ---- the operators either side of the conv path, run on the same kernel ------------------------------- */

/* include/tracea.hpp:84-87. */
typedef struct {
  TraceaEpilogueKind epilogue;
  void *stream;
} TraceaGemmParams;

/* c = epilogue(a[M,K] * b[K,N]): replaces include/tracea.hpp:139-144 and src/interface/c_bindings.rs:375-440.
 * Rank-2 views, strides in elements (NULL = row-major). It runs as the 1x1 convolution it is: `a` rows are the
 * pixels, `b` columns the output channels. The zero-copy form is a with stride[1] == 1 and b with stride[0] == 1
 * and stride[1] == K (memory [N][K], e.g. a transposed view of a Linear layer's weight, or the buffer
 * tracea_gemm_prepack_b wrote); a row-major b is transposed into scratch on every call. bias: rank-1, length N;
 * residual: [M,N], dtype of c. Dtypes as tracea_conv2d (fp32 runs as TF32; the reference's entry took fp16 only).
 * rank != 2 or a shape mismatch -> INVALID_PARAMS. */
TraceaStatus tracea_gemm(TraceaTensorView a, TraceaTensorView b, const TraceaTensorView *bias,
                         const TraceaTensorView *residual, TraceaTensorView *c, TraceaGemmParams params);

/* include/tracea.hpp:118-131. */
typedef struct {
  uint32_t stride_h;
  uint32_t stride_w;
  uint32_t padding_h;
  uint32_t padding_w;
  uint32_t output_padding_h;
  uint32_t output_padding_w;
  uint32_t dilation_h;
  uint32_t dilation_w;
  uint32_t groups;
  TraceaEpilogueKind epilogue;
  void *stream;
} TraceaConvTranspose2dParams;

/* out = epilogue(conv_transpose2d(x, w)): replaces include/tracea.hpp:133-137 and
 * src/interface/c_bindings.rs:292-372. Shapes are the ones that entry reads (c_bindings.rs:301-311;
 * tracea-python/python/tracea/ops.py:72-88): x [N,H,W,C], w [K,R,S,C], out and residual [N,Ho,Wo,K] with
 * Ho = (H-1)*stride_h - 2*padding_h + R + output_padding_h; strides in elements decide the memory layout
 * (NULL = row-major, i.e. NHWC / KRSC memory). The reference's kernel reads its weights as [C*R*S][K] memory
 * (src/emitter/conv_transpose.rs:232-243): pass that buffer as shape [K,R,S,C] with strides {1, S*K, K, R*S*K}.
 * out[n,ho,wo,k] = sum over (hi,r), (wi,s), c with ho = hi*stride_h - padding_h + r of x[n,hi,wi,c]*w[k,r,s,c]
 * (examples/verify_conv_transpose.rs:12-52). It runs as stride_h*stride_w stride-1 convolutions, one per output
 * phase, each over the filter taps that reach that phase.
 * dilation != 1 or groups != 1 -> UNSUPPORTED_CONFIG (the reference ignores both fields); output_padding must be
 * smaller than the stride; other validation as tracea_conv2d. Device tensors and host tensors (device_id -1,
 * staged through the current GPU) are accepted. */
TraceaStatus tracea_conv_transpose2d(TraceaTensorView x, TraceaTensorView w, const TraceaTensorView *b,
                                     const TraceaTensorView *residual, TraceaTensorView *out,
                                     TraceaConvTranspose2dParams params);

/* The plan tracea_conv_transpose2d follows along one axis, for inspection and tests (pure arithmetic, no device).
 * For each output phase a0 in [0, stride) it writes 8 values to phases[8*a0 ..]:
 *   {a0, T, a, taps, x_off, in, pad_lo, pad_hi}
 * outputs a0 + stride*t, t < T, are a stride-1 correlation of input rows [x_off, x_off + in), zero-padded by pad_lo
 * in front and pad_hi behind, with the `taps` filter taps a + stride*(taps-1-j), j = 0..taps-1 (reversed order);
 * a = -1 marks a phase no tap reaches (one zero tap). T = 0: the phase has no outputs. Returns stride, or -1 on
 * bad arguments. No counterpart in the reference. */
int32_t tracea_b200_conv_transpose_plan(uint32_t in_extent, uint32_t out_extent, uint32_t filter, uint32_t stride,
                                        uint32_t padding, int64_t *phases);

/* Weight prepacking, so that the documented OIHW / row-major surface costs nothing in steady state. No
 * counterpart in the reference, whose kernels fix one weight layout per back end (src/emitter/cuda/conv.rs:248-266).
 *
 * tracea_conv2d_prepack writes w (logical [K,C,R,S], any strides, device memory) into `dst` as dense
 * [K][R][S][Cp] memory, Cp = C rounded up to 16 bytes' worth of elements with zero fill, on `stream`, and fills
 * `packed_shape` / `packed_stride` with the logical [K,Cp,R,S] view of dst to hand to tracea_conv2d (which then
 * reads it in place). When Cp != C the activations passed with it must carry Cp channels too (zero padded).
 * tracea_gemm_prepack_b does the same for b[K,N]: dst becomes [N][K] memory and packed_stride = {1, K}.
 * `dst_bytes` must be at least tracea_conv2d_prepack_bytes(w) / tracea_gemm_prepack_b_bytes(b) (0 on a bad view);
 * dst must be 16-byte aligned and on w.device_id. */
uint64_t tracea_conv2d_prepack_bytes(TraceaTensorView w);
TraceaStatus tracea_conv2d_prepack(TraceaTensorView w, void *dst, uint64_t dst_bytes, uint64_t packed_shape[4],
                                   int64_t packed_stride[4], void *stream);
uint64_t tracea_gemm_prepack_b_bytes(TraceaTensorView b);
TraceaStatus tracea_gemm_prepack_b(TraceaTensorView b, void *dst, uint64_t dst_bytes, int64_t packed_stride[2],
                                   void *stream);

/* Thread-local last error text: tracea-ffi/src/lib.rs:87-109. Returns bytes copied (without the
 * terminating NUL), -1 when buf is NULL or len is 0. */
int32_t tracea_get_last_error(uint8_t *buf, size_t len);
void tracea_clear_error(void);

/* Version 0.1.0, as tracea-ffi/src/lib.rs:244-251. */
uint32_t tracea_version_major(void);
uint32_t tracea_version_minor(void);
uint32_t tracea_version_patch(void);

/* Optional, idempotent runtime bring-up / tear-down (include/tracea.h:26-31,
 * src/interface/c_bindings.rs:103-119). tracea_conv2d initialises lazily, so neither is required.
 * tracea_init returns 0 on success, -1 if no CUDA device can be opened. */
int tracea_init(void);
void tracea_shutdown(void);

/* Reads and clears the device-side status words of `device_id`: 0 when every conv kernel launched
 * so far on that device finished normally, otherwise the code of the first bounded wait that ran
 * out inside a kernel (see conv2d_sm100.cuh). Covers both the kernels of tracea_conv2d (words in pinned host
 * memory) and those of tracea_conv2d_noalloc (words in device memory, fetched with a blocking copy once that
 * entry has been used on the device). Call after synchronising the stream. The reference
 * has no counterpart: its kernels spin without limit. */
uint32_t tracea_b200_device_status(int32_t device_id);

/* For tests of the failure path only. Every wait inside the kernels is bounded; a wait that runs out makes its role
 * record a code, the CTA unwind and the kernel return normally. wait_limit_cycles > 0 replaces the limit of a single
 * wait (default about two seconds) for the launches that follow; producer_stop_after >= 0 makes the TMA producer of
 * every CTA of those launches stop after that many pipeline stages and leave normally, so that the waits downstream
 * of it run out -- nothing faults, traps or spins without limit. (0, -1) restores normal operation. Process-wide.
 * No counterpart in the reference (its kernels wait without limit, src/backend/cuda/primitives.rs:70-121). */
void tracea_b200_test_hooks(int64_t wait_limit_cycles, int32_t producer_stop_after);

/* Byte counters of the library's stream-ordered scratch pool on `device_id`:
 * stats = {reserved now, reserved high-water mark, in use now, in-use high-water mark}; reset_high != 0 resets
 * the two high-water marks after reading. Returns 1, 0 when the device has no pool yet (stats all zero), -1 on
 * bad arguments. Lets a test show that a call took nothing from the pool. No counterpart in the reference. */
int32_t tracea_b200_pool_stats(int32_t device_id, uint64_t stats[4], int32_t reset_high);

/* Number of GPU kernels this library has launched in this process so far (conv kernels and layout adapters;
 * a call may launch more than one: a layout adapter per staged operand, one conv launch per phase of a transposed
 * convolution). Benchmarks read it before and after a timed region. No counterpart in the reference. */
uint64_t tracea_b200_launch_count(void);

/* The same count for one kind of kernel: 0 the general implicit-GEMM conv kernel, 1 its instantiations that cut tiles
 * over K, 2 the resident-filter kernel (stride-1 small filters over 64-channel activations), 3 layout adapters,
 * 4 the row-band kernel (few-channel 16-bit images such as the RGB stem).
 * Lets tests and benchmarks see which path a call took. 0 for any other `kind`. No counterpart in the reference. */
uint64_t tracea_b200_launch_count_of(int32_t kind);

#ifdef __cplusplus
}
#endif
#endif /* TRACEA_B200_H_ */
