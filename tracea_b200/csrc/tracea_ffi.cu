// Host side of libtracea_b200.so: the C ABI of include/tracea_b200.h on top of the sm_100a conv
// kernel. It takes the place of three pieces of the reference for this one path: the FFI shim
// (tracea-ffi/src/lib.rs:121-238, whose CUDA body is a stub), the NVRTC code emitter + compile
// cache (src/emitter/cuda/conv.rs, src/runtime/manager/kernel.rs:123-327) and the tile-config
// search (src/policy/standard.rs:73-113) -- kernels are compiled ahead of time and the tile
// width is picked by a closed-form cost rule.
//
// There is no CPU compute path in this library: every call ends in a kernel launch on a CUDA
// device or in an error status.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <exception>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../../include/tracea_b200.h"
#include "conv2d_sm100.cuh"
#include "conv2d_window_sm100.cuh"
#include "conv2d_rowband_sm100.cuh"
#include "layout_kernels.cuh"

namespace {

using tb200::ConvKernelArgs;

// ------------------------------------------------------------------ last error (thread local)
thread_local std::string g_last_error;

void set_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

struct StatusError {
  TraceaStatus status;
};

#define TB_FAIL(status_, ...)        \
  do {                               \
    set_error(__VA_ARGS__);          \
    throw StatusError{status_};      \
  } while (0)

#define TB_CUDA(expr)                                                                   \
  do {                                                                                  \
    cudaError_t e_ = (expr);                                                            \
    if (e_ != cudaSuccess) {                                                            \
      TB_FAIL(TRACEA_CUDA_ERROR, "%s failed: %s", #expr, cudaGetErrorString(e_));       \
    }                                                                                   \
  } while (0)

// ------------------------------------------------------------------ driver entry points
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

struct DeviceState {
  std::atomic<bool> ready{false};
  int dev = 0;
  int num_sms = 0;
  cudaMemPool_t pool = nullptr;
  uint32_t* status = nullptr;  // pinned, mapped: kernels write error codes the host reads directly
  std::mutex host_mu;          // one host-memory call at a time per device (it owns the copy streams below)
  // Scratch of the K-split schedule (fp32 partial sums, then the counters), one block per stream that has used it:
  // launches on one stream run one after another, so they can share a block, and the kernels leave the counters
  // at zero, so nothing has to be cleared between launches. Allocated once per stream with cudaMalloc.
  std::mutex ws_mu;
  std::unordered_map<unsigned long long, void*> split_ws;
  size_t split_partial_bytes = 0, split_counter_bytes = 0;
  // host-memory path only: copy streams and events for the chunked H2D / compute / D2H pipeline
  static constexpr int kMaxChunks = 16;
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t ev_entry = nullptr, ev_done = nullptr;
  cudaEvent_t ev_in[kMaxChunks] = {}, ev_out[kMaxChunks] = {};
};

constexpr int kMaxDevices = 64;
// Locking: each device's state is brought up once under its own mutex and is read-only afterwards, so host
// threads that drive different GPUs (or the same GPU on different streams) do not serialise on the call path:
// validation, tensor-map encoding and the launch itself run without any lock.
std::mutex g_dev_mu[kMaxDevices];
std::mutex g_driver_mu;
DeviceState g_dev[kMaxDevices];
// Test hooks (tracea_b200_test_hooks): a shortened wait limit and a producer that goes silent, so that a test can
// make a bounded wait run out without hanging anything. Off (0 / -1) unless a test sets them.
std::atomic<long long> g_test_wait_limit{0};
std::atomic<int> g_test_producer_stop{-1};
// "opt-in shared memory size has been set for this kernel variant on this device":
// [device][dtype][bn index][tiling: single CTA / CTA pair / two row blocks; x3: plain, coop epilogue, K-split].
// Setting the attribute twice is harmless, so a relaxed flag is enough.
std::atomic<bool> g_attr_set[kMaxDevices][3][3][9];
std::atomic<unsigned long long> g_kernel_launches{0};   // every kernel this library has launched (conv + layout adapters)
// the same, by kind: 0 general implicit-GEMM kernel, 1 its K-split instantiations, 2 resident-filter kernel, 3 layout adapters
std::atomic<unsigned long long> g_launches_by_kind[5];
EncodeTiledFn g_encode_tiled = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;

void load_driver_entry_points() {
  std::lock_guard<std::mutex> lock(g_driver_mu);
  if (g_encode_tiled != nullptr && g_encode_im2col != nullptr) return;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  TB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
    TB_FAIL(TRACEA_CUDA_ERROR, "driver does not export cuTensorMapEncodeTiled");
  g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  fn = nullptr;
  TB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres));
  if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
    TB_FAIL(TRACEA_CUDA_ERROR, "driver does not export cuTensorMapEncodeIm2col");
  g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
}

// The per-device state, brought up on first use (with `dev` current).
DeviceState& device_state(int dev) {
  if (dev < 0 || dev >= kMaxDevices) TB_FAIL(TRACEA_INVALID_PARAMS, "device_id %d out of range", dev);
  DeviceState& st = g_dev[dev];
  if (st.ready.load(std::memory_order_acquire)) return st;
  std::lock_guard<std::mutex> lock(g_dev_mu[dev]);
  if (st.ready.load(std::memory_order_relaxed)) return st;
  cudaDeviceProp prop;
  TB_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG,
            "device %d is sm_%d%d; this library only carries sm_100a kernels", dev, prop.major,
            prop.minor);
  st.dev = dev;
  st.num_sms = prop.multiProcessorCount;
  // the largest split any launch can ask for: 2 slots per worker of 256 x 256 fp32, 8 counter pairs per split tile
  st.split_partial_bytes = 2ull * st.num_sms * 256 * 256 * sizeof(float);
  st.split_counter_bytes = 2 * static_cast<size_t>(st.num_sms) * 8 * 2 * sizeof(uint32_t);   // up to two waves of tiles
  load_driver_entry_points();
  cudaMemPoolProps pp = {};
  pp.allocType = cudaMemAllocationTypePinned;
  pp.handleTypes = cudaMemHandleTypeNone;
  pp.location.type = cudaMemLocationTypeDevice;
  pp.location.id = dev;
  TB_CUDA(cudaMemPoolCreate(&st.pool, &pp));
  uint64_t keep = ~0ull;  // keep freed scratch cached in the pool instead of returning it to the OS
  TB_CUDA(cudaMemPoolSetAttribute(st.pool, cudaMemPoolAttrReleaseThreshold, &keep));
  TB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&st.status), 4 * sizeof(uint32_t),
                        cudaHostAllocMapped | cudaHostAllocPortable));
  memset(st.status, 0, 4 * sizeof(uint32_t));
  st.ready.store(true, std::memory_order_release);
  return st;
}

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int dev) {
    TB_CUDA(cudaGetDevice(&prev));
    if (prev != dev) {
      TB_CUDA(cudaSetDevice(dev));
      switched = true;
    }
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

// Stream-ordered scratch from the library's pool; released (stream-ordered) by the destructor.
struct Scratch {
  void* ptr = nullptr;
  cudaStream_t stream = nullptr;
  Scratch() = default;
  Scratch(const Scratch&) = delete;
  Scratch& operator=(const Scratch&) = delete;
  void alloc(DeviceState& st, size_t bytes, cudaStream_t s) {
    stream = s;
    TB_CUDA(cudaMallocFromPoolAsync(&ptr, bytes == 0 ? 16 : bytes, st.pool, s));
  }
  ~Scratch() {
    if (ptr != nullptr) cudaFreeAsync(ptr, stream);
  }
};

// The K-split scratch block of `stream` on this device (created on first use). A block's counters start at zero
// and every kernel leaves them at zero. Not for launches that are being captured into a graph: those take
// stream-ordered pool memory, which the graph owns.
void* split_workspace(DeviceState& st, cudaStream_t stream) {
  unsigned long long key = reinterpret_cast<unsigned long long>(stream);
  if (stream == cudaStreamPerThread)   // one handle, a different stream in every host thread
    key ^= static_cast<unsigned long long>(std::hash<std::thread::id>()(std::this_thread::get_id())) << 8;
  std::lock_guard<std::mutex> lock(st.ws_mu);
  auto it = st.split_ws.find(key);
  if (it != st.split_ws.end()) return it->second;
  void* base = nullptr;
  TB_CUDA(cudaMalloc(&base, st.split_partial_bytes + st.split_counter_bytes));
  TB_CUDA(cudaMemset(static_cast<char*>(base) + st.split_partial_bytes, 0, st.split_counter_bytes));
  st.split_ws.emplace(key, base);
  return base;
}

// After a kernel gave up a wait its counters may be anywhere: clear every block of the device.
void reset_split_workspaces(DeviceState& st) {
  std::lock_guard<std::mutex> lock(st.ws_mu);
  for (auto& kv : st.split_ws)
    cudaMemset(static_cast<char*>(kv.second) + st.split_partial_bytes, 0, st.split_counter_bytes);
}

// ------------------------------------------------------------------ views
struct View4 {
  void* ptr = nullptr;
  long long shape[4] = {0, 0, 0, 0};
  long long stride[4] = {0, 0, 0, 0};
  TraceaDType dtype = TRACEA_DTYPE_FLOAT32;
  int device = -1;
};

int elem_size(TraceaDType t) {
  switch (t) {
    case TRACEA_DTYPE_FLOAT32: return 4;
    case TRACEA_DTYPE_FLOAT16: return 2;
    case TRACEA_DTYPE_BFLOAT16: return 2;
    default: return 0;
  }
}

const char* dtype_name(TraceaDType t) {
  switch (t) {
    case TRACEA_DTYPE_FLOAT32: return "float32";
    case TRACEA_DTYPE_FLOAT16: return "float16";
    case TRACEA_DTYPE_BFLOAT16: return "bfloat16";
    case TRACEA_DTYPE_INT32: return "int32";
    case TRACEA_DTYPE_INT8: return "int8";
    default: return "?";
  }
}

View4 load_view4(const TraceaTensorView& v, const char* name) {
  if (v.rank != 4) TB_FAIL(TRACEA_INVALID_PARAMS, "Expected 4D tensors (NCHW): %s has rank %u", name, v.rank);
  if (v.shape == nullptr) TB_FAIL(TRACEA_INVALID_PARAMS, "%s: shape array is NULL", name);
  View4 o;
  o.ptr = v.ptr;
  o.dtype = v.dtype;
  o.device = v.device_id;
  for (int i = 0; i < 4; ++i) {
    o.shape[i] = static_cast<long long>(v.shape[i]);
    // an empty batch (shape[0] == 0) is legal and is a no-op; every other extent must be positive
    if ((o.shape[i] <= 0 && !(i == 0 && o.shape[i] == 0)) || o.shape[i] > 0x7fffffffLL)
      TB_FAIL(TRACEA_INVALID_PARAMS, "%s: shape[%d] = %llu is out of range", name, i,
              (unsigned long long)v.shape[i]);
  }
  if (v.stride != nullptr) {
    for (int i = 0; i < 4; ++i) o.stride[i] = v.stride[i];
  } else {  // contiguous row-major, what tracea::TensorView builds (include/tracea.hpp:218-228)
    long long s = 1;
    for (int i = 3; i >= 0; --i) {
      o.stride[i] = s;
      s *= o.shape[i];
    }
  }
  for (int i = 0; i < 4; ++i)
    if (o.stride[i] < 0) TB_FAIL(TRACEA_INVALID_PARAMS, "%s: negative stride[%d]", name, i);
  return o;
}

// Number of elements from the first to the last addressed element, inclusive.
long long span_elems(const View4& v) {
  long long s = 1;
  for (int i = 0; i < 4; ++i) s += (v.shape[i] - 1) * v.stride[i];
  return s;
}
long long num_elems(const View4& v) { return v.shape[0] * v.shape[1] * v.shape[2] * v.shape[3]; }

// Strides of extent-1 dimensions carry no information (torch reports arbitrary values for them);
// when the channel axis is innermost, rewrite them to the dense channels-last values so that the
// layout tests below and the TMA stride rules see a consistent picture.
void canon_channels_last(View4& v) {
  if (v.shape[1] != 1 && v.stride[1] != 1) return;
  if (v.shape[1] == 1) v.stride[1] = 1;
  if (v.shape[3] == 1) v.stride[3] = v.shape[1];
  if (v.shape[2] == 1) v.stride[2] = v.shape[3] * v.stride[3];
  if (v.shape[0] == 1) v.stride[0] = v.shape[2] * v.stride[2];
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------ epilogue decoding
struct Epilogue {
  bool bias = false;
  bool residual = false;
  int act = tb200::kActNone;
};

// Kind -> op list, after src/interface/c_bindings.rs:144-197.
Epilogue decode_epilogue(TraceaEpilogueKind kind, bool have_bias, bool have_res) {
  Epilogue e;
  switch (kind) {
    case TRACEA_EPILOGUE_IDENTITY: break;
    case TRACEA_EPILOGUE_BIAS_ADD: e.bias = have_bias; break;
    case TRACEA_EPILOGUE_RELU: e.act = tb200::kActRelu; break;
    case TRACEA_EPILOGUE_GELU: e.act = tb200::kActGelu; break;
    case TRACEA_EPILOGUE_SILU: e.act = tb200::kActSilu; break;
    case TRACEA_EPILOGUE_BIAS_RELU: e.bias = have_bias; e.act = tb200::kActRelu; break;
    case TRACEA_EPILOGUE_BIAS_SILU:
      // the reference emits the fused BiasAddSiLU functor only when a bias is present
      e.bias = have_bias;
      e.act = have_bias ? tb200::kActSilu : tb200::kActNone;
      break;
    case TRACEA_EPILOGUE_RESIDUAL: e.residual = have_res; break;
    case TRACEA_EPILOGUE_RESIDUAL_RELU: e.residual = have_res; e.act = tb200::kActRelu; break;
    case TRACEA_EPILOGUE_BIAS_RESIDUAL_RELU:
      e.bias = have_bias; e.residual = have_res; e.act = tb200::kActRelu; break;
    case TRACEA_EPILOGUE_BIAS_RESIDUAL: e.bias = have_bias; e.residual = have_res; break;
    default:
      TB_FAIL(TRACEA_INVALID_PARAMS, "unknown epilogue kind %d", static_cast<int>(kind));
  }
  return e;
}

// ------------------------------------------------------------------ environment knobs
int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v != nullptr && *v != '\0') ? atoi(v) : dflt;
}

// Bring-up / test knobs, read from the environment once per process (a getenv per knob per call is a measurable
// part of the ~6 us a call costs on the host). TRACEA_B200_HOST_CHUNKS is read per call and is not in here.
struct Knobs {
  int force_bn, force_stages, force_chunk, no_tma_store, no_tma_residual, tiled_a, force_staging, no_window,
      pair, rows2, panel, pdl, split_k, no_window3, no_row_band;
};
const Knobs& knobs() {
  static const Knobs k = {
      env_int("TRACEA_B200_FORCE_BN", 0),      env_int("TRACEA_B200_FORCE_STAGES", 0),
      env_int("TRACEA_B200_FORCE_CHUNK", 0),   env_int("TRACEA_B200_NO_TMA_STORE", 0),
      env_int("TRACEA_B200_NO_TMA_RESIDUAL", 0), env_int("TRACEA_B200_TILED_A", 0),
      env_int("TRACEA_B200_FORCE_STAGING", 0), env_int("TRACEA_B200_NO_WINDOW", 0),
      env_int("TRACEA_B200_PAIR", -1),         env_int("TRACEA_B200_ROWS2", -1),
      env_int("TRACEA_B200_PANEL", 0),         env_int("TRACEA_B200_PDL", 1),
      env_int("TRACEA_B200_SPLIT_K", 0),       env_int("TRACEA_B200_NO_RESIDENT_FILTER", 0),
      env_int("TRACEA_B200_NO_ROW_BAND", 0)};
  return k;
}

// ------------------------------------------------------------------ tile selection
// Relative cost of one 128-byte k-step of a 128-row x BN tile on one SM, measured on the ResNet-50 layers rather
// than derived: the tensor pipe alone would give 512 / 256 / 192 cycles (BN/2 per MMA, 48 at BN = 64 where the
// shared-memory operand reads bind), but the narrower tiles pull (128 + BN) * 128 bytes per step through L2 -> SM
// paths that deliver ~70 B/cycle/SM when every SM loads, so a BN = 128 step costs ~400 and a BN = 64 step ~300.
// The widest tile wins ties: it re-reads A least.
int pick_bn(long long m_tiles, int k_out, int num_sms) {
  const int bns[3] = {256, 128, 64};
  const int step_cost[3] = {512, 400, 300};
  long long best_cost = -1;
  int best = 64;
  for (int i = 0; i < 3; ++i) {
    const long long n_tiles = (k_out + bns[i] - 1) / bns[i];
    const long long waves = (m_tiles * n_tiles + num_sms - 1) / num_sms;
    const long long cost = waves * step_cost[i];
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bns[i];
    }
  }
  return best;
}

int pick_stages(int bn, bool pair, bool rows2, bool shared_bias) {
  const int stage_bytes = tb200::conv_smem_bytes(bn, 1, pair, rows2) - tb200::conv_smem_bytes(bn, 0, pair, rows2);
  const int fixed = tb200::conv_smem_bytes(bn, 0, pair, rows2, shared_bias);
  int s = (232448 - fixed) / stage_bytes;  // 227 KB opt-in limit per CTA
  return std::min(s, tb200::kMaxStages);
}

template <typename OutT, int BN, bool kPair, bool kRows2, bool kCoop, bool kSplit>
void launch_one_variant(DeviceState& st, int dt_idx, int bn_idx, const CUtensorMap& tx, const CUtensorMap& tw,
                const CUtensorMap& to, const CUtensorMap& tr, const ConvKernelArgs& args, int grid, int smem,
                cudaStream_t stream) {
  auto kern = tb200::conv2d_igemm_sm100_kernel<OutT, BN, kPair, kRows2, kCoop, kSplit>;
  constexpr int kVariant = (kPair ? 1 : (kRows2 ? 2 : 0)) + (kCoop ? 3 : (kSplit ? 6 : 0));
  std::atomic<bool>& attr_done = g_attr_set[st.dev][dt_idx][bn_idx][kVariant];
  if (!attr_done.load(std::memory_order_relaxed)) {
    TB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    attr_done.store(true, std::memory_order_relaxed);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kRows2 ? tb200::kNumThreadsRows2 : tb200::kNumThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n_attr = 0;
  if constexpr (kPair) {
    // clusters of two CTAs on neighbouring SMs; no multicast load is used anywhere in the kernel
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (knobs().pdl != 0) {
    // programmatic dependent launch: this kernel's prologue (barrier init, TMEM allocation, descriptor prefetch)
    // may run while the previous kernel on the stream drains; the kernel waits for it before touching global memory
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  TB_CUDA(cudaLaunchKernelEx(&cfg, kern, tx, tw, to, tr, args));
  TB_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  g_launches_by_kind[kSplit ? 1 : 0].fetch_add(1, std::memory_order_relaxed);
}

// The K-split kernels exist for the TMA-store / per-lane epilogues only (the host never splits a coop launch).
template <typename OutT, int BN, bool kPair, bool kRows2, bool kCoop>
void launch_one(DeviceState& st, int dt_idx, int bn_idx, const CUtensorMap& tx, const CUtensorMap& tw,
                const CUtensorMap& to, const CUtensorMap& tr, const ConvKernelArgs& args, int grid, int smem,
                cudaStream_t stream) {
  if constexpr (!kCoop) {
    if (args.sk_tiles > 0) {
      launch_one_variant<OutT, BN, kPair, kRows2, false, true>(st, dt_idx, bn_idx, tx, tw, to, tr, args, grid, smem, stream);
      return;
    }
  }
  launch_one_variant<OutT, BN, kPair, kRows2, kCoop, false>(st, dt_idx, bn_idx, tx, tw, to, tr, args, grid, smem, stream);
}

// `coop`: the kernel variant whose epilogue moves its staging boxes to a strided, channel-contiguous output itself.
template <typename OutT, bool kCoop>
void launch_tiling(DeviceState& st, int dt_idx, int bn, bool pair, bool rows2, const CUtensorMap& tx,
                   const CUtensorMap& tw, const CUtensorMap& to, const CUtensorMap& tr, const ConvKernelArgs& args,
                   int grid, int smem, cudaStream_t stream) {
  if (rows2) {
    if (bn == 64) launch_one<OutT, 64, false, true, kCoop>(st, dt_idx, 0, tx, tw, to, tr, args, grid, smem, stream);
    else launch_one<OutT, 128, false, true, kCoop>(st, dt_idx, 1, tx, tw, to, tr, args, grid, smem, stream);
    return;
  }
  if (pair) {
    if (bn == 128) launch_one<OutT, 128, true, false, kCoop>(st, dt_idx, 1, tx, tw, to, tr, args, grid, smem, stream);
    else launch_one<OutT, 256, true, false, kCoop>(st, dt_idx, 2, tx, tw, to, tr, args, grid, smem, stream);
    return;
  }
  switch (bn) {
    case 64: launch_one<OutT, 64, false, false, kCoop>(st, dt_idx, 0, tx, tw, to, tr, args, grid, smem, stream); break;
    case 128: launch_one<OutT, 128, false, false, kCoop>(st, dt_idx, 1, tx, tw, to, tr, args, grid, smem, stream); break;
    default: launch_one<OutT, 256, false, false, kCoop>(st, dt_idx, 2, tx, tw, to, tr, args, grid, smem, stream); break;
  }
}

template <typename OutT>
void launch_bn(DeviceState& st, int dt_idx, int bn, bool pair, bool rows2, bool coop, const CUtensorMap& tx,
               const CUtensorMap& tw, const CUtensorMap& to, const CUtensorMap& tr, const ConvKernelArgs& args, int grid,
               int smem, cudaStream_t stream) {
  if (coop) launch_tiling<OutT, true>(st, dt_idx, bn, pair, rows2, tx, tw, to, tr, args, grid, smem, stream);
  else launch_tiling<OutT, false>(st, dt_idx, bn, pair, rows2, tx, tw, to, tr, args, grid, smem, stream);
}

CUtensorMapDataType tmap_dtype(TraceaDType t) {
  switch (t) {
    case TRACEA_DTYPE_FLOAT16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case TRACEA_DTYPE_BFLOAT16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  }
}

CUtensorMapSwizzle tmap_swizzle(int chunk_bytes) {
  switch (chunk_bytes) {
    case 128: return CU_TENSOR_MAP_SWIZZLE_128B;
    case 64: return CU_TENSOR_MAP_SWIZZLE_64B;
    case 32: return CU_TENSOR_MAP_SWIZZLE_32B;
    default: return CU_TENSOR_MAP_SWIZZLE_NONE;
  }
}

// ------------------------------------------------------------------ static scratch (no-alloc entry)
// Staging memory for tracea_conv2d_noalloc: a fixed array inside the library's device image, so
// that entry point never has to ask the CUDA allocator for anything. Every GPU that loads the
// library carries these bytes until the process exits. The symbol below is only a host-side
// handle; the device address kernels must be given comes from cudaGetSymbolAddress (noalloc_state).
constexpr size_t kStaticScratchBytes = 16u << 20;   // 16 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
// Error words of the kernels tracea_conv2d_noalloc launches ({code, block, detail, 0}, first error wins). The
// allocating path keeps its words in pinned host memory; this path may not allocate, so its words live in the
// device image as well and tracea_b200_device_status copies them back on request.
static __device__ __align__(16) uint32_t g_noalloc_status[4];

// Bump allocator over the static array for the duration of one call.
struct StaticArena {
  unsigned char* base = nullptr;
  size_t capacity = 0;
  size_t used = 0;
  void* take(size_t bytes, const char* what) {
    const size_t start = (used + 255u) & ~static_cast<size_t>(255u);
    if (start + bytes > capacity)
      TB_FAIL(TRACEA_UNSUPPORTED_CONFIG,
              "tracea_conv2d_noalloc: staging %s needs %zu bytes on top of %zu already in use, but the "
              "built-in scratch holds %zu bytes; use tracea_conv2d or pass channels-last tensors",
              what, bytes, start, capacity);
    used = start + bytes;
    return base + start;
  }
};

struct NoAllocState {
  std::atomic<bool> ready{false};
  int num_sms = 0;
  unsigned char* scratch = nullptr;   // device address of g_static_scratch on this device
  uint32_t* status = nullptr;         // device address of g_noalloc_status on this device
};
NoAllocState g_noalloc[kMaxDevices];

// First call on a device (with that device current): queries the SM count, resolves the driver entry
// points and the device addresses of the static scratch and of the status words. Nothing here allocates.
NoAllocState& noalloc_state(int dev) {
  if (dev < 0 || dev >= kMaxDevices) TB_FAIL(TRACEA_INVALID_PARAMS, "device_id %d out of range", dev);
  NoAllocState& na = g_noalloc[dev];
  if (na.ready.load(std::memory_order_acquire)) return na;
  std::lock_guard<std::mutex> lock(g_dev_mu[dev]);
  if (na.ready.load(std::memory_order_relaxed)) return na;
  int major = 0, sms = 0;
  TB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "device %d is not sm_100; this library only carries sm_100a kernels", dev);
  TB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  load_driver_entry_points();
  void* addr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&addr, g_static_scratch);
  if (e != cudaSuccess || addr == nullptr)
    TB_FAIL(TRACEA_CUDA_ERROR, "cudaGetSymbolAddress(g_static_scratch) failed on device %d: %s", dev,
            cudaGetErrorString(e));
  void* status_addr = nullptr;
  const cudaError_t e2 = cudaGetSymbolAddress(&status_addr, g_noalloc_status);
  if (e2 != cudaSuccess || status_addr == nullptr)
    TB_FAIL(TRACEA_CUDA_ERROR, "cudaGetSymbolAddress(g_noalloc_status) failed on device %d: %s", dev,
            cudaGetErrorString(e2));
  na.num_sms = sms;
  na.scratch = static_cast<unsigned char*>(addr);
  na.status = static_cast<uint32_t*>(status_addr);   // zero-initialised with the device image
  na.ready.store(true, std::memory_order_release);
  return na;
}

// ------------------------------------------------------------------ weight packing
// w[k, c, r, s] through element strides -> dst[k][r][Sd][Cp] (channels >= C and tap slots >= S zero-filled).
void launch_weight_pack(const void* src, void* dst, int es, long long K, long long C, long long R, long long S,
                        long long Sd, long long Cp, const long long stride[4], cudaStream_t stream) {
  const long long total = K * R * Sd * Cp;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  if (R == 1 && Sd == 1 && (Cp + 31) / 32 <= 65535) {
    // a 1x1 filter is a [K][C] matrix: the tiled transpose keeps both sides coalesced when w arrives C-major
    // (a row-major GEMM B operand)
    dim3 grid(static_cast<unsigned>((K + 31) / 32), static_cast<unsigned>((Cp + 31) / 32), 1u);
    dim3 block(32, 8);
    if (es == 2)
      tb200::to_channels_last_kernel<uint16_t><<<grid, block, 0, stream>>>(
          static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), (int)C, 1, (int)K, (int)Cp, 0LL, stride[1], 0LL,
          stride[0]);
    else
      tb200::to_channels_last_kernel<uint32_t><<<grid, block, 0, stream>>>(
          static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), (int)C, 1, (int)K, (int)Cp, 0LL, stride[1], 0LL,
          stride[0]);
  } else if (es == 2) {
    tb200::pack_weights_krsc_kernel<uint16_t><<<blocks, threads, 0, stream>>>(
        static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), total, (int)C, (int)R, (int)S, (int)Sd, (int)Cp,
        stride[0], stride[1], stride[2], stride[3]);
  } else {
    tb200::pack_weights_krsc_kernel<uint32_t><<<blocks, threads, 0, stream>>>(
        static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), total, (int)C, (int)R, (int)S, (int)Sd, (int)Cp,
        stride[0], stride[1], stride[2], stride[3]);
  }
  TB_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  g_launches_by_kind[3].fetch_add(1, std::memory_order_relaxed);
}


// ------------------------------------------------------------------ the device path
// The conv geometry the kernel runs: the public parameters plus a separate padding behind the last row /
// column. padding_h / padding_w pad in front; the output extents are out.shape[2], out.shape[3] and must equal
// (H + padding_h + pad_h_hi - dilation_h*(R-1) - 1) / stride_h + 1 (same for w). tracea_conv2d always pads
// symmetrically; the phases of a transposed convolution do not.
struct CoreParams : TraceaConv2dParams {
  long long pad_h_hi = 0, pad_w_hi = 0;
  // Set by callers that issue several launches which do not depend on each other (the phases of a transposed
  // convolution): *chain is 0 until one of them has been launched as the head of a chain (see ConvKernelArgs::pdl_mode).
  int* chain = nullptr;
  CoreParams() : TraceaConv2dParams() {}
  CoreParams(const TraceaConv2dParams& p) : TraceaConv2dParams(p), pad_h_hi(p.padding_h), pad_w_hi(p.padding_w) {}
};

// All pointers are device pointers on `dev`. x: [N,C,H,W], w: [K,C,R,S], out: [N,K,Ho,Wo] (logical).
// ------------------------------------------------------------------ row-band kernel (few-channel images, e.g. the RGB stem)
// Tries the kernel of conv2d_rowband_sm100.cuh: 16-bit images of up to 8 channels whose horizontal step is 16 bytes
// of (channel-padded) input -- 4-channel pixels under stride_w 2, 8-channel pixels under stride_w 1. Stages the
// padded channels-last copy of x and the packed filter bank itself (`staging` hands out the scratch), then launches.
// Returns false (nothing launched, nothing staged) when the layer does not qualify.
std::atomic<bool> g_rowband_attr_set[kMaxDevices][2];

template <typename Staging>
bool try_row_band_conv(DeviceState& st, Staging&& staging, const View4& x, const View4& w, const View4* bias,
                       const View4& out, const CoreParams& p, const Epilogue& epi, cudaStream_t stream) {
  const long long N = x.shape[0], C = x.shape[1], H = x.shape[2], W = x.shape[3];
  const long long K = w.shape[0], R = w.shape[2], S = w.shape[3];
  const long long Ho = out.shape[2], Wo = out.shape[3];
  if (knobs().no_row_band != 0 || st.status == nullptr) return false;
  if (x.dtype == TRACEA_DTYPE_FLOAT32 || C > 8 || K > 64 || (K % 8) != 0 || epi.residual) return false;
  const long long Cw = C <= 4 ? 4 : 8;                     // channels per pixel of the padded copy
  const long long px_bytes = Cw * 2;
  if ((long long)p.stride_w * px_bytes != 16 || p.dilation_w != 1 || S < 2) return false;
  const long long kmma = (S * px_bytes + 31) / 32;         // K = 16 MMAs per filter row
  if (kmma > 4 || R > 16 || p.dilation_h > 8) return false;
  const bool ovec = out.stride[1] == 1 && aligned16(out.ptr) && (out.stride[0] * 2) % 16 == 0 &&
                    (out.stride[2] * 2) % 16 == 0 && (out.stride[3] * 2) % 16 == 0;
  if (!ovec || N > 0x3fffffffLL / (Ho + 1)) return false;
  // row pitch: the padded row, and at least what the last output pixel's taps (zero-weight ones included) read
  const long long px_per_128 = 128 / px_bytes;
  const long long need_px = std::max<long long>(W + p.padding_w + p.pad_w_hi, (Wo - 1) * p.stride_w + kmma * 32 / px_bytes);
  const long long Wpitch = (need_px + px_per_128 - 1) / px_per_128 * px_per_128;
  const long long row_bytes = Wpitch * px_bytes;
  if (row_bytes / 128 > 256 || Wo < 32) return false;
  const long long wtiles = (Wo + 127) / 128;
  if (Wo * 100 < wtiles * 128 * 60) return false;          // mostly dropped rows: the general kernel packs pixels densely
  const uint32_t w_bytes = static_cast<uint32_t>(R * kmma) * 2048u;

  // band height: the cheapest of 16, 8, 4, 2, 1 output rows by a simple cycle model (MMA time + copy time, times
  // the bands the busiest CTA gets); at least two slots must fit
  long long hb = 0, best_cost = 0, in_rows = 0, slot_bytes = 0, num_slots = 0;
  for (long long h = 16; h >= 1; h >>= 1) {
    if (h > Ho && h > 1) continue;
    const long long rows_in = (h - 1) * p.stride_h + (R - 1) * p.dilation_h + 1;
    if (rows_in > 256) continue;
    const long long slot = (rows_in * row_bytes + 2048 + 128 + 1023) / 1024 * 1024;
    const long long fixed = tb200::rowband_smem_bytes(w_bytes, 0, 0);
    const long long slots = std::min<long long>(tb200::kBandMaxSlots, (232448 - fixed) / slot);
    if (slots < 2) continue;
    const long long bands = N * ((Ho + h - 1) / h);
    const long long ctas = std::min<long long>(bands, st.num_sms);
    const long long per_cta = (bands + ctas - 1) / ctas;
    const long long cost = per_cta * (h * wtiles * R * kmma * 55 + rows_in * row_bytes / 32);
    if (hb == 0 || cost < best_cost) {
      hb = h; best_cost = cost; in_rows = rows_in; slot_bytes = slot; num_slots = slots;
    }
  }
  if (hb == 0) return false;
  const long long bands_per_img = (Ho + hb - 1) / hb, n_bands = N * bands_per_img;
  if (n_bands > 0x3fffffffLL) return false;

  // ---- staging: the padded channels-last copy of x, the packed filter bank
  Scratch x_scratch, w_scratch;
  const long long pixels = N * H * Wpitch;
  void* x_stage = staging(x_scratch, static_cast<size_t>(pixels * px_bytes), "the padded channels-last copy of x");
  {
    const int threads = 256;
    const unsigned blocks = static_cast<unsigned>((pixels + threads - 1) / threads);
    const bool dense_rgb = C == 3 && x.stride[1] == 1 && x.stride[3] == 3 && (W % 4) == 0 && (x.stride[2] % 4) == 0 &&
                           (x.stride[0] % 4) == 0 && (reinterpret_cast<uintptr_t>(x.ptr) % 8) == 0 &&
                           N * H <= 0x7fffffffLL;
    if (dense_rgb)
      tb200::rgb16_rows_to_padded4_kernel<<<static_cast<unsigned>(N * H), 64, 0, stream>>>(
          static_cast<const uint16_t*>(x.ptr), static_cast<uint16_t*>(x_stage), (int)H, (int)W, (int)Wpitch,
          (int)p.padding_w, x.stride[0], x.stride[2]);
    else if (Cw == 4)
      tb200::to_channels_last_wpad_kernel<uint16_t, 4><<<blocks, threads, 0, stream>>>(
          static_cast<const uint16_t*>(x.ptr), static_cast<uint16_t*>(x_stage), (int)C, (int)H, (int)W, (int)Wpitch,
          (int)p.padding_w, pixels, x.stride[0], x.stride[1], x.stride[2], x.stride[3]);
    else
      tb200::to_channels_last_wpad_kernel<uint16_t, 8><<<blocks, threads, 0, stream>>>(
          static_cast<const uint16_t*>(x.ptr), static_cast<uint16_t*>(x_stage), (int)C, (int)H, (int)W, (int)Wpitch,
          (int)p.padding_w, pixels, x.stride[0], x.stride[1], x.stride[2], x.stride[3]);
    TB_CUDA(cudaGetLastError());
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    g_launches_by_kind[3].fetch_add(1, std::memory_order_relaxed);
  }
  const long long Sd = kmma * 32 / px_bytes;               // tap slots per filter row in the packed bank
  void* w_stage = staging(w_scratch, static_cast<size_t>(K * R * Sd * px_bytes), "the packed filter bank");
  launch_weight_pack(w.ptr, w_stage, 2, K, C, R, S, Sd, Cw, w.stride, stream);

  CUtensorMap tmap_x;
  {
    const cuuint64_t gdim[4] = {64, (cuuint64_t)(row_bytes / 128), (cuuint64_t)H, (cuuint64_t)N};
    const cuuint64_t gstr[3] = {128, (cuuint64_t)row_bytes, (cuuint64_t)(H * row_bytes)};
    const cuuint32_t box[4] = {64u, (cuuint32_t)(row_bytes / 128), (cuuint32_t)in_rows, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = g_encode_tiled(&tmap_x, tmap_dtype(x.dtype), 4, x_stage, gdim, gstr, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TB_FAIL(TRACEA_CUDA_ERROR, "cuTensorMapEncodeTiled (row band) failed with %d", (int)r);
  }
  CUtensorMap tmap_out;
  {
    // the output as {channel, column, row, image}; a warp stores 32 pixels x 64 channels, clipped at Wo and K_out
    const cuuint64_t gdim[4] = {(cuuint64_t)K, (cuuint64_t)Wo, (cuuint64_t)Ho, (cuuint64_t)N};
    const cuuint64_t gstr[3] = {(cuuint64_t)(out.stride[3] * 2), (cuuint64_t)(out.stride[2] * 2),
                                (cuuint64_t)(out.stride[0] * 2)};
    const cuuint32_t box[4] = {64u, 32u, 1u, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = g_encode_tiled(&tmap_out, tmap_dtype(out.dtype), 4, out.ptr, gdim, gstr, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TB_FAIL(TRACEA_CUDA_ERROR, "cuTensorMapEncodeTiled (row band output) failed with %d", (int)r);
  }

  tb200::RowBandKernelArgs a;
  memset(&a, 0, sizeof(a));
  a.R = (int)R; a.stride_h = (int)p.stride_h; a.pad_h = (int)p.padding_h; a.dil_h = (int)p.dilation_h;
  a.Ho = (int)Ho; a.Wo = (int)Wo;
  a.hb = (int)hb; a.bands_per_img = (int)bands_per_img; a.n_bands = (int)n_bands;
  a.wtiles = (int)wtiles; a.kmma = (int)kmma; a.num_slots = (int)num_slots;
  a.row_bytes = static_cast<uint32_t>(row_bytes);
  a.box_bytes = static_cast<uint32_t>(in_rows * row_bytes);
  a.slot_bytes = static_cast<uint32_t>(slot_bytes);
  a.w_bytes = w_bytes;
  a.idesc = tb200::ptx::make_idesc(x.dtype == TRACEA_DTYPE_FLOAT16 ? 0u : 1u, 128, tb200::kBandBN);
  a.w = w_stage;
  a.K_out = (int)K;
  if (epi.bias && bias != nullptr) {
    a.bias = bias->ptr;
    a.bias_is_f32 = bias->dtype == TRACEA_DTYPE_FLOAT32 ? 1 : 0;
  }
  a.act = epi.act;
  a.status = st.status;
  {
    const long long lim = g_test_wait_limit.load(std::memory_order_relaxed);
    a.wait_limit = lim > 0 ? lim : tb200::kWaitLimitCycles;
    a.test_producer_stop = g_test_producer_stop.load(std::memory_order_relaxed);
  }

#ifdef TB200_PROFILE
  {
    const char* pp = getenv("TRACEA_B200_PROF_PTR");
    a.prof = pp != nullptr ? reinterpret_cast<long long*>(strtoull(pp, nullptr, 0)) : nullptr;
  }
#endif
  const int smem = static_cast<int>(tb200::rowband_smem_bytes(w_bytes, a.slot_bytes, a.num_slots));
  const int grid = static_cast<int>(std::min<long long>(n_bands, st.num_sms));
  const bool bf16 = x.dtype == TRACEA_DTYPE_BFLOAT16;
  auto kern_bf = tb200::conv2d_rowband_sm100_kernel<__nv_bfloat16>;
  auto kern_h = tb200::conv2d_rowband_sm100_kernel<__half>;
  std::atomic<bool>& attr_done = g_rowband_attr_set[st.dev][bf16 ? 0 : 1];
  if (!attr_done.load(std::memory_order_relaxed)) {
    if (bf16) TB_CUDA(cudaFuncSetAttribute(kern_bf, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    else TB_CUDA(cudaFuncSetAttribute(kern_h, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    attr_done.store(true, std::memory_order_relaxed);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(tb200::kBandThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  unsigned n_attr = 0;
  if (knobs().pdl != 0) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  if (bf16) TB_CUDA(cudaLaunchKernelEx(&cfg, kern_bf, tmap_x, tmap_out, a));
  else TB_CUDA(cudaLaunchKernelEx(&cfg, kern_h, tmap_x, tmap_out, a));
  TB_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  g_launches_by_kind[4].fetch_add(1, std::memory_order_relaxed);
  return true;
}

void conv2d_core(DeviceState& st, StaticArena* arena, const View4& x_in, const View4& w_in, const View4* bias,
                 const View4* residual, const View4& out, const CoreParams& p, const Epilogue& epi);

void conv2d_device(int dev, const View4& x_in, const View4& w_in, const View4* bias,
                   const View4* residual, const View4& out, const CoreParams& p,
                   const Epilogue& epi) {
  DeviceGuard guard(dev);
  DeviceState& st = device_state(dev);

  if (st.status[0] != 0u) {
    const uint32_t code = st.status[0], blk = st.status[1], det = st.status[2];
    memset(st.status, 0, 4 * sizeof(uint32_t));
    cudaDeviceSynchronize();
    reset_split_workspaces(st);
    TB_FAIL(TRACEA_CUDA_ERROR,
            "an earlier conv kernel on device %d gave up a bounded wait (code %u, block %u, detail %u)",
            dev, code, blk, det);
  }
  conv2d_core(st, nullptr, x_in, w_in, bias, residual, out, p, epi);
}

// Same device path with every staging buffer carved out of the library's static scratch: no call
// below this point allocates or frees device or pinned memory.
void conv2d_device_noalloc(int dev, const View4& x_in, const View4& w_in, const View4* bias,
                           const View4* residual, const View4& out, const CoreParams& p,
                           const Epilogue& epi) {
  DeviceGuard guard(dev);
  NoAllocState& na = noalloc_state(dev);
  DeviceState st;                       // a view for conv2d_core, not a registered device state
  st.dev = dev;
  st.num_sms = na.num_sms;
  // Device-resident status words: reading them back means waiting for the GPU, so this entry does not look at
  // them on the way in (tracea_conv2d does, its words are in host memory); tracea_b200_device_status reports them.
  st.status = na.status;
  StaticArena arena;
  arena.base = na.scratch;
  arena.capacity = kStaticScratchBytes;
  conv2d_core(st, &arena, x_in, w_in, bias, residual, out, p, epi);
}

// ------------------------------------------------------------------ resident-filter kernel (stride-1 small filters, C = 64)
// Tries the kernel of conv2d_window_sm100.cuh: filter bank resident in shared memory, one halo'd window copy per
// tile, filter taps as shifted descriptors over the window. `x` is channels-last with 64 channels, `w_ptr` dense
// [K][R][S][64]. Returns false (nothing launched) when the layer does not qualify.
std::atomic<bool> g_window_attr_set[kMaxDevices][2];

bool try_resident_filter_conv(DeviceState& st, const View4& x, const void* w_ptr, const View4* bias, const View4& out,
                              const CoreParams& p, const Epilogue& epi, long long K, long long R, long long S,
                              bool out_vec, cudaStream_t stream) {
  const long long N = x.shape[0], H = x.shape[2], W = x.shape[3];
  const long long Ho = out.shape[2], Wo = out.shape[3];
  if (knobs().no_window3 != 0 || x.dtype == TRACEA_DTYPE_FLOAT32 || x.shape[1] != 64 || K > 64 || (K % 8) != 0) return false;
  if (p.stride_h != 1 || p.stride_w != 1 || p.dilation_h != 1 || p.dilation_w != 1) return false;
  if (R > 3 || S > 3 || R * S < 4 || !out_vec || (epi.residual)) return false;
  if (p.pad_w_hi > (long long)p.padding_w || W + p.padding_w > 256 || N > 0x3fffffffLL / (Ho + 1)) return false;
  const long long Wp = W + p.padding_w, dummy = Wp - Wo;
  if (dummy < 0) return false;
  const uint32_t w_bytes = static_cast<uint32_t>(R * S) * 4096u;
  long long ht = 0, nblk = 0, slot_bytes = 0, box_rows = 0;
  for (long long nb = tb200::kWinMaxBlocks; nb >= 1; --nb) {
    long long h = std::min<long long>((128 * nb + dummy) / Wp, Ho);
    if (h < 1 || h + R - 1 > 256) continue;
    const long long rows = (h + R - 1) * Wp;                            // what a window copy fills
    const long long reach = 128 * nb + (R - 1) * Wp + (S - 1);         // what the MMAs of nb blocks read
    const long long slot = (std::max(rows + p.pad_w_hi, reach) * 128 + 1023) / 1024 * 1024;
    if (tb200::window_smem_bytes(w_bytes, static_cast<uint32_t>(slot)) > 232448u) continue;
    ht = h; nblk = nb; slot_bytes = slot; box_rows = rows;
    break;
  }
  if (ht == 0) return false;
  const long long nblk_full = (ht * Wp - dummy + 127) / 128;
  const long long tiles_per_img = Ho / ht, ht_short = Ho % ht;
  const long long nblk_short = ht_short > 0 ? (ht_short * Wp - dummy + 127) / 128 : 0;
  // worth it only when the 128-row MMA blocks are mostly real pixels and the launch fills the GPU at least once
  const long long blocks_per_img = tiles_per_img * nblk_full + nblk_short;
  if (Ho * Wo * 100 < blocks_per_img * 128 * 85) return false;
  const long long n_full = N * tiles_per_img, n_short = ht_short > 0 ? N : 0;
  const long long pair_full = (n_full + 1) / 2, pair_tiles = pair_full + (n_short + 1) / 2;
  if (pair_tiles < st.num_sms / 2 || pair_tiles > 0x3fffffffLL) return false;
  (void)nblk;

  auto encode_x = [&](CUtensorMap* m, long long box_h) {
    const int es = 2;
    const cuuint64_t gdim[4] = {64, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    const cuuint64_t gstr[3] = {(cuuint64_t)(x.stride[3] * es), (cuuint64_t)(x.stride[2] * es),
                                (cuuint64_t)(x.stride[0] * es)};
    const cuuint32_t box[4] = {64u, (cuuint32_t)Wp, (cuuint32_t)box_h, 1u};
    const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = g_encode_tiled(m, tmap_dtype(x.dtype), 4, x.ptr, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TB_FAIL(TRACEA_CUDA_ERROR, "cuTensorMapEncodeTiled (window) failed with %d", (int)r);
  };
  CUtensorMap tmap_full, tmap_short, tmap_w;
  encode_x(&tmap_full, ht + R - 1);
  // a short tile's copy takes one row more than it needs: the right-hand padding of its last row reads there
  // (below a full tile's copy the slot is kept zero instead)
  encode_x(&tmap_short, ht_short > 0 ? ht_short + R : ht + R - 1);
  {
    const cuuint64_t gdim[2] = {(cuuint64_t)(R * S * 64), (cuuint64_t)K};
    const cuuint64_t gstr[1] = {(cuuint64_t)(R * S * 64 * 2)};
    const cuuint32_t box[2] = {64u, 32u};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult r = g_encode_tiled(&tmap_w, tmap_dtype(x.dtype), 2, const_cast<void*>(w_ptr), gdim, gstr, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TB_FAIL(TRACEA_CUDA_ERROR, "cuTensorMapEncodeTiled (filter bank) failed with %d", (int)r);
  }

  tb200::WindowKernelArgs a;
  memset(&a, 0, sizeof(a));
  a.R = (int)R; a.S = (int)S; a.pad_h = (int)p.padding_h; a.pad_w = (int)p.padding_w;
  a.Wp = (int)Wp; a.Ho = (int)Ho; a.Wo = (int)Wo;
  a.ht_full = (int)ht; a.nblk_full = (int)nblk_full; a.ht_short = (int)ht_short; a.nblk_short = (int)nblk_short;
  a.tiles_per_img = (int)tiles_per_img; a.n_full = (int)n_full; a.n_short = (int)n_short;
  a.pair_tiles_full = (int)pair_full; a.pair_tiles = (int)pair_tiles;
  a.box_bytes_full = static_cast<uint32_t>(box_rows * 128);
  a.box_bytes_short = static_cast<uint32_t>((ht_short > 0 ? ht_short + R : ht + R - 1) * Wp * 128);
  a.w_bytes = w_bytes;
  a.slot_bytes = static_cast<uint32_t>(slot_bytes);
  a.zero_from = a.box_bytes_full;
  a.idesc = tb200::ptx::make_idesc(x.dtype == TRACEA_DTYPE_FLOAT16 ? 0u : 1u, 256, tb200::kWinBN);
  a.K_out = (int)K;
  a.out = out.ptr;
  a.out_sn = out.stride[0]; a.out_sh = out.stride[2]; a.out_sw = out.stride[3];
  if (epi.bias && bias != nullptr) {
    a.bias = bias->ptr;
    a.bias_is_f32 = bias->dtype == TRACEA_DTYPE_FLOAT32 ? 1 : 0;
  }
  a.act = epi.act;
  a.status = st.status;
  {
    const long long lim = g_test_wait_limit.load(std::memory_order_relaxed);
    a.wait_limit = lim > 0 ? lim : tb200::kWaitLimitCycles;
    a.test_producer_stop = g_test_producer_stop.load(std::memory_order_relaxed);
  }
#ifdef TB200_PROFILE
  {
    const char* pp = getenv("TRACEA_B200_PROF_PTR");
    a.prof = pp != nullptr ? reinterpret_cast<long long*>(strtoull(pp, nullptr, 0)) : nullptr;
  }
#endif

  const int smem = static_cast<int>(tb200::window_smem_bytes(w_bytes, a.slot_bytes));
  const int grid = 2 * static_cast<int>(std::min<long long>(pair_tiles, st.num_sms / 2));
  const bool bf16 = x.dtype == TRACEA_DTYPE_BFLOAT16;
  auto kern_bf = tb200::conv2d_window_sm100_kernel<__nv_bfloat16>;
  auto kern_h = tb200::conv2d_window_sm100_kernel<__half>;
  std::atomic<bool>& attr_done = g_window_attr_set[st.dev][bf16 ? 0 : 1];
  if (!attr_done.load(std::memory_order_relaxed)) {
    if (bf16) TB_CUDA(cudaFuncSetAttribute(kern_bf, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    else TB_CUDA(cudaFuncSetAttribute(kern_h, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    attr_done.store(true, std::memory_order_relaxed);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(tb200::kWinThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n_attr = 0;
  attr[n_attr].id = cudaLaunchAttributeClusterDimension;   // CTA pairs; no multicast load anywhere in the kernel
  attr[n_attr].val.clusterDim.x = 2;
  attr[n_attr].val.clusterDim.y = 1;
  attr[n_attr].val.clusterDim.z = 1;
  ++n_attr;
  if (knobs().pdl != 0) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  if (bf16) TB_CUDA(cudaLaunchKernelEx(&cfg, kern_bf, tmap_full, tmap_short, tmap_w, a));
  else TB_CUDA(cudaLaunchKernelEx(&cfg, kern_h, tmap_full, tmap_short, tmap_w, a));
  TB_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  g_launches_by_kind[2].fetch_add(1, std::memory_order_relaxed);
  return true;
}

void conv2d_core(DeviceState& st, StaticArena* arena, const View4& x_in, const View4& w_in, const View4* bias,
                 const View4* residual, const View4& out, const CoreParams& p, const Epilogue& epi) {
  cudaStream_t stream = static_cast<cudaStream_t>(p.stream);
  // staging comes from the stream-ordered pool, or from the static scratch for the no-alloc entry
  bool staged = false;   // this call launches layout adapters in front of its conv kernel
  auto staging = [&](Scratch& s, size_t bytes, const char* what) -> void* {
    staged = true;
    if (arena != nullptr) return arena->take(bytes, what);
    s.alloc(st, bytes, stream);
    return s.ptr;
  };

  const int es = elem_size(x_in.dtype);
  const long long N = x_in.shape[0], C = x_in.shape[1], H = x_in.shape[2], W = x_in.shape[3];
  const long long K = w_in.shape[0], R = w_in.shape[2], S = w_in.shape[3];
  const long long Ho = out.shape[2], Wo = out.shape[3];
  const long long M = N * Ho * Wo;
  if (M > 0x7fffff00LL) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "N*Ho*Wo = %lld exceeds 2^31", M);
  if (p.stride_h > 8 || p.stride_w > 8)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "stride > 8 is not supported (TMA traversal stride limit)");
  if ((S - 1) * p.dilation_w > 255 || (R - 1) * p.dilation_h > 255)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "filter extent > 256 is not supported (TMA im2col offset limit)");
  if (p.padding_h > 32767 || p.padding_w > 32767 || p.pad_h_hi > 32767 || p.pad_w_hi > 32767 || p.pad_h_hi < 0 ||
      p.pad_w_hi < 0)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "padding > 32767 is not supported");

  const int vec_elems = 16 / es;
  const long long Cp = (C + vec_elems - 1) / vec_elems * vec_elems;

  // ---- few-channel 16-bit images with a 16-byte horizontal step: the row-band kernel reads them in place
  if (C <= 8 && es == 2 && try_row_band_conv(st, staging, x_in, w_in, bias, out, p, epi, stream)) return;

  // ---- small-channel inputs (a pixel is 16 bytes after channel padding, e.g. the RGB stem): copy x with the
  // horizontal padding materialised; one filter row of a pixel is then 8 adjacent pixels = one 128-byte
  // k-chunk, fetched by a single im2col copy over an overlapping view (pixel pitch 16 B, "pixel" size 128 B).
  const bool window = Cp * es == 16 && S > 1 && S <= 8 && p.dilation_w == 1 && W + 2LL * p.padding_w < (1LL << 30) &&
                      p.pad_w_hi == (long long)p.padding_w && knobs().no_window == 0;
  const long long Wpitch = W + 2LL * p.padding_w + 8;   // row pitch of the padded copy, in pixels

  // ---- activations: consume channels-last memory directly, otherwise transpose into scratch
  View4 x = x_in;
  Scratch x_scratch;
  const bool x_direct = x.stride[1] == 1 && C == Cp && aligned16(x.ptr) &&
                        (x.stride[3] * es) % 16 == 0 && (x.stride[2] * es) % 16 == 0 &&
                        (x.stride[0] * es) % 16 == 0 && x.stride[3] >= C;
  if (window) {
    const long long pixels = N * H * Wpitch;
    void* x_stage = staging(x_scratch, static_cast<size_t>(pixels * Cp) * es, "the padded channels-last copy of x");
    const int threads = 256;
    const unsigned blocks = static_cast<unsigned>((pixels + threads - 1) / threads);
    if (es == 2)
      tb200::to_channels_last_wpad_kernel<uint16_t, 8><<<blocks, threads, 0, stream>>>(
          static_cast<const uint16_t*>(x.ptr), static_cast<uint16_t*>(x_stage), (int)C, (int)H, (int)W, (int)Wpitch,
          (int)p.padding_w, pixels, x.stride[0], x.stride[1], x.stride[2], x.stride[3]);
    else
      tb200::to_channels_last_wpad_kernel<uint32_t, 4><<<blocks, threads, 0, stream>>>(
          static_cast<const uint32_t*>(x.ptr), static_cast<uint32_t*>(x_stage), (int)C, (int)H, (int)W, (int)Wpitch,
          (int)p.padding_w, pixels, x.stride[0], x.stride[1], x.stride[2], x.stride[3]);
    TB_CUDA(cudaGetLastError());
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    g_launches_by_kind[3].fetch_add(1, std::memory_order_relaxed);
    x.ptr = x_stage;
    x.stride[0] = H * Wpitch * Cp;
    x.stride[1] = 1;
    x.stride[2] = Wpitch * Cp;
    x.stride[3] = Cp;
  } else if (!x_direct || knobs().force_staging) {
    void* x_stage = staging(x_scratch, static_cast<size_t>(N * H * W * Cp) * es, "the channels-last copy of x");
    dim3 grid(static_cast<unsigned>((H * W + 31) / 32), static_cast<unsigned>((Cp + 31) / 32),
              static_cast<unsigned>(N));
    if (grid.y > 65535u || grid.z > 65535u)
      TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "layout adapter: N or C too large");
    dim3 block(32, 8);
    if (es == 2)
      tb200::to_channels_last_kernel<uint16_t><<<grid, block, 0, stream>>>(
          static_cast<const uint16_t*>(x.ptr), static_cast<uint16_t*>(x_stage), (int)C, (int)H,
          (int)W, (int)Cp, x.stride[0], x.stride[1], x.stride[2], x.stride[3]);
    else
      tb200::to_channels_last_kernel<uint32_t><<<grid, block, 0, stream>>>(
          static_cast<const uint32_t*>(x.ptr), static_cast<uint32_t*>(x_stage), (int)C, (int)H,
          (int)W, (int)Cp, x.stride[0], x.stride[1], x.stride[2], x.stride[3]);
    TB_CUDA(cudaGetLastError());
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    g_launches_by_kind[3].fetch_add(1, std::memory_order_relaxed);
    x.ptr = x_stage;
    x.stride[0] = H * W * Cp;
    x.stride[1] = 1;
    x.stride[2] = W * Cp;
    x.stride[3] = Cp;
  }

  // ---- k-chunking: the widest power-of-two row (<= 128 B) that divides one pixel's channels
  // In window mode the kernel sees a conv with one tap per filter row over "pixels" of 8 * Cp channels.
  const long long Cg = window ? 8 * Cp : Cp;      // channel extent of the kernel's view
  const long long Sg = window ? 1 : S;            // taps per filter row of the kernel's view
  const long long row_bytes = Cg * es;
  int chunk_bytes = 16;
  for (int cb = 128; cb >= 16; cb >>= 1) {
    if (row_bytes % cb == 0) {
      chunk_bytes = cb;
      break;
    }
  }
  const int forced_chunk = knobs().force_chunk;
  if (forced_chunk == 16 || forced_chunk == 32 || forced_chunk == 64 || forced_chunk == 128) {
    if (row_bytes % forced_chunk == 0) chunk_bytes = forced_chunk;
  }
  const int chunk_elems = chunk_bytes / es;
  const int chunks_per_tap = static_cast<int>(Cg / chunk_elems);
  const long long total_chunks_ll = R * Sg * chunks_per_tap;
  if (total_chunks_ll > 0x7fffffffLL / 128) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "R*S*C too large");

  // ---- weights. Read in place when every output channel's taps are channel-contiguous and lie inside its own
  // row of a [K][row] matrix: the dense [K][R][S][C] layout, and -- with 128-byte k-chunks, where the loader walks
  // Kgemm one tap-slice at a time -- any tap order reachable by strides (reversed / subsampled taps: the phase
  // filters of a transposed convolution). The loader then starts at column b_k0 and adds b_jump_s / b_jump_r to its
  // column at every tap / filter-row boundary. Anything else is repacked into scratch.
  const void* w_ptr = w_in.ptr;
  Scratch w_scratch;
  long long w_row_elems = R * S * C, w_pitch = R * S * C, b_k0 = 0, b_jump_s = 0, b_jump_r = 0;
  const bool w_dense = C == Cp && (w_in.stride[1] == 1) && w_in.stride[3] == C &&
                       w_in.stride[2] == S * C && w_in.stride[0] == R * S * C && aligned16(w_in.ptr);
  bool w_direct = w_dense, w_remap = false;
  if (!w_dense && !window && C == Cp && w_in.stride[1] == 1 && chunk_bytes == 128) {
    const long long ss = S == 1 ? C : w_in.stride[3], sr = R == 1 ? S * ss : w_in.stride[2], sk = w_in.stride[0];
    const long long lo = std::min(0LL, (R - 1) * sr) + std::min(0LL, (S - 1) * ss);
    const long long hi = std::max(0LL, (R - 1) * sr) + std::max(0LL, (S - 1) * ss) + C;
    const char* base = static_cast<const char*>(w_in.ptr) + lo * es;
    const bool taps_apart = (ss >= C || ss <= -C) && (R == 1 || sr >= C || sr <= -C);
    if (taps_apart && (K == 1 || sk >= hi - lo) && (sk * es) % 16 == 0 && (ss * es) % 16 == 0 && (sr * es) % 16 == 0 &&
        aligned16(base) && hi - lo < (1LL << 31)) {
      w_direct = w_remap = true;
      w_ptr = base;
      w_row_elems = hi - lo;
      w_pitch = K == 1 ? hi - lo : sk;
      b_k0 = -lo;
      b_jump_s = ss - C;
      b_jump_r = sr - S * ss;
    }
  }
  const long long Sd = window ? 8 : S;   // tap slots per filter row in the packed weights
  if (!w_direct || window) {
    void* w_stage = staging(w_scratch, static_cast<size_t>(K * R * Sd * Cp) * es, "the repacked weights");
    launch_weight_pack(w_in.ptr, w_stage, es, K, C, R, S, Sd, Cp, w_in.stride, stream);
    w_ptr = w_stage;
  }

  const long long Kgemm = R * Sg * Cg;

  // ---- stride-1 small filters over 64-channel activations: the resident-filter kernel, when the layer qualifies
  {
    const bool ovec = (out.stride[1] == 1) && aligned16(out.ptr) && (out.stride[0] * es) % 16 == 0 &&
                      (out.stride[2] * es) % 16 == 0 && (out.stride[3] * es) % 16 == 0 && (K % vec_elems) == 0;
    if (!window && !w_remap && Cp == 64 && C == 64 && st.status != nullptr &&
        try_resident_filter_conv(st, x, w_ptr, bias, out, p, epi, K, R, S, ovec, stream))
      return;
  }

  // ---- tiling of the whole problem
  const long long m_tiles_128 = (M + tb200::kBlockM - 1) / tb200::kBlockM;
  int bn = pick_bn(m_tiles_128, static_cast<int>(K), st.num_sms);
  const int forced_bn = knobs().force_bn;
  if (forced_bn == 64 || forced_bn == 128 || forced_bn == 256) bn = forced_bn;
  // CTA pairs (cta_group::2): a pair of SMs owns a 256 x bn tile and each CTA brings in only half of B's rows
  // Worth it when the main loop is long enough to dominate the tile (>= 8 k-steps); short-K, epilogue-bound
  // layers lose more from coupling two SMs' epilogues than they gain. TRACEA_B200_PAIR=0/1 forces the choice.
  const int pair_env = knobs().pair;
  const bool pair_ok = chunk_bytes == 128 && bn == 256 && st.num_sms >= 2;
  const bool pair = pair_ok && (pair_env == 1 || (pair_env != 0 && total_chunks_ll >= 8));
  // Two row blocks per CTA for narrow outputs (bn <= 128): twice the tensor work per barrier probe and per tile.
  const int rows2_env = knobs().rows2;
  // A 256-row tile costs an SM about 1.6x what a 128-row tile costs it (measured; the narrow tile is bound by the
  // shared-memory fill rate, which B's reuse across two row blocks relieves): taken when it shortens the launch,
  // wave quantisation included.
  const long long n_tiles = (K + bn - 1) / bn;
  const long long waves_128 = (m_tiles_128 * n_tiles + st.num_sms - 1) / st.num_sms;
  const long long waves_256 = ((m_tiles_128 + 1) / 2 * n_tiles + st.num_sms - 1) / st.num_sms;
  const bool rows2 = !pair && chunk_bytes == 128 && bn <= 128 && rows2_env != 0 &&
                     (rows2_env == 1 || (total_chunks_ll >= 7 && 8 * waves_256 < 5 * waves_128));

  // ---- tensor maps shared by every launch of this call
  CUtensorMap tmap_x, tmap_out, tmap_res;
  memset(&tmap_out, 0, sizeof(tmap_out));
  memset(&tmap_res, 0, sizeof(tmap_res));
  // A 1x1 / stride-1 / unpadded conv over dense NHWC memory is a plain [M][C] x [C][K] GEMM; the
  // tiled map is kept as a cross-check of the im2col path (TRACEA_B200_TILED_A=1).
  const bool a_tiled = !pair && !rows2 && !window && knobs().tiled_a != 0 && R == 1 && S == 1 && p.stride_h == 1 &&
                       p.stride_w == 1 && p.padding_h == 0 && p.padding_w == 0 && p.pad_h_hi == 0 && p.pad_w_hi == 0 &&
                       x.stride[3] == Cp &&
                       x.stride[2] == W * Cp && x.stride[0] == H * W * Cp;
  if (a_tiled) {
    const cuuint64_t gdim[2] = {(cuuint64_t)Cp, (cuuint64_t)M};
    const cuuint64_t gstr[1] = {(cuuint64_t)(Cp * es)};
    const cuuint32_t box[2] = {(cuuint32_t)chunk_elems, (cuuint32_t)tb200::kBlockM};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult r = g_encode_tiled(&tmap_x, tmap_dtype(x.dtype), 2, x.ptr, gdim, gstr, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, tmap_swizzle(chunk_bytes),
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TB_FAIL(TRACEA_CUDA_ERROR, "cuTensorMapEncodeTiled (A) failed with %d", (int)r);
  } else {
    // window mode: "pixel" w of the view starts at padded pixel w and spans 8 of them (pitch 16 B, extent
    // 128 B, overlapping); the horizontal padding is in memory, so the W corners only trim the filter width
    const cuuint64_t gdim[4] = {(cuuint64_t)Cg, (cuuint64_t)(window ? W + 2LL * p.padding_w : W), (cuuint64_t)H,
                                (cuuint64_t)N};
    const cuuint64_t gstr[3] = {(cuuint64_t)(x.stride[3] * es), (cuuint64_t)(x.stride[2] * es),
                                (cuuint64_t)(x.stride[0] * es)};
    const int lower[2] = {window ? 0 : -(int)p.padding_w, -(int)p.padding_h};
    const int upper[2] = {window ? -(int)(S - 1) : (int)p.pad_w_hi - (int)((S - 1) * p.dilation_w),
                          (int)p.pad_h_hi - (int)((R - 1) * p.dilation_h)};
    const cuuint32_t estr[4] = {1u, p.stride_w, p.stride_h, 1u};
    CUresult r = g_encode_im2col(&tmap_x, tmap_dtype(x.dtype), 4, x.ptr, gdim, gstr, lower, upper,
                                 (cuuint32_t)chunk_elems, (cuuint32_t)tb200::kBlockM, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, tmap_swizzle(chunk_bytes),
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      TB_FAIL(TRACEA_CUDA_ERROR,
              "cuTensorMapEncodeIm2col failed with %d (C=%lld W=%lld H=%lld N=%lld chunk=%d B lower=(%d,%d) "
              "upper=(%d,%d) stride=(%u,%u))",
              (int)r, Cg, W, H, N, chunk_bytes, lower[0], lower[1], upper[0], upper[1], p.stride_w,
              p.stride_h);
  }

  // ---- kernel arguments common to every launch
  ConvKernelArgs a;
  memset(&a, 0, sizeof(a));
  a.K_out = static_cast<int>(K);
  a.Ho = static_cast<int>(Ho);
  a.Wo = static_cast<int>(Wo);
  a.stride_h = p.stride_h;
  a.stride_w = p.stride_w;
  a.pad_h = p.padding_h;
  a.pad_w = window ? 0 : p.padding_w;
  a.dil_h = p.dilation_h;
  a.dil_w = p.dilation_w;
  a.S = static_cast<int>(Sg);
  a.chunk_elems = chunk_elems;
  a.chunk_bytes = chunk_bytes;
  a.chunks_per_tap = chunks_per_tap;
  a.total_chunks = static_cast<int>(total_chunks_ll);
  a.C = static_cast<int>(Cg);
  a.a_tiled = a_tiled ? 1 : 0;
  a.num_n_tiles = static_cast<int>(n_tiles);
  a.b_k0 = static_cast<int>(b_k0);
  a.b_jump_s = static_cast<int>(b_jump_s);
  a.b_jump_r = static_cast<int>(b_jump_r);
  // K-major operand descriptors. Swizzled rows of chunk_bytes: 8-row groups are 8*chunk_bytes apart
  // (SBO) and one MMA (32 B of K) stays inside a row. Unswizzled 16-byte chunks: an 8-row x 16 B core
  // matrix is 128 contiguous bytes (SBO) and the MMA's second K half is the next chunk (LBO).
  const uint32_t a_chunk = tb200::kBlockM * chunk_bytes, b_chunk = bn * chunk_bytes;
  if (chunk_bytes >= 32) {
    a.swizzle_mode = chunk_bytes == 128 ? 2u : (chunk_bytes == 64 ? 4u : 6u);
    a.a_sbo = a.b_sbo = 8u * chunk_bytes;
    a.a_lbo = a.b_lbo = 0u;
    const int mma_per_chunk = chunk_bytes / 32;
    for (int k = 0; k < 4; ++k) {
      a.a_mma_off[k] = (k / mma_per_chunk) * a_chunk + (k % mma_per_chunk) * 32u;
      a.b_mma_off[k] = (k / mma_per_chunk) * b_chunk + (k % mma_per_chunk) * 32u;
    }
  } else {
    a.swizzle_mode = 0u;
    a.a_sbo = a.b_sbo = 128u;
    a.a_lbo = a_chunk;
    a.b_lbo = b_chunk;
    for (int k = 0; k < 4; ++k) {
      a.a_mma_off[k] = 2u * k * a_chunk;
      a.b_mma_off[k] = 2u * k * b_chunk;
    }
  }
  a.out = out.ptr;
  a.out_sn = out.stride[0];
  a.out_sc = out.stride[1];
  a.out_sh = out.stride[2];
  a.out_sw = out.stride[3];
  auto vec_legal = [&](const View4& v) {
    return (v.stride[1] == 1) && aligned16(v.ptr) && (v.stride[0] * es) % 16 == 0 &&
           (v.stride[2] * es) % 16 == 0 && (v.stride[3] * es) % 16 == 0 && (K % vec_elems) == 0;
  };
  a.out_vec = vec_legal(out) ? 1 : 0;
  // Output rows that are linear in m = (n*Ho + ho)*Wo + wo form a [M][pitch] matrix: the epilogue
  // stages 32-pixel x 128-byte boxes in shared memory and the TMA unit writes them out.
  const bool out_rows_linear = out.stride[2] == Wo * out.stride[3] && out.stride[0] == Ho * out.stride[2];
  if (a.out_vec && out_rows_linear && knobs().no_tma_store == 0) {
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t gstr[1] = {(cuuint64_t)(out.stride[3] * es)};
    const cuuint32_t box[2] = {(cuuint32_t)(128 / es), 32u};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult r = g_encode_tiled(&tmap_out, tmap_dtype(x.dtype), 2, out.ptr, gdim, gstr, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) TB_FAIL(TRACEA_CUDA_ERROR, "cuTensorMapEncodeTiled (out) failed with %d", (int)r);
    a.out_tma = 1;
  }
  if (epi.bias && bias != nullptr) {
    a.bias = bias->ptr;
    a.bias_is_f32 = bias->dtype == TRACEA_DTYPE_FLOAT32 ? 1 : 0;
  }
  if (epi.residual && residual != nullptr) {
    a.residual = residual->ptr;
    a.res_sn = residual->stride[0];
    a.res_sc = residual->stride[1];
    a.res_sh = residual->stride[2];
    a.res_sw = residual->stride[3];
    a.res_vec = vec_legal(*residual) ? 1 : 0;
    // a residual with the same dense row-linear form is TMA-loaded into the epilogue's staging boxes
    const bool res_rows_linear = residual->stride[2] == Wo * residual->stride[3] &&
                                 residual->stride[0] == Ho * residual->stride[2];
    if (a.out_tma && a.res_vec && res_rows_linear && knobs().no_tma_residual == 0) {
      const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
      const cuuint64_t gstr[1] = {(cuuint64_t)(residual->stride[3] * es)};
      const cuuint32_t box[2] = {(cuuint32_t)(128 / es), 32u};
      const cuuint32_t estr[2] = {1u, 1u};
      CUresult r = g_encode_tiled(&tmap_res, tmap_dtype(x.dtype), 2, residual->ptr, gdim, gstr, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) TB_FAIL(TRACEA_CUDA_ERROR, "cuTensorMapEncodeTiled (residual) failed with %d", (int)r);
      a.res_tma = 1;
    } else {
      a.out_tma = 0;   // the kernel's TMA epilogue takes its residual through TMA or not at all
    }
  }
  a.act = epi.act;
  a.status = st.status;
  {
    const long long lim = g_test_wait_limit.load(std::memory_order_relaxed);
    a.wait_limit = lim > 0 ? lim : tb200::kWaitLimitCycles;
    a.test_producer_stop = g_test_producer_stop.load(std::memory_order_relaxed);
  }
  if (p.chain != nullptr && knobs().pdl != 0) {
    // the head of a chain waits before it lets its successor start; a later member starts without waiting, unless
    // an adapter kernel of its own sits between it and the member before it
    if (*p.chain == 0) { a.pdl_mode = 1; *p.chain = 1; }
    else a.pdl_mode = staged ? 0 : 2;
  }
  // channel-contiguous output (and residual, if any) that the TMA unit cannot address as one matrix: the kernel
  // variant whose epilogue writes its staging boxes out itself, whole 128-byte rows at a time
  const bool coop = !a.out_tma && a.out_vec && (a.residual == nullptr || a.res_vec);
#ifdef TB200_PROFILE
  {  // bring-up builds only: TRACEA_B200_PROF_PTR carries a device pointer to 8 counters per CTA
    const char* pp = getenv("TRACEA_B200_PROF_PTR");
    a.prof = pp != nullptr ? reinterpret_cast<long long*>(strtoull(pp, nullptr, 0)) : nullptr;
  }
#endif
  const uint32_t fmt = x.dtype == TRACEA_DTYPE_FLOAT16 ? 0u : (x.dtype == TRACEA_DTYPE_BFLOAT16 ? 1u : 2u);

  // ---- one launch over output pixels [row_begin, row_end) with the given tiling. (Splitting a partly filled last
  // wave off into a second launch with 128-row tiles was measured and is slower: a CTA pair's 256-row tile costs
  // each SM exactly what a 128-row tile costs it, so the tail does not get shorter, and the launch boundary adds
  // ~10 us.)
  auto launch_rows = [&](bool pair_v, bool rows2_v, long long row_begin, long long row_end) {
    const long long rows = row_end - row_begin;
    const long long tile_rows = (pair_v || rows2_v) ? 2 * tb200::kBlockM : tb200::kBlockM;
    const long long m_tiles = (rows + tile_rows - 1) / tile_rows;
    if (m_tiles * n_tiles > 0x7fffffffLL) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "too many tiles");
    // an output one tile wide never changes its bias: one copy per CTA instead of one per epilogue warp leaves
    // room for a fifth stage of the CTA-pair tiling
    const bool shared_bias = n_tiles == 1;
    int stages = pick_stages(bn, pair_v, rows2_v, shared_bias);
    const int forced_stages = knobs().force_stages;
    if (forced_stages >= 2 && forced_stages <= stages) stages = forced_stages;
    const int smem = tb200::conv_smem_bytes(bn, stages, pair_v, rows2_v, shared_bias);

    CUtensorMap tmap_w;
    // repacked or dense weights: one row is the whole Kgemm axis; in-place strided taps: one row spans the taps
    const cuuint64_t gdim[2] = {(cuuint64_t)(w_remap ? w_row_elems : Kgemm), (cuuint64_t)K};
    const cuuint64_t gstr[1] = {(cuuint64_t)((w_remap ? w_pitch : Kgemm) * es)};
    const cuuint32_t box[2] = {(cuuint32_t)chunk_elems, (cuuint32_t)(pair_v ? bn / 2 : bn)};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult r = g_encode_tiled(&tmap_w, tmap_dtype(x.dtype), 2, const_cast<void*>(w_ptr), gdim, gstr,
                                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, tmap_swizzle(chunk_bytes),
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      TB_FAIL(TRACEA_CUDA_ERROR, "cuTensorMapEncodeTiled failed with %d (Kgemm=%lld K=%lld bn=%d)", (int)r,
              Kgemm, K, bn);

    ConvKernelArgs la = a;
    la.m_begin = static_cast<int>(row_begin);
    la.M = static_cast<int>(row_end);
    la.num_m_tiles = static_cast<int>(m_tiles);
    // Tile order: wide outputs are walked in panels of 8 column tiles so that a wave of CTAs shares its B columns
    // and A rows through L2 instead of streaming all of B once per wave (TRACEA_B200_PANEL overrides the width).
    long long panel = n_tiles > 8 ? 8 : n_tiles;
    if (knobs().panel > 0) panel = std::min<long long>(knobs().panel, n_tiles);
    if (m_tiles * panel > 0x7fffffffLL) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "too many tiles");
    la.panel_width = static_cast<int>(panel);
    la.panel_tiles = static_cast<int>(m_tiles * panel);
    la.num_stages = stages;
    la.shared_bias = shared_bias ? 1 : 0;
    la.idesc = tb200::ptx::make_idesc(fmt, pair_v ? 2 * tb200::kBlockM : tb200::kBlockM, bn);
    const long long tiles = m_tiles * n_tiles;
    const long long workers_max = pair_v ? st.num_sms / 2 : st.num_sms;   // CTAs, or CTA pairs
    long long workers = std::min<long long>(tiles, workers_max);

    // ---- work schedule. A layer whose tile count is not a multiple of the worker count leaves SMs idle in its
    // last wave; a layer with fewer tiles than SMs leaves them idle throughout. Cutting tiles over K evens that
    // out: the k-steps of a "split region" of tiles are laid end to end and dealt out in equal shares, so that
    // several workers compute one tile, each over a slice of K, and exchange fp32 partial sums through scratch
    // memory (the piece that finishes last adds them up and runs the epilogue).
    //  * more than one wave: the split region is the partial wave plus one whole wave, so every share is longer
    //    than one tile and no tile is cut into more than two pieces; the waves before it stay whole tiles;
    //  * less than one wave: every tile is in the region, shares of at least four k-steps.
    // OFF unless TRACEA_B200_SPLIT_K=1 (2: also when it saves a single k-step). Measured on B200 it loses: a
    // 256 x 256 fp32 partial sum is as many bytes as the operands of four k-steps, and these kernels already run at
    // the rate L2 can feed the SMs, so the exchange costs more than the idle tail it removes (1x1 1024->256 at
    // 256 images: 31 -> 55 us; 3x3 256->256: 46 -> 61 us; 3x3 512->512 at 64 images: 27 -> 31 us). Kept as a
    // tested option for parts with a different balance. 128-byte k-chunks only.
    la.dp_tiles = static_cast<int>(tiles);
    Scratch sk_scratch;
    const long long k_iters = total_chunks_ll;   // 128-byte chunks: one per pipeline stage
    const int split_env = knobs().split_k;
    if (chunk_bytes == 128 && !a_tiled && !coop && split_env != 0 && arena == nullptr && k_iters >= 2 &&
        2 * workers_max * k_iters < (1LL << 30)) {
      const long long rem = tiles % workers_max;       // tiles of the last, partly filled wave (all of them if < 1 wave)
      if (rem > 0) {
        long long region = 0, sk_workers = 0, saved = 0, min_saved = 0;
        if (tiles > workers_max) {
          region = rem + workers_max;
          sk_workers = workers_max;
          saved = 2 * k_iters - (region * k_iters + sk_workers - 1) / sk_workers;
          min_saved = split_env == 2 ? 1 : 4;
        } else {
          const long long min_share = split_env == 2 ? 1 : 4;
          region = rem;
          sk_workers = std::min<long long>(workers_max, rem * k_iters / min_share);
          saved = sk_workers > rem ? k_iters - (region * k_iters + sk_workers - 1) / sk_workers : 0;
          min_saved = split_env == 2 ? 1 : 8;
        }
        {
          const long long rem = region;   // the tiles of the split region
          if (saved >= min_saved) {
            la.sk_slot_floats = 256LL * bn;
            const size_t partial_bytes = static_cast<size_t>(2 * sk_workers * la.sk_slot_floats) * sizeof(float);
            const size_t counter_bytes = static_cast<size_t>(rem) * 8 * 2 * sizeof(uint32_t);
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) {
              cudaGetLastError();   // e.g. another thread is capturing in global mode: run this call unsplit
              cap = cudaStreamCaptureStatusInvalidated;
            }
            // a graph may be replayed at any time, next to anything: it never shares a stream's block
            void* ws = cap == cudaStreamCaptureStatusNone ? split_workspace(st, stream) : nullptr;
            if (ws != nullptr) {
              la.sk_partials = static_cast<float*>(ws);
              la.sk_counters = reinterpret_cast<uint32_t*>(static_cast<char*>(ws) + st.split_partial_bytes);
            } else if (cap == cudaStreamCaptureStatusActive) {
              // inside a graph capture on a stream without a block: memory the graph owns, cleared by a memset node
              sk_scratch.alloc(st, partial_bytes + counter_bytes, stream);
              la.sk_partials = static_cast<float*>(sk_scratch.ptr);
              la.sk_counters = reinterpret_cast<uint32_t*>(static_cast<char*>(sk_scratch.ptr) + partial_bytes);
              TB_CUDA(cudaMemsetAsync(la.sk_counters, 0, counter_bytes, stream));
            }
            if (la.sk_partials != nullptr) {
              la.sk_tiles = static_cast<int>(rem);
              la.dp_tiles = static_cast<int>(tiles - rem);
              la.sk_workers = static_cast<int>(sk_workers);
              workers = tiles >= workers_max ? workers_max : sk_workers;
              // the exchange scratch belongs to the stream: a launch that uses it must not run beside the launch in
              // front of it, which may be using it too
              if (la.pdl_mode == 2) la.pdl_mode = 0;
            }
          }
        }
      }
    }
    const int grid = static_cast<int>(pair_v ? 2 * workers : workers);
    switch (x.dtype) {
      case TRACEA_DTYPE_BFLOAT16:
        launch_bn<__nv_bfloat16>(st, 0, bn, pair_v, rows2_v, coop, tmap_x, tmap_w, tmap_out, tmap_res, la, grid, smem, stream);
        break;
      case TRACEA_DTYPE_FLOAT16:
        launch_bn<__half>(st, 1, bn, pair_v, rows2_v, coop, tmap_x, tmap_w, tmap_out, tmap_res, la, grid, smem, stream);
        break;
      default:
        launch_bn<float>(st, 2, bn, pair_v, rows2_v, coop, tmap_x, tmap_w, tmap_out, tmap_res, la, grid, smem, stream);
        break;
    }
  };
  launch_rows(pair, rows2, 0, M);
}

// ------------------------------------------------------------------ host-memory staging
struct Staged {
  Scratch buf;
  View4 view;
};

void stage_in(DeviceState& st, const View4& host, Staged& s, cudaStream_t stream, bool copy) {
  const size_t bytes = static_cast<size_t>(span_elems(host)) * elem_size(host.dtype);
  s.buf.alloc(st, bytes, stream);
  s.view = host;
  s.view.ptr = s.buf.ptr;
  if (copy) TB_CUDA(cudaMemcpyAsync(s.buf.ptr, host.ptr, bytes, cudaMemcpyHostToDevice, stream));
}

// ------------------------------------------------------------------ validation + dispatch
void conv2d_checked(const TraceaTensorView& xv, const TraceaTensorView& wv, const TraceaTensorView* bv,
                    const TraceaTensorView* rv, TraceaTensorView* ov, const TraceaConv2dParams& p,
                    bool no_alloc = false) {
  if (xv.ptr == nullptr || wv.ptr == nullptr || ov == nullptr || ov->ptr == nullptr)
    TB_FAIL(TRACEA_INVALID_PARAMS, "Null pointer in input tensors");
  if (p.groups != 1) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "Unsupported groups: %u", p.groups);
  if (p.stride_h == 0 || p.stride_w == 0) TB_FAIL(TRACEA_INVALID_PARAMS, "stride must be >= 1");
  if (p.dilation_h == 0 || p.dilation_w == 0) TB_FAIL(TRACEA_INVALID_PARAMS, "dilation must be >= 1");
  const int es = elem_size(xv.dtype);
  if (es == 0)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "Unsupported dtype %s (float32, float16, bfloat16 are supported)",
            dtype_name(xv.dtype));
  if (wv.dtype != xv.dtype)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "x is %s but w is %s", dtype_name(xv.dtype), dtype_name(wv.dtype));
  if (ov->dtype != xv.dtype)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "x is %s but out is %s", dtype_name(xv.dtype), dtype_name(ov->dtype));

  View4 x = load_view4(xv, "x");
  View4 w = load_view4(wv, "w");
  View4 out = load_view4(*ov, "out");
  canon_channels_last(x);
  canon_channels_last(w);
  canon_channels_last(out);
  const long long N = x.shape[0], C = x.shape[1], H = x.shape[2], W = x.shape[3];
  const long long K = w.shape[0], R = w.shape[2], S = w.shape[3];
  if (w.shape[1] != C)
    TB_FAIL(TRACEA_INVALID_PARAMS, "Channel mismatch: x has %lld channels, w has %lld", C, w.shape[1]);
  const long long eff_h = H + 2LL * p.padding_h - (long long)p.dilation_h * (R - 1) - 1;
  const long long eff_w = W + 2LL * p.padding_w - (long long)p.dilation_w * (S - 1) - 1;
  if (eff_h < 0 || eff_w < 0)
    TB_FAIL(TRACEA_INVALID_PARAMS, "filter %lldx%lld does not fit the padded %lldx%lld input", R, S, H, W);
  const long long Ho = eff_h / p.stride_h + 1, Wo = eff_w / p.stride_w + 1;
  if (out.shape[0] != N || out.shape[1] != K || out.shape[2] != Ho || out.shape[3] != Wo)
    TB_FAIL(TRACEA_INVALID_PARAMS, "out shape [%lld,%lld,%lld,%lld] does not match expected [%lld,%lld,%lld,%lld]",
            out.shape[0], out.shape[1], out.shape[2], out.shape[3], N, K, Ho, Wo);

  const int dev = x.device;
  if (w.device != dev || out.device != dev)
    TB_FAIL(TRACEA_INVALID_PARAMS, "x, w and out must live on the same device");
  if (w.shape[0] == 0) TB_FAIL(TRACEA_INVALID_PARAMS, "w: shape[0] = 0 is out of range");

  View4 bias4, res4;
  const View4* bias = nullptr;
  const View4* res = nullptr;
  if (bv != nullptr) {
    if (bv->ptr == nullptr) TB_FAIL(TRACEA_INVALID_PARAMS, "bias view has a NULL pointer");
    if (bv->rank != 1 || bv->shape == nullptr || (long long)bv->shape[0] != K)
      TB_FAIL(TRACEA_INVALID_PARAMS, "bias must be a rank-1 tensor of length %lld", K);
    if (bv->stride != nullptr && bv->stride[0] != 1)
      TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "bias must be contiguous");
    if (bv->dtype != TRACEA_DTYPE_FLOAT32 && bv->dtype != xv.dtype)
      TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "bias must be float32 or %s", dtype_name(xv.dtype));
    if (bv->device_id != dev) TB_FAIL(TRACEA_INVALID_PARAMS, "bias must live on the same device as x");
    bias4.ptr = bv->ptr;
    bias4.dtype = bv->dtype;
    bias4.device = bv->device_id;
    bias4.shape[0] = K;
    bias4.shape[1] = bias4.shape[2] = bias4.shape[3] = 1;
    bias4.stride[0] = 1;
    bias = &bias4;
  }
  if (rv != nullptr) {
    if (rv->ptr == nullptr) TB_FAIL(TRACEA_INVALID_PARAMS, "residual view has a NULL pointer");
    res4 = load_view4(*rv, "residual");
    canon_channels_last(res4);
    if (res4.dtype != xv.dtype)
      TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "residual must be %s", dtype_name(xv.dtype));
    for (int i = 0; i < 4; ++i)
      if (res4.shape[i] != out.shape[i])
        TB_FAIL(TRACEA_INVALID_PARAMS, "residual shape must equal the out shape");
    if (res4.device != dev) TB_FAIL(TRACEA_INVALID_PARAMS, "residual must live on the same device as x");
    res = &res4;
  }
  const Epilogue epi = decode_epilogue(p.epilogue, bias != nullptr, res != nullptr);
  if (N == 0) return;  // empty batch: nothing to compute, nothing to launch

  if (no_alloc) {
    if (dev < 0)
      TB_FAIL(TRACEA_INVALID_PARAMS,
              "tracea_conv2d_noalloc takes device tensors only: staging host memory would need an allocation");
    conv2d_device_noalloc(dev, x, w, bias, res, out, p, epi);
    return;
  }
  if (dev >= 0) {
    conv2d_device(dev, x, w, bias, res, out, p, epi);
    return;
  }

  // Host memory: stage through the current CUDA device, run the same device path, copy back and
  // wait, so that the result is in the caller's buffer when the call returns. Large batches are cut
  // into chunks of images so that the copy in of chunk i+1, the kernels of chunk i and the copy out
  // of chunk i-1 overlap (PCIe is full duplex; the kernels are a small fraction of the copy time).
  int cur = 0;
  TB_CUDA(cudaGetDevice(&cur));
  cudaStream_t stream = static_cast<cudaStream_t>(p.stream);
  DeviceState& st_cur = device_state(cur);
  std::lock_guard<std::mutex> host_lock(st_cur.host_mu);
  const bool use_bias = bias != nullptr && epi.bias, use_res = res != nullptr && epi.residual;
  auto image_major = [](const View4& v) {   // images do not interleave: one image's span fits in stride[0]
    long long span = 1;
    for (int i = 1; i < 4; ++i) span += (v.shape[i] - 1) * v.stride[i];
    return v.shape[0] == 1 || v.stride[0] >= span;
  };
  auto image_span = [](const View4& v) {
    long long span = 1;
    for (int i = 1; i < 4; ++i) span += (v.shape[i] - 1) * v.stride[i];
    return span;
  };
  const long long total_bytes = (span_elems(x) + span_elems(out) + (use_res ? span_elems(*res) : 0)) * es;
  int chunks = 1;
  if (N >= 16 && total_bytes >= (8LL << 20) && image_major(x) && image_major(out) && span_elems(out) == num_elems(out) &&
      (!use_res || image_major(*res)) && env_int("TRACEA_B200_HOST_CHUNKS", 8) > 1) {
    chunks = std::min<long long>({(long long)env_int("TRACEA_B200_HOST_CHUNKS", 8), (long long)DeviceState::kMaxChunks, N / 2});
  }
  Staged sx, sw, sb, sr, so;
  DeviceState* stp = nullptr;
  {
    DeviceState& st = st_cur;
    stp = &st;
    stage_in(st, x, sx, stream, chunks == 1);
    stage_in(st, w, sw, stream, true);
    if (use_bias) stage_in(st, *bias, sb, stream, true);
    if (use_res) stage_in(st, *res, sr, stream, chunks == 1);
    // a strided `out` has gaps the copy back must not clobber: seed the staging buffer with them
    stage_in(st, out, so, stream, span_elems(out) != num_elems(out));
    if (chunks > 1 && st.copy_in == nullptr) {
      TB_CUDA(cudaStreamCreateWithFlags(&st.copy_in, cudaStreamNonBlocking));
      TB_CUDA(cudaStreamCreateWithFlags(&st.copy_out, cudaStreamNonBlocking));
      TB_CUDA(cudaEventCreateWithFlags(&st.ev_entry, cudaEventDisableTiming));
      TB_CUDA(cudaEventCreateWithFlags(&st.ev_done, cudaEventDisableTiming));
      for (int i = 0; i < DeviceState::kMaxChunks; ++i) {
        TB_CUDA(cudaEventCreateWithFlags(&st.ev_in[i], cudaEventDisableTiming));
        TB_CUDA(cudaEventCreateWithFlags(&st.ev_out[i], cudaEventDisableTiming));
      }
    }
  }
  if (chunks == 1) {
    conv2d_device(cur, sx.view, sw.view, use_bias ? &sb.view : nullptr, use_res ? &sr.view : nullptr, so.view, p, epi);
    TB_CUDA(cudaMemcpyAsync(out.ptr, so.buf.ptr, static_cast<size_t>(span_elems(out)) * es,
                            cudaMemcpyDeviceToHost, stream));
  } else {
    DeviceState& st = *stp;
    // the staging buffers were allocated in stream order on `stream`: the copy streams start after that point
    TB_CUDA(cudaEventRecord(st.ev_entry, stream));
    TB_CUDA(cudaStreamWaitEvent(st.copy_in, st.ev_entry, 0));
    TB_CUDA(cudaStreamWaitEvent(st.copy_out, st.ev_entry, 0));
    auto chunk_of = [&](const View4& dev_view, long long n0, long long n1) {
      View4 c = dev_view;
      c.ptr = static_cast<char*>(dev_view.ptr) + n0 * dev_view.stride[0] * es;
      c.shape[0] = n1 - n0;
      return c;
    };
    auto copy_chunk = [&](void* dst_base, const void* src_base, const View4& v, long long n0, long long n1,
                          cudaMemcpyKind kind, cudaStream_t s) {
      const size_t off = static_cast<size_t>(n0 * v.stride[0]) * es;
      const size_t len = static_cast<size_t>((n1 - n0 - 1) * v.stride[0] + image_span(v)) * es;
      TB_CUDA(cudaMemcpyAsync(static_cast<char*>(dst_base) + off, static_cast<const char*>(src_base) + off, len, kind, s));
    };
    for (int c = 0; c < chunks; ++c) {
      const long long n0 = N * c / chunks, n1 = N * (c + 1) / chunks;
      copy_chunk(sx.buf.ptr, x.ptr, x, n0, n1, cudaMemcpyHostToDevice, st.copy_in);
      if (use_res) copy_chunk(sr.buf.ptr, res->ptr, *res, n0, n1, cudaMemcpyHostToDevice, st.copy_in);
      TB_CUDA(cudaEventRecord(st.ev_in[c], st.copy_in));
      TB_CUDA(cudaStreamWaitEvent(stream, st.ev_in[c], 0));
      const View4 xc = chunk_of(sx.view, n0, n1), oc = chunk_of(so.view, n0, n1);
      View4 rc;
      if (use_res) rc = chunk_of(sr.view, n0, n1);
      conv2d_device(cur, xc, sw.view, use_bias ? &sb.view : nullptr, use_res ? &rc : nullptr, oc, p, epi);
      TB_CUDA(cudaEventRecord(st.ev_out[c], stream));
      TB_CUDA(cudaStreamWaitEvent(st.copy_out, st.ev_out[c], 0));
      copy_chunk(out.ptr, so.buf.ptr, out, n0, n1, cudaMemcpyDeviceToHost, st.copy_out);
    }
    TB_CUDA(cudaEventRecord(st.ev_done, st.copy_out));
    TB_CUDA(cudaStreamWaitEvent(stream, st.ev_done, 0));
  }
  TB_CUDA(cudaStreamSynchronize(stream));
  const uint32_t code = tracea_b200_device_status(cur);
  if (code != 0u) TB_FAIL(TRACEA_CUDA_ERROR, "conv kernel gave up a bounded wait (code %u)", code);
}

// ------------------------------------------------------------------ GEMM: the 1x1 convolution it is
struct Rank2 {
  long long shape[2];
  long long stride[2];
};

Rank2 load_rank2(const TraceaTensorView& v, const char* name) {
  if (v.rank != 2) TB_FAIL(TRACEA_INVALID_PARAMS, "Expected 2D tensors: %s has rank %u", name, v.rank);
  if (v.shape == nullptr) TB_FAIL(TRACEA_INVALID_PARAMS, "%s: shape array is NULL", name);
  Rank2 r;
  for (int i = 0; i < 2; ++i) {
    r.shape[i] = static_cast<long long>(v.shape[i]);
    if (r.shape[i] < 0 || r.shape[i] > 0x7fffffffLL)
      TB_FAIL(TRACEA_INVALID_PARAMS, "%s: shape[%d] = %llu is out of range", name, i, (unsigned long long)v.shape[i]);
  }
  r.stride[0] = v.stride != nullptr ? v.stride[0] : r.shape[1];
  r.stride[1] = v.stride != nullptr ? v.stride[1] : 1;
  if (r.stride[0] < 0 || r.stride[1] < 0) TB_FAIL(TRACEA_INVALID_PARAMS, "%s: negative stride", name);
  return r;
}

// A rank-2 [rows, cols] matrix as the rank-4 view {1, cols, 1, rows}: rows are pixels along W, cols channels.
struct AsConvView {
  uint64_t shape[4];
  int64_t stride[4];
  TraceaTensorView view;
  AsConvView(const TraceaTensorView& v, const Rank2& r) {
    shape[0] = 1; shape[1] = (uint64_t)r.shape[1]; shape[2] = 1; shape[3] = (uint64_t)r.shape[0];
    stride[1] = r.stride[1];
    stride[3] = r.stride[0];
    stride[2] = stride[0] = r.stride[0] * r.shape[0];
    view = v;
    view.rank = 4;
    view.shape = shape;
    view.stride = stride;
  }
};

void gemm_checked(const TraceaTensorView& av, const TraceaTensorView& bv, const TraceaTensorView* biasv,
                  const TraceaTensorView* rv, TraceaTensorView* cv, const TraceaGemmParams& gp) {
  if (av.ptr == nullptr || bv.ptr == nullptr || cv == nullptr || cv->ptr == nullptr)
    TB_FAIL(TRACEA_INVALID_PARAMS, "Null pointer in input tensors");
  const Rank2 a = load_rank2(av, "a"), b = load_rank2(bv, "b"), c = load_rank2(*cv, "c");
  const long long M = a.shape[0], K = a.shape[1], N = b.shape[1];
  if (b.shape[0] != K)
    TB_FAIL(TRACEA_INVALID_PARAMS, "Inner dimension mismatch: a is [%lld,%lld], b is [%lld,%lld]", M, K, b.shape[0], N);
  if (c.shape[0] != M || c.shape[1] != N)
    TB_FAIL(TRACEA_INVALID_PARAMS, "c shape [%lld,%lld] does not match expected [%lld,%lld]", c.shape[0], c.shape[1], M, N);
  if (K == 0 || N == 0) TB_FAIL(TRACEA_INVALID_PARAMS, "K = %lld, N = %lld: both must be positive", K, N);
  Rank2 r2 = c;
  if (rv != nullptr) {
    if (rv->ptr == nullptr) TB_FAIL(TRACEA_INVALID_PARAMS, "residual view has a NULL pointer");
    r2 = load_rank2(*rv, "residual");
    if (r2.shape[0] != M || r2.shape[1] != N) TB_FAIL(TRACEA_INVALID_PARAMS, "residual shape must equal the c shape");
  }
  if (M == 0) {   // nothing to compute; still reject what tracea_conv2d would reject
    if (elem_size(av.dtype) == 0) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "Unsupported dtype %s", dtype_name(av.dtype));
    return;
  }

  AsConvView x4(av, a), o4(*cv, c);
  // b[K,N] is the filter bank w[N, K, 1, 1]: output channel n reads column n of b
  uint64_t wshape[4] = {(uint64_t)N, (uint64_t)K, 1, 1};
  int64_t wstride[4] = {b.stride[1], b.stride[0], 0, 0};
  if (b.stride[0] == 1) wstride[2] = wstride[3] = K;
  TraceaTensorView w4 = bv;
  w4.rank = 4;
  w4.shape = wshape;
  w4.stride = wstride;
  TraceaTensorView res_view;
  AsConvView* r4 = nullptr;
  AsConvView r4_storage(rv != nullptr ? *rv : *cv, r2);
  if (rv != nullptr) {
    r4 = &r4_storage;
    res_view = r4->view;
  }
  TraceaConv2dParams p;
  p.stride_h = p.stride_w = 1;
  p.padding_h = p.padding_w = 0;
  p.dilation_h = p.dilation_w = 1;
  p.groups = 1;
  p.epilogue = gp.epilogue;
  p.stream = gp.stream;
  try {
    conv2d_checked(x4.view, w4, biasv, r4 != nullptr ? &res_view : nullptr, &o4.view, p);
  } catch (const StatusError&) {
    g_last_error = "tracea_gemm (run as a 1x1 conv: a is x, b is w, c is out): " + g_last_error;
    throw;
  }
}

// ------------------------------------------------------------------ ConvTranspose2d: one stride-1 conv per output phase
// 16 zero bytes in device memory: the "filter" of an output phase that no tap reaches.
static __device__ __align__(16) unsigned int g_zero_words[4];

// One axis of one output phase. Outputs o = a0 + stride*t (t < T) receive x[i] * w[r] for i*stride - pad + r = o,
// i.e. taps r = a + stride*j (j < taps) with a = (a0 + pad) % stride, from i = t + q0 - j, q0 = (a0 + pad) / stride.
// With the taps reversed (j' = taps-1-j) that is a stride-1 correlation: i = t - pad_lo + j', pad_lo = taps-1-q0.
// A negative pad_lo / pad_hi crops input rows instead (x_off rows from the front, extent `in` kept).
struct PhaseAxis {
  long long a0 = 0, T = 0, a = 0, taps = 0, x_off = 0, in = 0, pad_lo = 0, pad_hi = 0;
  bool empty = false;   // no tap or no input row reaches this phase: its outputs are epilogue(0)
};

PhaseAxis phase_axis(long long in_extent, long long out_extent, long long filt, long long stride, long long pad,
                     long long a0) {
  PhaseAxis ax;
  ax.a0 = a0;
  ax.T = a0 < out_extent ? (out_extent - a0 + stride - 1) / stride : 0;
  ax.a = (a0 + pad) % stride;
  const long long q0 = (a0 + pad) / stride;
  ax.taps = ax.a < filt ? (filt - ax.a + stride - 1) / stride : 0;
  ax.in = in_extent;
  ax.pad_lo = ax.taps - 1 - q0;
  if (ax.pad_lo < 0) {
    ax.x_off = -ax.pad_lo;
    ax.in -= ax.x_off;
    ax.pad_lo = 0;
  }
  ax.pad_hi = ax.T - ax.in - ax.pad_lo + (ax.taps - 1);
  if (ax.pad_hi < 0) {
    ax.in += ax.pad_hi;
    ax.pad_hi = 0;
  }
  ax.empty = ax.taps == 0 || ax.in <= 0;
  return ax;
}

// Geometry of an axis of an empty phase: a single zero tap over as much of the input as the outputs need.
void make_empty_axis(PhaseAxis& ax, long long in_extent) {
  ax.taps = 1;
  ax.x_off = 0;
  ax.in = std::min(in_extent, ax.T);
  ax.pad_lo = 0;
  ax.pad_hi = ax.T - ax.in;
}

// x, w, out, residual: device views in the conv's logical index order (x [N,C,H,W], w [K,C,R,S], out [N,K,Ho,Wo]).
void conv_transpose_phases(int dev, const View4& x, const View4& w, const View4* bias, const View4* res,
                           const View4& out, const TraceaConvTranspose2dParams& tp, const Epilogue& epi) {
  const int es = elem_size(x.dtype);
  const long long H = x.shape[2], W = x.shape[3], R = w.shape[2], S = w.shape[3];
  const long long Ho = out.shape[2], Wo = out.shape[3];
  const long long sh = tp.stride_h, sw = tp.stride_w;
  void* zero_ptr = nullptr;
  int chain = 0;   // the phases write disjoint outputs and read the same inputs: a chain of independent launches
  for (long long ah = 0; ah < sh; ++ah) {
    for (long long aw = 0; aw < sw; ++aw) {
      PhaseAxis ph = phase_axis(H, Ho, R, sh, tp.padding_h, ah);
      PhaseAxis pw = phase_axis(W, Wo, S, sw, tp.padding_w, aw);
      if (ph.T == 0 || pw.T == 0) continue;
      const bool empty = ph.empty || pw.empty;
      if (empty) {
        make_empty_axis(ph, H);
        make_empty_axis(pw, W);
      }
      View4 xp = x, wp = w, op = out, rp;
      xp.ptr = static_cast<char*>(x.ptr) + (ph.x_off * x.stride[2] + pw.x_off * x.stride[3]) * es;
      xp.shape[2] = ph.in;
      xp.shape[3] = pw.in;
      wp.shape[2] = ph.taps;
      wp.shape[3] = pw.taps;
      if (empty) {
        if (zero_ptr == nullptr) {
          DeviceGuard guard(dev);
          TB_CUDA(cudaGetSymbolAddress(&zero_ptr, g_zero_words));
        }
        wp.ptr = zero_ptr;
        wp.stride[0] = wp.stride[1] = wp.stride[2] = wp.stride[3] = 0;
      } else {
        // reversed taps: tap j' of the phase filter is w[.., a + stride*(taps-1-j'), ..]
        wp.ptr = static_cast<char*>(w.ptr) +
                 ((ph.a + sh * (ph.taps - 1)) * w.stride[2] + (pw.a + sw * (pw.taps - 1)) * w.stride[3]) * es;
        wp.stride[2] = -sh * w.stride[2];
        wp.stride[3] = -sw * w.stride[3];
      }
      auto phase_of = [&](const View4& v) {
        View4 o = v;
        o.ptr = static_cast<char*>(v.ptr) + (ah * v.stride[2] + aw * v.stride[3]) * es;
        o.shape[2] = ph.T;
        o.shape[3] = pw.T;
        o.stride[2] = sh * v.stride[2];
        o.stride[3] = sw * v.stride[3];
        return o;
      };
      op = phase_of(out);
      if (res != nullptr) rp = phase_of(*res);
      CoreParams cp;
      cp.stride_h = cp.stride_w = 1;
      cp.dilation_h = cp.dilation_w = 1;
      cp.groups = 1;
      cp.epilogue = tp.epilogue;
      cp.stream = tp.stream;
      cp.padding_h = static_cast<uint32_t>(ph.pad_lo);
      cp.padding_w = static_cast<uint32_t>(pw.pad_lo);
      cp.pad_h_hi = ph.pad_hi;
      cp.pad_w_hi = pw.pad_hi;
      cp.chain = &chain;
      conv2d_device(dev, xp, wp, bias, res != nullptr ? &rp : nullptr, op, cp, epi);
    }
  }
}

// [d0, d1, d2, d3] view in (n, h, w, c) index order -> the conv's logical (n, c, h, w) order.
View4 nhwc_to_logical(const View4& v) {
  View4 o = v;
  o.shape[1] = v.shape[3]; o.shape[2] = v.shape[1]; o.shape[3] = v.shape[2];
  o.stride[1] = v.stride[3]; o.stride[2] = v.stride[1]; o.stride[3] = v.stride[2];
  return o;
}

void conv_transpose2d_checked(const TraceaTensorView& xv, const TraceaTensorView& wv, const TraceaTensorView* bv,
                              const TraceaTensorView* rv, TraceaTensorView* ov, const TraceaConvTranspose2dParams& tp) {
  if (xv.ptr == nullptr || wv.ptr == nullptr || ov == nullptr || ov->ptr == nullptr)
    TB_FAIL(TRACEA_INVALID_PARAMS, "Null pointer in input tensors");
  if (tp.groups != 1) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "Unsupported groups: %u", tp.groups);
  if (tp.stride_h == 0 || tp.stride_w == 0) TB_FAIL(TRACEA_INVALID_PARAMS, "stride must be >= 1");
  if (tp.stride_h > 16 || tp.stride_w > 16) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "stride > 16 is not supported");
  if (tp.dilation_h != 1 || tp.dilation_w != 1)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "Unsupported dilation: (%u, %u)", tp.dilation_h, tp.dilation_w);
  if (tp.output_padding_h >= tp.stride_h || tp.output_padding_w >= tp.stride_w)
    TB_FAIL(TRACEA_INVALID_PARAMS, "output_padding must be smaller than the stride");
  const int es = elem_size(xv.dtype);
  if (es == 0)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "Unsupported dtype %s (float32, float16, bfloat16 are supported)",
            dtype_name(xv.dtype));
  if (wv.dtype != xv.dtype)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "x is %s but w is %s", dtype_name(xv.dtype), dtype_name(wv.dtype));
  if (ov->dtype != xv.dtype)
    TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "x is %s but out is %s", dtype_name(xv.dtype), dtype_name(ov->dtype));

  View4 x = nhwc_to_logical(load_view4(xv, "x"));
  View4 w = nhwc_to_logical(load_view4(wv, "w"));
  View4 out = nhwc_to_logical(load_view4(*ov, "out"));
  canon_channels_last(x);
  canon_channels_last(out);
  const long long N = x.shape[0], C = x.shape[1], H = x.shape[2], W = x.shape[3];
  const long long K = w.shape[0], R = w.shape[2], S = w.shape[3];
  if (w.shape[1] != C)
    TB_FAIL(TRACEA_INVALID_PARAMS, "Channel mismatch: x has %lld channels, w has %lld", C, w.shape[1]);
  if (K == 0) TB_FAIL(TRACEA_INVALID_PARAMS, "w: shape[0] = 0 is out of range");
  const long long Ho = (H - 1) * tp.stride_h - 2LL * tp.padding_h + R + tp.output_padding_h;
  const long long Wo = (W - 1) * tp.stride_w - 2LL * tp.padding_w + S + tp.output_padding_w;
  if (Ho <= 0 || Wo <= 0)
    TB_FAIL(TRACEA_INVALID_PARAMS, "padding (%u, %u) leaves no output for a %lldx%lld input and a %lldx%lld filter",
            tp.padding_h, tp.padding_w, H, W, R, S);
  if (out.shape[0] != N || out.shape[1] != K || out.shape[2] != Ho || out.shape[3] != Wo)
    TB_FAIL(TRACEA_INVALID_PARAMS, "out shape [%lld,%lld,%lld,%lld] does not match expected [%lld,%lld,%lld,%lld]",
            out.shape[0], out.shape[2], out.shape[3], out.shape[1], N, Ho, Wo, K);
  const int dev = x.device;
  if (w.device != dev || out.device != dev)
    TB_FAIL(TRACEA_INVALID_PARAMS, "x, w and out must live on the same device");

  View4 bias4, res4;
  const View4* bias = nullptr;
  const View4* res = nullptr;
  if (bv != nullptr) {
    if (bv->ptr == nullptr) TB_FAIL(TRACEA_INVALID_PARAMS, "bias view has a NULL pointer");
    if (bv->rank != 1 || bv->shape == nullptr || (long long)bv->shape[0] != K)
      TB_FAIL(TRACEA_INVALID_PARAMS, "bias must be a rank-1 tensor of length %lld", K);
    if (bv->stride != nullptr && bv->stride[0] != 1) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "bias must be contiguous");
    if (bv->dtype != TRACEA_DTYPE_FLOAT32 && bv->dtype != xv.dtype)
      TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "bias must be float32 or %s", dtype_name(xv.dtype));
    if (bv->device_id != dev) TB_FAIL(TRACEA_INVALID_PARAMS, "bias must live on the same device as x");
    bias4.ptr = bv->ptr;
    bias4.dtype = bv->dtype;
    bias4.device = bv->device_id;
    bias4.shape[0] = K;
    bias4.shape[1] = bias4.shape[2] = bias4.shape[3] = 1;
    bias4.stride[0] = 1;
    bias = &bias4;
  }
  if (rv != nullptr) {
    if (rv->ptr == nullptr) TB_FAIL(TRACEA_INVALID_PARAMS, "residual view has a NULL pointer");
    res4 = nhwc_to_logical(load_view4(*rv, "residual"));
    canon_channels_last(res4);
    if (res4.dtype != xv.dtype) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "residual must be %s", dtype_name(xv.dtype));
    for (int i = 0; i < 4; ++i)
      if (res4.shape[i] != out.shape[i]) TB_FAIL(TRACEA_INVALID_PARAMS, "residual shape must equal the out shape");
    if (res4.device != dev) TB_FAIL(TRACEA_INVALID_PARAMS, "residual must live on the same device as x");
    res = &res4;
  }
  const Epilogue epi = decode_epilogue(tp.epilogue, bias != nullptr, res != nullptr);
  if (N == 0) return;

  if (dev >= 0) {
    conv_transpose_phases(dev, x, w, bias, res, out, tp, epi);
    return;
  }
  // host memory: stage whole tensors through the current device, run the phases, copy back and wait
  int cur = 0;
  TB_CUDA(cudaGetDevice(&cur));
  cudaStream_t stream = static_cast<cudaStream_t>(tp.stream);
  DeviceState& st_cur = device_state(cur);
  std::lock_guard<std::mutex> host_lock(st_cur.host_mu);
  const bool use_bias = bias != nullptr && epi.bias, use_res = res != nullptr && epi.residual;
  Staged sx, sw, sb, sr, so;
  {
    DeviceState& st = st_cur;
    stage_in(st, x, sx, stream, true);
    stage_in(st, w, sw, stream, true);
    if (use_bias) stage_in(st, *bias, sb, stream, true);
    if (use_res) stage_in(st, *res, sr, stream, true);
    stage_in(st, out, so, stream, span_elems(out) != num_elems(out));
  }
  conv_transpose_phases(cur, sx.view, sw.view, use_bias ? &sb.view : nullptr, use_res ? &sr.view : nullptr, so.view, tp,
                        epi);
  TB_CUDA(cudaMemcpyAsync(out.ptr, so.buf.ptr, static_cast<size_t>(span_elems(out)) * es, cudaMemcpyDeviceToHost,
                          stream));
  TB_CUDA(cudaStreamSynchronize(stream));
  const uint32_t code = tracea_b200_device_status(cur);
  if (code != 0u) TB_FAIL(TRACEA_CUDA_ERROR, "conv kernel gave up a bounded wait (code %u)", code);
}

// ------------------------------------------------------------------ weight prepacking
long long padded_channels(long long c, int es) {
  const long long v = 16 / es;
  return (c + v - 1) / v * v;
}

void conv2d_prepack_checked(const TraceaTensorView& wv, void* dst, uint64_t dst_bytes, uint64_t* packed_shape,
                            int64_t* packed_stride, void* stream) {
  if (wv.ptr == nullptr || dst == nullptr || packed_shape == nullptr || packed_stride == nullptr)
    TB_FAIL(TRACEA_INVALID_PARAMS, "Null pointer in prepack arguments");
  const int es = elem_size(wv.dtype);
  if (es == 0) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "Unsupported dtype %s", dtype_name(wv.dtype));
  const View4 w = load_view4(wv, "w");
  if (w.shape[0] == 0) TB_FAIL(TRACEA_INVALID_PARAMS, "w: shape[0] = 0 is out of range");
  if (w.device < 0) TB_FAIL(TRACEA_INVALID_PARAMS, "prepacking takes device tensors (device_id >= 0)");
  if (!aligned16(dst)) TB_FAIL(TRACEA_INVALID_PARAMS, "dst must be 16-byte aligned");
  const long long K = w.shape[0], C = w.shape[1], R = w.shape[2], S = w.shape[3];
  const long long Cp = padded_channels(C, es);
  const unsigned long long need = (unsigned long long)(K * R * S * Cp) * es;
  if (dst_bytes < need) TB_FAIL(TRACEA_INVALID_PARAMS, "dst holds %llu bytes, the packed weights need %llu",
                                (unsigned long long)dst_bytes, need);
  DeviceGuard guard(w.device);
  launch_weight_pack(w.ptr, dst, es, K, C, R, S, S, Cp, w.stride, static_cast<cudaStream_t>(stream));
  packed_shape[0] = (uint64_t)K; packed_shape[1] = (uint64_t)Cp; packed_shape[2] = (uint64_t)R; packed_shape[3] = (uint64_t)S;
  packed_stride[0] = R * S * Cp; packed_stride[1] = 1; packed_stride[2] = S * Cp; packed_stride[3] = Cp;
}

void gemm_prepack_b_checked(const TraceaTensorView& bv, void* dst, uint64_t dst_bytes, int64_t* packed_stride,
                            void* stream) {
  if (bv.ptr == nullptr || dst == nullptr || packed_stride == nullptr)
    TB_FAIL(TRACEA_INVALID_PARAMS, "Null pointer in prepack arguments");
  const int es = elem_size(bv.dtype);
  if (es == 0) TB_FAIL(TRACEA_UNSUPPORTED_CONFIG, "Unsupported dtype %s", dtype_name(bv.dtype));
  const Rank2 b = load_rank2(bv, "b");
  if (b.shape[0] == 0 || b.shape[1] == 0) TB_FAIL(TRACEA_INVALID_PARAMS, "b must not be empty");
  if (bv.device_id < 0) TB_FAIL(TRACEA_INVALID_PARAMS, "prepacking takes device tensors (device_id >= 0)");
  if (!aligned16(dst)) TB_FAIL(TRACEA_INVALID_PARAMS, "dst must be 16-byte aligned");
  const long long K = b.shape[0], N = b.shape[1];
  const unsigned long long need = (unsigned long long)(K * N) * es;
  if (dst_bytes < need) TB_FAIL(TRACEA_INVALID_PARAMS, "dst holds %llu bytes, the packed matrix needs %llu",
                                (unsigned long long)dst_bytes, need);
  DeviceGuard guard(bv.device_id);
  const long long stride[4] = {b.stride[1], b.stride[0], 0, 0};   // filter bank [N, K, 1, 1]
  launch_weight_pack(bv.ptr, dst, es, N, K, 1, 1, 1, K, stride, static_cast<cudaStream_t>(stream));
  packed_stride[0] = 1;
  packed_stride[1] = K;
}

template <typename F>
TraceaStatus guarded(const char* what, F&& f) {
  // mirrors the catch_unwind wrapper of tracea-ffi/src/lib.rs:130-141: nothing escapes the C boundary
  try {
    f();
    return TRACEA_SUCCESS;
  } catch (const StatusError& e) {
    return e.status;
  } catch (const std::exception& e) {
    set_error("Exception in %s: %s", what, e.what());
    return TRACEA_UNKNOWN_ERROR;
  } catch (...) {
    set_error("Unknown exception in %s", what);
    return TRACEA_UNKNOWN_ERROR;
  }
}

}  // namespace

// ==================================================================== exported C ABI
extern "C" {

TraceaStatus tracea_conv2d(TraceaTensorView x, TraceaTensorView w, const TraceaTensorView* b,
                           const TraceaTensorView* residual, TraceaTensorView* out,
                           TraceaConv2dParams params) {
  return guarded("tracea_conv2d", [&] { conv2d_checked(x, w, b, residual, out, params); });
}

TraceaStatus tracea_conv2d_v0(TraceaTensorView x, TraceaTensorView w, const TraceaTensorView* b,
                              TraceaTensorView* out, TraceaConv2dParamsV0 params) {
  TraceaConv2dParams p;
  p.stride_h = params.stride_h;
  p.stride_w = params.stride_w;
  p.padding_h = params.padding_h;
  p.padding_w = params.padding_w;
  p.dilation_h = params.dilation_h;
  p.dilation_w = params.dilation_w;
  p.groups = params.groups;
  p.epilogue = b != nullptr ? TRACEA_EPILOGUE_BIAS_ADD : TRACEA_EPILOGUE_IDENTITY;
  p.stream = params.stream;
  return guarded("tracea_conv2d_v0", [&] { conv2d_checked(x, w, b, nullptr, out, p); });
}

TraceaStatus tracea_conv2d_noalloc(TraceaTensorView x, TraceaTensorView w, const TraceaTensorView* b,
                                   const TraceaTensorView* residual, TraceaTensorView* out,
                                   TraceaConv2dParams params) {
  return guarded("tracea_conv2d_noalloc", [&] { conv2d_checked(x, w, b, residual, out, params, true); });
}

TraceaStatus tracea_gemm(TraceaTensorView a, TraceaTensorView b, const TraceaTensorView* bias,
                         const TraceaTensorView* residual, TraceaTensorView* c, TraceaGemmParams params) {
  return guarded("tracea_gemm", [&] { gemm_checked(a, b, bias, residual, c, params); });
}

TraceaStatus tracea_conv_transpose2d(TraceaTensorView x, TraceaTensorView w, const TraceaTensorView* b,
                                     const TraceaTensorView* residual, TraceaTensorView* out,
                                     TraceaConvTranspose2dParams params) {
  return guarded("tracea_conv_transpose2d", [&] { conv_transpose2d_checked(x, w, b, residual, out, params); });
}

uint64_t tracea_conv2d_prepack_bytes(TraceaTensorView w) {
  const int es = elem_size(w.dtype);
  if (es == 0 || w.rank != 4 || w.shape == nullptr) return 0;
  return w.shape[0] * w.shape[2] * w.shape[3] * static_cast<uint64_t>(padded_channels((long long)w.shape[1], es)) * es;
}

TraceaStatus tracea_conv2d_prepack(TraceaTensorView w, void* dst, uint64_t dst_bytes, uint64_t packed_shape[4],
                                   int64_t packed_stride[4], void* stream) {
  return guarded("tracea_conv2d_prepack",
                 [&] { conv2d_prepack_checked(w, dst, dst_bytes, packed_shape, packed_stride, stream); });
}

uint64_t tracea_gemm_prepack_b_bytes(TraceaTensorView b) {
  const int es = elem_size(b.dtype);
  if (es == 0 || b.rank != 2 || b.shape == nullptr) return 0;
  return b.shape[0] * b.shape[1] * es;
}

TraceaStatus tracea_gemm_prepack_b(TraceaTensorView b, void* dst, uint64_t dst_bytes, int64_t packed_stride[2],
                                   void* stream) {
  return guarded("tracea_gemm_prepack_b", [&] { gemm_prepack_b_checked(b, dst, dst_bytes, packed_stride, stream); });
}

int32_t tracea_get_last_error(uint8_t* buf, size_t len) {
  if (buf == nullptr || len == 0) return -1;
  const size_t n = std::min(g_last_error.size(), len - 1);
  memcpy(buf, g_last_error.data(), n);
  buf[n] = 0;
  return static_cast<int32_t>(n);
}

void tracea_clear_error(void) { g_last_error.clear(); }

uint32_t tracea_version_major(void) { return 0; }
uint32_t tracea_version_minor(void) { return 1; }
uint32_t tracea_version_patch(void) { return 0; }

int tracea_init(void) {
  const TraceaStatus s = guarded("tracea_init", [&] {
    int count = 0;
    TB_CUDA(cudaGetDeviceCount(&count));
    if (count <= 0) TB_FAIL(TRACEA_CUDA_ERROR, "no CUDA device");
    int cur = 0;
    TB_CUDA(cudaGetDevice(&cur));
    device_state(cur);
  });
  return s == TRACEA_SUCCESS ? 0 : -1;
}

void tracea_shutdown(void) {
  for (int d = 0; d < kMaxDevices; ++d) {
    std::lock_guard<std::mutex> lock(g_dev_mu[d]);
    DeviceState& st = g_dev[d];
    if (!st.ready.load(std::memory_order_acquire)) continue;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(d);
    cudaDeviceSynchronize();
    if (st.copy_in != nullptr) {
      cudaStreamDestroy(st.copy_in);
      cudaStreamDestroy(st.copy_out);
      cudaEventDestroy(st.ev_entry);
      cudaEventDestroy(st.ev_done);
      for (int i = 0; i < DeviceState::kMaxChunks; ++i) {
        cudaEventDestroy(st.ev_in[i]);
        cudaEventDestroy(st.ev_out[i]);
      }
    }
    if (st.pool != nullptr) cudaMemPoolDestroy(st.pool);
    if (st.status != nullptr) cudaFreeHost(st.status);
    {
      std::lock_guard<std::mutex> ws_lock(st.ws_mu);
      for (auto& kv : st.split_ws) cudaFree(kv.second);
      st.split_ws.clear();
    }
    st.pool = nullptr;
    st.status = nullptr;
    st.copy_in = st.copy_out = nullptr;
    st.ev_entry = st.ev_done = nullptr;
    st.ready.store(false, std::memory_order_release);
    cudaSetDevice(prev);
  }
}

int32_t tracea_b200_conv_transpose_plan(uint32_t in_extent, uint32_t out_extent, uint32_t filter, uint32_t stride,
                                        uint32_t padding, int64_t* phases) {
  if (phases == nullptr || stride == 0 || stride > 16 || in_extent == 0 || filter == 0) return -1;
  for (uint32_t a0 = 0; a0 < stride; ++a0) {
    PhaseAxis ax = phase_axis(in_extent, out_extent, filter, stride, padding, a0);
    if (ax.T > 0 && ax.empty) make_empty_axis(ax, in_extent);
    int64_t* o = phases + 8 * a0;
    o[0] = ax.a0; o[1] = ax.T; o[2] = ax.a; o[3] = ax.taps; o[4] = ax.x_off; o[5] = ax.in; o[6] = ax.pad_lo; o[7] = ax.pad_hi;
    if (ax.T > 0 && ax.empty) o[2] = -1;   // no tap reaches this phase: its single tap is a zero
  }
  return static_cast<int32_t>(stride);
}

void tracea_b200_test_hooks(int64_t wait_limit_cycles, int32_t producer_stop_after) {
  g_test_wait_limit.store(wait_limit_cycles > 0 ? wait_limit_cycles : 0, std::memory_order_relaxed);
  g_test_producer_stop.store(producer_stop_after >= 0 ? producer_stop_after : -1, std::memory_order_relaxed);
}

uint64_t tracea_b200_launch_count(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

uint64_t tracea_b200_launch_count_of(int32_t kind) {
  if (kind < 0 || kind >= 5) return 0;
  return g_launches_by_kind[kind].load(std::memory_order_relaxed);
}

uint32_t tracea_b200_device_status(int32_t device_id) {
  if (device_id < 0 || device_id >= kMaxDevices) return 0;
  DeviceState& st = g_dev[device_id];
  uint32_t code = 0;
  if (st.ready.load(std::memory_order_acquire) && st.status != nullptr) {
    code = st.status[0];
    if (code != 0u) memset(st.status, 0, 4 * sizeof(uint32_t));
  }
  // the no-alloc entry's words are in device memory: a blocking copy, which is why this is a call to make after
  // synchronising and not on a latency path
  NoAllocState& na = g_noalloc[device_id];
  if (na.ready.load(std::memory_order_acquire) && na.status != nullptr) {
    int prev = -1;
    if (cudaGetDevice(&prev) == cudaSuccess && (prev == device_id || cudaSetDevice(device_id) == cudaSuccess)) {
      uint32_t words[4] = {0, 0, 0, 0};
      if (cudaMemcpy(words, na.status, sizeof(words), cudaMemcpyDeviceToHost) == cudaSuccess && words[0] != 0u) {
        if (code == 0u) code = words[0];
        cudaMemset(na.status, 0, sizeof(words));
      }
      if (prev != device_id) cudaSetDevice(prev);
    }
  }
  return code;
}

int32_t tracea_b200_pool_stats(int32_t device_id, uint64_t stats[4], int32_t reset_high) {
  if (device_id < 0 || device_id >= kMaxDevices || stats == nullptr) return -1;
  stats[0] = stats[1] = stats[2] = stats[3] = 0;
  DeviceState& st = g_dev[device_id];
  if (!st.ready.load(std::memory_order_acquire) || st.pool == nullptr) return 0;   // no pool yet: all zeros
  const cudaMemPoolAttr attrs[4] = {cudaMemPoolAttrReservedMemCurrent, cudaMemPoolAttrReservedMemHigh,
                                    cudaMemPoolAttrUsedMemCurrent, cudaMemPoolAttrUsedMemHigh};
  for (int i = 0; i < 4; ++i) {
    cuuint64_t v = 0;
    if (cudaMemPoolGetAttribute(st.pool, attrs[i], &v) != cudaSuccess) return -1;
    stats[i] = v;
  }
  if (reset_high != 0) {
    cuuint64_t zero = 0;
    cudaMemPoolSetAttribute(st.pool, cudaMemPoolAttrReservedMemHigh, &zero);
    cudaMemPoolSetAttribute(st.pool, cudaMemPoolAttrUsedMemHigh, &zero);
  }
  return 1;
}

}  // extern "C"
