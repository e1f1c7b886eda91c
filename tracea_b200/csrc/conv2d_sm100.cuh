// Implicit-GEMM Conv2d for sm_100a: TMA im2col loads -> smem ring -> tcgen05.mma -> TMEM ->
// fused bias / residual / activation epilogue.
//
// GEMM view (same as the reference kernel, src/emitter/cuda/conv.rs:40-41, 209-210):
//   M = N*Ho*Wo output pixels, Ngemm = K_out, Kgemm = R*S*C walked in (r, s, c) order.
//   A[m, k] = x[n, ho*stride - pad + r*dil, wo*stride - pad + s*dil, c]   (zero outside the image)
//   B[k, n] = w[n, r, s, c]
// Where the reference recovers (n, ho, wo) / (r, s, c) per 16-byte chunk with mul-shift divmods
// (conv.rs:144-151, 202-247), the TMA unit walks the pixels itself here: one im2col-mode copy
// brings 128 consecutive output pixels x one k-chunk of one filter tap into swizzled shared memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ptx_sm100.cuh"

// Role-level cycle accounting for kernel bring-up: compiled in only with -DTB200_PROFILE, in which
// case ConvKernelArgs::prof points at 16 counters per CTA (waits and totals per role).
#ifdef TB200_PROFILE
#define TB200_PROF_T(var) const long long var = clock64()
#define TB200_PROF_ADD(acc, t0) acc += clock64() - (t0)
#define TB200_PROF_STORE(idx, val) \
  if (args.prof != nullptr) args.prof[blockIdx.x * 16 + (idx)] = (val)
#define TB200_PROF_NOW(idx)                                                              \
  if (args.prof != nullptr && threadIdx.x == 0) {                                        \
    unsigned long long t_;                                                               \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                               \
    args.prof[blockIdx.x * 16 + (idx)] = static_cast<long long>(t_);                     \
  }
#else
#define TB200_PROF_NOW(idx)
#define TB200_PROF_T(var)
#define TB200_PROF_ADD(acc, t0)
#define TB200_PROF_STORE(idx, val)
#endif

namespace tb200 {

constexpr int kBlockM = 128;          // output pixels per tile = TMEM lanes
constexpr int kStageKBytes = 128;     // bytes of K per smem row per pipeline stage
constexpr int kNumThreads = 320;      // warp 0 TMA, warp 1 MMA, warps 2..5 and 6..9 two epilogue groups
constexpr int kNumThreadsRows2 = 352; // 256-row tiles of one CTA: warp 10 is a second MMA issuer (the tile's second block)
constexpr int kMaxStages = 12;
constexpr long long kWaitLimitCycles = 4000000000LL;  // default limit of one wait: ~2 s at 1.9 GHz (ConvKernelArgs::wait_limit)

// Device-side error codes written to ConvKernelArgs::status (0 = fine).
enum : uint32_t {
  kErrNone = 0,
  kErrProducerWait = 1,   // TMA producer: a stage never became free
  kErrMmaWaitFull = 2,    // MMA issuer: a stage's bytes never landed
  kErrMmaWaitTmem = 3,    // MMA issuer: accumulator never drained
  kErrEpilogueWait = 4,   // epilogue: accumulator never became ready
  kErrResidualWait = 5,   // epilogue: a residual box never landed
  kErrSplitWait = 6,      // epilogue: the partial sums of a tile split over K never all arrived
};

enum : int { kActNone = 0, kActRelu = 1, kActGelu = 2, kActSilu = 3 };

struct ConvKernelArgs {
  // problem
  int M;            // one past the last output pixel (row of the implicit GEMM) this launch owns
  int m_begin;      // first output pixel this launch owns: tile t covers rows m_begin + t * rows-per-tile ...
  int K_out;        // output channels
  int Ho, Wo;
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int S;            // filter width (taps per filter row)
  // k-chunking: one chunk = chunk_elems channels of one tap
  int chunk_elems;        // elements per chunk (chunk_bytes / element size)
  int chunk_bytes;        // 128, 64, 32 or 16
  int chunks_per_tap;     // C / chunk_elems
  int total_chunks;       // R * S * chunks_per_tap
  int C;                  // input channels (c coordinate >= C reads zeros)
  int a_tiled;            // 1: A is a plain [M][C] matrix (1x1, stride 1, no padding) read by tiled TMA
  // B's column (element index inside one output channel's weight row) of tap (r, s), channel c is
  // b_k0 + r * (row stride) + s * (tap stride) + c. The loader walks it incrementally: +chunk_elems per k-step,
  // +b_jump_s at every tap boundary, +b_jump_r more at every filter-row boundary. Dense [R][S][C] rows: all 0.
  // Non-zero jumps are only used with 128-byte chunks (one chunk per stage).
  int b_k0, b_jump_s, b_jump_r;
  // tiling / pipeline
  int num_m_tiles, num_n_tiles;
  int panel_width;  // column tiles per panel of the tile order (>= 1; num_n_tiles = one panel = row-major order)
  int panel_tiles;  // num_m_tiles * panel_width
  int num_stages;
  int shared_bias;  // 1: one bias copy per CTA (num_n_tiles == 1) instead of one per epilogue warp
  // Work schedule. Tiles [0, dp_tiles) are dealt whole to the workers (CTAs, or CTA pairs) round robin. The k-steps
  // of the remaining sk_tiles tiles -- the partly filled last wave of a large layer, or every tile of a layer with
  // fewer tiles than SMs -- are laid end to end and cut into equal shares for the first sk_workers workers, so a
  // tile may be computed by several workers, each over a slice of K. sk_tiles == 0: no tile is split.
  int dp_tiles, sk_tiles, sk_workers;
  float* sk_partials;       // fp32 partial accumulators: 2 slots per worker, sk_slot_floats each
  uint32_t* sk_counters;    // per split tile and epilogue warp: {tickets taken, partials written}; zero at launch
  long long sk_slot_floats;
  // tcgen05 descriptors (host-built constants)
  uint32_t idesc;
  uint32_t a_lbo, a_sbo, b_lbo, b_sbo, swizzle_mode;
  uint32_t a_mma_off[4];  // byte offset of each of the 4 MMAs' A operand inside a stage
  uint32_t b_mma_off[4];
  // epilogue
  // out / residual are addressed as base + n*sn + ho*sh + wo*sw + k*sc (element strides), so both
  // channels-last (sc == 1) and NCHW (sw == 1) memory are written without a transpose pass.
  void* out;
  long long out_sn, out_sh, out_sw, out_sc;
  int out_vec;            // sc == 1 and 16-byte vector stores are legal
  const void* bias;       // [K_out], fp32 or OutT
  int bias_is_f32;
  const void* residual;   // same dtype as out
  long long res_sn, res_sh, res_sw, res_sc;
  int res_vec;
  int act;
  int out_tma;            // 1: out is dense row-major [M][pitch] and is written by TMA stores
  int res_tma;            // 1: residual is dense row-major too and is TMA-loaded into the staging boxes
  // error reporting: 4 words {code, block, detail, 0}; first error wins
  uint32_t* status;
  long long wait_limit;   // cycles any single wait may take before the role gives up (args.wait_limit unless a test shortens it)
  int pdl_mode;           // 0: start the next launch, then wait for the previous one; 1 / 2: see the kernel
  int test_producer_stop; // test hook, -1 in normal use: the TMA producer stops issuing after this many stages and
                          // leaves normally, so that the waits downstream of it run out
  long long* prof;        // cycle counters, only written by -DTB200_PROFILE builds
};

template <typename T> struct OutTraits;
template <> struct OutTraits<__nv_bfloat16> {
  static constexpr bool kTf32 = false;
  static constexpr bool kIsBf16 = true;
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct OutTraits<__half> {
  static constexpr bool kTf32 = false;
  static constexpr bool kIsBf16 = false;
  __device__ static float to_f(__half v) { return __half2float(v); }
  __device__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct OutTraits<float> {
  static constexpr bool kTf32 = true;
  static constexpr bool kIsBf16 = false;
  __device__ static float to_f(float v) { return v; }
  __device__ static float from_f(float v) { return v; }
};

// Activation formulas follow src/kernels/gpu/epilogue.cuh:12-63 (fp32 math). The branch on the
// activation kind is taken once per 32-value block, not per value. For 16-bit outputs exp / tanh
// use the hardware approximations (error far below the output rounding); fp32 outputs keep the
// library functions.
template <bool kFast>
__device__ __forceinline__ void apply_act32(float (&f)[32], int act) {
  if (act == kActRelu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = fmaxf(0.0f, f[j]);
  } else if (act == kActSilu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if constexpr (kFast) f[j] = __fdividef(f[j], 1.0f + __expf(-f[j]));
      else f[j] = f[j] / (1.0f + expf(-f[j]));
    }
  } else if (act == kActGelu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float x = f[j];
      const float u = 0.79788456f * (x + 0.044715f * x * x * x);
      float t;
      if constexpr (kFast) asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
      else t = tanhf(u);
      f[j] = 0.5f * x * (1.0f + t);
    }
  }
}

// Records the first error of the device in `status` ({code, block, detail, 0}) and raises the CTA's abort flag.
__device__ __forceinline__ void report_error_status(uint32_t* status, volatile uint32_t* abort_flag, uint32_t code,
                                                    uint32_t detail) {
  *abort_flag = 1u;
  if (status != nullptr && atomicCAS(status, 0u, code) == 0u) {
    status[1] = blockIdx.x;
    status[2] = detail;
    __threadfence_system();
  }
}
__device__ __forceinline__ void report_error(const ConvKernelArgs& a, volatile uint32_t* abort_flag,
                                             uint32_t code, uint32_t detail) {
  report_error_status(a.status, abort_flag, code, detail);
}

// Shared memory map (offsets from a 1024-byte aligned base):
//   [0, stages * stage_bytes)        operand ring: per stage A (128 rows x 128 B) then B (BN rows x 128 B)
//   + kStagingBytes                  per epilogue warp 2 alternating 4 KB boxes (32 pixels x 128 B): the residual
//                                    is TMA-loaded into a box, combined in place, and the box is TMA-stored
//   + 8 * BN * 4                     per-epilogue-warp copy of the tile's bias, as fp32 (one BN * 4 copy for the
//                                    whole CTA when the output is a single tile wide: the bias never changes)
//   + 256                            mbarriers, TMEM base slot, abort flag
constexpr int kStagingBoxBytes = 32 * 128;
constexpr int kStagingDepth = 2;
constexpr int kNumEpilogueWarps = 8;
constexpr int kStagingBytes = kNumEpilogueWarps * kStagingDepth * kStagingBoxBytes;
// `pair`: two CTAs on neighbouring SMs work on one 256-row tile and each holds only half of B's rows.
// `rows2`: one CTA owns a 256-row tile (two 128-row blocks of A per stage against one B).
__host__ __device__ constexpr int conv_smem_bytes(int bn, int stages, bool pair = false, bool rows2 = false,
                                                  bool shared_bias = false) {
  return stages * ((rows2 ? 2 : 1) * kBlockM * kStageKBytes + (pair ? bn / 2 : bn) * kStageKBytes) + kStagingBytes +
         (shared_bias ? 1 : kNumEpilogueWarps) * bn * 4 + 512 + 1024;
}

// 8 consecutive fp32 values -> one 16-byte vector of OutT (16-bit types) / 4 values (fp32).
template <typename OutT>
__device__ __forceinline__ uint4 pack16(const float* f) {
  uint4 r;
  if constexpr (sizeof(OutT) == 4) {
    r.x = __float_as_uint(f[0]); r.y = __float_as_uint(f[1]);
    r.z = __float_as_uint(f[2]); r.w = __float_as_uint(f[3]);
  } else {
    OutT* e = reinterpret_cast<OutT*>(&r);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = OutTraits<OutT>::from_f(f[j]);
  }
  return r;
}

// (a, b) += (c, d) as one packed fp32x2 add.
__device__ __forceinline__ void add2(float& a, float& b, float c, float d) {
  asm("{\n"
      ".reg .b64 x, y;\n"
      "mov.b64 x, {%0, %1};\n"
      "mov.b64 y, {%2, %3};\n"
      "add.rn.f32x2 x, x, y;\n"
      "mov.b64 {%0, %1}, x;\n"
      "}\n"
      : "+f"(a), "+f"(b)
      : "f"(c), "f"(d));
}

// Two consecutive fp32 values -> one packed word of the 16-bit output type (element 0 in the low
// half), optionally with ReLU folded into the conversion instruction.
template <typename OutT, bool kRelu>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if constexpr (sizeof(OutT) == 2 && OutTraits<OutT>::kIsBf16) {
    if constexpr (kRelu) asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    if constexpr (kRelu) asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

// One packed word of the 16-bit type -> two fp32 values.
template <typename OutT>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
  if constexpr (OutTraits<OutT>::kIsBf16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
}

// 32 fp32 values (acc + bias [+ residual from 16-byte chunks]) -> packed output chunks, for the TMA
// epilogue. 16-bit outputs: kChunks = 4 chunks of 8; fp32 outputs: 8 chunks of 4.
template <typename OutT, bool kRelu>
__device__ __forceinline__ void finish32(float (&f)[32], const uint4* res_chunks, bool has_res, uint4* packed) {
  if constexpr (sizeof(OutT) == 2) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (has_res) {
        const uint4 r = res_chunks[c];
        float lo, hi;
        unpack2<OutT>(r.x, lo, hi); add2(f[c * 8 + 0], f[c * 8 + 1], lo, hi);
        unpack2<OutT>(r.y, lo, hi); add2(f[c * 8 + 2], f[c * 8 + 3], lo, hi);
        unpack2<OutT>(r.z, lo, hi); add2(f[c * 8 + 4], f[c * 8 + 5], lo, hi);
        unpack2<OutT>(r.w, lo, hi); add2(f[c * 8 + 6], f[c * 8 + 7], lo, hi);
      }
      packed[c].x = pack2<OutT, kRelu>(f[c * 8 + 0], f[c * 8 + 1]);
      packed[c].y = pack2<OutT, kRelu>(f[c * 8 + 2], f[c * 8 + 3]);
      packed[c].z = pack2<OutT, kRelu>(f[c * 8 + 4], f[c * 8 + 5]);
      packed[c].w = pack2<OutT, kRelu>(f[c * 8 + 6], f[c * 8 + 7]);
    }
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (has_res) {
        const uint4 r = res_chunks[c];
        add2(f[c * 4 + 0], f[c * 4 + 1], __uint_as_float(r.x), __uint_as_float(r.y));
        add2(f[c * 4 + 2], f[c * 4 + 3], __uint_as_float(r.z), __uint_as_float(r.w));
      }
      if constexpr (kRelu) {
#pragma unroll
        for (int j = 0; j < 4; ++j) f[c * 4 + j] = fmaxf(0.0f, f[c * 4 + j]);
      }
      packed[c] = make_uint4(__float_as_uint(f[c * 4 + 0]), __float_as_uint(f[c * 4 + 1]),
                             __float_as_uint(f[c * 4 + 2]), __float_as_uint(f[c * 4 + 3]));
    }
  }
}

template <typename OutT>
__device__ __forceinline__ void add16(float* f, const uint4& raw) {
  constexpr int kVec = 16 / sizeof(OutT);
  const OutT* e = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
  for (int j = 0; j < kVec; ++j) f[j] += OutTraits<OutT>::to_f(e[j]);
}

// Out-of-line path for outputs / residuals the TMA boxes cannot address (NCHW or irregular
// strides, K_out not a multiple of the vector width): finishes one 32-column block of one pixel --
// residual, activation, store. `f` holds accumulator + bias. Kept out of line so that the common
// path's instruction footprint stays small.
template <typename OutT>
__device__ __noinline__ void epilogue_block_generic(const ConvKernelArgs& args, float* f, const OutT* res_px,
                                                    OutT* out_px, int n_first, bool row_ok) {
  constexpr int kVec = 16 / sizeof(OutT);
  if (res_px != nullptr && row_ok) {
    if (args.res_vec) {
#pragma unroll
      for (int c = 0; c < 32 / kVec; ++c)
        if (n_first + c * kVec < args.K_out) add16<OutT>(f + c * kVec, __ldg(reinterpret_cast<const uint4*>(res_px) + c));
    } else {
#pragma unroll 4
      for (int j = 0; j < 32; ++j)
        if (n_first + j < args.K_out) f[j] += OutTraits<OutT>::to_f(res_px[j * args.res_sc]);
    }
  }
  apply_act32<sizeof(OutT) == 2>(*reinterpret_cast<float(*)[32]>(f), args.act);
  if (!row_ok) return;
  if (args.out_vec) {
#pragma unroll
    for (int c = 0; c < 32 / kVec; ++c)
      if (n_first + c * kVec < args.K_out) reinterpret_cast<uint4*>(out_px)[c] = pack16<OutT>(f + c * kVec);
  } else {
    // lanes are consecutive pixels: for NCHW memory (sw == 1) each store instruction is coalesced
#pragma unroll 4
    for (int j = 0; j < 32; ++j)
      if (n_first + j < args.K_out) out_px[j * args.out_sc] = OutTraits<OutT>::from_f(f[j]);
  }
}

// kPair: launched as clusters of two CTAs (cta_group::2). The pair owns a 256 x BN tile: each CTA loads its own
// 128 pixels of A and its own half of B's rows (no multicast), the leader CTA issues M = 256 MMAs that span both
// SMs, each CTA drains its own 128 TMEM lanes. Per CTA this halves the B bytes brought in per MMA.
// kRows2 (single CTA, narrow outputs): the CTA owns a 256 x BN tile as two 128-row blocks with one accumulator
// each; a stage carries both A blocks and one B; two warps issue the MMAs, one block each (a single thread issues
// too slowly for MMAs this narrow), and the two epilogue groups drain the two halves of the same tile instead of
// alternate tiles.
// Staging box (32 pixel rows x 128 bytes, SWIZZLE_128B layout: 16-byte chunk c of row r at r*128 + ((c ^ (r & 7)) << 4))
// <-> global memory, moved by the warp itself for outputs the TMA unit cannot address as one matrix. Lane l handles
// chunk l & 7 of rows (l >> 3) + 4 i, so each instruction covers four whole 128-byte rows. `row_base` points at the
// first element of the group's columns in pixel 0's row; `row_off` is this lane's own pixel offset (in elements),
// `row_ok` whether its pixel exists; `cols_left` = K_out - first column of the group. Only instantiated in the kCoop kernels.
template <typename OutT>
__device__ __noinline__ void coop_store_box(uint32_t stg, OutT* row_base, long long row_off, bool row_ok, int cols_left,
                                            int lane) {
  constexpr int kVec = 16 / sizeof(OutT);
  __syncwarp();   // every lane's row is in the box
  const uint32_t ok_rows = __ballot_sync(0xffffffffu, row_ok);
  const uint32_t chunk = static_cast<uint32_t>(lane) & 7u;
  const bool chunk_ok = static_cast<int>(chunk) * kVec < cols_left;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    const long long off = __shfl_sync(0xffffffffu, row_off, r);
    const uint4 v = ptx::ld_shared_v4(stg + static_cast<uint32_t>(r) * 128u + ((chunk ^ (static_cast<uint32_t>(r) & 7u)) << 4));
    if (chunk_ok && ((ok_rows >> r) & 1u)) *(reinterpret_cast<uint4*>(row_base + off) + chunk) = v;
  }
  __syncwarp();   // the box may be rewritten once every lane has read it out
}

template <typename OutT>
__device__ __noinline__ void coop_load_box(uint32_t stg, const OutT* row_base, long long row_off, bool row_ok,
                                           int cols_left, int lane) {
  constexpr int kVec = 16 / sizeof(OutT);
  const uint32_t ok_rows = __ballot_sync(0xffffffffu, row_ok);
  const uint32_t chunk = static_cast<uint32_t>(lane) & 7u;
  const bool chunk_ok = static_cast<int>(chunk) * kVec < cols_left;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    const long long off = __shfl_sync(0xffffffffu, row_off, r);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (chunk_ok && ((ok_rows >> r) & 1u)) v = __ldg(reinterpret_cast<const uint4*>(row_base + off) + chunk);
    ptx::st_shared_v4(stg + static_cast<uint32_t>(r) * 128u + ((chunk ^ (static_cast<uint32_t>(r) & 7u)) << 4), v);
  }
  __syncwarp();   // rows were written by other lanes than the ones that read them next
}

// One unit of work of a worker: k-steps [k_begin, k_end) of tile `tile`. A whole tile has k_begin == 0 and
// k_end == k_iters; anything else is one piece of a tile that is split over K between several workers.
struct WorkItem {
  int tile, k_begin, k_end;
};

// Split region: `total` k-steps (sk_tiles * k_iters, kept below 2^30 by the host) shared by `workers` workers;
// worker w owns [w * total / workers, (w + 1) * total / workers).
__device__ __forceinline__ int sk_share_begin(int total, int workers, int w) {
  return static_cast<int>(static_cast<long long>(w) * total / workers);
}
// The worker whose share contains position `pos` (the largest w with sk_share_begin(w) <= pos).
__device__ __forceinline__ int sk_owner_of(int total, int workers, int pos) {
  return static_cast<int>(((static_cast<long long>(pos) + 1) * workers - 1) / total);
}

// Walks a worker's items in the order every role of the CTA follows: first the pieces its share of the split
// region cuts off (the tail of the tile the share starts in, the head of the tile it ends in: at most two, both
// short), then the whole tiles of the share, then its whole tiles of the rest. The pieces come first so that the
// exchange of partial sums and their short main loops sit in front of long main loops that hide them -- a short
// item between two long ones would leave the tensor pipe waiting for an accumulator to drain.
struct WorkIter {
  int sk_b, sk_e;           // this worker's share of the split region [sk_b, sk_e), in k-steps
  int idx;                  // items handed out so far
  int whole_next;           // next whole tile of the share (index inside the split region)
  int dp_next;              // next whole tile outside the split region
  template <bool kSplit>
  __device__ __forceinline__ void init(const ConvKernelArgs& a, int worker, int k_iters) {
    sk_b = sk_e = 0;
    if (kSplit && a.sk_tiles > 0 && worker < a.sk_workers) {
      const int total = a.sk_tiles * k_iters;
      sk_b = sk_share_begin(total, a.sk_workers, worker);
      sk_e = sk_share_begin(total, a.sk_workers, worker + 1);
    }
    idx = 0;
    whole_next = (sk_b + k_iters - 1) / k_iters;
    dp_next = worker;
  }
  template <bool kSplit>
  __device__ __forceinline__ bool next(WorkItem& it, const ConvKernelArgs& a, int num_workers, int k_iters) {
    if constexpr (kSplit) {
      if (sk_b < sk_e) {
        const int tb = sk_b / k_iters, te = sk_e / k_iters;          // tiles the share starts / ends in
        const int kb = sk_b - tb * k_iters, ke = sk_e - te * k_iters;
        const bool has_tail = kb != 0;                               // [sk_b, end of tile tb) -- or [sk_b, sk_e)
        const bool has_head = ke != 0 && !(has_tail && te == tb);    // [start of tile te, sk_e)
        const int n_pieces = (has_tail ? 1 : 0) + (has_head ? 1 : 0);
        if (idx < n_pieces) {
          if (idx == 0 && has_tail) {
            it.tile = a.dp_tiles + tb;
            it.k_begin = kb;
            it.k_end = te == tb ? ke : k_iters;
          } else {
            it.tile = a.dp_tiles + te;
            it.k_begin = 0;
            it.k_end = ke;
          }
          ++idx;
          return true;
        }
        if (whole_next < te) {
          it.tile = a.dp_tiles + whole_next++;
          it.k_begin = 0;
          it.k_end = k_iters;
          ++idx;
          return true;
        }
      }
    }
    if (dp_next < a.dp_tiles) {
      it.tile = dp_next;
      it.k_begin = 0;
      it.k_end = k_iters;
      dp_next += num_workers;
      ++idx;
      return true;
    }
    return false;
  }
};

// Slot `end` (1: the piece starts at the tile's first k-step) of worker w in the partial-sum scratch. Inside a
// slot: [epilogue-warp position 0..7][32-column chunk][8][lane] float4, so that every load / store instruction of
// a warp covers 512 contiguous bytes.
__device__ __forceinline__ float4* sk_slot(const ConvKernelArgs& a, int w, int end) {
  return reinterpret_cast<float4*>(a.sk_partials + (2LL * w + end) * a.sk_slot_floats);
}

// ---- exchange of partial sums between the pieces of a tile that is split over K (one epilogue warp's part: the
// warp owns 32 rows x `chunks` * 32 columns of the accumulator at TMEM address taddr0). Every piece takes a ticket
// per warp position. All but the last ticket write their fp32 accumulators to their slot of the scratch
// (sk_dump_partial), hand the TMEM buffer back and count themselves done. The last ticket keeps its accumulator,
// waits until the others are done -- they all hold earlier tickets, so they are running their stores right now
// and wait for nobody: no piece ever waits for a CTA that is not running -- then adds the partial sums in piece
// order (its own taken at its position, so the result does not depend on which piece came last), writes the total
// back to TMEM (sk_reduce_two / sk_reduce_many) and runs the ordinary epilogue on it. The counters are left at
// zero for the next launch. Each step is a function of its own, out of line: the kernel has 168 registers per
// thread and a spilled register goes all the way to L2 (shared memory leaves the L1 almost no room), so neither
// the epilogue nor any of these may be made to spill by the others.

// Writes the warp's accumulator to `dst` (this lane's first float4 of the warp's region of a slot) and hands the
// TMEM buffer back (arrive on `release_bar`, a shared::cluster address when kPair) once the last chunk is in registers.
template <bool kPair>
__device__ __noinline__ void sk_dump_partial(uint32_t taddr0, int chunks, float4* dst, uint32_t release_bar, int lane) {
  using namespace ptx;
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(taddr0 + c * 32, v);
    tmem_ld_wait();
    if (c == chunks - 1) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) mbar_arrive_cluster(release_bar);
        else mbar_arrive(release_bar);
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q)
      __stcg(dst + (c * 8 + q) * 32,
             make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                         __uint_as_float(v[4 * q + 3])));
  }
}

// Lane 0 waits until `expected` other pieces have counted themselves done on cnt[1], then zeroes the tile's two
// counters (every party has passed both by then). False when the wait gave up.
__device__ __noinline__ bool sk_wait_partials(uint32_t* cnt, uint32_t expected, volatile uint32_t* abort_flag,
                                              long long limit_cycles, int lane) {
  bool all_in = true;
  if (lane == 0) {
    const long long t_start = clock64();
    uint32_t spins = 0;
    while (ptx::ld_acquire_gpu(cnt + 1) != expected) {
      if ((++spins & 0xffu) == 0 && (*abort_flag != 0u || clock64() - t_start > limit_cycles)) {
        all_in = false;
        break;
      }
    }
    if (all_in) {
      cnt[0] = 0u;
      cnt[1] = 0u;
    }
  }
  // lane 0's acquire load, then the warp-wide vote: the other lanes' reads below come after both
  all_in = __all_sync(0xffffffffu, all_in);
  return all_in;
}

// Two pieces (a split region of more than one wave never cuts a tile into more): own + other, which is the same
// number whichever of the two does the adding. `src` is this lane's first float4 of the other piece's values; the
// block of the next chunk is in flight while this chunk is added and written back.
__device__ __noinline__ void sk_reduce_two(uint32_t taddr0, int chunks, const float4* src) {
  using namespace ptx;
  float4 nb[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) nb[q] = __ldcg(src + q * 32);
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(taddr0 + c * 32, v);
    float4 cur[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) cur[q] = nb[q];
    if (c + 1 < chunks) {
#pragma unroll
      for (int q = 0; q < 8; ++q) nb[q] = __ldcg(src + (c + 1) * 256 + q * 32);
    }
    tmem_ld_wait();
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + cur[q].x);
      v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + cur[q].y);
      v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + cur[q].z);
      v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + cur[q].w);
    }
    tmem_st_32x32(taddr0 + c * 32, v);
  }
  tmem_st_wait();
}

// Any number of pieces, added in piece order: pieces 0 .. me-1 from scratch, this piece's own values from TMEM,
// pieces me+1 .. from scratch. `first` is the worker of piece 0, `warp_off` the lane's float4 offset inside a slot.
// (One block of 32 columns is fetched while the previous one is added; layers with fewer tiles than SMs, whose
// tiles are cut into three or more pieces, come through here.)
__device__ __noinline__ void sk_reduce_many(const ConvKernelArgs& a, uint32_t taddr0, int chunks, int first, int pieces,
                                            int me, long long warp_off) {
  using namespace ptx;
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    float acc[32];
    float4 nb[8];
    // a tile's first piece starts at k-step 0 (slot end 1); every later piece is the head of its worker's share
    auto fetch = [&](int pc) {
      const float4* src = sk_slot(a, first + pc, pc == 0 ? 1 : 0) + warp_off + c * 256;
#pragma unroll
      for (int q = 0; q < 8; ++q) nb[q] = __ldcg(src + q * 32);
    };
    auto own_values = [&](bool init) {
      uint32_t v[32];
      tmem_ld_32x32(taddr0 + c * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = init ? __uint_as_float(v[j]) : acc[j] + __uint_as_float(v[j]);
    };
    if (me != 0) fetch(0);
#pragma unroll 1
    for (int pc = 0; pc < pieces; ++pc) {
      if (pc == me) {
        own_values(pc == 0);
        if (pc == 0 && pieces > 1) fetch(1);
        continue;
      }
      float4 cur[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) cur[q] = nb[q];
      const int nxt = pc + 1 == me ? pc + 2 : pc + 1;   // next piece that comes from scratch
      if (nxt < pieces) fetch(nxt);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (pc == 0) {
          acc[4 * q] = cur[q].x; acc[4 * q + 1] = cur[q].y; acc[4 * q + 2] = cur[q].z; acc[4 * q + 3] = cur[q].w;
        } else {
          acc[4 * q] += cur[q].x; acc[4 * q + 1] += cur[q].y; acc[4 * q + 2] += cur[q].z; acc[4 * q + 3] += cur[q].w;
        }
      }
    }
    uint32_t v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(acc[j]);
    tmem_st_32x32(taddr0 + c * 32, v);
  }
  tmem_st_wait();
}

// kSplit: the launch cuts some tiles over K (ConvKernelArgs::sk_tiles > 0). A separate instantiation, so that the
// launches that split nothing -- most of them -- carry none of the exchange code: the call to it alone costs the
// epilogue registers, and a spilled register here goes all the way to L2.
template <typename OutT, int BN, bool kPair, bool kRows2, bool kCoop, bool kSplit>
__global__ void __launch_bounds__(kRows2 ? kNumThreadsRows2 : kNumThreads, 1)
conv2d_igemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_x,
                          const __grid_constant__ CUtensorMap tmap_w,
                          const __grid_constant__ CUtensorMap tmap_out,
                          const __grid_constant__ CUtensorMap tmap_res,
                          const __grid_constant__ ConvKernelArgs args) {
  using namespace ptx;
  static_assert(!(kPair && kRows2), "one tiling variant at a time");
  static_assert(!kRows2 || BN <= 128, "two accumulator pairs of a 256-row tile must fit 512 TMEM columns");
  constexpr uint32_t kABlockBytes = kBlockM * kStageKBytes;            // one 128-pixel block of A: 16 KB
  constexpr uint32_t kABytes = (kRows2 ? 2u : 1u) * kABlockBytes;
  constexpr uint32_t kBRows = kPair ? BN / 2 : BN;       // rows of B this CTA keeps in shared memory
  constexpr uint32_t kBBytes = kBRows * kStageKBytes;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr int kTileM = (kPair || kRows2) ? 2 * kBlockM : kBlockM;   // output pixels per tile
  const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0u;
  // tiles are dealt to CTAs (or CTA pairs) round robin
  const int worker = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int num_workers = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr uint32_t kAccCols = (kRows2 ? 2 : 1) * BN;   // TMEM columns of one tile's accumulator(s)
  constexpr uint32_t kTmemCols = 2 * kAccCols;           // double-buffered: 128, 256 or 512 columns
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN");

  TB200_PROF_NOW(12);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int num_stages = args.num_stages;
  const uint32_t ring_bytes = static_cast<uint32_t>(num_stages) * kStageBytes;
  const uint32_t staging_base = smem_base + ring_bytes;
  const uint32_t bias_off = ring_bytes + kStagingBytes;
  const uint32_t bar_off = bias_off + (args.shared_bias ? 1u : static_cast<uint32_t>(kNumEpilogueWarps)) * BN * 4u;
  const uint32_t bar_base = smem_base + bar_off;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + 2 + b); };
  auto res_bar = [&](int q, int b) { return bar_base + 8u * (2 * kMaxStages + 4 + q * kStagingDepth + b); };
  constexpr uint32_t kNumBars = 2 * kMaxStages + 4 + kNumEpilogueWarps * kStagingDepth;
  const uint32_t tmem_slot = bar_base + 8u * kNumBars;
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(smem_gen + bar_off + 8u * kNumBars);
  volatile uint32_t* abort_p = tmem_slot_p + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kRows2 ? 2 : 1);   // one commit per MMA-issuing warp
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), kRows2 ? 2 : 1);
      // one arrival per epilogue warp that drains the buffer: 4, or 8 when both groups / both CTAs of a pair do
      mbar_init(tempty_bar(b), (kPair || kRows2) ? 8 : 4);
    }
    for (int q = 0; q < kNumEpilogueWarps; ++q)
      for (int b = 0; b < kStagingDepth; ++b) mbar_init(res_bar(q, b), 1);
    *abort_p = 0u;
    fence_mbar_init();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_w);
    if (args.out_tma) prefetch_tmap(&tmap_out);
    if (args.res_tma) prefetch_tmap(&tmap_res);
  }
  if (warp == 1) {
    if constexpr (kPair) {
      tmem_alloc_pair<kTmemCols>(tmem_slot);
      tmem_relinquish_pair();
    } else {
      tmem_alloc<kTmemCols>(tmem_slot);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (kPair) cluster_sync();   // the peer's barriers are initialised before anything signals them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;
  // Everything above touched only this CTA's shared memory, TMEM and the kernel's own parameters, so under a
  // programmatic dependent launch it overlaps the tail of the previous kernel on the stream. From here on global
  // memory is read and written: wait for that kernel to finish (a no-op without such a dependency). The next
  // kernel may be scheduled onto SMs as this grid's CTAs leave them; it waits at the same point.
  // pdl_mode 1 / 2: a chain of launches that do not depend on each other (the phases of a transposed convolution).
  // Its head waits BEFORE it lets the next launch start; the members after it start without waiting -- whatever
  // came before the chain is complete by then -- so their CTAs fill the SMs the previous member's last wave leaves
  // idle, and wait at their very end instead, which keeps the launches completing in stream order.
  if (args.pdl_mode == 1) {
    griddep_wait();
    griddep_launch_dependents();
  } else {
    griddep_launch_dependents();
    if (args.pdl_mode != 2) griddep_wait();
  }
  TB200_PROF_NOW(13);

  const int chunks_per_stage = kStageKBytes / args.chunk_bytes;
  const int k_iters = (args.total_chunks + chunks_per_stage - 1) / chunks_per_stage;
  // Tile order: the output is cut into panels of `panel_width` column tiles; inside a panel tiles run row by row.
  // One wave of CTAs then works on a block of rows x panel_width columns whose A rows and B columns stay in L2
  // (with a single panel -- panel_width = num_n_tiles -- this is plain row-major order). Two divisions per tile.
  auto tile_coords = [&](int tile, int& mt, int& nt) {
    const int panel = tile / args.panel_tiles;
    const int rem = tile - panel * args.panel_tiles;
    const int n0 = panel * args.panel_width;
    const int width = min(args.panel_width, args.num_n_tiles - n0);
    mt = rem / width;
    nt = n0 + rem - mt * width;
  };
  const uint32_t full_bar0 = bar_base, empty_bar0 = bar_base + 8u * kMaxStages;
  const uint32_t full_leader0 = kPair ? mapa_cluster(full_bar0, 0u) : full_bar0;   // leader's full barriers
  const uint32_t ring_end = smem_base + ring_bytes;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // One thread; the loop body is kept to a handful of instructions per stage, because at
    // 256 cycles of tensor work per stage (BN = 128) the issuing thread itself can become the limit.
    if (lane == 0) {
      uint32_t stage_addr = smem_base;             // A buffer of the current stage
      uint32_t full_addr = full_bar0, empty_addr = empty_bar0;
      uint32_t phase = 0;
      const uint32_t a_chunk_bytes = kBlockM * args.chunk_bytes;
      const uint32_t b_chunk_bytes = BN * args.chunk_bytes;
      const bool one_chunk = (chunks_per_stage == 1) && !args.a_tiled;
      bool ok = true;
      int issued = 0;
      int m_tile = 0, n_tile = 0;
      long long prof_wait = 0;
      (void)prof_wait;
      TB200_PROF_T(prof_t0);
      bool slot_free = mbar_test_wait(empty_addr, phase ^ 1u);
      WorkIter witer;
      witer.template init<kSplit>(args, worker, k_iters);
      WorkItem item;
      bool stopped = false;
      while (ok && !stopped && witer.template next<kSplit>(item, args, num_workers, k_iters)) {
        tile_coords(item.tile, m_tile, n_tile);
        const int m0 = args.m_begin + m_tile * kTileM + static_cast<int>(cta_rank) * kBlockM;   // this CTA's 128 pixels
        const int q0 = m0 % args.Wo;
        const int t = m0 / args.Wo;
        const int p0 = t % args.Ho;
        const int img0 = t / args.Ho;
        const int w_start = q0 * args.stride_w - args.pad_w;
        const int h_start = p0 * args.stride_h - args.pad_h;
        const int n_coord = n_tile * BN + static_cast<int>(cta_rank * kBRows);   // this CTA's rows of B
        int w_start1 = 0, h_start1 = 0, img1 = 0;   // start pixel of the tile's second 128-row block
        if constexpr (kRows2) {
          const int m1 = m0 + kBlockM;
          const int t1 = m1 / args.Wo;
          w_start1 = (m1 % args.Wo) * args.stride_w - args.pad_w;
          h_start1 = (t1 % args.Ho) * args.stride_h - args.pad_h;
          img1 = t1 / args.Ho;
        }
        if (one_chunk) {
          // common case: one 128-byte chunk per stage = 64 (16-bit) or 32 (fp32) channels of one tap.
          // Position of k-step k_begin: tap (r, s), channel chunk cc (a whole tile starts at 0, 0, 0)
          int c_coord = 0, k_coord = args.b_k0, tap_s = 0;
          uint32_t off_w = 0, off_h = 0;
          if (item.k_begin != 0) {
            const int tap = item.k_begin / args.chunks_per_tap;
            const int cc = item.k_begin - tap * args.chunks_per_tap;
            const int tap_r = tap / args.S;
            tap_s = tap - tap_r * args.S;
            c_coord = cc * args.chunk_elems;
            off_w = static_cast<uint32_t>(tap_s * args.dil_w);
            off_h = static_cast<uint32_t>(tap_r * args.dil_h);
            k_coord += item.k_begin * args.chunk_elems + tap * args.b_jump_s + tap_r * args.b_jump_r;
          }
          for (int it = item.k_begin; it < item.k_end; ++it) {
            if (issued == args.test_producer_stop) {   // test hook: go silent, leave normally
              stopped = true;
              break;
            }
            TB200_PROF_T(tw);
            if (!slot_free && !mbar_wait_bounded(empty_addr, phase ^ 1u, abort_p, args.wait_limit)) {
              report_error(args, abort_p, kErrProducerWait, (uint32_t)it);
              ok = false;
              break;
            }
            TB200_PROF_ADD(prof_wait, tw);
            // probe the next slot now; the answer is read at the top of the next iteration
            uint32_t nstage = stage_addr + kStageBytes, nfull = full_addr + 8u, nempty = empty_addr + 8u, nphase = phase;
            if (nstage == ring_end) { nstage = smem_base; nfull = full_bar0; nempty = empty_bar0; nphase ^= 1u; }
            bool next_free;
            if constexpr (kPair) {
              // both CTAs' copies complete on the leader's full barrier; the leader arms it for both
              next_free = tma_stage_probe_pair(stage_addr, stage_addr + kABytes, full_addr,
                                               full_leader0 + (full_addr - full_bar0), leader ? 2u * kStageBytes : 0u,
                                               &tmap_x, c_coord, w_start, h_start, img0, (uint16_t)off_w,
                                               (uint16_t)off_h, &tmap_w, k_coord, n_coord, nempty, nphase ^ 1u);
            } else if constexpr (kRows2) {
              next_free = tma_stage_probe_rows2(stage_addr, stage_addr + kABlockBytes, stage_addr + kABytes, full_addr,
                                                kStageBytes, &tmap_x, c_coord, w_start, h_start, img0, w_start1,
                                                h_start1, img1, (uint16_t)off_w, (uint16_t)off_h, &tmap_w, k_coord,
                                                n_coord, nempty, nphase ^ 1u);
            } else {
              next_free = tma_stage_probe(stage_addr, stage_addr + kABytes, full_addr, kStageBytes, &tmap_x, c_coord,
                                          w_start, h_start, img0, (uint16_t)off_w, (uint16_t)off_h, &tmap_w, k_coord,
                                          n_coord, nempty, nphase ^ 1u);
            }
            k_coord += args.chunk_elems;
            c_coord += args.chunk_elems;
            if (c_coord == args.C) {
              c_coord = 0;
              off_w += args.dil_w;
              k_coord += args.b_jump_s;
              if (++tap_s == args.S) { tap_s = 0; off_w = 0; off_h += args.dil_h; k_coord += args.b_jump_r; }
            }
            ++issued;
            stage_addr = nstage; full_addr = nfull; empty_addr = nempty; phase = nphase;
            slot_free = next_free;
          }
        } else {
          // narrow k-chunks (several per stage): whole tiles only, the host never splits these over K
          int chunk = 0, tap_r = 0, tap_s = 0, cc = 0;
          for (int it = 0; it < k_iters; ++it) {
            if (!mbar_wait_bounded(empty_addr, phase ^ 1u, abort_p, args.wait_limit)) {
              report_error(args, abort_p, kErrProducerWait, (uint32_t)it);
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(full_addr, kStageBytes);
            const uint32_t a_dst = stage_addr;
            const uint32_t b_dst = a_dst + kABytes;
            for (int j = 0; j < chunks_per_stage; ++j, ++chunk) {
              // chunks past the end of Kgemm read zeros: channel coordinate C / column Kgemm are out of range
              const bool pad_chunk = chunk >= args.total_chunks;
              const int c_coord = pad_chunk ? args.C : cc * args.chunk_elems;
              const int k_coord = pad_chunk ? args.total_chunks * args.chunk_elems
                                            : chunk * args.chunk_elems;
              if (args.a_tiled) {
                tma_load_2d(a_dst + j * a_chunk_bytes, &tmap_x, full_addr, c_coord, m0);
              } else {
                tma_load_im2col_4d(a_dst + j * a_chunk_bytes, &tmap_x, full_addr, c_coord,
                                   w_start, h_start, img0, (uint16_t)(tap_s * args.dil_w),
                                   (uint16_t)(tap_r * args.dil_h));
              }
              tma_load_2d(b_dst + j * b_chunk_bytes, &tmap_w, full_addr, k_coord, n_coord);
              if (!pad_chunk) {
                if (++cc == args.chunks_per_tap) {
                  cc = 0;
                  if (++tap_s == args.S) { tap_s = 0; ++tap_r; }
                }
              }
            }
            ++issued;
            stage_addr += kStageBytes; full_addr += 8u; empty_addr += 8u;
            if (stage_addr == ring_end) { stage_addr = smem_base; full_addr = full_bar0; empty_addr = empty_bar0; phase ^= 1u; }
          }
          slot_free = false;   // this path waits in full every time
        }
      }
      TB200_PROF_STORE(0, prof_wait);
      TB200_PROF_STORE(1, clock64() - prof_t0);
      // Never leave with copies in flight into this CTA's shared memory: wait (bounded) until the
      // MMA side has released every stage that was filled.
      if (ok) {
        const int pending = issued < num_stages ? issued : num_stages;
        for (int i = 0; i < pending; ++i) {
          if (!mbar_wait_bounded(empty_addr, phase ^ 1u, abort_p, args.wait_limit)) break;
          stage_addr += kStageBytes; empty_addr += 8u;
          if (stage_addr == ring_end) { stage_addr = smem_base; empty_addr = empty_bar0; phase ^= 1u; }
        }
      } else {
        // aborted: give outstanding copies a bounded time to land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1 || (kRows2 && warp == 10)) {
    // ------------------------------------------------------------ MMA issuer
    // One thread. Descriptor low words are precomputed per k-slice; per stage they only move by the
    // stage pitch, so an MMA costs two adds and one instruction here (the tensor pipe needs a new
    // 128 x BN x 32-byte MMA every BN/2 cycles).
    // kRows2 (BN <= 128): one thread cannot issue that fast -- measured about 90 cycles per MMA in this loop against
    // the 64 an N = 128 MMA takes -- so the tile's two 128-row blocks have an issuer each (warps 1 and 10): separate
    // accumulators, the same stages; a stage is released, and a tile handed over, when both have committed.
    if (lane == 0 && leader) {
      const uint32_t blk = (kRows2 && warp == 10) ? 1u : 0u;
      constexpr bool kTf32 = OutTraits<OutT>::kTf32;
      const uint32_t desc_hi = ((args.a_sbo >> 4) & 0x3FFFu) | (1u << 14) | ((args.swizzle_mode & 7u) << 29);
      uint32_t a_k[4], b_k[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        a_k[k] = ((smem_base + args.a_mma_off[k] + blk * kABlockBytes) >> 4) | (((args.a_lbo >> 4) & 0x3FFFu) << 16);
        b_k[k] = ((smem_base + kABytes + args.b_mma_off[k]) >> 4) | (((args.b_lbo >> 4) & 0x3FFFu) << 16);
      }
      constexpr uint32_t kStageUnits = kStageBytes >> 4;
      const uint32_t ring_units = ring_bytes >> 4;
      const uint32_t idesc = args.idesc;
      uint32_t s_off = 0;                          // current stage's offset in 16-byte units
      uint32_t full_addr = full_bar0, empty_addr = empty_bar0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      long long prof_wfull = 0, prof_wtmem = 0;
      (void)prof_wfull; (void)prof_wtmem;
      TB200_PROF_T(prof_t0);
      bool stage_ready = mbar_test_wait(full_addr, phase);
      WorkIter witer;
      witer.template init<kSplit>(args, worker, k_iters);
      WorkItem item;
      for (; ok && witer.template next<kSplit>(item, args, num_workers, k_iters); ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t use = static_cast<uint32_t>(local_tile >> 1);
        TB200_PROF_T(tw0);
        if (!mbar_wait_bounded(tempty_bar(buf), (use & 1u) ^ 1u, abort_p, args.wait_limit)) {
          report_error(args, abort_p, kErrMmaWaitTmem, (uint32_t)local_tile);
          ok = false;
          break;
        }
        TB200_PROF_ADD(prof_wtmem, tw0);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf) * kAccCols + blk * BN;
        for (int it = item.k_begin; it < item.k_end; ++it) {
          const bool first = it == item.k_begin;   // the piece's first MMA overwrites the accumulator
          TB200_PROF_T(tw1);
          if (!stage_ready && !mbar_wait_bounded(full_addr, phase, abort_p, args.wait_limit)) {
            report_error(args, abort_p, kErrMmaWaitFull, (uint32_t)it);
            ok = false;
            break;
          }
          TB200_PROF_ADD(prof_wfull, tw1);
          // probe the next stage now; the MMAs below are issued while the answer is on its way
          uint32_t n_off = s_off + kStageUnits, nfull = full_addr + 8u, nempty = empty_addr + 8u, nphase = phase;
          if (n_off == ring_units) { n_off = 0; nfull = full_bar0; nempty = empty_bar0; nphase ^= 1u; }
          tc_fence_after();
          bool next_ready;
          if constexpr (kPair) {
            if (first)
              next_ready = mma_stage4_probe_pair<kTf32, false>(d_tmem, a_k[0] + s_off, a_k[1] + s_off, a_k[2] + s_off,
                                                               a_k[3] + s_off, b_k[0] + s_off, b_k[1] + s_off,
                                                               b_k[2] + s_off, b_k[3] + s_off, desc_hi, idesc,
                                                               empty_addr, nfull, nphase);
            else
              next_ready = mma_stage4_probe_pair<kTf32, true>(d_tmem, a_k[0] + s_off, a_k[1] + s_off, a_k[2] + s_off,
                                                              a_k[3] + s_off, b_k[0] + s_off, b_k[1] + s_off,
                                                              b_k[2] + s_off, b_k[3] + s_off, desc_hi, idesc,
                                                              empty_addr, nfull, nphase);
          } else {
            if (first)
              next_ready = mma_stage4_probe<kTf32, false>(d_tmem, a_k[0] + s_off, a_k[1] + s_off, a_k[2] + s_off,
                                                          a_k[3] + s_off, b_k[0] + s_off, b_k[1] + s_off, b_k[2] + s_off,
                                                          b_k[3] + s_off, desc_hi, idesc, empty_addr, nfull, nphase);
            else
              next_ready = mma_stage4_probe<kTf32, true>(d_tmem, a_k[0] + s_off, a_k[1] + s_off, a_k[2] + s_off,
                                                         a_k[3] + s_off, b_k[0] + s_off, b_k[1] + s_off, b_k[2] + s_off,
                                                         b_k[3] + s_off, desc_hi, idesc, empty_addr, nfull, nphase);
          }
          s_off = n_off; full_addr = nfull; empty_addr = nempty; phase = nphase;
          stage_ready = next_ready;
        }
        if (ok) {                                 // accumulator complete (in both CTAs of a pair)
          if constexpr (kPair) mma_commit_pair(tfull_bar(buf));
          else mma_commit(tfull_bar(buf));
        }
      }
      if (blk == 0u) {
        TB200_PROF_STORE(2, prof_wfull);
        TB200_PROF_STORE(3, prof_wtmem);
        TB200_PROF_STORE(4, clock64() - prof_t0);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..9)
    // Two groups of four warps take alternate tiles of this CTA (group e drains TMEM accumulator e), so
    // one tile's epilogue may take as long as two main loops before it holds the tensor pipe up.
    // Warp w may only read TMEM lanes [32*(w%4), 32*(w%4)+32): it owns those 32 output pixels of
    // the tile, one pixel per lane. Columns are processed in groups of 128 bytes of output.
    const int ew = warp - 2;                       // 0..7
    const int egroup = ew >> 2;                    // which accumulator / which tiles
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    OutT* __restrict__ out = static_cast<OutT*>(args.out);
    const OutT* __restrict__ res = static_cast<const OutT*>(args.residual);
    constexpr int kVec = 16 / sizeof(OutT);        // elements per 16-byte vector
    constexpr int kGroupCols = 128 / sizeof(OutT); // columns per 128-byte staging row
    constexpr int kGroups = BN / kGroupCols;
    constexpr int kLdPerGroup = kGroupCols / 32;
    constexpr int kChunksPerLd = 32 / kVec;        // 16-byte chunks produced per 32-column TMEM load
    // with a shared copy every warp writes the same values to the same words before it reads them
    const int bias_slot = args.shared_bias ? 0 : ew * BN;
    float* bias_w = reinterpret_cast<float*>(smem_gen + bias_off) + bias_slot;
    const uint32_t bias_w_s = smem_base + bias_off + static_cast<uint32_t>(bias_slot) * 4u;
    const uint32_t stg0 = staging_base + static_cast<uint32_t>(ew) * (kStagingDepth * kStagingBoxBytes);
    const bool res_tma = args.res_tma != 0;
    // this lane's 16-byte chunk c of its staging row lives at row*128 + ((c ^ (row & 7)) << 4): the
    // SWIZZLE_128B pattern of the out / residual tensor maps (bank-conflict free for 8-lane phases)
    const uint32_t lane_row_off = static_cast<uint32_t>(lane) * 128u;
    const uint32_t lane_xor = static_cast<uint32_t>(lane) & 7u;
    uint32_t box = 0;                              // staging box the next live group uses (0..1)
    uint32_t box_phase = 0;                        // bit b = parity of the next residual load into box b
    int bias_tile = -1;
    constexpr int kBiasPerLane = BN / 32;
    float bias_next[kBiasPerLane];
    auto fetch_bias = [&](int nt) {   // independent loads: all in flight together
#pragma unroll
      for (int j = 0; j < kBiasPerLane; ++j) {
        const int n = nt * BN + j * 32 + lane;
        float b = 0.0f;
        if (args.bias != nullptr && n < args.K_out) {
          b = args.bias_is_f32 ? __ldg(static_cast<const float*>(args.bias) + n)
                               : OutTraits<OutT>::to_f(static_cast<const OutT*>(args.bias)[n]);
        }
        bias_next[j] = b;
      }
    };
    // This group's items: every second item of the worker (group e drains TMEM accumulator e) -- or, with
    // two-row-block tiles, every item, of which the group takes the 128-row block `egroup`. The iterator runs one
    // item ahead so that the next tile's bias can be fetched early.
    // The worker's LAST item is shared by both groups: nothing overlaps its epilogue any more (the next kernel
    // cannot start before this one ends), so the group that would idle takes every second 128-byte column group of
    // it -- the same TMEM lanes belong to warp w and warp w + 4 -- and the exposed tail of the launch is halved.
    int last_item = -1;
    if constexpr (!kRows2 && kGroups >= 2) {
      WorkIter cnt;
      cnt.template init<kSplit>(args, worker, k_iters);
      WorkItem t;
      while (cnt.template next<kSplit>(t, args, num_workers, k_iters)) ++last_item;
    }
    WorkIter witer;
    witer.template init<kSplit>(args, worker, k_iters);
    int local_next = 0;                            // local index of the item witer.next() yields next
    auto next_mine = [&](WorkItem& it, int& local) -> bool {
      while (witer.template next<kSplit>(it, args, num_workers, k_iters)) {
        const int l = local_next++;
        if (kRows2 || (l & 1) == egroup || l == last_item) {
          local = l;
          return true;
        }
      }
      return false;
    };
    WorkItem item = {0, 0, 0};
    int m_tile = 0, n_tile = 0;
    // bias of the next item of this group, if its column tile differs from `cur_n` (-1: always): looked up on a
    // copy of the iterator, so that no look-ahead state stays live across the epilogue body
    auto prefetch_next_bias = [&](int cur_n) {
      WorkIter pk = witer;
      int pl = local_next;
      WorkItem ni;
      while (pk.template next<kSplit>(ni, args, num_workers, k_iters)) {
        const int l = pl++;
        if (kRows2 || (l & 1) == egroup || l == last_item) {
          int mm, nn;
          tile_coords(ni.tile, mm, nn);
          if (nn != cur_n) fetch_bias(nn);
          return;
        }
      }
    };
    prefetch_next_bias(-1);
    int local_tile = 0;
    bool ok = true;
    long long prof_wacc = 0, prof_wres = 0, prof_ld = 0, prof_math = 0, prof_stage = 0, prof_wstore = 0;
    (void)prof_wacc; (void)prof_wres; (void)prof_ld; (void)prof_math; (void)prof_stage; (void)prof_wstore;
    TB200_PROF_T(prof_t0);
    const bool need_coords = !args.out_tma || (res != nullptr && !res_tma);
    // kCoop kernels serve channel-contiguous outputs whose pixels are not one dense [M][pitch] matrix (a strided
    // view, one phase of a transposed convolution; the host launches them only then, with out_tma = 0): same staging
    // boxes as the TMA path, but the warp moves them itself, 8 lanes per pixel and 16 bytes each, so every store /
    // residual load instruction covers 4 whole 128-byte rows. A separate instantiation, because inside the TMA
    // kernels this code cost 1.3 % through register spills.
    const bool res_staged = res_tma || (kCoop && res != nullptr);
    // ---- exchange of partial sums, ahead of the main loop. The pieces of split tiles are the first (at most two)
    // items of a worker. For each piece this warp owns rows of: wait for its accumulator, take a ticket, then either
    // write the partial sums out and release the accumulator (bit stays 0: the main loop skips the item), or -- last
    // ticket -- add the others' partial sums into the accumulator in TMEM (bit set: the main loop treats the item
    // as a whole tile). Kept out of the main loop so that its calls cost the loop no registers.
    uint32_t sk_reduced = 0;
    if constexpr (kSplit) {
      WorkIter pre;
      pre.template init<kSplit>(args, worker, k_iters);
      WorkItem pi;
      for (int l = 0; ok && l < 2 && pre.template next<kSplit>(pi, args, num_workers, k_iters); ++l) {
        if (pi.k_end - pi.k_begin == k_iters) break;          // whole tiles from here on
        if (!kRows2 && (l & 1) != egroup) continue;           // the other group's item
        const int buf = kRows2 ? (l & 1) : egroup;
        const bool ready = mbar_wait_bounded(tfull_bar(buf), 0u, abort_p, 2 * args.wait_limit);   // first use of the buffer
        if (!__all_sync(0xffffffffu, ready)) {
          if (lane == 0) report_error(args, abort_p, kErrEpilogueWait, (uint32_t)l);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                static_cast<uint32_t>(buf) * kAccCols + (kRows2 ? static_cast<uint32_t>(egroup * BN) : 0u);
        const int sk_t = pi.tile - args.dp_tiles;
        const int sk_total = args.sk_tiles * k_iters;
        const int sk_first = sk_owner_of(sk_total, args.sk_workers, sk_t * k_iters);
        const int sk_pieces = sk_owner_of(sk_total, args.sk_workers, sk_t * k_iters + k_iters - 1) - sk_first + 1;
        const int sk_me = worker - sk_first;
        const int row_block = kPair ? static_cast<int>(cta_rank) : (kRows2 ? egroup : 0);
        const int sk_pos = row_block * 4 + quarter;   // which 32 rows of the tile this warp owns, 0..7
        uint32_t* cnt = args.sk_counters + (static_cast<long long>(sk_t) * 8 + sk_pos) * 2;
        const long long warp_off = static_cast<long long>(sk_pos) * (BN / 32) * 256 + lane;   // float4s inside a slot
        uint32_t ticket = 0;
        if (lane == 0) ticket = atomicAdd(cnt, 1u);
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        if (ticket + 1u != static_cast<uint32_t>(sk_pieces)) {
          TB200_PROF_T(tsd);
          sk_dump_partial<kPair>(taddr0, BN / 32, sk_slot(args, worker, pi.k_begin == 0 ? 1 : 0) + warp_off,
                                 kPair ? mapa_cluster(tempty_bar(buf), 0u) : tempty_bar(buf), lane);
          // every lane's stores, then the warp barrier, then lane 0's release at GPU scope (no full fence: a
          // sequentially consistent one waits for every copy the SM has in flight)
          __syncwarp();
          if (lane == 0) red_release_gpu_add(cnt + 1, 1u);
          TB200_PROF_ADD(prof_wres, tsd);
          continue;
        }
        TB200_PROF_T(tsw);
        if (!sk_wait_partials(cnt, static_cast<uint32_t>(sk_pieces - 1), abort_p, args.wait_limit, lane)) {
          if (lane == 0) report_error(args, abort_p, kErrSplitWait, (uint32_t)l);
          ok = false;
          break;
        }
        if (sk_pieces == 2)
          sk_reduce_two(taddr0, BN / 32, sk_slot(args, sk_first + 1 - sk_me, sk_me == 0 ? 0 : 1) + warp_off);
        else
          sk_reduce_many(args, taddr0, BN / 32, sk_first, sk_pieces, sk_me, warp_off);
        TB200_PROF_ADD(prof_wstore, tsw);
        sk_reduced |= 1u << l;
      }
    }
    while (ok && next_mine(item, local_tile)) {
      const int tile = item.tile;
      tile_coords(tile, m_tile, n_tile);
      const int buf = local_tile & 1;              // = egroup for the group's own items
      const bool partial = kSplit && item.k_end - item.k_begin != k_iters;   // one piece of a tile split over K
      // column groups this warp takes: all of them, or -- on the shared last item -- every second one
      const bool shared = !kRows2 && local_tile == last_item && !partial;
      const int g_first = shared && (local_tile & 1) != egroup ? 1 : 0;
      const int g_step = shared ? 2 : 1;
      const uint32_t use = static_cast<uint32_t>(local_tile >> 1);
      const int n_base = n_tile * BN;
      const int row_block = kPair ? static_cast<int>(cta_rank) : (kRows2 ? egroup : 0);   // which 128 rows of the tile
      const int m_row0 = args.m_begin + m_tile * kTileM + row_block * kBlockM + quarter * 32;

      // this warp's fp32 copy of the tile's bias (zeros when there is none / past K_out); the values
      // were fetched into registers during the previous tile, and the next tile's are fetched now
      if (n_tile != bias_tile) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kBiasPerLane; ++j) bias_w[j * 32 + lane] = bias_next[j];
        __syncwarp();
        bias_tile = n_tile;
      }
      prefetch_next_bias(n_tile);

      const int m = args.m_begin + m_tile * kTileM + row_block * kBlockM + row;
      const bool row_ok = m < args.M;
      long long out_off = 0, res_off = 0;
      if (need_coords) {   // only the per-lane store / load paths need (n, ho, wo); the TMA paths do not
        const int pq = m / args.Wo;
        const int wo = m - pq * args.Wo;
        const int img = pq / args.Ho;
        const int ho = pq - img * args.Ho;
        out_off = img * args.out_sn + ho * args.out_sh + wo * args.out_sw;
        res_off = img * args.res_sn + ho * args.res_sh + wo * args.res_sw;
      }
      const OutT* res_row = res + res_off + static_cast<long long>(n_base) * args.res_sc;

      // Residual box of the tile's first live group: requested before the accumulator is waited for.
      // Box `box` was last stored from two groups ago; only the newer store may still be pending.
      auto request_first_residual = [&]() {
        if (res_tma && n_base + g_first * kGroupCols < args.K_out) {
          if (lane == 0) {
            bulk_wait_group_read<1>();
            mbar_arrive_expect_tx(res_bar(ew, box), kStagingBoxBytes);
            tma_load_2d(stg0 + box * kStagingBoxBytes, &tmap_res, res_bar(ew, box), n_base + g_first * kGroupCols, m_row0);
          }
        }
      };
      if constexpr (kSplit) {
        // a piece whose partial sums went to another CTA is finished; one that collected the others' is a whole tile
        // now (for the group that collected them: a piece is never shared between the groups, except that both
        // groups drain their own row block of a two-row-block tile)
        if (partial && (((sk_reduced >> local_tile) & 1u) == 0u || (!kRows2 && (local_tile & 1) != egroup))) continue;
      }
      if (!partial) request_first_residual();

      TB200_PROF_T(tw2);
      const bool ready = mbar_wait_bounded(tfull_bar(buf), use & 1u, abort_p, 2 * args.wait_limit);
      TB200_PROF_ADD(prof_wacc, tw2);
      if (!__all_sync(0xffffffffu, ready)) {      // keep the warp converged for tcgen05.ld
        if (lane == 0) report_error(args, abort_p, kErrEpilogueWait, (uint32_t)local_tile);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr0 =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf) * kAccCols +
          (kRows2 ? static_cast<uint32_t>(egroup * BN) : 0u);

      if constexpr (kSplit) {
        if (partial) request_first_residual();   // the exchange left the tile's total in TMEM: an ordinary tile now
      }

#pragma unroll 1
      for (int g = g_first; g < kGroups; g += g_step) {
        const int n0 = n_base + g * kGroupCols;
        const bool group_live = n0 < args.K_out;   // warp-uniform: false when the group is past K_out
        const uint32_t stg = stg0 + box * kStagingBoxBytes;
        uint32_t v[kLdPerGroup][32];
        TB200_PROF_T(tl);
#pragma unroll
        for (int h = 0; h < kLdPerGroup; ++h) tmem_ld_32x32(taddr0 + g * kGroupCols + h * 32, v[h]);
        tmem_ld_wait();
        TB200_PROF_ADD(prof_ld, tl);
        if (g == kGroups - 1 && !shared) {
          // the accumulator is in registers now: hand the TMEM buffer back to the MMA issuer (nobody waits for
          // the buffer of the worker's last item, which two groups drain)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) mbar_arrive_cluster(mapa_cluster(tempty_bar(buf), 0u));   // the leader's barrier
            else mbar_arrive(tempty_bar(buf));
          }
        }
        if (!group_live) continue;

        if (res_tma) {
          TB200_PROF_T(tw3);
          const bool landed = mbar_wait_bounded(res_bar(ew, box), (box_phase >> box) & 1u, abort_p,
                                                args.wait_limit);
          TB200_PROF_ADD(prof_wres, tw3);
          if (!__all_sync(0xffffffffu, landed)) {
            if (lane == 0) report_error(args, abort_p, kErrResidualWait, (uint32_t)local_tile);
            ok = false;
            break;
          }
          box_phase ^= (1u << box);
          // Now that this group's residual has landed, fetch the NEXT group's into the other box. That
          // box was stored from one group ago; its store has had this group's wait to be read out.
          if (g + g_step < kGroups && n0 + g_step * kGroupCols < args.K_out) {
            if (lane == 0) {
              const uint32_t nb = box ^ 1u;
              bulk_wait_group_read<0>();
              mbar_arrive_expect_tx(res_bar(ew, nb), kStagingBoxBytes);
              tma_load_2d(stg0 + nb * kStagingBoxBytes, &tmap_res, res_bar(ew, nb), n0 + g_step * kGroupCols, m_row0);
            }
          }
        } else if (args.out_tma) {
          TB200_PROF_T(ts);
          if (lane == 0) bulk_wait_group_read<1>();   // this box's previous store (two groups ago) has been read out
          __syncwarp();
          TB200_PROF_ADD(prof_wstore, ts);
        }
        if constexpr (kCoop) {
          if (res != nullptr) coop_load_box<OutT>(stg, res + n0, res_off, row_ok, args.K_out - n0, lane);
        }

        TB200_PROF_T(tm);
        uint4 packed[8];
#pragma unroll
        for (int h = 0; h < kLdPerGroup; ++h) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[h][j]);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 b4 = ld_shared_f4(bias_w_s + static_cast<uint32_t>(g * kGroupCols + h * 32 + j4 * 4) * 4u);
            add2(f[j4 * 4 + 0], f[j4 * 4 + 1], b4.x, b4.y);
            add2(f[j4 * 4 + 2], f[j4 * 4 + 3], b4.z, b4.w);
          }
          if (!kCoop && !args.out_tma) {
            float fg[32];   // a copy the out-of-line path may keep in local memory; f stays in registers
#pragma unroll
            for (int j = 0; j < 32; ++j) fg[j] = f[j];
            epilogue_block_generic<OutT>(
                args, fg, res != nullptr ? res_row + static_cast<long long>(g * kGroupCols + h * 32) * args.res_sc : nullptr,
                out + out_off + static_cast<long long>(n0 + h * 32) * args.out_sc, n0 + h * 32, row_ok);
            continue;
          }
          // TMA output; a residual, if any, sits in this lane's row of the staging box (the host
          // guarantees a residual is TMA-loaded whenever the output is TMA-stored)
          uint4 rchunks[kChunksPerLd];
          if (res_staged) {
#pragma unroll
            for (int c = 0; c < kChunksPerLd; ++c) {
              const uint32_t cc = static_cast<uint32_t>(h * kChunksPerLd + c);
              rchunks[c] = ld_shared_v4(stg + lane_row_off + ((cc ^ lane_xor) << 4));
            }
          }
          if (args.act == kActRelu) {
            finish32<OutT, true>(f, rchunks, res_staged, packed + h * kChunksPerLd);
          } else {
            if (res_staged) {
#pragma unroll
              for (int c = 0; c < kChunksPerLd; ++c) add16<OutT>(f + c * kVec, rchunks[c]);
            }
            apply_act32<sizeof(OutT) == 2>(f, args.act);
            finish32<OutT, false>(f, rchunks, false, packed + h * kChunksPerLd);
          }
        }
        TB200_PROF_ADD(prof_math, tm);
        TB200_PROF_T(tg);
        if (args.out_tma) {
          // the lane's pixel row goes to its swizzled 128-byte row of the box; one TMA store writes the box
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared_v4(stg + lane_row_off + ((static_cast<uint32_t>(c) ^ lane_xor) << 4), packed[c]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_out, stg, n0, m_row0);
            bulk_commit_group();
          }
          box ^= 1u;
        } else if constexpr (kCoop) {
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared_v4(stg + lane_row_off + ((static_cast<uint32_t>(c) ^ lane_xor) << 4), packed[c]);
          coop_store_box<OutT>(stg, out + n0, out_off, row_ok, args.K_out - n0, lane);
          box ^= 1u;
        }
        TB200_PROF_ADD(prof_stage, tg);
      }
    }
    if (args.out_tma && lane == 0) bulk_wait_group0();
    if (warp == 2 && lane == 0) {
      TB200_PROF_STORE(5, prof_wacc);
      TB200_PROF_STORE(6, prof_wres);
      TB200_PROF_STORE(7, clock64() - prof_t0);
      TB200_PROF_STORE(8, prof_ld);
      TB200_PROF_STORE(9, prof_math);
      TB200_PROF_STORE(10, prof_stage);
      TB200_PROF_STORE(11, prof_wstore);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  if constexpr (kPair) cluster_sync();   // neither CTA frees TMEM or exits while the other may still use the pair
  else __syncthreads();
  TB200_PROF_NOW(14);
  if (warp == 1) {
    tc_fence_after();
    if constexpr (kPair) tmem_dealloc_pair<kTmemCols>(tmem_base);
    else tmem_dealloc<kTmemCols>(tmem_base);
  }
  if (args.pdl_mode == 2) griddep_wait();   // do not complete before the launch in front of this one has
  TB200_PROF_NOW(15);
}

}  // namespace tb200
