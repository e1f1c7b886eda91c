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

namespace tb200 {

constexpr int kBlockM = 128;          // output pixels per tile = TMEM lanes
constexpr int kStageKBytes = 128;     // bytes of K per smem row per pipeline stage
constexpr int kNumThreads = 192;      // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int kMaxStages = 12;
constexpr long long kWaitLimitCycles = 4000000000LL;  // ~2 s at 1.9 GHz, per wait

// Device-side error codes written to ConvKernelArgs::status (0 = fine).
enum : uint32_t {
  kErrNone = 0,
  kErrProducerWait = 1,   // TMA producer: a stage never became free
  kErrMmaWaitFull = 2,    // MMA issuer: a stage's bytes never landed
  kErrMmaWaitTmem = 3,    // MMA issuer: accumulator never drained
  kErrEpilogueWait = 4,   // epilogue: accumulator never became ready
};

enum : int { kActNone = 0, kActRelu = 1, kActGelu = 2, kActSilu = 3 };

struct ConvKernelArgs {
  // problem
  int M;            // N * Ho * Wo
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
  // tiling / pipeline
  int num_m_tiles, num_n_tiles;
  int num_stages;
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
  // error reporting: 4 words {code, block, detail, 0}; first error wins
  uint32_t* status;
};

template <typename T> struct OutTraits;
template <> struct OutTraits<__nv_bfloat16> {
  static constexpr bool kTf32 = false;
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct OutTraits<__half> {
  static constexpr bool kTf32 = false;
  __device__ static float to_f(__half v) { return __half2float(v); }
  __device__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct OutTraits<float> {
  static constexpr bool kTf32 = true;
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

__device__ __forceinline__ void report_error(const ConvKernelArgs& a, volatile uint32_t* abort_flag,
                                             uint32_t code, uint32_t detail) {
  *abort_flag = 1u;
  if (a.status != nullptr && atomicCAS(a.status, 0u, code) == 0u) {
    a.status[1] = blockIdx.x;
    a.status[2] = detail;
    __threadfence_system();
  }
}

// Shared memory map (offsets from a 1024-byte aligned base):
//   [0, stages * stage_bytes)        operand ring: per stage A (128 rows x 128 B) then B (BN rows x 128 B)
//   + kStagingBytes                  4 x 4 KB output staging, one 32-row x 128 B box per epilogue warp
//   + 4 * BN * 4                     per-epilogue-warp copy of the tile's bias, as fp32
//   + 256                            mbarriers, TMEM base slot, abort flag
constexpr int kStagingBytes = 4 * 32 * 128;
__host__ __device__ constexpr int conv_smem_bytes(int bn, int stages) {
  return stages * (kBlockM * kStageKBytes + bn * kStageKBytes) + kStagingBytes + 4 * bn * 4 + 256 + 1024;
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

template <typename OutT>
__device__ __forceinline__ void add16(float* f, const uint4& raw) {
  constexpr int kVec = 16 / sizeof(OutT);
  const OutT* e = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
  for (int j = 0; j < kVec; ++j) f[j] += OutTraits<OutT>::to_f(e[j]);
}

template <typename OutT, int BN>
__global__ void __launch_bounds__(kNumThreads, 1)
conv2d_igemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_x,
                          const __grid_constant__ CUtensorMap tmap_w,
                          const __grid_constant__ CUtensorMap tmap_out,
                          const __grid_constant__ ConvKernelArgs args) {
  using namespace ptx;
  constexpr uint32_t kABytes = kBlockM * kStageKBytes;   // 16 KB
  constexpr uint32_t kBBytes = BN * kStageKBytes;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;                 // two accumulators: 128, 256 or 512 columns
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int num_stages = args.num_stages;
  const uint32_t ring_bytes = static_cast<uint32_t>(num_stages) * kStageBytes;
  const uint32_t staging_base = smem_base + ring_bytes;
  const uint32_t bias_off = ring_bytes + kStagingBytes;
  const uint32_t bar_off = bias_off + 4u * BN * 4u;
  const uint32_t bar_base = smem_base + bar_off;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * kMaxStages + 4);
  volatile uint32_t* tmem_slot_p =
      reinterpret_cast<volatile uint32_t*>(smem_gen + bar_off + 8u * (2 * kMaxStages + 4));
  volatile uint32_t* abort_p = tmem_slot_p + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);   // one arrival per epilogue warp
    }
    *abort_p = 0u;
    fence_mbar_init();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_w);
    if (args.out_tma) prefetch_tmap(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc<kTmemCols>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;

  const int num_tiles = args.num_m_tiles * args.num_n_tiles;
  const int chunks_per_stage = kStageKBytes / args.chunk_bytes;
  const int k_iters = (args.total_chunks + chunks_per_stage - 1) / chunks_per_stage;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t a_chunk_bytes = kBlockM * args.chunk_bytes;
      const uint32_t b_chunk_bytes = BN * args.chunk_bytes;
      bool ok = true;
      int issued = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_tile = tile / args.num_n_tiles;
        const int n_tile = tile - m_tile * args.num_n_tiles;
        const int m0 = m_tile * kBlockM;
        const int q0 = m0 % args.Wo;
        const int t = m0 / args.Wo;
        const int p0 = t % args.Ho;
        const int img0 = t / args.Ho;
        const int w_start = q0 * args.stride_w - args.pad_w;
        const int h_start = p0 * args.stride_h - args.pad_h;
        int chunk = 0, tap_r = 0, tap_s = 0, cc = 0;
        for (int it = 0; it < k_iters; ++it) {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_p, kWaitLimitCycles)) {
            report_error(args, abort_p, kErrProducerWait, (uint32_t)it);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          for (int j = 0; j < chunks_per_stage; ++j, ++chunk) {
            // chunks past the end of Kgemm read zeros: channel coordinate C / column Kgemm are out of range
            const bool pad_chunk = chunk >= args.total_chunks;
            const int c_coord = pad_chunk ? args.C : cc * args.chunk_elems;
            const int k_coord = pad_chunk ? args.total_chunks * args.chunk_elems
                                          : chunk * args.chunk_elems;
            if (args.a_tiled) {
              tma_load_2d(a_dst + j * a_chunk_bytes, &tmap_x, full_bar(stage), c_coord, m0);
            } else {
              tma_load_im2col_4d(a_dst + j * a_chunk_bytes, &tmap_x, full_bar(stage), c_coord,
                                 w_start, h_start, img0, (uint16_t)(tap_s * args.dil_w),
                                 (uint16_t)(tap_r * args.dil_h));
            }
            tma_load_2d(b_dst + j * b_chunk_bytes, &tmap_w, full_bar(stage), k_coord, n_tile * BN);
            if (!pad_chunk) {
              if (++cc == args.chunks_per_tap) {
                cc = 0;
                if (++tap_s == args.S) { tap_s = 0; ++tap_r; }
              }
            }
          }
          ++issued;
          if (++stage == num_stages) { stage = 0; phase ^= 1u; }
        }
      }
      // Never leave with copies in flight into this CTA's shared memory: wait (bounded) until the
      // MMA side has released every stage that was filled.
      if (ok) {
        const int pending = issued < num_stages ? issued : num_stages;
        for (int i = 0; i < pending; ++i) {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_p, kWaitLimitCycles)) break;
          if (++stage == num_stages) { stage = 0; phase ^= 1u; }
        }
      } else {
        // aborted: give outstanding copies a bounded time to land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t use = static_cast<uint32_t>(local_tile >> 1);
        if (!mbar_wait_bounded(tempty_bar(buf), (use & 1u) ^ 1u, abort_p, kWaitLimitCycles)) {
          report_error(args, abort_p, kErrMmaWaitTmem, (uint32_t)local_tile);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int it = 0; it < k_iters; ++it) {
          if (!mbar_wait_bounded(full_bar(stage), phase, abort_p, kWaitLimitCycles)) {
            report_error(args, abort_p, kErrMmaWaitFull, (uint32_t)it);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_base + stage * kStageBytes;
          const uint32_t b_base = a_base + kABytes;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t adesc =
                make_smem_desc(a_base + args.a_mma_off[k], args.a_lbo, args.a_sbo, args.swizzle_mode);
            const uint64_t bdesc =
                make_smem_desc(b_base + args.b_mma_off[k], args.b_lbo, args.b_sbo, args.swizzle_mode);
            const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
            if constexpr (OutTraits<OutT>::kTf32) {
              mma_tf32_ss(d_tmem, adesc, bdesc, args.idesc, acc);
            } else {
              mma_f16_ss(d_tmem, adesc, bdesc, args.idesc, acc);
            }
          }
          mma_commit(empty_bar(stage));           // stage reusable once these MMAs retire
          if (++stage == num_stages) { stage = 0; phase ^= 1u; }
        }
        if (ok) mma_commit(tfull_bar(buf));       // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5)
    // Warp w may only read TMEM lanes [32*(w%4), 32*(w%4)+32): it owns those 32 output pixels of
    // the tile, one pixel per lane.
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    OutT* __restrict__ out = static_cast<OutT*>(args.out);
    const OutT* __restrict__ res = static_cast<const OutT*>(args.residual);
    constexpr int kVec = 16 / sizeof(OutT);        // elements per 16-byte vector
    constexpr int kGroupCols = 128 / sizeof(OutT); // columns per 128-byte staging row
    constexpr int kGroups = BN / kGroupCols;
    constexpr int kLdPerGroup = kGroupCols / 32;
    float* bias_w = reinterpret_cast<float*>(smem_gen + bias_off) + quarter * BN;
    const uint32_t stg = staging_base + static_cast<uint32_t>(quarter) * 4096u;
    const bool use_res_vec = (res != nullptr) && args.res_vec;
    int bias_tile = -1;
    int local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      const int m_tile = tile / args.num_n_tiles;
      const int n_tile = tile - m_tile * args.num_n_tiles;
      const int buf = local_tile & 1;
      const uint32_t use = static_cast<uint32_t>(local_tile >> 1);
      const int n_base = n_tile * BN;

      // this warp's fp32 copy of the tile's bias (zeros when there is none / past K_out)
      if (n_tile != bias_tile) {
        __syncwarp();
        for (int i = lane; i < BN; i += 32) {
          const int n = n_base + i;
          float b = 0.0f;
          if (args.bias != nullptr && n < args.K_out) {
            b = args.bias_is_f32 ? __ldg(static_cast<const float*>(args.bias) + n)
                                 : OutTraits<OutT>::to_f(static_cast<const OutT*>(args.bias)[n]);
          }
          bias_w[i] = b;
        }
        __syncwarp();
        bias_tile = n_tile;
      }

      const int m = m_tile * kBlockM + row;
      const bool row_ok = m < args.M;
      const int pq = m / args.Wo;
      const int wo = m - pq * args.Wo;
      const int img = pq / args.Ho;
      const int ho = pq - img * args.Ho;
      const long long out_off = img * args.out_sn + ho * args.out_sh + wo * args.out_sw;
      const long long res_off = img * args.res_sn + ho * args.res_sh + wo * args.res_sw;
      const OutT* res_row = res + res_off + static_cast<long long>(n_base) * args.res_sc;

      // residual for column group g, 8 x 16 B of this lane's pixel; issued one group ahead of its use
      uint4 rv[2][8];
      auto load_res_group = [&](uint4 (&dst)[8], int g) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int n = n_base + g * kGroupCols + c * kVec;
          if (row_ok && n < args.K_out)
            dst[c] = __ldg(reinterpret_cast<const uint4*>(res_row + g * kGroupCols) + c);
          else
            dst[c] = make_uint4(0u, 0u, 0u, 0u);
        }
      };
      if (use_res_vec) load_res_group(rv[0], 0);

      const bool ready = mbar_wait_bounded(tfull_bar(buf), use & 1u, abort_p, kWaitLimitCycles);
      if (!__all_sync(0xffffffffu, ready)) {      // keep the warp converged for tcgen05.ld
        if (lane == 0) report_error(args, abort_p, kErrEpilogueWait, (uint32_t)local_tile);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr0 =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * BN);

#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        if (use_res_vec && g + 1 < kGroups) load_res_group(rv[(g + 1) & 1], g + 1);
        const int n0 = n_base + g * kGroupCols;
        const bool group_live = n0 < args.K_out;   // warp-uniform: false when the group is past K_out
        uint4 packed[8];
        constexpr int kChunksPerLd = 32 / kVec;    // 16-byte chunks produced per 32-column TMEM load
#pragma unroll
        for (int h = 0; h < kLdPerGroup; ++h) {
          uint32_t v[32];
          tmem_ld_32x32(taddr0 + g * kGroupCols + h * 32, v);
          tmem_ld_wait();
          if (g == kGroups - 1 && h == kLdPerGroup - 1) {
            // the accumulator is in registers now: hand the TMEM buffer back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(buf));
          }
          if (!group_live) continue;
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) + bias_w[g * kGroupCols + h * 32 + j];
          if (res != nullptr) {
            if (use_res_vec) {
#pragma unroll
              for (int c = 0; c < kChunksPerLd; ++c) add16<OutT>(f + c * kVec, rv[g & 1][h * kChunksPerLd + c]);
            } else if (row_ok) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + h * 32 + j < args.K_out)
                  f[j] += OutTraits<OutT>::to_f(res_row[(g * kGroupCols + h * 32 + j) * args.res_sc]);
            }
          }
          apply_act32<sizeof(OutT) == 2>(f, args.act);
          if (args.out_tma || args.out_vec) {
#pragma unroll
            for (int c = 0; c < kChunksPerLd; ++c) packed[h * kChunksPerLd + c] = pack16<OutT>(f + c * kVec);
          } else if (row_ok) {
            // lanes are consecutive pixels: for NCHW memory (sw == 1) each store instruction is coalesced
            OutT* op = out + out_off + static_cast<long long>(n0 + h * 32) * args.out_sc;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + h * 32 + j < args.K_out) op[j * args.out_sc] = OutTraits<OutT>::from_f(f[j]);
          }
        }
        if (!group_live) continue;
        if (args.out_tma) {
          // lane's pixel row -> its 128-byte row of the warp's staging box, 16-byte chunks XOR-swizzled
          // the way the tensor map (SWIZZLE_128B) expects; one TMA store writes the 32 x 128 B box.
          if (lane == 0) bulk_wait_group_read0();  // previous box has been read out of staging
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared_v4(stg + lane * 128u + ((static_cast<uint32_t>(c) ^ (lane & 7u)) << 4), packed[c]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_out, stg, n0, m_tile * kBlockM + quarter * 32);
            bulk_commit_group();
          }
        } else if (args.out_vec && row_ok) {
          OutT* op = out + out_off + static_cast<long long>(n0) * args.out_sc;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            if (n0 + c * kVec < args.K_out) reinterpret_cast<uint4*>(op)[c] = packed[c];
        }
      }
    }
    if (args.out_tma && lane == 0) bulk_wait_group0();
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

}  // namespace tb200
