// Conv2d over few-channel 16-bit images whose horizontal step is exactly 16 bytes of input: 4-channel pixels
// (8 bytes, e.g. RGB + one zero channel) under stride_w = 2, or 8-channel pixels under stride_w = 1. The case that
// matters is the 7x7 / 2 RGB stem of the ResNet family (ResNet-50 conv1; the reference runs it through its generic
// implicit GEMM, src/emitter/conv.rs + src/interface/c_bindings.rs:144-197), sm_100a.
//
// The general kernel gathers one im2col block per filter row: every input pixel travels L2 -> shared memory about
// R * S / stride_w times and the K axis is padded to 64 per filter row. Here the im2col matrix is never built:
//   * a band of `hb` output rows needs (hb - 1) * stride_h + (R - 1) * dil_h + 1 input rows; they arrive as ONE tiled
//     TMA copy into shared memory, each row once, rows above / below the image zero-filled by the copy, the
//     horizontal padding already in memory (the padded channels-last copy the host adapter writes);
//   * for one output row and one filter row r, output pixel wo reads the S pixels that start 16 * wo bytes into input
//     row ho * stride_h + r * dil_h. The A operand of the MMA is therefore a matrix whose rows are 16 bytes apart
//     and 32 * kmma bytes long -- overlapping rows. A no-swizzle K-major tcgen05 descriptor describes exactly that:
//     8-row x 16-byte core matrices, row pitch 16 B inside a core matrix, stride 128 B between 8-row groups (SBO)
//     and 16 B between core matrices along K (LBO). The descriptor reads the band in place;
//   * the filter bank ([K_out][R][kmma * 16] elements, taps past S zero) stays in shared memory for the whole kernel
//     in the same core-matrix form.
// One MMA group per (output row, 128-pixel column tile): R * kmma MMAs of M = 128, N = 64, K = 16 into one of eight
// 64-column TMEM accumulators, drained by two groups of four epilogue warps that alternate accumulators; every warp
// writes its 32 pixels x 64 channels through a swizzled 4 KB box and one TMA store (shared-memory bandwidth is what
// MMAs this narrow are bound by, so the epilogue touches shared memory as little as it can).
// Rows of a tile past Wo read whatever follows in shared memory; they are computed and clipped by the store.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "conv2d_sm100.cuh"

namespace tb200 {

constexpr int kBandThreads = 352;   // warp 0 TMA, warps 1 and 10 MMA, warps 2..9 epilogue (two groups of four)
constexpr int kBandBN = 64;         // output channels per MMA (K_out <= 64)
constexpr int kBandAccs = 8;        // 64-column accumulators in TMEM
constexpr int kBandMaxSlots = 4;    // band slots in shared memory
constexpr uint32_t kBandBoxBytes = 32 * 128;   // staging box of one epilogue warp: 32 pixels x 64 channels; two per warp

struct RowBandKernelArgs {
  int R, stride_h, pad_h, dil_h;
  int Ho, Wo;
  int hb;                  // output rows per band
  int bands_per_img;       // ceil(Ho / hb)
  int n_bands;             // images * bands_per_img
  int wtiles;              // ceil(Wo / 128)
  int kmma;                // K = 16 MMAs per filter row: ceil(S * pixel_bytes / 32)
  int num_slots;           // band slots in the ring (2 .. kBandMaxSlots)
  uint32_t row_bytes;      // pitch of one input row, in memory and in a slot (multiple of 128)
  uint32_t box_bytes;      // bytes one band copy delivers: in_rows * row_bytes
  uint32_t slot_bytes;     // pitch of the slots: box_bytes + slack for the dropped rows' reads, 1024-byte multiple
  uint32_t w_bytes;        // filter bank: R * kmma * 2048
  uint32_t idesc;          // M = 128, N = 64, fp32 accumulate
  const void* w;           // packed filter bank in global memory: [K_out][R][kmma * 16] elements
  int K_out;
  const void* bias;
  int bias_is_f32;
  int act;
  uint32_t* status;
  long long wait_limit;    // cycles any single wait may take before the role gives up
  int test_producer_stop;  // test hook, -1 in normal use: the TMA producer stops after this many bands
  long long* prof;         // cycle counters, only written by -DTB200_PROFILE builds
};

__host__ __device__ constexpr uint32_t rowband_smem_bytes(uint32_t w_bytes, uint32_t slot_bytes, int num_slots) {
  return w_bytes + static_cast<uint32_t>(num_slots) * slot_bytes + 16u * kBandBoxBytes + kBandBN * 4u + 512u + 1024u;
}

namespace ptx {
// Tiled 4-D load into this CTA's shared memory: coordinates {c0 (innermost), c1, c2, c3}. No multicast.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Tiled 4-D store shared -> global (bulk-group completion); coordinates outside the tensor are clipped.
__device__ __forceinline__ void tma_store_4d(const void* tmap, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// M = 128 MMAs of a single CTA, kind::f16 (fp16 / bf16 operands, fp32 accumulate), meant to be executed by a whole
// converged warp: every lane carries the (identical) operands, the instructions themselves are predicated on `issue`
// (1 in one lane). The rate at which a thread can feed the tensor pipe is what bounds MMAs with a narrow N: with the
// operand arithmetic in uniform control flow the compiler keeps it in uniform registers, where the MMA instruction
// reads its descriptors from; issued from inside an `if (lane == 0)` block the same loop runs about three times
// slower (measured: 141 against 48 cycles per M128 N64 K16 MMA).
// The kMma MMAs of one filter row as one block: K slices 32 bytes (2 units) apart in A, 2048 bytes (128 units) apart
// in B; the first one overwrites the accumulator when `accumulate` is 0.
template <int kMma>
__device__ __forceinline__ void mma_filter_row(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                               uint32_t idesc, uint32_t accumulate, uint32_t issue) {
  static_assert(kMma >= 1 && kMma <= 4, "one to four K slices per filter row");
#define TB200_ROW_MMA(K)                                      \
  "add.u32 a, %1, " #K "*2;\n"                                \
  "add.u32 b, %2, " #K "*128;\n"                              \
  "mov.b64 da, {a, %3};\n"                                    \
  "mov.b64 db, {b, %3};\n"                                    \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, t;\n"
#define TB200_ROW_HEAD                                        \
  "{\n"                                                       \
  ".reg .pred p, q, t;\n"                                     \
  ".reg .b64 da, db;\n"                                       \
  ".reg .b32 a, b;\n"                                         \
  "setp.ne.b32 p, %5, 0;\n"                                   \
  "setp.ne.b32 q, %6, 0;\n"                                   \
  "setp.eq.b32 t, 0, 0;\n"                                    \
  "mov.b64 da, {%1, %3};\n"                                   \
  "mov.b64 db, {%2, %3};\n"                                   \
  "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n"
#define TB200_ROW_ARGS \
  ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(issue) : "memory"
  if constexpr (kMma == 1) {
    asm volatile(TB200_ROW_HEAD "}\n" TB200_ROW_ARGS);
  } else if constexpr (kMma == 2) {
    asm volatile(TB200_ROW_HEAD TB200_ROW_MMA(1) "}\n" TB200_ROW_ARGS);
  } else if constexpr (kMma == 3) {
    asm volatile(TB200_ROW_HEAD TB200_ROW_MMA(1) TB200_ROW_MMA(2) "}\n" TB200_ROW_ARGS);
  } else {
    asm volatile(TB200_ROW_HEAD TB200_ROW_MMA(1) TB200_ROW_MMA(2) TB200_ROW_MMA(3) "}\n" TB200_ROW_ARGS);
  }
#undef TB200_ROW_MMA
#undef TB200_ROW_HEAD
#undef TB200_ROW_ARGS
}
}  // namespace ptx

template <typename OutT>
__global__ void __launch_bounds__(kBandThreads, 1)
conv2d_rowband_sm100_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_out,
                            const __grid_constant__ RowBandKernelArgs args) {
  using namespace ptx;
  static_assert(sizeof(OutT) == 2, "16-bit activations only");
  constexpr uint32_t kTmemCols = kBandAccs * kBandBN;   // 512

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t w_s = smem_base;                                                   // filter bank
  const uint32_t band_s = smem_base + args.w_bytes;                                 // band slots
  const uint32_t stg_off = args.w_bytes + static_cast<uint32_t>(args.num_slots) * args.slot_bytes;
  const uint32_t stg_s = smem_base + stg_off;                                       // epilogue staging, two 4 KB boxes per warp
  const uint32_t bias_off = stg_off + 16u * kBandBoxBytes;
  const uint32_t bar_base = smem_base + bias_off + kBandBN * 4u;
  auto band_full = [&](uint32_t s) { return bar_base + 8u * s; };
  auto band_empty = [&](uint32_t s) { return bar_base + 8u * (kBandMaxSlots + s); };
  auto tfull_bar = [&](uint32_t b) { return bar_base + 8u * (2 * kBandMaxSlots + b); };
  auto tempty_bar = [&](uint32_t b) { return bar_base + 8u * (2 * kBandMaxSlots + kBandAccs + b); };
  constexpr uint32_t kBarBytes = 8u * (2 * kBandMaxSlots + 2 * kBandAccs);
  const uint32_t tmem_slot = bar_base + kBarBytes;
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(smem_gen + bias_off + kBandBN * 4u + kBarBytes);
  volatile uint32_t* abort_p = tmem_slot_p + 1;
  float* bias_s = reinterpret_cast<float*>(smem_gen + bias_off);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // the same in every lane, provably
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kBandMaxSlots; ++s) {
      mbar_init(band_full(s), 1);
      mbar_init(band_empty(s), 2);   // both MMA-issuing warps commit
    }
    for (uint32_t b = 0; b < kBandAccs; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);   // the four warps of the epilogue group that drains this accumulator
    }
    *abort_p = 0u;
    fence_mbar_init();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc<kTmemCols>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot_p, 0);
  TB200_PROF_NOW(12);
  griddep_launch_dependents();
  griddep_wait();   // the packed filter bank and the padded image copy come from the launches before this one

  // ---- filter bank -> shared memory, core-matrix form: 16-byte k-core kc of filter row r, output channel n at
  //      (r * 2 kmma + kc) * 1024 + (n / 8) * 128 + (n % 8) * 16
  {
    const int cores = args.kmma * 2;
    const int total = kBandBN * args.R * cores;
    const uint4* __restrict__ wg = static_cast<const uint4*>(args.w);
    for (int i = threadIdx.x; i < total; i += kBandThreads) {
      const int kc = i % cores;
      const int t = i / cores;
      const int r = t % args.R;
      const int n = t / args.R;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (n < args.K_out) v = __ldg(wg + (static_cast<long long>(n) * args.R + r) * cores + kc);
      st_shared_v4(w_s + static_cast<uint32_t>(r * cores + kc) * 1024u + static_cast<uint32_t>(n >> 3) * 128u +
                       static_cast<uint32_t>(n & 7) * 16u, v);
    }
    fence_proxy_async_smem();   // the tensor pipe reads these bytes through the async proxy
  }
  __syncthreads();
  TB200_PROF_NOW(13);

  const int first_band = static_cast<int>(blockIdx.x);
  const int band_step = static_cast<int>(gridDim.x);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      uint32_t it = 0, slot = 0, use = 0;
      bool ok = true;
      long long prof_wait = 0;
      (void)prof_wait;
      TB200_PROF_T(prof_t0);
      for (int b = first_band; b < args.n_bands; b += band_step, ++it) {
        if (static_cast<int>(it) == args.test_producer_stop) break;   // test hook: go silent, leave normally
        TB200_PROF_T(tw);
        if (!mbar_wait_bounded(band_empty(slot), (use & 1u) ^ 1u, abort_p, args.wait_limit)) {
          report_error_status(args.status, abort_p, kErrProducerWait, it);
          ok = false;
          break;
        }
        TB200_PROF_ADD(prof_wait, tw);
        const int img = b / args.bands_per_img;
        const int ho0 = (b - img * args.bands_per_img) * args.hb;
        mbar_arrive_expect_tx(band_full(slot), args.box_bytes);
        tma_load_4d(band_s + slot * args.slot_bytes, &tmap_x, band_full(slot), 0, 0, ho0 * args.stride_h - args.pad_h,
                    img);
        if (++slot == static_cast<uint32_t>(args.num_slots)) { slot = 0; ++use; }
      }
      TB200_PROF_STORE(0, prof_wait);
      TB200_PROF_STORE(1, clock64() - prof_t0);
      // never leave with a copy in flight into shared memory: wait (bounded) until the last bands have been used
      if (ok) {
        const uint32_t pending = it < static_cast<uint32_t>(args.num_slots) ? it : static_cast<uint32_t>(args.num_slots);
        for (uint32_t i = 0; i < pending; ++i) {
          // walk back from the slot after the last one filled: slot, use name the NEXT fill
          const uint32_t q = it - pending + i;
          const uint32_t qs = q % static_cast<uint32_t>(args.num_slots), qu = q / static_cast<uint32_t>(args.num_slots);
          if (!mbar_wait_bounded(band_empty(qs), qu & 1u, abort_p, args.wait_limit)) break;
        }
      } else {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ------------------------------------------------------------ MMA issuers (two whole warps, one lane of each issues)
    // Feeding N = 64 MMAs is bound by how fast a warp gets through the issuing instruction stream, so two warps
    // issue: warp 1 the even units, warp 10 the odd ones -- the accumulators the epilogue group of the same parity drains.
    {
      const uint32_t issuer = warp == 1 ? 0u : 1u;
      const uint32_t issue = elect_one_lane();
      const uint32_t desc_hi = (128u >> 4) | (1u << 14);        // SBO 128 B between 8-row groups, no swizzle
      const uint32_t a_lbo = (16u >> 4) << 16;                  // A: k-cores 16 B apart -- the overlapping rows
      const uint32_t b_lbo = (1024u >> 4) << 16;                // B: k-cores 1024 B apart
      const uint32_t row_units = args.row_bytes >> 4;
      const uint32_t a_step = static_cast<uint32_t>(args.dil_h) * row_units;
      const uint32_t b_step = static_cast<uint32_t>(args.kmma) * 128u;
      const uint32_t j_step = static_cast<uint32_t>(args.stride_h) * row_units;
      const uint32_t b_first = (w_s >> 4) | b_lbo;
      uint32_t slot = 0, use = 0, unit = 0, it = 0;
      bool ok = true, acc_free = false;
      long long prof_wfull = 0, prof_wtmem = 0, prof_loop = 0;
      (void)prof_wfull; (void)prof_wtmem; (void)prof_loop;
      TB200_PROF_T(prof_t0);
      for (int b = first_band; b < args.n_bands && ok; b += band_step, ++it) {
        const int ho0 = (b % args.bands_per_img) * args.hb;
        const int rows = min(args.hb, args.Ho - ho0);
        TB200_PROF_T(tw1);
        if (!mbar_wait_bounded_uniform(band_full(slot), use & 1u, abort_p, args.wait_limit)) {
          if (issue) report_error_status(args.status, abort_p, kErrMmaWaitFull, it);
          ok = false;
          break;
        }
        TB200_PROF_ADD(prof_wfull, tw1);
        tc_fence_after();
        // descriptor low word of the first output row's first filter row; rows of the band follow j_step apart
        uint32_t a_j = ((band_s + slot * args.slot_bytes) >> 4) | a_lbo;
        for (int j = 0; j < rows && ok; ++j, a_j += j_step) {
          uint32_t a_unit = a_j;
          for (int wt = 0; wt < args.wtiles; ++wt, ++unit, a_unit += 128u) {
            if ((unit & 1u) != issuer) continue;
            // accumulator `buf` is free once its previous drain (the use before this one) has arrived
            const uint32_t buf = unit & (kBandAccs - 1), buf_parity = (unit / kBandAccs) & 1u;
            TB200_PROF_T(tw0);
            if (!acc_free && !mbar_wait_bounded_uniform(tempty_bar(buf), buf_parity ^ 1u, abort_p, args.wait_limit)) {
              if (issue) report_error_status(args.status, abort_p, kErrMmaWaitTmem, unit);
              ok = false;
              break;
            }
            TB200_PROF_ADD(prof_wtmem, tw0);
            tc_fence_after();
            // ask about this warp's next accumulator now; the answer comes back while this unit's MMAs are issued
            const uint32_t d = tmem_base + buf * kBandBN;
            const uint32_t commit_bar = tfull_bar(buf);
            const uint32_t nbuf = (unit + 2u) & (kBandAccs - 1), nparity = ((unit + 2u) / kBandAccs) & 1u;
            const bool probe = mbar_test_wait(tempty_bar(nbuf), nparity ^ 1u);
            uint32_t a_row = a_unit;
            uint32_t b_lo = b_first;
            uint32_t acc = 0u;
            // one filter row per step; the loop is kept this tight on purpose (it is the pace of the tensor pipe)
            TB200_PROF_T(tl);
            if (args.kmma == 2) {
#pragma unroll 1
              for (int r = 0; r < args.R; ++r, a_row += a_step, b_lo += b_step, acc = 1u)
                mma_filter_row<2>(d, a_row, b_lo, desc_hi, args.idesc, acc, issue);
            } else if (args.kmma == 1) {
#pragma unroll 1
              for (int r = 0; r < args.R; ++r, a_row += a_step, b_lo += b_step, acc = 1u)
                mma_filter_row<1>(d, a_row, b_lo, desc_hi, args.idesc, acc, issue);
            } else if (args.kmma == 3) {
#pragma unroll 1
              for (int r = 0; r < args.R; ++r, a_row += a_step, b_lo += b_step, acc = 1u)
                mma_filter_row<3>(d, a_row, b_lo, desc_hi, args.idesc, acc, issue);
            } else {
#pragma unroll 1
              for (int r = 0; r < args.R; ++r, a_row += a_step, b_lo += b_step, acc = 1u)
                mma_filter_row<4>(d, a_row, b_lo, desc_hi, args.idesc, acc, issue);
            }
            TB200_PROF_ADD(prof_loop, tl);
            if (issue) mma_commit(commit_bar);   // this accumulator is complete
            acc_free = __all_sync(0xffffffffu, probe);
          }
        }
        if (issue) mma_commit(band_empty(slot));     // the band may be overwritten
        __syncwarp();
        if (++slot == static_cast<uint32_t>(args.num_slots)) { slot = 0; ++use; }
      }
      if (issue && issuer == 0u) {
        TB200_PROF_STORE(2, prof_wfull);
        TB200_PROF_STORE(3, prof_wtmem);
        TB200_PROF_STORE(6, prof_loop);
        TB200_PROF_STORE(4, clock64() - prof_t0);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..9)
    // Group e (warps 2..5 / 6..9) drains the accumulators e, e + 2, ...; warp w owns TMEM lanes 32 * (w % 4) ...,
    // one output pixel per lane: its 64 channels are one swizzled 128-byte row of the warp's staging box.
    const int ew = warp - 2;
    const uint32_t egroup = static_cast<uint32_t>(ew >> 2);
    const int quarter = warp & 3;
    const uint32_t stg0 = stg_s + static_cast<uint32_t>(ew) * 2u * kBandBoxBytes;
    const uint32_t lane_row = static_cast<uint32_t>(lane) * 128u;
    const uint32_t lane_xor = static_cast<uint32_t>(lane) & 7u;
    if (ew == 0) {
      for (int n = lane; n < kBandBN; n += 32) {
        float b = 0.0f;
        if (args.bias != nullptr && n < args.K_out)
          b = args.bias_is_f32 ? __ldg(static_cast<const float*>(args.bias) + n)
                               : OutTraits<OutT>::to_f(static_cast<const OutT*>(args.bias)[n]);
        bias_s[n] = b;
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps only
    const uint32_t bias_addr = smem_base + bias_off;
    uint32_t unit = 0, box = 0;
    bool ok = true;
    long long prof_wacc = 0;
    (void)prof_wacc;
    TB200_PROF_T(prof_t0);
    for (int b = first_band; b < args.n_bands && ok; b += band_step) {
      const int img = b / args.bands_per_img;
      const int ho0 = (b - img * args.bands_per_img) * args.hb;
      const int rows = min(args.hb, args.Ho - ho0);
      for (int j = 0; j < rows && ok; ++j) {
        for (int wt = 0; wt < args.wtiles; ++wt, ++unit) {
          if ((unit & 1u) != egroup) continue;
          const uint32_t buf = unit & (kBandAccs - 1), buse = unit / kBandAccs;
          TB200_PROF_T(tw2);
          const bool ready = mbar_wait_bounded_warp<true>(tfull_bar(buf), buse & 1u, abort_p, 2 * args.wait_limit, lane);
          TB200_PROF_ADD(prof_wacc, tw2);
          if (!ready) {
            if (lane == 0) report_error_status(args.status, abort_p, kErrEpilogueWait, unit);
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t v[2][32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBandBN;
          tmem_ld_32x32(taddr, v[0]);
          tmem_ld_32x32(taddr + 32, v[1]);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(tempty_bar(buf));
            bulk_wait_group_read<1>();   // the store that last used this box (two units ago) has read it out
          }
          __syncwarp();
          const uint32_t stg = stg0 + box * kBandBoxBytes;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float f[32];
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) f[jj] = __uint_as_float(v[h][jj]);
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              const float4 b4 = ld_shared_f4(bias_addr + static_cast<uint32_t>(h * 32 + j4 * 4) * 4u);
              add2(f[j4 * 4 + 0], f[j4 * 4 + 1], b4.x, b4.y);
              add2(f[j4 * 4 + 2], f[j4 * 4 + 3], b4.z, b4.w);
            }
            uint4 packed[4];
            if (args.act == kActRelu) {
              finish32<OutT, true>(f, nullptr, false, packed);
            } else {
              apply_act32<true>(f, args.act);
              finish32<OutT, false>(f, nullptr, false, packed);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c)
              st_shared_v4(stg + lane_row + ((static_cast<uint32_t>(h * 4 + c) ^ lane_xor) << 4), packed[c]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&tmap_out, stg, 0, wt * 128 + quarter * 32, ho0 + j, img);
            bulk_commit_group();
          }
          box ^= 1u;
        }
      }
    }
    if (lane == 0) bulk_wait_group0();   // the stores have left shared memory and reached global memory
    if (warp == 2 && lane == 0) {
      TB200_PROF_STORE(5, prof_wacc);
      TB200_PROF_STORE(7, clock64() - prof_t0);
    }
    if (warp == 6 && lane == 0) {
      TB200_PROF_STORE(8, prof_wacc);
      TB200_PROF_STORE(9, clock64() - prof_t0);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  TB200_PROF_NOW(14);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

}  // namespace tb200
