// Stride-1 small-filter Conv2d for 64-channel 16-bit activations (the ResNet 3x3 64->64 layer the reference's own
// benchmark is built around: examples/resnet_bench.rs:28-47, src/optimizer/benchmark.rs:474-509), sm_100a.
//
// The general kernel (conv2d_sm100.cuh) fetches one 128-pixel x 128-byte im2col block per filter tap, i.e. every
// input pixel travels L2 -> shared memory R*S times, and re-fetches the weights with every stage; with only 64
// output channels per MMA that traffic, not the tensor pipe, sets the pace. Here
//   * the filter bank stays in shared memory for the whole kernel (each CTA of a pair keeps half the output
//     channels: R*S blocks of 32 rows x 128 bytes);
//   * the activations of a tile -- `ht` output rows of one image plus the R-1 halo rows -- arrive as ONE tiled TMA
//     copy: a box of (ht + R - 1) rows x Wp pixels x 64 channels that starts pad_w pixels left of the image, so the
//     zero fill of out-of-range coordinates is the padding. Wp = W + pad_w: the box ends where the image ends, and
//     the right-hand padding of a row is the left-hand padding of the next row of the box;
//   * in that window pixel (h, w) sits in 128-byte row (h - h0) * Wp + (w + pad_w), so the operand of filter tap
//     (r, s) for the output pixels g = (ho - ho0) * Wp + wo, g = 0, 1, 2 ..., is simply the window shifted down by
//     r * Wp + s rows. tcgen05 shared-memory descriptors apply the 128-byte swizzle to absolute address bits, so a
//     descriptor may start at any row of the window: the R*S taps are R*S descriptors over the same bytes.
// One output pixel in Wp is a dummy (wo = Wo .. Wp-1: its taps straddle two image rows); it is computed and dropped.
// MMAs are M = 256 over a CTA pair (each CTA its own tile / window, 128 pixels per block), N = 64, K = 16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "conv2d_sm100.cuh"

namespace tb200 {

constexpr int kWinThreads = 352;        // warp 0 TMA, warps 1 and 10 MMA, warps 2..9 epilogue (two groups of four)
constexpr int kWinBN = 64;              // output channels per MMA (K_out <= 64)
constexpr int kWinMaxBlocks = 4;        // 128-pixel blocks per tile: 4 x 64 TMEM columns, double-buffered = 512
constexpr int kWinStageBytes = 32 * 64; // per epilogue warp: 32 pixels x 64 bytes (half of the 64 channels)

struct WindowKernelArgs {
  // geometry (stride 1, dilation 1)
  int R, S, pad_h, pad_w;
  int Wp;                 // window row pitch in pixels: W + pad_w
  int Ho, Wo;
  // tiles: every image is cut into tiles_per_img tiles of ht_full output rows, plus -- when ht_short > 0 -- one tile of
  // ht_short rows at the bottom. Tiles are numbered full tiles first ([0, n_full): image-major), then the short ones
  // ([n_full, n_full + n_short): one per image), and handed to CTA pairs two at a time, so that both CTAs of a pair
  // always work on tiles of the same kind (same box, same block count).
  int ht_full, nblk_full, ht_short, nblk_short;
  int tiles_per_img, n_full, n_short;
  int pair_tiles_full, pair_tiles;     // pair-tiles made of full tiles / in total
  uint32_t box_bytes_full, box_bytes_short;   // bytes one CTA's window copy delivers
  uint32_t w_bytes;        // this CTA's filter bank: R*S * 4096
  uint32_t slot_bytes;     // pitch of the two window slots (1024-byte multiple)
  uint32_t zero_from;      // bytes of a slot a full tile's copy fills; [zero_from, slot_bytes) is cleared once and stays
                           // zero: the right-hand padding of the window's last row reads there
  uint32_t idesc;          // M = 256, N = 64, fp32 accumulate
  // epilogue
  int K_out;
  void* out;
  long long out_sn, out_sh, out_sw;   // element strides of (image, row, column); channels are contiguous
  const void* bias;
  int bias_is_f32;
  int act;
  uint32_t* status;
  long long wait_limit;   // cycles any single wait may take before the role gives up
  int test_producer_stop; // test hook, -1 in normal use: the TMA producer stops after this many windows
  long long* prof;        // cycle counters, only written by -DTB200_PROFILE builds
};

__host__ __device__ constexpr uint32_t window_smem_bytes(uint32_t w_bytes, uint32_t slot_bytes) {
  return w_bytes + 2u * slot_bytes + 8u * kWinStageBytes + kWinBN * 4u + 256u + 1024u;
}

namespace ptx {
// Tiled loads for a CTA pair: the copy lands in this CTA's shared memory and completes on `bar`, a shared::cluster
// address (the leader's barrier). No multicast: each CTA fetches what it needs itself.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                                 int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// The four K = 16 MMAs of one filter tap (64 channels) as a single block: M = 256 over a CTA pair, kind::f16 (fp16 /
// bf16 operands, fp32 accumulate). a_lo / b_lo are descriptor low words of the first K slice; the others follow 32
// bytes (2 units) apart inside the 128-byte rows. kFirstAccumulates = false: the first MMA overwrites the accumulator.
// Executed by the whole (converged) MMA warp with identical operands in every lane; the instructions are predicated
// on `issue`, 1 in one lane: operand arithmetic in uniform control flow stays in uniform registers, where the MMA
// reads its descriptors from, and that is what lets one warp feed N = 64 MMAs at the tensor pipe's pace.
template <bool kFirstAccumulates>
__device__ __forceinline__ void mma_tap4_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                              uint32_t idesc, uint32_t issue) {
  asm volatile(
      "{\n"
      ".reg .pred p0, p1, q;\n"
      ".reg .b64 da, db;\n"
      ".reg .b32 a, b;\n"
      "setp.ne.b32 p0, %5, 0;\n"
      "setp.eq.b32 p1, 0, 0;\n"
      "setp.ne.b32 q, %6, 0;\n"
      "mov.b64 da, {%1, %3};\n"
      "mov.b64 db, {%2, %3};\n"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p0;\n"
      "add.u32 a, %1, 2;\n"
      "add.u32 b, %2, 2;\n"
      "mov.b64 da, {a, %3};\n"
      "mov.b64 db, {b, %3};\n"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p1;\n"
      "add.u32 a, %1, 4;\n"
      "add.u32 b, %2, 4;\n"
      "mov.b64 da, {a, %3};\n"
      "mov.b64 db, {b, %3};\n"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p1;\n"
      "add.u32 a, %1, 6;\n"
      "add.u32 b, %2, 6;\n"
      "mov.b64 da, {a, %3};\n"
      "mov.b64 db, {b, %3};\n"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p1;\n"
      "}\n" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(kFirstAccumulates ? 1 : 0), "r"(issue)
      : "memory");
}
}  // namespace ptx

// The MMAs of one tile: for each of its `nblk` 128-pixel blocks (accumulators 64 TMEM columns apart), every filter
// tap (r, s) reads the window shifted by r * Wp + s pixel rows (8 descriptor units each) against the tap's 4 KB of
// the filter bank. k3x3: the common 3x3 filter as straight-line code. Whole-warp code, see mma_tap4_pair. Feeding
// N = 64 MMAs is bound by how fast a warp gets through this instruction stream (about 65 cycles per MMA here against
// the 43 the tensor pipe needs), so two warps issue, one block each in turn.
template <bool k3x3>
__device__ __forceinline__ void window_issue_tile(uint32_t tmem_d0, uint32_t win_units, uint32_t w_units,
                                                  uint32_t desc_hi, uint32_t idesc, int blk0, int nblk, int R, int S,
                                                  uint32_t row_units, uint32_t issue) {
  using namespace ptx;
  for (int blk = blk0; blk < nblk; blk += 2) {   // the two issuing warps take every second block
    const uint32_t d = tmem_d0 + static_cast<uint32_t>(blk) * kWinBN;
    uint32_t a_lo = win_units + static_cast<uint32_t>(blk) * (128u * 8u);
    uint32_t b_lo = w_units;
    if constexpr (k3x3) {
      mma_tap4_pair<false>(d, a_lo, b_lo, desc_hi, idesc, issue);
      mma_tap4_pair<true>(d, a_lo + 8u, b_lo + 256u, desc_hi, idesc, issue);
      mma_tap4_pair<true>(d, a_lo + 16u, b_lo + 512u, desc_hi, idesc, issue);
      mma_tap4_pair<true>(d, a_lo + row_units, b_lo + 768u, desc_hi, idesc, issue);
      mma_tap4_pair<true>(d, a_lo + row_units + 8u, b_lo + 1024u, desc_hi, idesc, issue);
      mma_tap4_pair<true>(d, a_lo + row_units + 16u, b_lo + 1280u, desc_hi, idesc, issue);
      mma_tap4_pair<true>(d, a_lo + 2u * row_units, b_lo + 1536u, desc_hi, idesc, issue);
      mma_tap4_pair<true>(d, a_lo + 2u * row_units + 8u, b_lo + 1792u, desc_hi, idesc, issue);
      mma_tap4_pair<true>(d, a_lo + 2u * row_units + 16u, b_lo + 2048u, desc_hi, idesc, issue);
    } else {
      const uint32_t row_step = row_units - static_cast<uint32_t>(S) * 8u;   // from a filter row's last tap to the next row
      mma_tap4_pair<false>(d, a_lo, b_lo, desc_hi, idesc, issue);
      for (int r = 0; r < R; ++r) {
        for (int s = (r == 0 ? 1 : 0); s < S; ++s) {
          a_lo += 8u;
          b_lo += 256u;
          mma_tap4_pair<true>(d, a_lo, b_lo, desc_hi, idesc, issue);
        }
        a_lo += row_step;
      }
    }
  }
}

// Staging box of one epilogue warp (32 pixel rows x 64 bytes; 16-byte chunk c of row r at
// r*64 + ((c ^ ((r >> 1) & 3)) << 4): conflict-free both for a lane writing its own row and for the read-out
// below) -> global memory. Lane l moves chunk l & 3 of rows (l >> 2) + 8 i, so every store instruction covers eight
// 64-byte row segments. `row_off` is this lane's own pixel offset in elements, `row_ok` whether its pixel exists;
// `col0` the first of the box's 32 output channels.
template <typename OutT>
__device__ __forceinline__ void window_store_box(uint32_t stg, OutT* out, long long row_off, bool row_ok, int col0,
                                                 int k_out, int lane) {
  __syncwarp();   // every lane's row is in the box
  const uint32_t ok_rows = __ballot_sync(0xffffffffu, row_ok);
  const uint32_t chunk = static_cast<uint32_t>(lane) & 3u;
  const bool chunk_ok = col0 + static_cast<int>(chunk) * 8 < k_out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2);
    const long long off = __shfl_sync(0xffffffffu, row_off, r);
    const uint4 v = ptx::ld_shared_v4(stg + static_cast<uint32_t>(r) * 64u +
                                      ((chunk ^ ((static_cast<uint32_t>(r) >> 1) & 3u)) << 4));
    if (chunk_ok && ((ok_rows >> r) & 1u)) *(reinterpret_cast<uint4*>(out + off + col0) + chunk) = v;
  }
  __syncwarp();   // the box may be rewritten once every lane has read it out
}

template <typename OutT>
__global__ void __launch_bounds__(kWinThreads, 1)
conv2d_window_sm100_kernel(const __grid_constant__ CUtensorMap tmap_x_full,
                           const __grid_constant__ CUtensorMap tmap_x_short,
                           const __grid_constant__ CUtensorMap tmap_w,
                           const __grid_constant__ WindowKernelArgs args) {
  using namespace ptx;
  static_assert(sizeof(OutT) == 2, "16-bit activations only");
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kBufCols = kWinMaxBlocks * kWinBN;   // 256 columns per accumulator buffer
  const uint32_t cta_rank = __shfl_sync(0xffffffffu, cluster_ctarank(), 0);   // the same in every lane, provably
  const bool leader = cta_rank == 0u;
  const int pair = static_cast<int>(blockIdx.x >> 1);
  const int num_pairs = static_cast<int>(gridDim.x >> 1);

  TB200_PROF_NOW(12);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t w_s = smem_base;                           // filter bank: tap t at t * 4096
  const uint32_t win_s = smem_base + args.w_bytes;          // two window slots
  const uint32_t stg_s = win_s + 2u * args.slot_bytes;      // epilogue staging, 2 KB per warp
  const uint32_t bias_off = args.w_bytes + 2u * args.slot_bytes + 8u * kWinStageBytes;
  const uint32_t bar_base = smem_base + bias_off + kWinBN * 4u;
  const uint32_t w_bar = bar_base;
  auto win_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto win_empty = [&](int s) { return bar_base + 8u * (3 + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (5 + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (7 + b); };
  const uint32_t tmem_slot = bar_base + 8u * 9u;
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(smem_gen + bias_off + kWinBN * 4u + 72u);
  volatile uint32_t* abort_p = tmem_slot_p + 1;
  float* bias_s = reinterpret_cast<float*>(smem_gen + bias_off);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);   // likewise
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(w_bar, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(win_full(s), 1);
      mbar_init(win_empty(s), 2);     // both MMA-issuing warps commit
      mbar_init(tfull_bar(s), 2);
      mbar_init(tempty_bar(s), 16);   // the eight epilogue warps of both CTAs
    }
    *abort_p = 0u;
    fence_mbar_init();
    for (uint32_t s = 0; s < 2; ++s)
      for (uint32_t b = args.zero_from; b < args.slot_bytes; b += 16u)
        st_shared_v4(win_s + s * args.slot_bytes + b, make_uint4(0u, 0u, 0u, 0u));
    fence_proxy_async_smem();   // the tensor pipe reads these bytes through the async proxy
    prefetch_tmap(&tmap_x_full);
    prefetch_tmap(&tmap_x_short);
    prefetch_tmap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair<kTmemCols>(tmem_slot);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot_p, 0);
  griddep_launch_dependents();
  griddep_wait();
  TB200_PROF_NOW(13);

  // tile of this CTA in pair-tile j: index, kind, image and first output row; `valid` is false for the partner-less
  // CTA of an odd tile count (it repeats its neighbour's copy so that every barrier sees its bytes, and stores nothing)
  struct Tile {
    bool full, valid;
    int img, ho0, ht, nblk;
  };
  auto tile_of = [&](int j) {
    Tile t;
    t.full = j < args.pair_tiles_full;
    int idx, count;
    if (t.full) {
      idx = 2 * j + static_cast<int>(cta_rank);
      count = args.n_full;
    } else {
      idx = 2 * (j - args.pair_tiles_full) + static_cast<int>(cta_rank);
      count = args.n_short;
    }
    t.valid = idx < count;
    if (!t.valid) idx = count - 1;
    if (t.full) {
      t.img = idx / args.tiles_per_img;
      t.ho0 = (idx - t.img * args.tiles_per_img) * args.ht_full;
      t.ht = args.ht_full;
      t.nblk = args.nblk_full;
    } else {
      t.img = idx;
      t.ho0 = args.tiles_per_img * args.ht_full;
      t.ht = args.ht_short;
      t.nblk = args.nblk_short;
    }
    return t;
  };

  // The pair's own sequence of pair-tiles, the same for every role: its full tiles (pair, pair + num_pairs, ...), then
  // its short ones. Short tiles are dealt so that they even the load out: when the full tiles do not divide by the
  // number of pairs, pairs [0, heavy) hold one full tile more than the others, and the others are given short tiles
  // first, up to the `catch_up` of them that weigh as much as one full tile; the rest go round robin over all pairs.
  // (Dealt round robin from where the full tiles ended, the busiest pair of the 256-image layer had 46 blocks
  // against a mean of 43.2; now 44.) Returns the index in the numbering tile_of() takes, -1 past the end.
  const int pf_tiles = args.pair_tiles_full, ps_tiles = args.pair_tiles - args.pair_tiles_full;
  const int my_fulls = pair < pf_tiles ? (pf_tiles - pair + num_pairs - 1) / num_pairs : 0;
  const int heavy = pf_tiles % num_pairs;
  const int light = num_pairs - heavy;
  const int catch_up = heavy == 0 || args.nblk_short <= 0 ? 0 : args.nblk_full / args.nblk_short;
  const int first_deal = min(ps_tiles, light * catch_up);            // short tiles that go to the light pairs only
  const int my_first = pair >= heavy && first_deal > pair - heavy ? (first_deal - (pair - heavy) + light - 1) / light : 0;
  auto my_pair_tile = [&](uint32_t it) -> int {
    const int i = static_cast<int>(it);
    if (i < my_fulls) return pair + i * num_pairs;
    int k = i - my_fulls, s;
    if (k < my_first) {
      s = (pair - heavy) + k * light;
    } else {
      k -= my_first;
      s = first_deal + pair + k * num_pairs;
    }
    return s < ps_tiles ? pf_tiles + s : -1;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread per CTA)
    if (lane == 0) {
      const uint32_t w_bar_leader = mapa_cluster(w_bar, 0u);
      if (leader) mbar_arrive_expect_tx(w_bar, 2u * args.w_bytes);
      const int taps = args.R * args.S;
      for (int t = 0; t < taps; ++t)
        tma_load_2d_pair(w_s + static_cast<uint32_t>(t) * 4096u, &tmap_w, w_bar_leader, t * 64,
                         static_cast<int>(cta_rank) * 32);
      uint32_t it = 0;
      bool ok = true;
      for (int j; ok && (j = my_pair_tile(it)) >= 0; ++it) {
        if (static_cast<int>(it) == args.test_producer_stop) break;   // test hook: go silent, leave normally
        const uint32_t slot = it & 1u, use = it >> 1;
        if (!mbar_wait_bounded(win_empty(slot), (use & 1u) ^ 1u, abort_p, args.wait_limit)) {
          report_error_status(args.status, abort_p, kErrProducerWait, it);
          ok = false;
          break;
        }
        const Tile t = tile_of(j);
        if (leader) mbar_arrive_expect_tx(win_full(slot), 2u * (t.full ? args.box_bytes_full : args.box_bytes_short));
        tma_load_4d_pair(win_s + slot * args.slot_bytes, t.full ? &tmap_x_full : &tmap_x_short,
                         mapa_cluster(win_full(slot), 0u), 0, -args.pad_w, t.ho0 - args.pad_h, t.img);
      }
      // never leave with a copy in flight into this CTA's shared memory: wait (bounded) for the last windows to be used
      if (ok) {
        const uint32_t pending = it < 2u ? it : 2u;
        for (uint32_t i = 0; i < pending; ++i) {
          const uint32_t q = it - pending + i;
          if (!mbar_wait_bounded(win_empty(q & 1u), (q >> 1) & 1u, abort_p, args.wait_limit)) break;
        }
      } else {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { __nanosleep(1000); }
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ------------------------------------------------------------ MMA issuers (warps 1 and 10 of the leader CTA; one lane issues)
    if (leader) {
      const int issuer = warp == 1 ? 0 : 1;
      const uint32_t issue = elect_one_lane();
      const uint32_t desc_hi = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);   // SBO 1024 B, SWIZZLE_128B
      bool ok = mbar_wait_bounded_uniform(w_bar, 0u, abort_p, args.wait_limit);
      if (!ok && issue) report_error_status(args.status, abort_p, kErrMmaWaitFull, 0xffffu);
      uint32_t it = 0;
      long long prof_wfull = 0, prof_wtmem = 0, prof_loop = 0;
      (void)prof_wfull; (void)prof_wtmem; (void)prof_loop;
      TB200_PROF_T(prof_t0);
      const uint32_t w_units = w_s >> 4;
      const uint32_t row_units = static_cast<uint32_t>(args.Wp) * 8u;          // one window row, in 16-byte units
      const uint32_t idesc = args.idesc;
      const bool three_by_three = args.R == 3 && args.S == 3;
      for (int j; ok && (j = my_pair_tile(it)) >= 0; ++it) {
        const uint32_t slot = it & 1u, use = it >> 1;   // window slot and accumulator buffer alternate together
        const int nblk = j < args.pair_tiles_full ? args.nblk_full : args.nblk_short;
        TB200_PROF_T(tw0);
        if (!mbar_wait_bounded_uniform(tempty_bar(slot), (use & 1u) ^ 1u, abort_p, args.wait_limit)) {
          if (issue) report_error_status(args.status, abort_p, kErrMmaWaitTmem, it);
          ok = false;
          break;
        }
        TB200_PROF_ADD(prof_wtmem, tw0);
        TB200_PROF_T(tw1);
        if (!mbar_wait_bounded_uniform(win_full(slot), use & 1u, abort_p, args.wait_limit)) {
          if (issue) report_error_status(args.status, abort_p, kErrMmaWaitFull, it);
          ok = false;
          break;
        }
        TB200_PROF_ADD(prof_wfull, tw1);
        tc_fence_after();
        // (the shuffles restate that these are the same in every lane, whatever the loop around them looks like)
        const uint32_t win_units = __shfl_sync(0xffffffffu, (win_s + slot * args.slot_bytes) >> 4, 0);   // 16-byte units
        const uint32_t tile_d = __shfl_sync(0xffffffffu, tmem_base + slot * kBufCols, 0);
        TB200_PROF_T(tl);
        if (three_by_three)
          window_issue_tile<true>(tile_d, win_units, w_units, desc_hi, idesc, issuer, nblk, 3, 3, row_units, issue);
        else
          window_issue_tile<false>(tile_d, win_units, w_units, desc_hi, idesc, issuer, nblk, args.R, args.S, row_units,
                                   issue);
        TB200_PROF_ADD(prof_loop, tl);
        if (issue) {
          mma_commit_pair(win_empty(slot));   // the window may be overwritten (both CTAs)
          mma_commit_pair(tfull_bar(slot));   // the accumulators are complete (both CTAs)
        }
        __syncwarp();
      }
      if (issue && issuer == 0) {
        TB200_PROF_STORE(2, prof_wfull);
        TB200_PROF_STORE(3, prof_wtmem);
        TB200_PROF_STORE(6, prof_loop);
        TB200_PROF_STORE(4, clock64() - prof_t0);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..9)
    // Group e (warps 2..5 / 6..9) takes the blocks e, e + 2 of every tile; warp w owns TMEM lanes 32 * (w % 4) ...,
    // one output pixel per lane. A block is 64 channels = two passes of 32 through the warp's 2 KB staging box.
    const int ew = warp - 2;
    const int egroup = ew >> 2;
    const int quarter = warp & 3;
    OutT* __restrict__ out = static_cast<OutT*>(args.out);
    const uint32_t stg = stg_s + static_cast<uint32_t>(ew) * kWinStageBytes;
    const uint32_t lane_row = static_cast<uint32_t>(lane) * 64u;
    const uint32_t lane_xor = (static_cast<uint32_t>(lane) >> 1) & 3u;
    // bias: one fp32 copy per CTA, written by the first epilogue warp (zeros past K_out / without a bias)
    if (ew == 0) {
      for (int n = lane; n < kWinBN; n += 32) {
        float b = 0.0f;
        if (args.bias != nullptr && n < args.K_out)
          b = args.bias_is_f32 ? __ldg(static_cast<const float*>(args.bias) + n)
                               : OutTraits<OutT>::to_f(static_cast<const OutT*>(args.bias)[n]);
        bias_s[n] = b;
      }
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps only
    const uint32_t bias_addr = smem_base + bias_off;
    uint32_t it = 0;
    bool ok = true;
    long long prof_wacc = 0;
    (void)prof_wacc;
    TB200_PROF_T(prof_t0);
    for (int j; ok && (j = my_pair_tile(it)) >= 0; ++it) {
      const uint32_t buf = it & 1u, use = it >> 1;
      const Tile t = tile_of(j);
      TB200_PROF_T(tw2);
      const bool ready = mbar_wait_bounded(tfull_bar(buf), use & 1u, abort_p, 2 * args.wait_limit);
      TB200_PROF_ADD(prof_wacc, tw2);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) report_error_status(args.status, abort_p, kErrEpilogueWait, it);
        ok = false;
        break;
      }
      tc_fence_after();
      const int last_blk = t.nblk - 1 - ((t.nblk - 1 - egroup) & 1);   // this group's last block (< egroup: none)
      for (int blk = egroup; blk < t.nblk; blk += 2) {
        uint32_t v[2][32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBufCols +
                               static_cast<uint32_t>(blk) * kWinBN;
        tmem_ld_32x32(taddr, v[0]);
        tmem_ld_32x32(taddr + 32, v[1]);
        tmem_ld_wait();
        if (blk == last_blk) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa_cluster(tempty_bar(buf), 0u));
        }
        // this lane's output pixel
        const int g = blk * 128 + quarter * 32 + lane;
        const int pq = g / args.Wp;
        const int wo = g - pq * args.Wp;
        const bool row_ok = t.valid && wo < args.Wo && pq < t.ht;
        const long long out_off = t.img * args.out_sn + (t.ho0 + pq) * args.out_sh + wo * args.out_sw;
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
            st_shared_v4(stg + lane_row + ((static_cast<uint32_t>(c) ^ lane_xor) << 4), packed[c]);
          window_store_box<OutT>(stg, out, out_off, row_ok, h * 32, args.K_out, lane);
        }
      }
      if (last_blk < egroup) {   // a tile with fewer blocks than groups: nothing to drain, but the buffer is still handed back
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_cluster(tempty_bar(buf), 0u));
      }
    }
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
  cluster_sync();   // neither CTA frees TMEM or exits while the other may still use the pair
  TB200_PROF_NOW(14);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair<kTmemCols>(tmem_base);
  }
}

}  // namespace tb200
