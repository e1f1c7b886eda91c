// Layout adapters for callers that hand over NCHW-contiguous activations or OIHW-contiguous
// weights (the layouts include/tracea.hpp:101-105 documents). The conv kernel itself reads
// channels-last memory, which is what the reference's kernel reads too (NHWC input, conv.rs:202-247).
// Both adapters read through arbitrary element strides and write dense, channel-padded buffers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {

// x[n, c, h, w] (element strides sn, sc, sh, sw) -> dst[n][h*W + w][Cp] with channels c >= C
// zero-filled. One CTA moves a 32 (channels) x 32 (pixels) tile through shared memory so that
// both sides are coalesced when the source is NCHW-contiguous.
template <typename T>
__global__ void to_channels_last_kernel(const T* __restrict__ src, T* __restrict__ dst, int C, int H,
                                        int W, int Cp, long long sn, long long sc, long long sh,
                                        long long sw) {
  __shared__ T tile[32][33];
  const int HW = H * W;
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * 32;
  const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x;  // 0..31
  const int ty = threadIdx.y;  // 0..7
  // read: consecutive tx -> consecutive pixels (contiguous for NCHW sources)
  const int p = p0 + tx;
  long long poff = 0;
  if (p < HW) {
    const int h = p / W;
    poff = h * sh + (p - h * W) * sw;
  }
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i;
    T v = T(0);
    if (p < HW && c < C) v = src[n * sn + c * sc + poff];
    tile[i][tx] = v;
  }
  __syncthreads();
  // write: consecutive tx -> consecutive channels
  const int c = c0 + tx;
  for (int i = ty; i < 32; i += 8) {
    const int pp = p0 + i;
    if (pp < HW && c < Cp) dst[(static_cast<long long>(n) * HW + pp) * Cp + c] = tile[tx][i];
  }
}

// Small-channel inputs (one pixel = 16 bytes after channel padding, e.g. RGB as 8 x bf16): x -> dst[n][h][Wp][Cp]
// with `pad` zero pixels in front of every row and zeros up to the row pitch Wp behind it. With the
// horizontal padding materialised, the S taps of one filter row are adjacent in memory, so the conv
// kernel fetches a whole filter row of a pixel (8 pixels x 16 B = one 128-byte k-chunk) with one copy.
// One thread writes one destination pixel (16 bytes).
template <typename T, int kCp>
__global__ void to_channels_last_wpad_kernel(const T* __restrict__ src, T* __restrict__ dst, int C, int H, int W,
                                             int Wp, int pad, long long total_pixels, long long sn, long long sc,
                                             long long sh, long long sw) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total_pixels) return;
  const int wp = static_cast<int>(i % Wp);
  const long long t = i / Wp;
  const int h = static_cast<int>(t % H);
  const long long n = t / H;
  const int w = wp - pad;
  T v[kCp];
#pragma unroll
  for (int c = 0; c < kCp; ++c) v[c] = T(0);
  if (w >= 0 && w < W) {
    const T* p = src + n * sn + h * sh + w * sw;
#pragma unroll
    for (int c = 0; c < kCp; ++c)
      if (c < C) v[c] = p[c * sc];
  }
  if constexpr (kCp * sizeof(T) == 16) *reinterpret_cast<uint4*>(dst + i * kCp) = *reinterpret_cast<const uint4*>(v);
  else *reinterpret_cast<uint2*>(dst + i * kCp) = *reinterpret_cast<const uint2*>(v);   // 8-byte pixels (4 x 16 bit)
}

// The same padded copy for the one layout that matters in practice -- a dense channels-last RGB image of 16-bit
// values (pixel pitch 3 elements) -> 4-channel pixels: a thread turns four source pixels (24 bytes, three 8-byte
// loads) into four destination pixels (32 bytes, four 8-byte stores), and the threads past the image's width write
// the zero pixels in front of and behind the row. One block per image row. `src_row` / `src_img`: element pitches.
__global__ void rgb16_rows_to_padded4_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int H, int W,
                                             int Wp, int pad, long long src_img, long long src_row) {
  const long long row = blockIdx.x;                       // n * H + h
  const long long n = row / H, h = row - n * H;
  const uint2* __restrict__ s = reinterpret_cast<const uint2*>(src + n * src_img + h * src_row);
  uint2* __restrict__ d = reinterpret_cast<uint2*>(dst + row * Wp * 4);
  const int groups = W >> 2;
  for (int t = threadIdx.x; t < groups; t += blockDim.x) {
    const uint2 a = s[3 * t], b = s[3 * t + 1], c = s[3 * t + 2];   // words w0..w5 = elements e0..e11, two per word
    uint2* o = d + pad + 4 * t;
    o[0] = make_uint2(a.x, a.y & 0xffffu);
    o[1] = make_uint2((a.y >> 16) | (b.x << 16), b.x >> 16);
    o[2] = make_uint2(b.y, c.x & 0xffffu);
    o[3] = make_uint2((c.x >> 16) | (c.y << 16), c.y >> 16);
  }
  const int zeros = Wp - W;                               // pad in front, the rest behind
  for (int z = threadIdx.x; z < zeros; z += blockDim.x) d[z < pad ? z : W + z] = make_uint2(0u, 0u);
}

// w[k, c, r, s] (element strides) -> dst[k][r][s][Cp], zero-padded channels: the K-major B operand
// whose Kgemm axis runs (r, s, c), the order the reference walks it (conv.rs:209-210).
// `Sd` >= S is the number of tap slots per filter row in the destination (slots s >= S are zero).
template <typename T>
__global__ void pack_weights_krsc_kernel(const T* __restrict__ src, T* __restrict__ dst,
                                         long long total, int C, int R, int S, int Sd, int Cp, long long sk,
                                         long long sc, long long sr, long long ss) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % Cp);
  long long t = i / Cp;
  const int s = static_cast<int>(t % Sd);
  t /= Sd;
  const int r = static_cast<int>(t % R);
  const long long k = t / R;
  dst[i] = (c < C && s < S) ? src[k * sk + c * sc + r * sr + s * ss] : T(0);
}

}  // namespace tb200
