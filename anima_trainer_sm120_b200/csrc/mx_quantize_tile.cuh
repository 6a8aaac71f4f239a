// Tile kernel shared by the MXFP8 quantiser and the fused LoKr merge + quantise:
// one CTA owns a 128 x 128 tile whose bf16 values come from a Loader functor
// (plain global loads, or W + alpha * kron(w1, w2) built on the fly).
#pragma once

#include <cuda_fp8.h>

#include "common.cuh"

namespace anima {
namespace mxq {

constexpr int kTile = 128;      // tile edge in elements
constexpr int kThreads = 256;
constexpr float kAmaxFloor = 1e-30f;  // mxfp8_gemm.py:114

struct QuantParams {
  int64_t rows, cols;
  uint8_t* codes_row;
  uint8_t* scales_row;
  uint8_t* codes_colT;
  uint8_t* scales_col;
  int tiled;  // scale layout
};

// e = ceil(log2(amax / 448)) clamped to [-127, 127], for amax >= 1e-30 (normal fp32).
__device__ __forceinline__ int mx_exponent(float amax) {
  const uint32_t u = __float_as_uint(amax);
  const int E = static_cast<int>(u >> 23) - 127;
  const uint32_t mant = u & 0x7fffffu;
  if (E == 128) return 127;  // inf / nan: log2 -> inf, clamped
  int e = E - 8 + (mant > 0x600000u ? 1 : 0);
  return max(-127, min(127, e));
}

// 2^-e as fp32 for e in [-127, 127]; 2^-127 is the subnormal 0x00400000.
__device__ __forceinline__ float mx_inv_scale(int e) {
  return e >= 127 ? __uint_as_float(0x00400000u) : __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
}

__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

// packed bf16 pair helpers (operands and results as raw 32-bit words)
__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ int tiled_offset(int r, int j) {
  return (r & 31) * 16 + (r >> 5) * 4 + j;
}

// Loader interface (device side), for one chunk of 8 values at (row, col .. col+7), both in range:
//   using Raw = ...;                                            what the chunk needs from HBM
//   Raw   fetch(int64_t row, int64_t col) const;                issues the long-latency loads only
//   uint4 finish(const Raw&, int64_t row, int64_t col) const;   the 8 bf16 values
//   static constexpr bool kZeroSafe;                            finish(Raw{}) == 0 and reads no memory
//   static constexpr int kSmemBytes; void prepare(void* smem);  per-CTA shared-memory state (a lookup table)
// All eight fetches of a thread are issued before the first finish, so a loader that computes
// (merge, GELU) does not serialise its chunks on memory latency.
template <bool ROW, bool COL, class Loader>
__global__ void __launch_bounds__(kThreads, COL ? 3 : 4) mx_quantize_kernel(const QuantParams p, const Loader load_arg) {
  __shared__ uint4 tile[COL ? kTile * 16 : 1];  // 128 rows x 256 B
  __shared__ __align__(16) uint8_t loader_smem[Loader::kSmemBytes > 0 ? Loader::kSmemBytes : 16];
  Loader load = load_arg;
  __shared__ __align__(16) uint8_t sc_row[ROW ? 512 : 16];
  __shared__ __align__(16) uint8_t sc_col[COL ? 512 : 16];

  const int t = threadIdx.x;
  const int64_t tile_r = static_cast<int64_t>(blockIdx.y) * kTile;
  const int64_t tile_c = static_cast<int64_t>(blockIdx.x) * kTile;
  const int c16 = t & 15;  // 16-byte chunk (8 elements) within the tile row
  const int r0 = t >> 4;   // 0..15
  const int64_t col = tile_c + c16 * 8;
  const bool col_ok = col < p.cols;  // cols % 32 == 0 or % 8 == 0: a chunk is all in or all out

  if (ROW) {
    // Padding entries of a partial tile must be 0 in the tiled layout.
    reinterpret_cast<uint16_t*>(sc_row)[t] = 0;
  }
  if (COL) reinterpret_cast<uint16_t*>(sc_col)[t] = 0;

  typename Loader::Raw fetched[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t r = tile_r + r0 + 16 * i;
    fetched[i] = typename Loader::Raw{};
    if (col_ok && r < p.rows) fetched[i] = load.fetch(r, col);
  }
  load.prepare(loader_smem);   // after the tile's loads are in flight; visible to all threads after the barrier
  __syncthreads();             // also: zero fill of sc_* visible before the byte stores

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r_in = r0 + 16 * i;
    // kZeroSafe loaders map an all-zero Raw to zeros without touching memory, so out-of-range chunks need no branch
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (Loader::kZeroSafe || (col_ok && tile_r + r_in < p.rows)) v = load.finish(fetched[i], tile_r + r_in, col);
    if (COL) tile[r_in * 16 + c16] = v;
    if (ROW) {
      float f[8];
      unpack8(v, f);
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[k]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, kAmaxFloor);
      const int e = mx_exponent(amax);
      const float inv = mx_inv_scale(e);
      uint2 codes;
      codes.x = e4m3x2(f[0] * inv, f[1] * inv) | (e4m3x2(f[2] * inv, f[3] * inv) << 16);
      codes.y = e4m3x2(f[4] * inv, f[5] * inv) | (e4m3x2(f[6] * inv, f[7] * inv) << 16);
      const int64_t r = tile_r + r_in;
      if (col_ok && r < p.rows) {
        *reinterpret_cast<uint2*>(p.codes_row + r * p.cols + col) = codes;
        if ((c16 & 3) == 0) {
          const int j = c16 >> 2;
          sc_row[p.tiled ? tiled_offset(r_in, j) : r_in * 4 + j] = static_cast<uint8_t>(e + 127);
        }
      }
    }
  }

  if (COL) {
    __syncthreads();
    const int cp = t & 63;  // column pair
    const int g = t >> 6;   // 32-row group within the tile
    const uint32_t* tile32 = reinterpret_cast<const uint32_t*>(tile);
    // one pass over the column pair: 32 packed bf16x2 words stay in registers for amax and conversion
    uint32_t cw[32];
    // amax of both columns at once on the packed bf16 pairs (|x| by clearing the sign bits, then a packed
    // max that ignores NaN like fmaxf); the scaling by 2^-e is a packed bf16 multiply, exact for a power of two
    uint32_t am = 0u;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      cw[i] = tile32[(32 * g + i) * 64 + cp];
      am = bf16x2_max(am, cw[i] & 0x7fff7fffu);
    }
    const int e0 = mx_exponent(fmaxf(__uint_as_float(am << 16), kAmaxFloor));
    const int e1 = mx_exponent(fmaxf(__uint_as_float(am & 0xffff0000u), kAmaxFloor));
    const uint32_t inv2 = (__float_as_uint(mx_inv_scale(e0)) >> 16) | (__float_as_uint(mx_inv_scale(e1)) & 0xffff0000u);
    uint32_t w0[8], w1[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float a[4], b[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t sc = bf16x2_mul(cw[4 * q + k], inv2);
        a[k] = __uint_as_float(sc << 16);
        b[k] = __uint_as_float(sc & 0xffff0000u);
      }
      w0[q] = e4m3x2(a[0], a[1]) | (e4m3x2(a[2], a[3]) << 16);
      w1[q] = e4m3x2(b[0], b[1]) | (e4m3x2(b[2], b[3]) << 16);
    }
    // Transposed codes go through shared memory (the input tile is dead once every thread holds its
    // column pair in registers) so that the global writes are full 128-byte lines: column c of the tile
    // owns 128 bytes = 8 pieces of 16; piece q is stored at q ^ ((c >> 1) & 7) to keep both the
    // per-thread writes and the cooperative reads free of bank conflicts.
    __syncthreads();
    {
      const int c0 = 2 * cp, sw = cp & 7;
      tile[c0 * 8 + ((2 * g) ^ sw)] = make_uint4(w0[0], w0[1], w0[2], w0[3]);
      tile[c0 * 8 + ((2 * g + 1) ^ sw)] = make_uint4(w0[4], w0[5], w0[6], w0[7]);
      tile[(c0 + 1) * 8 + ((2 * g) ^ sw)] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
      tile[(c0 + 1) * 8 + ((2 * g + 1) ^ sw)] = make_uint4(w1[4], w1[5], w1[6], w1[7]);
      if (tile_c + c0 < p.cols && tile_r + 32 * g < p.rows) {
        sc_col[p.tiled ? tiled_offset(c0, g) : c0 * 4 + g] = static_cast<uint8_t>(e0 + 127);
        if (tile_c + c0 + 1 < p.cols)
          sc_col[p.tiled ? tiled_offset(c0 + 1, g) : (c0 + 1) * 4 + g] = static_cast<uint8_t>(e1 + 127);
      }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const int idx = t + h * kThreads;  // 1024 pieces: column idx / 8, piece idx % 8
      const int c = idx >> 3, q = idx & 7;
      const int64_t col_g = tile_c + c, row_g = tile_r + q * 16;  // rows % 32 == 0: a piece is all in or all out
      if (col_g < p.cols && row_g < p.rows)
        stg_stream16(p.codes_colT + col_g * p.rows + row_g, tile[c * 8 + (q ^ ((c >> 1) & 7))]);
    }
  }

  __syncthreads();
  // Scale bytes of the tile: 128 "rows" x 4 k-blocks, staged in shared memory.
  if (ROW) {
    const int64_t kb = p.cols / 32;
    if (p.tiled) {
      if (t < 128) {
        const int64_t chunk = blockIdx.y * ceil_div(kb, 4) + blockIdx.x;
        reinterpret_cast<uint32_t*>(p.scales_row + chunk * 512)[t] =
            reinterpret_cast<const uint32_t*>(sc_row)[t];
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int idx = t + h * kThreads;
        const int64_t r = tile_r + (idx >> 2), k = tile_c / 32 + (idx & 3);
        if (r < p.rows && k < kb) p.scales_row[r * kb + k] = sc_row[idx];
      }
    }
  }
  if (COL) {
    const int64_t kb = p.rows / 32;
    if (p.tiled) {
      if (t < 128) {
        const int64_t chunk = blockIdx.x * ceil_div(kb, 4) + blockIdx.y;
        reinterpret_cast<uint32_t*>(p.scales_col + chunk * 512)[t] =
            reinterpret_cast<const uint32_t*>(sc_col)[t];
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int idx = t + h * kThreads;
        const int64_t c = tile_c + (idx >> 2), k = tile_r / 32 + (idx & 3);
        if (c < p.cols && k < kb) p.scales_col[c * kb + k] = sc_col[idx];
      }
    }
  }
}

}  // namespace mxq
}  // namespace anima
