// TMA-fed, persistent form of the MXFP8 quantiser (same arithmetic and outputs as
// mx_quantize_kernel<ROW, COL, Loader>; see mx_quantize_tile.cuh for the tile algorithm).
//
// A CTA walks tiles b, b + gridDim.x, ... of 128 x 128 bf16 values. Two shared-memory stages hold input
// tiles; one elected thread keeps a `cp.async.bulk.tensor.2d` load of the NEXT tile in flight while the CTA
// works on the current one, so HBM reads overlap the arithmetic inside a CTA (the non-persistent kernel
// overlaps only across the CTAs of an SM) at no register cost, and the row pass reads its 16-byte chunks from
// shared memory instead of issuing global loads and shared stores itself. Tiles past the edge of the tensor
// are zero-filled by the copy engine; stores are predicated as in the tile kernel.
// Stage s, once its tile is in registers, doubles as the staging buffer for the transposed codes.
// Every mbarrier wait is bounded; a CTA that gives up raises g_quantize_timeout and leaves the loop.
//
// A loader that computes (GELU, GELU gradient) transforms the raw tile in place during the row pass: each
// thread rewrites the chunks it reads, a barrier follows, and the column pass sees the transformed tile. Its
// lookup table is copied to shared memory once per CTA instead of once per tile, and a second input (the
// incoming gradient) is fetched into registers one tile ahead, right after the row pass has consumed the
// current one. What the loader adds to the interface of mx_quantize_tile.cuh:
//   static constexpr bool kIdentity;        finish() returns the raw chunk (no rewrite, no extra barrier)
//   static constexpr bool kSecond;          there is a second input
//   static constexpr int kTmaCtasPerSm;     resident CTAs the kernel is compiled for (shared memory: two 32 KB
//                                           stages plus the table)
//   uint4 second(int64_t row, int64_t col) const;                         the second input's chunk (a load)
//   uint4 transform(const uint4& raw, const uint4& second, int64_t row, int64_t col) const;
#pragma once

#include "mx_quantize_tile.cuh"
#include "tma_util.cuh"

namespace anima {
namespace mxq {

constexpr int kTmaStageBytes = kTile * kTile * 2;                      // 32 KB
constexpr int kTmaSmemBytes = 2 * kTmaStageBytes + 128 /*alignment*/;  // + the loader's table; barriers and scale staging are static

__device__ int g_quantize_timeout;  // sticky; read by anima_mx_quantize_status()

template <bool ROW, bool COL, class Loader>
__global__ void __launch_bounds__(kThreads, Loader::kTmaCtasPerSm)
mx_quantize_tma_kernel(const __grid_constant__ CUtensorMap map_x, const QuantParams p, const Loader load_arg) {
  extern __shared__ uint8_t smem_raw[];
  Loader load = load_arg;
  __shared__ __align__(8) uint64_t full_bar[2];
  __shared__ volatile int abort_flag;
  __shared__ __align__(16) uint8_t sc_row[ROW ? 512 : 16];
  __shared__ __align__(16) uint8_t sc_col[COL ? 512 : 16];

  const int t = threadIdx.x;
  const int c16 = t & 15;  // 16-byte chunk (8 elements) within the tile row
  const int r0 = t >> 4;   // 0..15
  // dynamic shared memory: the loader's table first (its lookups pack two addresses into 16-bit halves, so it
  // must sit low), then the two stages
  constexpr uint32_t kTableBytes = (Loader::kSmemBytes + 127u) & ~127u;
  const uint32_t table0 = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* const table_ptr = smem_raw + (table0 - smem_u32(smem_raw));
  const uint32_t stage0 = table0 + kTableBytes;
  uint8_t* const stage_ptr0 = table_ptr + kTableBytes;
  const int64_t tiles_x = ceil_div(p.cols, static_cast<int64_t>(kTile));
  const int64_t n_tiles = tiles_x * ceil_div(p.rows, static_cast<int64_t>(kTile));
  const int64_t first = blockIdx.x, step = gridDim.x;

  if (ROW) reinterpret_cast<uint16_t*>(sc_row)[t] = 0;  // padding entries of a partial tile must be 0
  if (COL) reinterpret_cast<uint16_t*>(sc_col)[t] = 0;
  auto issue = [&](int64_t tile_id, int s) {  // one thread: arm the stage's barrier and start the copy
    const int64_t ty = tile_id / tiles_x, tx = tile_id - ty * tiles_x;
    mbar_expect_tx(smem_u32(&full_bar[s]), kTmaStageBytes);
    tma_load_2d(stage0 + s * kTmaStageBytes, &map_x, smem_u32(&full_bar[s]), static_cast<int>(tx * kTile),
                static_cast<int>(ty * kTile));
  };
  if (t == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&full_bar[0]), 1);
    mbar_init(smem_u32(&full_bar[1]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    if (first < n_tiles) issue(first, 0);
    if (first + step < n_tiles) issue(first + step, 1);
  }
  load.prepare(table_ptr);  // the table, once per CTA, behind the first copies
  // chunk i of this thread: tile row r0 + 16 i, columns 8 c16 .. + 7
  auto chunk_in_range = [&](int64_t tile_id, int i) {
    const int64_t ty = tile_id / tiles_x, tx = tile_id - ty * tiles_x;
    return tx * kTile + c16 * 8 < p.cols && ty * kTile + r0 + 16 * i < p.rows;
  };
  uint4 second[Loader::kSecond ? 8 : 1];
  auto fetch_second = [&](int64_t tile_id) {
    const int64_t ty = tile_id / tiles_x, tx = tile_id - ty * tiles_x;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      second[i] = make_uint4(0u, 0u, 0u, 0u);
      if (chunk_in_range(tile_id, i)) second[i] = load.second(ty * kTile + r0 + 16 * i, tx * kTile + c16 * 8);
    }
  };
  if (Loader::kSecond && first < n_tiles) fetch_second(first);
  __syncthreads();

  int it = 0;
  for (int64_t tile_id = first; tile_id < n_tiles; tile_id += step, ++it) {
    const int s = it & 1;
    const int64_t tile_y = tile_id / tiles_x, tile_x = tile_id - tile_y * tiles_x;
    const int64_t tile_r = tile_y * kTile, tile_c = tile_x * kTile;
    const int64_t col = tile_c + c16 * 8;
    const bool col_ok = col < p.cols;
    const uint4* tile = reinterpret_cast<const uint4*>(stage_ptr0 + s * kTmaStageBytes);
    uint4* tile_w = reinterpret_cast<uint4*>(stage_ptr0 + s * kTmaStageBytes);

    if (!mbar_wait(smem_u32(&full_bar[s]), (it >> 1) & 1u, &abort_flag)) break;

    if (ROW || !Loader::kIdentity) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r_in = r0 + 16 * i;
        const int64_t r = tile_r + r_in;
        uint4 v = tile[r_in * 16 + c16];
        if (!Loader::kIdentity) {
          v = (col_ok && r < p.rows) ? load.transform(v, second[Loader::kSecond ? i : 0], r, col)
                                     : make_uint4(0u, 0u, 0u, 0u);
          if (COL) tile_w[r_in * 16 + c16] = v;
        }
        if (!ROW) continue;
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
        if (col_ok && r < p.rows) {
          *reinterpret_cast<uint2*>(p.codes_row + r * p.cols + col) = codes;
          if ((c16 & 3) == 0) {
            const int j = c16 >> 2;
            sc_row[p.tiled ? tiled_offset(r_in, j) : r_in * 4 + j] = static_cast<uint8_t>(e + 127);
          }
        }
      }
    }

    if (Loader::kSecond && tile_id + step < n_tiles) fetch_second(tile_id + step);  // lands under the column pass

    if (COL) {
      if (!Loader::kIdentity) __syncthreads();  // the transformed tile is complete
      const int cp = t & 63;  // column pair
      const int g = t >> 6;   // 32-row group within the tile
      const uint32_t* tile32 = reinterpret_cast<const uint32_t*>(tile);
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
      __syncthreads();  // every thread holds its part of the input tile: the stage becomes the staging buffer
      {
        const int c0 = 2 * cp, sw = cp & 7;  // piece q of column c at q ^ ((c >> 1) & 7): conflict-free both ways
        tile_w[c0 * 8 + ((2 * g) ^ sw)] = make_uint4(w0[0], w0[1], w0[2], w0[3]);
        tile_w[c0 * 8 + ((2 * g + 1) ^ sw)] = make_uint4(w0[4], w0[5], w0[6], w0[7]);
        tile_w[(c0 + 1) * 8 + ((2 * g) ^ sw)] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        tile_w[(c0 + 1) * 8 + ((2 * g + 1) ^ sw)] = make_uint4(w1[4], w1[5], w1[6], w1[7]);
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
        const int64_t col_g = tile_c + c, row_g = tile_r + q * 16;
        if (col_g < p.cols && row_g < p.rows)
          stg_stream16(p.codes_colT + col_g * p.rows + row_g, tile[c * 8 + (q ^ ((c >> 1) & 7))]);
      }
    } else {
      __syncthreads();  // scale bytes of the row pass visible
    }

    // Scale bytes of the tile; each entry is zeroed again by the thread that stored it.
    if (ROW) {
      const int64_t kb = p.cols / 32;
      if (p.tiled) {
        if (t < 128) {
          const int64_t chunk = tile_y * ceil_div(kb, static_cast<int64_t>(4)) + tile_x;
          uint32_t* src = reinterpret_cast<uint32_t*>(sc_row) + t;
          reinterpret_cast<uint32_t*>(p.scales_row + chunk * 512)[t] = *src;
          *src = 0u;
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int idx = t + h * kThreads;
          const int64_t r = tile_r + (idx >> 2), k = tile_c / 32 + (idx & 3);
          if (r < p.rows && k < kb) p.scales_row[r * kb + k] = sc_row[idx];
          sc_row[idx] = 0;
        }
      }
    }
    if (COL) {
      const int64_t kb = p.rows / 32;
      if (p.tiled) {
        if (t < 128) {
          const int64_t chunk = tile_x * ceil_div(kb, static_cast<int64_t>(4)) + tile_y;
          uint32_t* src = reinterpret_cast<uint32_t*>(sc_col) + t;
          reinterpret_cast<uint32_t*>(p.scales_col + chunk * 512)[t] = *src;
          *src = 0u;
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int idx = t + h * kThreads;
          const int64_t c = tile_c + (idx >> 2), k = tile_r / 32 + (idx & 3);
          if (c < p.cols && k < kb) p.scales_col[c * kb + k] = sc_col[idx];
          sc_col[idx] = 0;
        }
      }
    }
    // this thread's generic-proxy accesses to the stage are ordered before the copy engine's next write to it
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();  // the stage and the scale staging are free
    if (t == 0 && tile_id + 2 * step < n_tiles) issue(tile_id + 2 * step, s);
  }
  if (abort_flag) {
    // copies may still be in flight into this CTA's shared memory: give them time to land before it is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (t == 0) atomicExch(&g_quantize_timeout, 1);
  }
}

}  // namespace mxq
}  // namespace anima
