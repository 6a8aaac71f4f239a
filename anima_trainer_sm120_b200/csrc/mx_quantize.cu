// MXFP8 quantiser: bf16 -> e4m3 codes + one e8m0 scale byte per 32 elements.
//
// Replaces anima-trainer's Triton quantiser (mxfp8_gemm.py:68-183) and its
// transpose -> quantise -> transpose construction of the column-wise operand
// (mxfp8_gemm.py:201-222). One CTA owns a 128 x 128 tile of x, reads it from HBM
// exactly once with 16-byte streaming loads, and can emit from that single read
//   * row-wise codes/scales (groups of 32 along the columns), and
//   * column-wise codes/scales (groups of 32 along the rows), written transposed
//     so that the result is again contiguous along its contraction axis.
// HBM-bound: 2 B read + 1.03 B (row) or 2.06 B (row + column) written per element.
//
// Exponent rule. The reference evaluates e = ceil(log2(amax) - log2(448)) in fp32.
// With amax = m * 2^E, 1 <= m < 2 and 448 = 1.75 * 2^8 this is, in exact
// arithmetic, e = E - 8 + (m > 1.75). The kernel uses that integer form: it does
// not depend on the accuracy of a hardware log2 near m == 1.75, the only mantissa
// a bf16 input can take that lands on the rounding boundary.
#include "mx_quantize_tile.cuh"

namespace anima {
namespace {

using namespace mxq;

struct PlainLoader {
  const __nv_bfloat16* x;
  int64_t ld;
  __device__ __forceinline__ uint4 operator()(int64_t r, int64_t c) const { return ldg_stream16(x + r * ld + c); }
};

__global__ void mx_dequantize_kernel(const uint8_t* __restrict__ codes,
                                     const uint8_t* __restrict__ scales, int64_t rows, int64_t k,
                                     int tiled, __nv_bfloat16* __restrict__ out) {
  const int64_t kb = k / 32;
  const int64_t total = rows * kb * 4;  // one thread per 8 codes
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / (kb * 4);
    const int64_t c8 = i % (kb * 4);
    const int64_t b = c8 / 4;
    uint8_t sb;
    if (tiled) {
      const int64_t chunk = (r / 128) * ceil_div(kb, 4) + b / 4;
      sb = scales[chunk * 512 + tiled_offset(static_cast<int>(r % 128), static_cast<int>(b % 4))];
    } else {
      sb = scales[r * kb + b];
    }
    // 2^(sb-127); byte 0 is the subnormal 2^-127.
    const float s = sb == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(static_cast<uint32_t>(sb) << 23);
    const uint2 cw = *reinterpret_cast<const uint2*>(codes + r * k + c8 * 8);
    const uint8_t* cb = reinterpret_cast<const uint8_t*>(&cw);
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __half_raw hr = __nv_cvt_fp8_to_halfraw(cb[j], __NV_E4M3);
      f[j] = __half2float(*reinterpret_cast<const __half*>(&hr)) * s;
    }
    *reinterpret_cast<uint4*>(out + r * k + c8 * 8) = pack8(f);
  }
}

__global__ void mx_scales_retile_kernel(const uint8_t* __restrict__ plain, int64_t rows, int64_t kb,
                                        uint8_t* __restrict__ tiled) {
  const int64_t kb4 = ceil_div(kb, 4);
  const int64_t total = ceil_div(rows, 128) * kb4 * 512;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t chunk = i / 512;
    const int off = static_cast<int>(i % 512);
    const int j = off & 3, r_in = ((off >> 2) & 3) * 32 + (off >> 4);
    const int64_t r = (chunk / kb4) * 128 + r_in, b = (chunk % kb4) * 4 + j;
    tiled[i] = (r < rows && b < kb) ? plain[r * kb + b] : 0;
  }
}

}  // namespace
}  // namespace anima

using namespace anima;

extern "C" int64_t anima_mx_scales_bytes(int64_t rows, int64_t k, int scale_layout) {
  if (rows < 0 || k < 0 || k % 32) return ANIMA_E_SHAPE;
  const int64_t kb = k / 32;
  return scale_layout == ANIMA_SCALES_TILED ? ceil_div(rows, 128) * ceil_div(kb, 4) * 512 : rows * kb;
}

extern "C" int anima_mx_quantize(const void* x, int64_t rows, int64_t cols, int64_t ld,
                                 uint8_t* codes_row, uint8_t* scales_row, uint8_t* codes_colT,
                                 uint8_t* scales_col, int scale_layout, void* stream) {
  const bool row = codes_row != nullptr, col = codes_colT != nullptr;
  ANIMA_REQUIRE(x != nullptr, ANIMA_E_ARG, "mx_quantize: x is null");
  ANIMA_REQUIRE(row || col, ANIMA_E_ARG, "mx_quantize: no output requested");
  ANIMA_REQUIRE((codes_row == nullptr) == (scales_row == nullptr) &&
                    (codes_colT == nullptr) == (scales_col == nullptr),
                ANIMA_E_ARG, "mx_quantize: codes and scales must be given in pairs");
  ANIMA_REQUIRE(scale_layout == ANIMA_SCALES_PLAIN || scale_layout == ANIMA_SCALES_TILED, ANIMA_E_ARG,
                "mx_quantize: bad scale_layout %d", scale_layout);
  ANIMA_REQUIRE(rows >= 0 && cols >= 0 && ld >= cols, ANIMA_E_ARG,
                "mx_quantize: bad sizes rows=%lld cols=%lld ld=%lld", (long long)rows, (long long)cols,
                (long long)ld);
  ANIMA_REQUIRE(!row || cols % 32 == 0, ANIMA_E_SHAPE,
                "mx_quantize: rowwise needs cols %% 32 == 0 (cols=%lld)", (long long)cols);
  ANIMA_REQUIRE(!col || rows % 32 == 0, ANIMA_E_SHAPE,
                "mx_quantize: columnwise needs rows %% 32 == 0 (rows=%lld)", (long long)rows);
  ANIMA_REQUIRE(cols % 8 == 0 && ld % 8 == 0, ANIMA_E_SHAPE,
                "mx_quantize: cols and ld must be multiples of 8");
  ANIMA_REQUIRE(aligned16(x) && (!row || aligned16(codes_row)) && (!col || aligned16(codes_colT)),
                ANIMA_E_ALIGN, "mx_quantize: x and code buffers must be 16-byte aligned");
  ANIMA_REQUIRE((!row || (reinterpret_cast<uintptr_t>(scales_row) & 3) == 0) &&
                    (!col || (reinterpret_cast<uintptr_t>(scales_col) & 3) == 0),
                ANIMA_E_ALIGN, "mx_quantize: scale buffers must be 4-byte aligned");
  if (rows == 0 || cols == 0) return ANIMA_OK;
  const int64_t gy = ceil_div(rows, kTile), gx = ceil_div(cols, kTile);
  ANIMA_REQUIRE(gy <= 65535, ANIMA_E_TOO_LARGE, "mx_quantize: rows=%lld exceeds 65535*128",
                (long long)rows);
  QuantParams p{rows, cols, codes_row, scales_row, codes_colT, scales_col,
                scale_layout == ANIMA_SCALES_TILED};
  const PlainLoader load{static_cast<const __nv_bfloat16*>(x), ld};
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (row && col)
    mx_quantize_kernel<true, true><<<grid, kThreads, 0, s>>>(p, load);
  else if (row)
    mx_quantize_kernel<true, false><<<grid, kThreads, 0, s>>>(p, load);
  else
    mx_quantize_kernel<false, true><<<grid, kThreads, 0, s>>>(p, load);
  ANIMA_CHECK_LAUNCH("mx_quantize");
  return ANIMA_OK;
}

extern "C" int anima_mx_dequantize(const uint8_t* codes, const uint8_t* scales, int64_t rows,
                                   int64_t k, int scale_layout, void* out, void* stream) {
  ANIMA_REQUIRE(codes && scales && out, ANIMA_E_ARG, "mx_dequantize: null pointer");
  ANIMA_REQUIRE(rows >= 0 && k >= 0 && k % 32 == 0, ANIMA_E_SHAPE, "mx_dequantize: k %% 32 != 0");
  ANIMA_REQUIRE(aligned16(out) && (reinterpret_cast<uintptr_t>(codes) & 7) == 0, ANIMA_E_ALIGN,
                "mx_dequantize: misaligned buffer");
  if (rows == 0 || k == 0) return ANIMA_OK;
  const int64_t total = rows * (k / 8);
  const int blocks = static_cast<int>(std::min<int64_t>(ceil_div(total, 256), sm_count() * 16));
  mx_dequantize_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      codes, scales, rows, k, scale_layout == ANIMA_SCALES_TILED, static_cast<__nv_bfloat16*>(out));
  ANIMA_CHECK_LAUNCH("mx_dequantize");
  return ANIMA_OK;
}

extern "C" int anima_mx_scales_retile(const uint8_t* plain, int64_t rows, int64_t k, uint8_t* tiled,
                                      void* stream) {
  ANIMA_REQUIRE(plain && tiled, ANIMA_E_ARG, "mx_scales_retile: null pointer");
  ANIMA_REQUIRE(rows >= 0 && k >= 0 && k % 32 == 0, ANIMA_E_SHAPE, "mx_scales_retile: k %% 32 != 0");
  if (rows == 0 || k == 0) return ANIMA_OK;
  const int64_t total = anima_mx_scales_bytes(rows, k, ANIMA_SCALES_TILED);
  const int blocks = static_cast<int>(std::min<int64_t>(ceil_div(total, 256), sm_count() * 16));
  mx_scales_retile_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(plain, rows, k / 32,
                                                                                 tiled);
  ANIMA_CHECK_LAUNCH("mx_scales_retile");
  return ANIMA_OK;
}
