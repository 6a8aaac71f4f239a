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
#include <cstdlib>
#include <mutex>

#include "mx_quantize_tile.cuh"
#include "mx_quantize_tma.cuh"

namespace anima {
namespace {

using namespace mxq;

struct PlainLoader {
  using Raw = uint4;
  static constexpr bool kZeroSafe = true;
  static constexpr int kSmemBytes = 0;
  static constexpr bool kIdentity = true, kSecond = false;
  static constexpr int kTmaCtasPerSm = 3;
  __device__ __forceinline__ void prepare(void*) {}
  __device__ __forceinline__ uint4 second(int64_t, int64_t) const { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ uint4 transform(const uint4& raw, const uint4&, int64_t, int64_t) const { return raw; }
  const __nv_bfloat16* x;
  int64_t ld;
  __device__ __forceinline__ Raw fetch(int64_t r, int64_t c) const { return ldg_stream16(x + r * ld + c); }
  __device__ __forceinline__ uint4 finish(const Raw& raw, int64_t, int64_t) const { return raw; }
};

// ---- GELU inside the quantiser ----------------------------------------------------------------
// A bf16 GELU is a function of 16 input bits, and so is the factor gelu'(x) that multiplies the incoming
// gradient. Both are tabulated for |x| in [2^-11, 8) (14 binades x 128 mantissas per sign): the table is
// filled once per device by evaluating, with the CUDA math library, exactly the expressions an eager bf16
// GELU kernel evaluates in fp32,
//     forward   x * 0.5 * (1 + erf(x / sqrt 2))                         stored rounded to bf16
//     backward  0.5 * (1 + erf(x / sqrt 2)) + x * exp(-x^2 / 2) / sqrt(2 pi)   stored as fp32, then dy * factor
// so the quantised codes equal those of quantising the materialised activation / gradient bit for bit,
// while a lookup costs a fraction of the ~25 instructions of an erf evaluation (which made this loader
// compute-bound). Inputs outside the table (|x| < 2^-11 or >= 8, NaN, inf: about 1 in 2500 for N(0,1) data)
// take the same expressions directly. A CTA copies the table it needs (7.5 or 15 KB) into shared memory: once per
// tile in the tile kernel, once for all its tiles in the persistent copy-engine-fed kernel (the default here).
//
// Index arithmetic runs on both bf16 values of a 32-bit word at once: clear the signs, clamp each half to the
// table's range with packed 16-bit max / min (a half that moved is outside the table), subtract the range
// start, and put the sign at bit 11 (negative inputs live at entries 2048..3839). One multiply-add turns the
// pair of indices into a pair of shared-memory byte addresses (each below 64 KB, so they fit their halves).
constexpr int kGeluLutMinExp = 127 - 11;   // biased exponent of 2^-11
constexpr int kGeluLutMaxExp = 127 + 3;    // first binade NOT in the table: [8, 16)
constexpr int kGeluLutHalf = (kGeluLutMaxExp - kGeluLutMinExp) * 128;   // 1792 magnitudes per sign
constexpr int kGeluLutNeg = 2048;                                       // first entry of the negative inputs
constexpr int kGeluLutSize = kGeluLutNeg + kGeluLutHalf;                // entries 1792..2047 are unused
constexpr uint32_t kGeluLo2 = static_cast<uint32_t>(kGeluLutMinExp << 7) * 0x10001u;
constexpr uint32_t kGeluHi2 = static_cast<uint32_t>((kGeluLutMaxExp << 7) - 1) * 0x10001u;
static_assert(kGeluLutHalf <= kGeluLutNeg && kGeluLutSize * 4 < 32768, "index pairs must fit 16 bits after scaling");
__device__ __align__(16) uint16_t g_gelu_lut[kGeluLutSize];
__device__ __align__(16) float g_gelu_grad_lut[kGeluLutSize];

__device__ __noinline__ float gelu_eager_f(float x) {   // rare path: kept out of line so the lookup loop stays small
  return x * 0.5f * (1.f + erff(x * 0.70710678118654752440f));
}
__device__ __noinline__ float gelu_grad_factor_eager_f(float x) {
  const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752440f));
  const float pdf = expf(-0.5f * x * x) * 0.39894228040143267794f;   // M_2_SQRTPI * M_SQRT1_2 * 0.5
  return cdf + x * pdf;
}
__device__ __forceinline__ uint32_t u16x2_max(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t u16x2_min(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("min.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// Both table indices of the bf16 pair `w`, one per 16-bit half; false when either value is outside the table.
__device__ __forceinline__ bool gelu_lut_index2(uint32_t w, uint32_t& idx2) {
  const uint32_t a = w & 0x7fff7fffu;
  const uint32_t c = u16x2_min(u16x2_max(a, kGeluLo2), kGeluHi2);
  idx2 = (c - kGeluLo2) | ((w >> 4) & 0x08000800u);   // no borrow between the halves: c >= range start in each
  return c == a;
}
// The table is written once per CTA before a barrier; volatile keeps the loads behind that barrier.
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

__global__ void gelu_lut_init_kernel() {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= kGeluLutSize) return;
  const int mag = i & (kGeluLutNeg - 1);
  if (mag >= kGeluLutHalf) {   // the gap between the two signs
    g_gelu_lut[i] = 0;
    g_gelu_grad_lut[i] = 0.f;
    return;
  }
  const uint32_t bits = static_cast<uint32_t>(mag + (kGeluLutMinExp << 7)) | (i >= kGeluLutNeg ? 0x8000u : 0u);
  const float x = __uint_as_float(bits << 16);
  g_gelu_lut[i] = __bfloat16_as_ushort(__float2bfloat16_rn(gelu_eager_f(x)));
  g_gelu_grad_lut[i] = gelu_grad_factor_eager_f(x);
}

template <class T>
__device__ __forceinline__ uint32_t copy_lut(void* smem, const T* table) {
  uint4* dst = static_cast<uint4*>(smem);
  const uint4* src = reinterpret_cast<const uint4*>(table);
  for (int i = threadIdx.x; i < kGeluLutSize * static_cast<int>(sizeof(T)) / 16; i += blockDim.x) dst[i] = src[i];
  return smem_u32(smem) * 0x10001u;   // the table's shared-memory address in both halves
}

__device__ __noinline__ uint32_t gelu_pair_eager(uint32_t w) {   // a pair with a value outside the table
  const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(gelu_eager_f(__uint_as_float(w << 16))));
  const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(gelu_eager_f(__uint_as_float(w & 0xffff0000u))));
  return lo | (hi << 16);
}

struct GeluLoader {
  using Raw = uint4;
  static constexpr bool kZeroSafe = false;  // finish may store the activation at (row, col)
  static constexpr int kSmemBytes = kGeluLutSize * 2;
  static constexpr bool kIdentity = false, kSecond = false;
  static constexpr int kTmaCtasPerSm = 3;     // 3 x (64 KB of stages + 7.5 KB table)
  __device__ __forceinline__ uint4 second(int64_t, int64_t) const { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ uint4 transform(const uint4& raw, const uint4&, int64_t r, int64_t c) const {
    return finish(raw, r, c);
  }
  const __nv_bfloat16* h;
  int64_t ld;
  __nv_bfloat16* act_out;                    // optional: the bf16 activation itself, [rows, cols] contiguous
  int64_t cols;
  uint32_t lut2;                             // shared-memory address of the table in both halves, set by prepare()
  __device__ __forceinline__ void prepare(void* smem) { lut2 = copy_lut(smem, g_gelu_lut); }
  __device__ __forceinline__ Raw fetch(int64_t r, int64_t c) const { return ldg_stream16(h + r * ld + c); }
  __device__ __forceinline__ uint32_t pair(uint32_t w) const {
    uint32_t idx2;
    if (!gelu_lut_index2(w, idx2)) return gelu_pair_eager(w);
    const uint32_t addr2 = idx2 * 2u + lut2;
    return lds_u16(addr2 & 0xffffu) | (lds_u16(addr2 >> 16) << 16);
  }
  __device__ __forceinline__ uint4 finish(const Raw& raw, int64_t r, int64_t c) const {
    const uint4 out = make_uint4(pair(raw.x), pair(raw.y), pair(raw.z), pair(raw.w));
    if (act_out) stg_stream16(act_out + r * cols + c, out);
    return out;
  }
};

__device__ __noinline__ float2 gelu_grad_factor_pair_eager(uint32_t w) {
  return make_float2(gelu_grad_factor_eager_f(__uint_as_float(w << 16)),
                     gelu_grad_factor_eager_f(__uint_as_float(w & 0xffff0000u)));
}

// d(pre-activation) = grad_act * gelu'(h), rounded to bf16.
struct GeluBwdLoader {
  using Raw = uint4;                           // the pre-activation; the incoming gradient is read in finish
  static constexpr bool kZeroSafe = false;     // (keeping both tiles in registers up front spills)
  static constexpr int kSmemBytes = kGeluLutSize * 4;
  static constexpr bool kIdentity = false, kSecond = true;
  static constexpr int kTmaCtasPerSm = 2;     // 2 x (64 KB of stages + 15 KB table)
  __device__ __forceinline__ uint4 second(int64_t r, int64_t c) const { return ldg_stream16(grad_act + r * ld + c); }
  const __nv_bfloat16* h;
  const __nv_bfloat16* grad_act;
  int64_t ld;
  __nv_bfloat16* act_out;                    // optional: the bf16 gradient itself, [rows, cols] contiguous
  int64_t cols;
  uint32_t lut2;
  __device__ __forceinline__ void prepare(void* smem) { lut2 = copy_lut(smem, g_gelu_grad_lut); }
  __device__ __forceinline__ Raw fetch(int64_t r, int64_t c) const { return ldg_stream16(h + r * ld + c); }
  __device__ __forceinline__ float2 factors(uint32_t w) const {
    uint32_t idx2;
    if (!gelu_lut_index2(w, idx2)) return gelu_grad_factor_pair_eager(w);
    const uint32_t addr2 = idx2 * 4u + lut2;
    return make_float2(lds_f32(addr2 & 0xffffu), lds_f32(addr2 >> 16));
  }
  __device__ __forceinline__ uint4 finish(const Raw& raw, int64_t r, int64_t c) const {
    return transform(raw, ldg_stream16(grad_act + r * ld + c), r, c);
  }
  __device__ __forceinline__ uint4 transform(const uint4& raw, const uint4& grad, int64_t r, int64_t c) const {
    float g[8], o[8];
    unpack8(grad, g);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = factors(w[k]);
      o[2 * k] = g[2 * k] * f.x;
      o[2 * k + 1] = g[2 * k + 1] * f.y;
    }
    const uint4 out = pack8(o);
    if (act_out) stg_stream16(act_out + r * cols + c, out);
    return out;
  }
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

// TILED scales of a code matrix [rows_in, k_in] -> TILED scales of the SAME codes viewed as
// [rows_out, k_out] (rows_in * k_in == rows_out * k_out): the 32-element blocks keep their row-major
// order, only their (row, block) coordinates and therefore their place in the 128 x 4 tiling change.
// Index arithmetic in Idx: 32-bit when every extent fits (64-bit divisions cost ~10x here and the kernel moves
// one byte per thread-iteration: 16 us for the 2 MB of scales of a [32768, 2048] operand before, 504 launches
// per T-LoKr step).
template <class Idx>
__global__ void mx_scales_regroup_kernel(const uint8_t* __restrict__ in, Idx kb_in, Idx rows_out, Idx kb_out, Idx total,
                                         uint8_t* __restrict__ out) {
  const Idx kb4_out = (kb_out + 3) / 4, kb4_in = (kb_in + 3) / 4;
  for (Idx i = blockIdx.x * static_cast<Idx>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<Idx>(gridDim.x) * blockDim.x) {
    const Idx chunk = i / 512;
    const int off = static_cast<int>(i % 512);
    const int j = off & 3, r_in = ((off >> 2) & 3) * 32 + (off >> 4);
    const Idx cr = chunk / kb4_out;
    const Idx r = cr * 128 + r_in, b = (chunk - cr * kb4_out) * 4 + j;
    uint8_t v = 0;
    if (r < rows_out && b < kb_out) {
      const Idx flat = r * kb_out + b;
      const Idx ri = flat / kb_in, bi = flat - ri * kb_in;
      v = in[((ri / 128) * kb4_in + bi / 4) * 512 + tiled_offset(static_cast<int>(ri % 128), static_cast<int>(bi % 4))];
    }
    out[i] = v;
  }
}

// Both block counts multiples of 4: the four scale bytes of a (row, 128-column) group are one aligned 32-bit
// word in either tiling and stay together, so the kernel moves words (a quarter of the index arithmetic, 4-byte
// accesses). rows_out % 128 may be anything: padded rows are written as zero.
__global__ void mx_scales_regroup_words_kernel(const uint32_t* __restrict__ in, uint32_t kb4_in, uint32_t rows_out,
                                               uint32_t kb4_out, uint32_t total_words, uint32_t* __restrict__ out) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total_words; i += gridDim.x * blockDim.x) {
    const uint32_t chunk = i >> 7, w = i & 127;                 // 128 words per chunk; word w = bytes 4w .. 4w+3
    const uint32_t r_in = (w & 3) * 32 + (w >> 2);              // tiled_offset(r, 0) / 4 = (r % 32) * 4 + r / 32
    const uint32_t cr = chunk / kb4_out;
    const uint32_t r = cr * 128 + r_in, q = chunk - cr * kb4_out;   // row, 128-column group
    uint32_t v = 0u;
    if (r < rows_out) {
      const uint32_t flat = r * kb4_out + q;                    // index of the group in row-major order
      const uint32_t ri = flat / kb4_in, qi = flat - ri * kb4_in;
      v = in[((ri >> 7) * kb4_in + qi) * 128 + (ri & 31) * 4 + ((ri >> 5) & 3)];
    }
    out[i] = v;
  }
}

// Test aid: the block exponent of `amax` by the integer rule the quantiser uses and by the reference's literal
// fp32 expression ceil(log2(amax) - log2(448)) (mxfp8_gemm.py:118-120) evaluated with the instruction its Triton
// kernel compiles to on a GPU (lg2.approx.f32), both clamped to [-127, 127].
__global__ void mx_exponent_probe_kernel(const float* __restrict__ amax, int64_t n, int32_t* __restrict__ by_rule,
                                         int32_t* __restrict__ by_lg2_approx) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const float a = fmaxf(amax[i], mxq::kAmaxFloor);
  by_rule[i] = mxq::mx_exponent(a);
  float la, l448;
  asm("lg2.approx.f32 %0, %1;" : "=f"(la) : "f"(a));
  asm("lg2.approx.f32 %0, %1;" : "=f"(l448) : "f"(448.0f));
  const float e = ceilf(la - l448);
  by_lg2_approx[i] = static_cast<int32_t>(fminf(fmaxf(e, -127.f), 127.f));
}

}  // namespace
}  // namespace anima

using namespace anima;

extern "C" int64_t anima_mx_scales_bytes(int64_t rows, int64_t k, int scale_layout) {
  if (rows < 0 || k < 0 || k % 32) return ANIMA_E_SHAPE;
  const int64_t kb = k / 32;
  return scale_layout == ANIMA_SCALES_TILED ? ceil_div(rows, 128) * ceil_div(kb, 4) * 512 : rows * kb;
}

namespace {

// Argument checks shared by the quantising entry points; returns ANIMA_OK or the failing status.
int check_quantize_args(const char* who, const void* x, int64_t rows, int64_t cols, int64_t ld,
                        const uint8_t* codes_row, const uint8_t* scales_row, const uint8_t* codes_colT,
                        const uint8_t* scales_col, int scale_layout) {
  const bool row = codes_row != nullptr, col = codes_colT != nullptr;
  ANIMA_REQUIRE(x != nullptr, ANIMA_E_ARG, "%s: x is null", who);
  ANIMA_REQUIRE(row || col, ANIMA_E_ARG, "%s: no output requested", who);
  ANIMA_REQUIRE((codes_row == nullptr) == (scales_row == nullptr) &&
                    (codes_colT == nullptr) == (scales_col == nullptr),
                ANIMA_E_ARG, "%s: codes and scales must be given in pairs", who);
  ANIMA_REQUIRE(scale_layout == ANIMA_SCALES_PLAIN || scale_layout == ANIMA_SCALES_TILED, ANIMA_E_ARG,
                "%s: bad scale_layout %d", who, scale_layout);
  ANIMA_REQUIRE(rows >= 0 && cols >= 0 && ld >= cols, ANIMA_E_ARG, "%s: bad sizes rows=%lld cols=%lld ld=%lld", who,
                (long long)rows, (long long)cols, (long long)ld);
  ANIMA_REQUIRE(!row || cols % 32 == 0, ANIMA_E_SHAPE, "%s: rowwise needs cols %% 32 == 0 (cols=%lld)", who,
                (long long)cols);
  ANIMA_REQUIRE(!col || rows % 32 == 0, ANIMA_E_SHAPE, "%s: columnwise needs rows %% 32 == 0 (rows=%lld)", who,
                (long long)rows);
  ANIMA_REQUIRE(cols % 8 == 0 && ld % 8 == 0, ANIMA_E_SHAPE, "%s: cols and ld must be multiples of 8", who);
  ANIMA_REQUIRE(aligned16(x) && (!row || aligned16(codes_row)) && (!col || aligned16(codes_colT)),
                ANIMA_E_ALIGN, "%s: x and code buffers must be 16-byte aligned", who);
  ANIMA_REQUIRE((!row || (reinterpret_cast<uintptr_t>(scales_row) & 3) == 0) &&
                    (!col || (reinterpret_cast<uintptr_t>(scales_col) & 3) == 0),
                ANIMA_E_ALIGN, "%s: scale buffers must be 4-byte aligned", who);
  ANIMA_REQUIRE(ceil_div(rows, kTile) <= 65535, ANIMA_E_TOO_LARGE, "%s: rows=%lld exceeds 65535*128", who,
                (long long)rows);
  return ANIMA_OK;
}

template <class Loader>
int launch_quantize(const char* who, const Loader& load, int64_t rows, int64_t cols, uint8_t* codes_row,
                    uint8_t* scales_row, uint8_t* codes_colT, uint8_t* scales_col, int scale_layout, void* stream) {
  const bool row = codes_row != nullptr, col = codes_colT != nullptr;
  QuantParams p{rows, cols, codes_row, scales_row, codes_colT, scales_col, scale_layout == ANIMA_SCALES_TILED};
  const dim3 grid(static_cast<unsigned>(ceil_div(cols, kTile)), static_cast<unsigned>(ceil_div(rows, kTile)));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (row && col)
    mx_quantize_kernel<true, true><<<grid, kThreads, 0, s>>>(p, load);
  else if (row)
    mx_quantize_kernel<true, false><<<grid, kThreads, 0, s>>>(p, load);
  else
    mx_quantize_kernel<false, true><<<grid, kThreads, 0, s>>>(p, load);
  ANIMA_CHECK_LAUNCH(who);
  return ANIMA_OK;
}

}  // namespace

namespace {

// 0 = choose (TMA-fed persistent kernel when the tensor map can be encoded), 1 = tile kernel with plain loads,
// 2 = TMA kernel or fail (ANIMA_MX_QUANTIZE_VARIANT, read per call; for tests).
int forced_quantize_variant() {
  const char* v = getenv("ANIMA_MX_QUANTIZE_VARIANT");
  return v ? atoi(v) : 0;
}

// bf16 [rows, cols] with row pitch ld elements; box = one 128 x 128 tile; reads outside the tensor give 0.
bool make_x_map(CUtensorMap* map, const void* x, int64_t rows, int64_t cols, int64_t ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {kTile, kTile};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool ROW, bool COL, class Loader>
int launch_tma(const CUtensorMap& map, const QuantParams& p, const Loader& load, unsigned grid, cudaStream_t s) {
  constexpr int kBytes = kTmaSmemBytes + ((Loader::kSmemBytes + 127) & ~127);
  static PerDeviceOnce once;
  const cudaError_t attr_rc = per_device_once(once, [] {
    return cudaFuncSetAttribute(mx_quantize_tma_kernel<ROW, COL, Loader>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                kBytes);
  });
  ANIMA_REQUIRE(attr_rc == cudaSuccess, ANIMA_E_CUDA, "mx_quantize: cannot reserve %d bytes of shared memory: %s",
                kBytes, cudaGetErrorString(attr_rc));
  mx_quantize_tma_kernel<ROW, COL, Loader><<<grid, kThreads, kBytes, s>>>(map, p, load);
  ANIMA_CHECK_LAUNCH("mx_quantize (TMA)");
  return ANIMA_OK;
}

// Returns ANIMA_OK when launched, 1 when this path does not apply (the caller then takes the tile kernel).
// x is the tensor the copy engine reads (the loader's first input).
template <class Loader>
int try_quantize_tma(const Loader& load, const void* x, int64_t rows, int64_t cols, int64_t ld, uint8_t* codes_row,
                     uint8_t* scales_row, uint8_t* codes_colT, uint8_t* scales_col, int scale_layout, void* stream) {
  if (rows >= (1ll << 31) || cols >= (1ll << 31)) return 1;
  CUtensorMap map;
  if (!make_x_map(&map, x, rows, cols, ld)) return 1;
  const bool row = codes_row != nullptr, col = codes_colT != nullptr;
  QuantParams p{rows, cols, codes_row, scales_row, codes_colT, scales_col, scale_layout == ANIMA_SCALES_TILED};
  const int64_t tiles = ceil_div(rows, static_cast<int64_t>(kTile)) * ceil_div(cols, static_cast<int64_t>(kTile));
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(tiles, static_cast<int64_t>(Loader::kTmaCtasPerSm) * sm_count()));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (row && col) return launch_tma<true, true>(map, p, load, grid, s);
  if (row) return launch_tma<true, false>(map, p, load, grid, s);
  return launch_tma<false, true>(map, p, load, grid, s);
}

// The kernel choice shared by the quantising entry points: `tma_by_default` says whether the copy-engine-fed
// kernel is the one to take when the variable does not force either.
template <class Loader>
int quantize_dispatch(const char* who, const Loader& load, bool tma_by_default, const void* x, int64_t rows, int64_t cols,
                      int64_t ld, uint8_t* codes_row, uint8_t* scales_row, uint8_t* codes_colT, uint8_t* scales_col,
                      int scale_layout, void* stream) {
  const int variant = forced_quantize_variant();
  if (variant == 2 || (variant == 0 && tma_by_default)) {
    const int rc = try_quantize_tma(load, x, rows, cols, ld, codes_row, scales_row, codes_colT, scales_col,
                                    scale_layout, stream);
    if (rc <= 0) return rc;
    ANIMA_REQUIRE(variant != 2, ANIMA_E_UNSUPPORTED, "%s: the TMA path is not available for this call", who);
  }
  return launch_quantize(who, load, rows, cols, codes_row, scales_row, codes_colT, scales_col, scale_layout, stream);
}

}  // namespace

extern "C" int anima_mx_quantize_status(void) {
  int flag = 0;
  const cudaError_t rc = cudaMemcpyFromSymbol(&flag, g_quantize_timeout, sizeof(int));   // synchronises
  ANIMA_REQUIRE(rc == cudaSuccess, ANIMA_E_CUDA, "mx_quantize_status: %s", cudaGetErrorString(rc));
  if (flag) {  // reported once: clear it so that a later check speaks about later launches
    const int zero = 0;
    const cudaError_t rc2 = cudaMemcpyToSymbol(g_quantize_timeout, &zero, sizeof(int));
    ANIMA_REQUIRE(rc2 == cudaSuccess, ANIMA_E_CUDA, "mx_quantize_status: %s", cudaGetErrorString(rc2));
  }
  return flag ? 1 : 0;
}

extern "C" int anima_mx_quantize(const void* x, int64_t rows, int64_t cols, int64_t ld,
                                 uint8_t* codes_row, uint8_t* scales_row, uint8_t* codes_colT,
                                 uint8_t* scales_col, int scale_layout, void* stream) {
  if (int rc = check_quantize_args("mx_quantize", x, rows, cols, ld, codes_row, scales_row, codes_colT, scales_col,
                                   scale_layout))
    return rc;
  if (rows == 0 || cols == 0) return ANIMA_OK;
  // The copy-engine-fed kernel wins whenever the column form is made (row+column 4401 -> 4930 GB/s, column only
  // 4966 -> 5517); the row-only form has no shared-memory tile and runs as well or better on plain loads (5758 vs 5675).
  const PlainLoader load{static_cast<const __nv_bfloat16*>(x), ld};
  return quantize_dispatch("mx_quantize", load, codes_colT != nullptr, x, rows, cols, ld, codes_row, scales_row,
                           codes_colT, scales_col, scale_layout, stream);
}

namespace {

// Fills the GELU tables of the current device on first use and waits for the fill (the one host
// synchronisation this entry point ever makes, once per device): every later call, on any stream and inside
// stream capture, then finds the tables complete without any event bookkeeping. The first call on a device
// must therefore be made outside stream capture.
int ensure_gelu_tables(cudaStream_t s) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static bool ready[kMaxDevices];
  int dev = 0;
  ANIMA_REQUIRE(cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices, ANIMA_E_CUDA,
                "mx_quantize_gelu: cannot identify the current device");
  std::lock_guard<std::mutex> lock(mu);
  if (ready[dev]) return ANIMA_OK;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  ANIMA_REQUIRE(cudaStreamIsCapturing(s, &capturing) == cudaSuccess && capturing == cudaStreamCaptureStatusNone,
                ANIMA_E_UNSUPPORTED, "mx_quantize_gelu: the first call on a device must be made outside stream capture");
  gelu_lut_init_kernel<<<ceil_div(kGeluLutSize, 256), 256, 0, s>>>();
  ANIMA_CHECK_LAUNCH("mx_quantize_gelu table fill");
  const cudaError_t rc = cudaStreamSynchronize(s);
  ANIMA_REQUIRE(rc == cudaSuccess, ANIMA_E_CUDA, "mx_quantize_gelu: table fill failed: %s", cudaGetErrorString(rc));
  ready[dev] = true;
  return ANIMA_OK;
}

}  // namespace

extern "C" int anima_mx_quantize_gelu(const void* h, const void* grad_act, int64_t rows, int64_t cols,
                                      int64_t ld, void* act_bf16, uint8_t* codes_row, uint8_t* scales_row,
                                      uint8_t* codes_colT, uint8_t* scales_col, int scale_layout,
                                      void* stream) {
  if (int rc = check_quantize_args("mx_quantize_gelu", h, rows, cols, ld, codes_row, scales_row, codes_colT,
                                   scales_col, scale_layout))
    return rc;
  ANIMA_REQUIRE((!grad_act || aligned16(grad_act)) && (!act_bf16 || aligned16(act_bf16)), ANIMA_E_ALIGN,
                "mx_quantize_gelu: grad_act and act_bf16 must be 16-byte aligned");
  if (rows == 0 || cols == 0) return ANIMA_OK;
  if (int rc = ensure_gelu_tables(static_cast<cudaStream_t>(stream))) return rc;
  if (grad_act) {
    const GeluBwdLoader load{static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(grad_act), ld,
                             static_cast<__nv_bfloat16*>(act_bf16), cols, 0u};
    return quantize_dispatch("mx_quantize_gelu", load, true, h, rows, cols, ld, codes_row, scales_row, codes_colT,
                             scales_col, scale_layout, stream);
  }
  const GeluLoader load{static_cast<const __nv_bfloat16*>(h), ld, static_cast<__nv_bfloat16*>(act_bf16), cols, 0u};
  return quantize_dispatch("mx_quantize_gelu", load, true, h, rows, cols, ld, codes_row, scales_row, codes_colT,
                           scales_col, scale_layout, stream);
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

extern "C" int anima_mx_scales_regroup(const uint8_t* tiled_in, int64_t rows_in, int64_t k_in, uint8_t* tiled_out,
                                       int64_t rows_out, int64_t k_out, void* stream) {
  ANIMA_REQUIRE(tiled_in && tiled_out, ANIMA_E_ARG, "mx_scales_regroup: null pointer");
  ANIMA_REQUIRE(rows_in >= 0 && rows_out >= 0 && k_in > 0 && k_out > 0 && k_in % 32 == 0 && k_out % 32 == 0,
                ANIMA_E_SHAPE, "mx_scales_regroup: k must be a positive multiple of 32");
  ANIMA_REQUIRE(rows_in * k_in == rows_out * k_out, ANIMA_E_SHAPE,
                "mx_scales_regroup: [%lld, %lld] and [%lld, %lld] hold different numbers of elements",
                (long long)rows_in, (long long)k_in, (long long)rows_out, (long long)k_out);
  if (rows_out == 0) return ANIMA_OK;
  const int64_t total = anima_mx_scales_bytes(rows_out, k_out, ANIMA_SCALES_TILED);
  const int blocks = static_cast<int>(std::min<int64_t>(ceil_div(total, 256), sm_count() * 16));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool small = (rows_out + 128) * (k_out / 32 + 4) < (1ll << 31) && (rows_in + 128) * (k_in / 32 + 4) < (1ll << 31);
  if (small && k_in % 128 == 0 && k_out % 128 == 0 && (reinterpret_cast<uintptr_t>(tiled_in) & 3) == 0 &&
      (reinterpret_cast<uintptr_t>(tiled_out) & 3) == 0) {
    const uint32_t words = static_cast<uint32_t>(total / 4);
    const int wblocks = static_cast<int>(std::min<int64_t>(ceil_div(static_cast<int64_t>(words), 256), sm_count() * 16));
    mx_scales_regroup_words_kernel<<<wblocks, 256, 0, s>>>(reinterpret_cast<const uint32_t*>(tiled_in),
                                                           static_cast<uint32_t>(k_in / 128), static_cast<uint32_t>(rows_out),
                                                           static_cast<uint32_t>(k_out / 128), words,
                                                           reinterpret_cast<uint32_t*>(tiled_out));
    ANIMA_CHECK_LAUNCH("mx_scales_regroup");
    return ANIMA_OK;
  }
  // 32-bit indices when the padded extents of both tilings (and r * kb_out + b for padded r) stay below 2^31
  if (small)
    mx_scales_regroup_kernel<uint32_t><<<blocks, 256, 0, s>>>(tiled_in, static_cast<uint32_t>(k_in / 32),
                                                               static_cast<uint32_t>(rows_out),
                                                               static_cast<uint32_t>(k_out / 32),
                                                               static_cast<uint32_t>(total), tiled_out);
  else
    mx_scales_regroup_kernel<int64_t><<<blocks, 256, 0, s>>>(tiled_in, k_in / 32, rows_out, k_out / 32, total, tiled_out);
  ANIMA_CHECK_LAUNCH("mx_scales_regroup");
  return ANIMA_OK;
}

extern "C" int anima_mx_exponent_probe(const float* amax, int64_t n, int32_t* by_rule, int32_t* by_lg2_approx,
                                       void* stream) {
  ANIMA_REQUIRE(amax && by_rule && by_lg2_approx && n >= 0, ANIMA_E_ARG, "mx_exponent_probe: bad argument");
  if (n == 0) return ANIMA_OK;
  mx_exponent_probe_kernel<<<static_cast<unsigned>(ceil_div(n, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      amax, n, by_rule, by_lg2_approx);
  ANIMA_CHECK_LAUNCH("mx_exponent_probe");
  return ANIMA_OK;
}
