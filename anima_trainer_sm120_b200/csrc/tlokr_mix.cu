// T-LoKr rank-space kernels: the 8x8 Kronecker-factor mix with the per-sample
// timestep rank mask, and the fp32 8x8 weight gradient of that mix.
//
// Replaces anima-trainer's tlokr_kernels.py: _rank_mix_kernel (:15-82) and
// _rank_mix_wgrad_kernel (:85-122). Both are HBM-bound on [batch, n, 8, rank]
// bf16 tensors:
//   rank_mix        reads hidden once, writes out once          (4 B/elem)
//   rank_mix_wgrad  reads grad_mixed and hidden ONCE each       (4 B/elem pair),
//                   contracting on the tensor cores (mma.sync m16n8k16: the output
//                   is 8 x 8, far below a tcgen05 tile); the reference launches one
//                   program per (i,j) pair and so reads both tensors 8 times.
// The wgrad reduction is two-stage (per-CTA partial 8x8 blocks in caller scratch,
// then a fixed-order sum) and therefore bit-reproducible.
#include "common.cuh"
#include "mx_quantize_tile.cuh"

namespace anima {
namespace {

template <bool TRANSPOSE, bool HAS_MASK>
__global__ void __launch_bounds__(256)
rank_mix_kernel(const __nv_bfloat16* __restrict__ hidden, const __nv_bfloat16* __restrict__ c,
                const __nv_bfloat16* __restrict__ mask, int64_t total, int64_t n_per_batch, int r8,
                __nv_bfloat16* __restrict__ out) {
  __shared__ float cw[64];  // cw[i*8+j] = weight applied to hidden row j for output row i
  if (threadIdx.x < 64) {
    const int i = threadIdx.x >> 3, j = threadIdx.x & 7;
    cw[threadIdx.x] = __bfloat162float(TRANSPOSE ? c[j * 8 + i] : c[i * 8 + j]);
  }
  __syncthreads();
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (idx >= total) return;
  const int64_t row = idx / r8;  // (b, n) flattened
  const int rc = static_cast<int>(idx - row * r8);
  const int64_t rank = static_cast<int64_t>(r8) * 8;
  const __nv_bfloat16* src = hidden + row * 8 * rank + rc * 8;

  uint4 h[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) h[j] = ldg_stream16(src + j * rank);
  float m[8];
  if (HAS_MASK) {
    unpack8(*reinterpret_cast<const uint4*>(mask + (row / n_per_batch) * rank + rc * 8), m);
  }
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float hf[8];
    unpack8(h[j], hf);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float w = cw[i * 8 + j];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(hf[e], w, acc[i][e]);
    }
  }
  __nv_bfloat16* dst = out + row * 8 * rank + rc * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (HAS_MASK) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][e] *= m[e];
    }
    stg_stream16(dst + i * rank, pack8(acc[i]));
  }
}

// rank_mix whose output leaves as MXFP8 operands (the factor GEMM that consumes the mixed tensor wants e4m3
// codes, and writing it in bf16 only to read it back in a quantiser launch costs 4 B/elem of the 4 + 3..4 the
// pair moves). The mix is computed and rounded to bf16 exactly as in rank_mix_kernel, then quantised with the
// arithmetic of the tile quantiser, so codes and scales equal those of quantising the bf16 tensor.
//   row form   [R, rank], R = items * 8: a block is 32 consecutive ranks of one row = the 8-rank chunks of four
//              adjacent lanes (two shuffles);
//   column form, stored transposed [rank, R]: a block is 32 consecutive rows of one rank = rows i = 0..7 of four
//              consecutive items, i.e. four threads r8 apart, which exchange their 8-row amax through shared
//              memory; a thread then writes 8 code bytes (its item's rows) per rank.
// The host guarantees rank in {128, 256, 512} (whole 128-column scale chunks, whole item groups per CTA) and
// items % 16 == 0 (every CTA full, R % 128 == 0: no padding entries in the tiled scale buffers).
struct MixCodes {
  uint8_t* codes_row;    // [R, rank] or null
  uint8_t* scales_row;   // tiled
  uint8_t* codes_colT;   // [rank, R] or null
  uint8_t* scales_col;   // tiled
  // Row form as eight planes: row i of item t goes to matrix row i * plane_rows + t instead of t * 8 + i
  // (plane_rows = items, a multiple of 128, so every plane is a whole number of scale row tiles). A GEMM over
  // the items can then take plane i as a K-major [items, rank] operand. 0 = the plain [R, rank] order.
  int64_t plane_rows;
};

template <bool TRANSPOSE, bool HAS_MASK, bool ROW, bool COL>
__global__ void __launch_bounds__(256, 2)
rank_mix_quant_kernel(const __nv_bfloat16* __restrict__ hidden, const __nv_bfloat16* __restrict__ c,
                      const __nv_bfloat16* __restrict__ mask, int64_t items, int64_t n_per_batch, int r8,
                      __nv_bfloat16* __restrict__ out, const MixCodes q) {
  __shared__ float cw[64];
  __shared__ __align__(16) float col_amax[COL ? 2048 : 4];   // [thread][8 ranks]
  __shared__ __align__(16) uint2 stage[COL ? 2048 : 2];      // transposed codes of the CTA: [rank][item] x 8 bytes
  if (threadIdx.x < 64) {
    const int i = threadIdx.x >> 3, j = threadIdx.x & 7;
    cw[threadIdx.x] = __bfloat162float(TRANSPOSE ? c[j * 8 + i] : c[i * 8 + j]);
  }
  __syncthreads();
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;   // < items * r8: every CTA is full
  const int64_t item = idx / r8;  // (b, n) flattened
  const int rc = static_cast<int>(idx - item * r8);
  const int rank = r8 * 8;
  const int64_t R = items * 8;
  const __nv_bfloat16* src = hidden + item * 8 * rank + rc * 8;

  uint4 h[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) h[j] = ldg_stream16(src + j * rank);
  float m[8];
  if (HAS_MASK) unpack8(*reinterpret_cast<const uint4*>(mask + (item / n_per_batch) * rank + rc * 8), m);
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float hf[8];
    unpack8(h[j], hf);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float w = cw[i * 8 + j];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(hf[e], w, acc[i][e]);
    }
  }
  float cmax[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) cmax[e] = 0.f;
  uint4 packed[8];   // the rows as rank_mix would have written them (bf16); the column pass re-reads them from here
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (HAS_MASK) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][e] *= m[e];
    }
    packed[i] = pack8(acc[i]);
    if (out != nullptr) stg_stream16(out + (item * 8 + i) * rank + rc * 8, packed[i]);
    float f[8];
    unpack8(packed[i], f);                         // quantise the rounded values
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float a = fabsf(f[e]);
      amax = fmaxf(amax, a);
      if (COL) cmax[e] = fmaxf(cmax[e], a);
    }
    if (ROW) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const int ex = mxq::mx_exponent(fmaxf(amax, mxq::kAmaxFloor));
      const float inv = mxq::mx_inv_scale(ex);
      uint2 codes;
      codes.x = mxq::e4m3x2(f[0] * inv, f[1] * inv) | (mxq::e4m3x2(f[2] * inv, f[3] * inv) << 16);
      codes.y = mxq::e4m3x2(f[4] * inv, f[5] * inv) | (mxq::e4m3x2(f[6] * inv, f[7] * inv) << 16);
      const int64_t row = q.plane_rows ? i * q.plane_rows + item : item * 8 + i;
      *reinterpret_cast<uint2*>(q.codes_row + row * rank + rc * 8) = codes;
      if ((rc & 3) == 0) {
        const int kb = rc >> 2;
        q.scales_row[((row >> 7) * (rank >> 7) + (kb >> 2)) * 512 + mxq::tiled_offset(static_cast<int>(row & 127), kb & 3)] =
            static_cast<uint8_t>(ex + 127);
      }
    }
  }
  if (COL) {
    float4* mine = reinterpret_cast<float4*>(col_amax + threadIdx.x * 8);
    mine[0] = make_float4(cmax[0], cmax[1], cmax[2], cmax[3]);
    mine[1] = make_float4(cmax[4], cmax[5], cmax[6], cmax[7]);
    __syncthreads();
    const int item_local = threadIdx.x / r8;
    const int group0 = (item_local & ~3) * r8 + rc;   // the thread of the group's first item with this rank chunk
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float4* other = reinterpret_cast<const float4*>(col_amax + (group0 + k * r8) * 8);
      const float4 lo = other[0], hi = other[1];
      cmax[0] = fmaxf(cmax[0], lo.x); cmax[1] = fmaxf(cmax[1], lo.y); cmax[2] = fmaxf(cmax[2], lo.z); cmax[3] = fmaxf(cmax[3], lo.w);
      cmax[4] = fmaxf(cmax[4], hi.x); cmax[5] = fmaxf(cmax[5], hi.y); cmax[6] = fmaxf(cmax[6], hi.z); cmax[7] = fmaxf(cmax[7], hi.w);
    }
    const int64_t blk = item >> 2;                    // 32-row block of R
    const int64_t kb4 = R >> 7;                       // scale chunks per 128 ranks
    // A rank owns P = 256 / r8 pieces of 8 bytes (one per item of the CTA), contiguous in the output. They are
    // staged in shared memory, piece p of rank chunk rc at p ^ (2 * (rc % (P/2))) (pairs stay together and the
    // stores of a half-warp spread over the banks), and leave as 16-byte stores in runs of 8 P bytes.
    const int P = 256 / r8;
    const int swz = (rc & (P / 2 - 1)) << 1;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int ex = mxq::mx_exponent(fmaxf(cmax[e], mxq::kAmaxFloor));
      const float inv = mxq::mx_inv_scale(ex);
      float v[8];   // rank e of rows 0..7: half e % 2 of word e / 2 of each packed row
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t w = reinterpret_cast<const uint32_t*>(&packed[i])[e >> 1];
        v[i] = __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
      }
      uint2 codes;
      codes.x = mxq::e4m3x2(v[0] * inv, v[1] * inv) | (mxq::e4m3x2(v[2] * inv, v[3] * inv) << 16);
      codes.y = mxq::e4m3x2(v[4] * inv, v[5] * inv) | (mxq::e4m3x2(v[6] * inv, v[7] * inv) << 16);
      const int col = rc * 8 + e;
      stage[col * P + (item_local ^ swz)] = codes;
      if ((item_local & 3) == 0)
        q.scales_col[((col >> 7) * kb4 + (blk >> 2)) * 512 + mxq::tiled_offset(col & 127, static_cast<int>(blk & 3))] =
            static_cast<uint8_t>(ex + 127);
    }
    __syncthreads();
    const int64_t row0 = static_cast<int64_t>(blockIdx.x) * P * 8;   // first row of R this CTA covers
    const int half = P / 2;                                           // 16-byte units per rank
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const int u = threadIdx.x + h * 256;          // 1024 units: rank u / half, unit u % half
      const int col = u / half, unit = u - col * half;
      const int s2 = ((col >> 3) & (half - 1)) << 1;
      const uint4 v = *reinterpret_cast<const uint4*>(&stage[col * P + ((2 * unit) ^ s2)]);
      stg_stream16(q.codes_colT + static_cast<int64_t>(col) * R + row0 + unit * 16, v);
    }
  }
}

constexpr int kWgradThreads = 256;
constexpr int kWgradWarps = kWgradThreads / 32;

// D(16x8, fp32) += A(16x16, bf16, row-major) * B(16x8, bf16): rows 8..15 of A are zero here.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// dc[i][j] = sum over (b, n, r) of grad[b,n,i,r] * hidden[b,n,j,r] * mask[b,r] is an 8 x 8 output with a
// contraction of millions: one m16n8k16 tensor-core instruction per 16 contraction elements replaces 1024
// scalar FMAs, which leaves the kernel bound by its two streaming reads. A warp owns one (b, n) item at a
// time; lane (g, t) = (lane / 4, lane % 4) loads 8 consecutive r of row g of both tensors. The contraction
// index may be permuted freely as long as A and B agree, so the lane's four 32-bit words feed the k-slots
// (2t, 2t+1) and (2t+8, 2t+9) of two instructions directly: no shuffles, 16-byte loads only.
// The mask multiplies hidden as bf16 pairs: exact for the 0 / 1 masks of the rank schedule.
template <bool HAS_MASK>
__global__ void __launch_bounds__(kWgradThreads)
rank_mix_wgrad_kernel(const __nv_bfloat16* __restrict__ grad, const __nv_bfloat16* __restrict__ hidden,
                      const __nv_bfloat16* __restrict__ mask, int64_t items, int64_t n_per_batch, int rank,
                      float* __restrict__ partial) {
  __shared__ float red[kWgradWarps][64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int steps = (rank + 31) / 32;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * kWgradWarps;
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWgradWarps + warp; item < items; item += warps_total) {
    const int64_t off = item * 8 * rank + static_cast<int64_t>(g) * rank + t * 8;
    const __nv_bfloat16* mp = HAS_MASK ? mask + (item / n_per_batch) * rank + t * 8 : nullptr;
#pragma unroll 4
    for (int s = 0; s < steps; ++s) {
      // rank % 8 == 0: a lane's chunk is all in or all out. Lanes past the tail feed zeros: the two
      // warp-wide instructions below are reached by all 32 lanes together, never from a divergent branch.
      uint4 a = make_uint4(0u, 0u, 0u, 0u), b = make_uint4(0u, 0u, 0u, 0u);
      if (s * 32 + t * 8 < rank) {
        a = ldg_stream16(grad + off + s * 32);
        b = ldg_stream16(hidden + off + s * 32);
        if (HAS_MASK) {
          const uint4 m = *reinterpret_cast<const uint4*>(mp + s * 32);
          b.x = bf16x2_mul(b.x, m.x);
          b.y = bf16x2_mul(b.y, m.y);
          b.z = bf16x2_mul(b.z, m.z);
          b.w = bf16x2_mul(b.w, m.w);
        }
      }
      __syncwarp();
      mma_bf16_16816(acc, a.x, a.y, b.x, b.y);
      mma_bf16_16816(acc, a.z, a.w, b.z, b.w);
    }
  }
  // acc[0], acc[1] = dc[g][2t], dc[g][2t+1] of this warp; rows 8..15 (acc[2], acc[3]) are padding
  red[warp][g * 8 + 2 * t] = acc[0];
  red[warp][g * 8 + 2 * t + 1] = acc[1];
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWgradWarps; ++w) s += red[w][threadIdx.x];
    partial[blockIdx.x * 64 + threadIdx.x] = s;
  }
}

__global__ void __launch_bounds__(kFinalizeThreads)
rank_mix_wgrad_finalize_kernel(const float* __restrict__ partial, int blocks, float* __restrict__ dc) {
  const float s = sum_partials_64(partial, blocks);
  if (threadIdx.x < 64) dc[threadIdx.x] = s;
}

// items = batch * n_per_batch; one warp per item at a time
int wgrad_blocks(int64_t items) {
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(ceil_div(items, kWgradWarps), 4LL * sm_count())));
}

}  // namespace
}  // namespace anima

using namespace anima;

extern "C" int anima_tlokr_rank_mix(const void* hidden, const void* c, const void* mask, int64_t batch,
                                    int64_t n_per_batch, int64_t rank, int transpose, void* out,
                                    void* stream) {
  ANIMA_REQUIRE(hidden && c && out, ANIMA_E_ARG, "tlokr_rank_mix: null pointer");
  ANIMA_REQUIRE(batch >= 0 && n_per_batch >= 0 && rank > 0, ANIMA_E_ARG, "tlokr_rank_mix: bad sizes");
  ANIMA_REQUIRE(rank % 8 == 0, ANIMA_E_SHAPE, "tlokr_rank_mix: rank=%lld must be a multiple of 8",
                (long long)rank);
  ANIMA_REQUIRE(aligned16(hidden) && aligned16(out) && (!mask || aligned16(mask)), ANIMA_E_ALIGN,
                "tlokr_rank_mix: tensors must be 16-byte aligned");
  const int64_t total = batch * n_per_batch * (rank / 8);
  if (total == 0) return ANIMA_OK;
  const unsigned grid = static_cast<unsigned>(ceil_div(total, 256));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* hp = static_cast<const __nv_bfloat16*>(hidden);
  const auto* cp = static_cast<const __nv_bfloat16*>(c);
  const auto* mp = static_cast<const __nv_bfloat16*>(mask);
  auto* op = static_cast<__nv_bfloat16*>(out);
  const int r8 = static_cast<int>(rank / 8);
#define ANIMA_MIX(T, M) rank_mix_kernel<T, M><<<grid, 256, 0, s>>>(hp, cp, mp, total, n_per_batch, r8, op)
  if (transpose) {
    if (mask) ANIMA_MIX(true, true); else ANIMA_MIX(true, false);
  } else {
    if (mask) ANIMA_MIX(false, true); else ANIMA_MIX(false, false);
  }
#undef ANIMA_MIX
  ANIMA_CHECK_LAUNCH("tlokr_rank_mix");
  return ANIMA_OK;
}

static int rank_mix_quant_impl(const void* hidden, const void* c, const void* mask, int64_t batch,
                               int64_t n_per_batch, int64_t rank, int transpose, void* out,
                               uint8_t* codes_row, uint8_t* scales_row, uint8_t* codes_colT,
                               uint8_t* scales_col, bool planes, void* stream) {
  ANIMA_REQUIRE(hidden && c, ANIMA_E_ARG, "tlokr_rank_mix_quant: null pointer");
  ANIMA_REQUIRE(codes_row || codes_colT, ANIMA_E_ARG, "tlokr_rank_mix_quant: no operand requested");
  ANIMA_REQUIRE((codes_row == nullptr) == (scales_row == nullptr) && (codes_colT == nullptr) == (scales_col == nullptr),
                ANIMA_E_ARG, "tlokr_rank_mix_quant: codes and scales must be given in pairs");
  ANIMA_REQUIRE(batch >= 0 && n_per_batch >= 0, ANIMA_E_ARG, "tlokr_rank_mix_quant: bad sizes");
  ANIMA_REQUIRE(rank == 128 || rank == 256 || rank == 512, ANIMA_E_SHAPE,
                "tlokr_rank_mix_quant: rank=%lld must be 128, 256 or 512", (long long)rank);
  const int64_t items = batch * n_per_batch;
  ANIMA_REQUIRE(items % 16 == 0, ANIMA_E_SHAPE, "tlokr_rank_mix_quant: batch * n = %lld must be a multiple of 16",
                (long long)items);
  ANIMA_REQUIRE(aligned16(hidden) && aligned16(out) && (!mask || aligned16(mask)) &&
                    (reinterpret_cast<uintptr_t>(codes_row) & 7) == 0 && (reinterpret_cast<uintptr_t>(codes_colT) & 7) == 0,
                ANIMA_E_ALIGN, "tlokr_rank_mix_quant: misaligned tensor");
  if (items == 0) return ANIMA_OK;
  const int r8 = static_cast<int>(rank / 8);
  const unsigned grid = static_cast<unsigned>(items * r8 / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* hp = static_cast<const __nv_bfloat16*>(hidden);
  const auto* cp = static_cast<const __nv_bfloat16*>(c);
  const auto* mp = static_cast<const __nv_bfloat16*>(mask);
  auto* op = static_cast<__nv_bfloat16*>(out);
  ANIMA_REQUIRE(!planes || (codes_row && items % 128 == 0), ANIMA_E_SHAPE,
                "tlokr_rank_mix_quant_planes: needs the row form and batch * n = %lld a multiple of 128", (long long)items);
  const MixCodes q{codes_row, scales_row, codes_colT, scales_col, planes ? items : 0};
#define ANIMA_MIXQ(T, M, R, C) rank_mix_quant_kernel<T, M, R, C><<<grid, 256, 0, s>>>(hp, cp, mp, items, n_per_batch, r8, op, q)
#define ANIMA_MIXQ_FORMS(T, M)                                     \
  do {                                                             \
    if (codes_row && codes_colT) ANIMA_MIXQ(T, M, true, true);     \
    else if (codes_row) ANIMA_MIXQ(T, M, true, false);             \
    else ANIMA_MIXQ(T, M, false, true);                            \
  } while (0)
  if (transpose) {
    if (mask) ANIMA_MIXQ_FORMS(true, true); else ANIMA_MIXQ_FORMS(true, false);
  } else {
    if (mask) ANIMA_MIXQ_FORMS(false, true); else ANIMA_MIXQ_FORMS(false, false);
  }
#undef ANIMA_MIXQ_FORMS
#undef ANIMA_MIXQ
  ANIMA_CHECK_LAUNCH("tlokr_rank_mix_quant");
  return ANIMA_OK;
}

extern "C" int anima_tlokr_rank_mix_quant(const void* hidden, const void* c, const void* mask, int64_t batch,
                                          int64_t n_per_batch, int64_t rank, int transpose, void* out,
                                          uint8_t* codes_row, uint8_t* scales_row, uint8_t* codes_colT,
                                          uint8_t* scales_col, void* stream) {
  return rank_mix_quant_impl(hidden, c, mask, batch, n_per_batch, rank, transpose, out, codes_row, scales_row, codes_colT,
                             scales_col, false, stream);
}

extern "C" int anima_tlokr_rank_mix_quant_planes(const void* hidden, const void* c, const void* mask, int64_t batch,
                                                 int64_t n_per_batch, int64_t rank, int transpose,
                                                 uint8_t* codes_planes, uint8_t* scales_planes, uint8_t* codes_colT,
                                                 uint8_t* scales_col, void* stream) {
  return rank_mix_quant_impl(hidden, c, mask, batch, n_per_batch, rank, transpose, nullptr, codes_planes, scales_planes,
                             codes_colT, scales_col, true, stream);
}

extern "C" int64_t anima_tlokr_rank_mix_wgrad_workspace_bytes(int64_t batch, int64_t n_per_batch,
                                                              int64_t rank) {
  if (batch < 0 || n_per_batch < 0 || rank <= 0 || rank % 8) return ANIMA_E_SHAPE;
  return static_cast<int64_t>(wgrad_blocks(batch * n_per_batch)) * 64 * sizeof(float);
}

extern "C" int anima_tlokr_rank_mix_wgrad(const void* grad_mixed, const void* hidden, const void* mask,
                                          int64_t batch, int64_t n_per_batch, int64_t rank, float* dc,
                                          void* workspace, int64_t workspace_bytes, void* stream) {
  ANIMA_REQUIRE(grad_mixed && hidden && dc, ANIMA_E_ARG, "tlokr_rank_mix_wgrad: null pointer");
  ANIMA_REQUIRE(batch >= 0 && n_per_batch >= 0 && rank > 0, ANIMA_E_ARG,
                "tlokr_rank_mix_wgrad: bad sizes");
  ANIMA_REQUIRE(rank % 8 == 0, ANIMA_E_SHAPE, "tlokr_rank_mix_wgrad: rank=%lld must be a multiple of 8",
                (long long)rank);
  ANIMA_REQUIRE(aligned16(grad_mixed) && aligned16(hidden) && (!mask || aligned16(mask)), ANIMA_E_ALIGN,
                "tlokr_rank_mix_wgrad: tensors must be 16-byte aligned");
  ANIMA_REQUIRE(rank < (1 << 30), ANIMA_E_TOO_LARGE, "tlokr_rank_mix_wgrad: rank too large");
  const int64_t items = batch * n_per_batch;
  const int64_t need = anima_tlokr_rank_mix_wgrad_workspace_bytes(batch, n_per_batch, rank);
  ANIMA_REQUIRE(workspace && workspace_bytes >= need, ANIMA_E_WORKSPACE,
                "tlokr_rank_mix_wgrad: workspace of %lld bytes required, got %lld", (long long)need,
                (long long)workspace_bytes);
  const int blocks = wgrad_blocks(items);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  const auto* gp = static_cast<const __nv_bfloat16*>(grad_mixed);
  const auto* hp = static_cast<const __nv_bfloat16*>(hidden);
  const auto* mp = static_cast<const __nv_bfloat16*>(mask);
  const int r = static_cast<int>(rank);
  if (mask)
    rank_mix_wgrad_kernel<true><<<blocks, kWgradThreads, 0, s>>>(gp, hp, mp, items, n_per_batch, r, ws);
  else
    rank_mix_wgrad_kernel<false><<<blocks, kWgradThreads, 0, s>>>(gp, hp, mp, items, n_per_batch, r, ws);
  ANIMA_CHECK_LAUNCH("tlokr_rank_mix_wgrad");
  rank_mix_wgrad_finalize_kernel<<<1, kFinalizeThreads, 0, s>>>(ws, blocks, dc);
  ANIMA_CHECK_LAUNCH("tlokr_rank_mix_wgrad finalize");
  return ANIMA_OK;
}
