// T-LoKr rank-space kernels: the 8x8 Kronecker-factor mix with the per-sample
// timestep rank mask, and the fp32 8x8 weight gradient of that mix.
//
// Replaces anima-trainer's tlokr_kernels.py: _rank_mix_kernel (:15-82) and
// _rank_mix_wgrad_kernel (:85-122). Both are HBM-bound on [batch, n, 8, rank]
// bf16 tensors:
//   rank_mix        reads hidden once, writes out once          (4 B/elem)
//   rank_mix_wgrad  reads grad_mixed and hidden ONCE each       (4 B/elem pair);
//                   the reference launches one program per (i,j) pair and so
//                   reads both tensors 8 times.
// The wgrad reduction is two-stage (per-CTA partial 8x8 blocks in caller scratch,
// then a fixed-order sum) and therefore bit-reproducible.
#include "common.cuh"

namespace anima {
namespace {

__device__ __forceinline__ float bf16_lane(const uint4& raw, int e) {
  const uint32_t w = reinterpret_cast<const uint32_t*>(&raw)[e >> 1];
  return __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
}

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

constexpr int kWgradThreads = 128;

template <bool HAS_MASK>
__global__ void __launch_bounds__(kWgradThreads)
rank_mix_wgrad_kernel(const __nv_bfloat16* __restrict__ grad, const __nv_bfloat16* __restrict__ hidden,
                      const __nv_bfloat16* __restrict__ mask, int64_t total, int64_t n_per_batch,
                      int r8, float* __restrict__ partial) {
  __shared__ float red[kWgradThreads / 32][64];
  const int64_t rank = static_cast<int64_t>(r8) * 8;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int64_t stride = static_cast<int64_t>(gridDim.x) * kWgradThreads;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(kWgradThreads) + threadIdx.x; idx < total;
       idx += stride) {
    const int64_t row = idx / r8;
    const int rc = static_cast<int>(idx - row * r8);
    const int64_t off = row * 8 * rank + rc * 8;
    uint4 g[8], h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      g[i] = ldg_stream16(grad + off + i * rank);
      h[i] = ldg_stream16(hidden + off + i * rank);
    }
    uint4 mraw = make_uint4(0u, 0u, 0u, 0u);
    if (HAS_MASK) mraw = *reinterpret_cast<const uint4*>(mask + (row / n_per_batch) * rank + rc * 8);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float gv[8], hv[8];
      const float mv = HAS_MASK ? bf16_lane(mraw, e) : 1.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        gv[i] = bf16_lane(g[i], e);
        hv[i] = bf16_lane(h[i], e) * mv;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(gv[i], hv[j], acc[i][j]);
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = warp_sum(acc[i][j]);
      if (lane == 0) red[warp][i * 8 + j] = s;
    }
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWgradThreads / 32; ++w) s += red[w][threadIdx.x];
    partial[blockIdx.x * 64 + threadIdx.x] = s;
  }
}

__global__ void rank_mix_wgrad_finalize_kernel(const float* __restrict__ partial, int blocks,
                                               float* __restrict__ dc) {
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[b * 64 + threadIdx.x];
  dc[threadIdx.x] = s;
}

int wgrad_blocks(int64_t total) {
  return static_cast<int>(std::max<int64_t>(
      1, std::min<int64_t>(ceil_div(total, kWgradThreads), 4LL * sm_count())));
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

extern "C" int64_t anima_tlokr_rank_mix_wgrad_workspace_bytes(int64_t batch, int64_t n_per_batch,
                                                              int64_t rank) {
  if (batch < 0 || n_per_batch < 0 || rank <= 0 || rank % 8) return ANIMA_E_SHAPE;
  return static_cast<int64_t>(wgrad_blocks(batch * n_per_batch * (rank / 8))) * 64 * sizeof(float);
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
  const int64_t total = batch * n_per_batch * (rank / 8);
  const int64_t need = anima_tlokr_rank_mix_wgrad_workspace_bytes(batch, n_per_batch, rank);
  ANIMA_REQUIRE(workspace && workspace_bytes >= need, ANIMA_E_WORKSPACE,
                "tlokr_rank_mix_wgrad: workspace of %lld bytes required, got %lld", (long long)need,
                (long long)workspace_bytes);
  const int blocks = wgrad_blocks(total);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  const auto* gp = static_cast<const __nv_bfloat16*>(grad_mixed);
  const auto* hp = static_cast<const __nv_bfloat16*>(hidden);
  const auto* mp = static_cast<const __nv_bfloat16*>(mask);
  const int r8 = static_cast<int>(rank / 8);
  if (mask)
    rank_mix_wgrad_kernel<true><<<blocks, kWgradThreads, 0, s>>>(gp, hp, mp, total, n_per_batch, r8, ws);
  else
    rank_mix_wgrad_kernel<false><<<blocks, kWgradThreads, 0, s>>>(gp, hp, mp, total, n_per_batch, r8, ws);
  ANIMA_CHECK_LAUNCH("tlokr_rank_mix_wgrad");
  rank_mix_wgrad_finalize_kernel<<<1, 64, 0, s>>>(ws, blocks, dc);
  ANIMA_CHECK_LAUNCH("tlokr_rank_mix_wgrad finalize");
  return ANIMA_OK;
}
