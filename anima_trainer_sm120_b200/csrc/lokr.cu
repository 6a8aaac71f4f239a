// LoKr weight kernels.
//
// (1) lokr_merge_quantize: builds merged = W + alpha * kron(w1, w2) for a wrapped
//     Linear and emits, from one read of W, the bf16 merged weight and/or its
//     row-wise and column-wise MXFP8 forms. Replaces the eager
//     get_weight -> cast -> add of lokr_patch.py:76-84 (which materialises the
//     [N,K] Kronecker product in HBM every forward and every checkpoint recompute)
//     plus the two weight quantisations of fp8_quant.py:234-235 / :501.
// (2) lokr_kron_backward: the adapter gradients from dW = dy^T x, i.e. the autograd
//     of torch.kron that lokr_patch.py:19-21 relies on, as one pass over dW.
//
// Rounding of the merged weight follows the eager bf16 path: the Kronecker product
// is rounded to bf16 (torch.kron of bf16 factors; an fp32 product cast to the
// weight dtype rounds the same way), then W + alpha * diff is evaluated in fp32 and
// rounded to bf16 once (torch.add(W, diff, alpha=alpha); alpha == 1 is W + diff).
#include "mx_quantize_tile.cuh"

namespace anima {
namespace {

using namespace mxq;

template <class F>
__device__ __forceinline__ float to_f32(F v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

static inline int log2_if_pow2(int64_t v) {
  if (v <= 0 || (v & (v - 1)) != 0) return -1;
  int s = 0;
  while ((int64_t{1} << s) < v) ++s;
  return s;
}

template <class F>
struct MergeLoader {
  const __nv_bfloat16* w;
  const F* w1;  // [up, uq]
  const F* w2;  // [vp, vq]
  __nv_bfloat16* merged;  // optional [N, K]
  float alpha;
  int64_t K, vp, vq, uq;
  int vp_shift, vq_shift;   // log2 when the block size is a power of two (then the divisions are shifts), else -1
  using Raw = uint4;
  static constexpr bool kZeroSafe = false;   // finish reads the factors at (row, col)
  static constexpr int kSmemBytes = 0;
  __device__ __forceinline__ void prepare(void*) {}
  __device__ __forceinline__ Raw fetch(int64_t r, int64_t c) const { return ldg_stream16(w + r * K + c); }
  __device__ __forceinline__ uint4 operator()(int64_t r, int64_t c) const { return finish(fetch(r, c), r, c); }
  // W comes from HBM (fetch); the factors are small and cache-resident and are read here.
  __device__ __forceinline__ uint4 finish(const Raw& raw, int64_t r, int64_t c) const {
    const int ri = static_cast<int>(r), ci = static_cast<int>(c);   // N, K < 2^31 is checked on the host
    const int i = vp_shift >= 0 ? ri >> vp_shift : ri / static_cast<int>(vp), p = ri - i * static_cast<int>(vp);
    const int j = vq_shift >= 0 ? ci >> vq_shift : ci / static_cast<int>(vq);    // vq % 8 == 0: the 8 columns share j
    const int q = ci - j * static_cast<int>(vq);
    const float a = to_f32(w1[i * uq + j]);
    float wv[8], o[8], f2[8];
    unpack8(raw, wv);
    const F* w2p = w2 + p * vq + q;  // 8 consecutive factors: vq % 8 == 0 keeps them 16/32-byte aligned
    if constexpr (sizeof(F) == 4) {
      const float4 lo = *reinterpret_cast<const float4*>(w2p), hi = *reinterpret_cast<const float4*>(w2p + 4);
      f2[0] = lo.x; f2[1] = lo.y; f2[2] = lo.z; f2[3] = lo.w;
      f2[4] = hi.x; f2[5] = hi.y; f2[6] = hi.z; f2[7] = hi.w;
    } else {
      unpack8(*reinterpret_cast<const uint4*>(w2p), f2);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float diff = __bfloat162float(__float2bfloat16_rn(a * f2[e]));
      o[e] = fmaf(alpha, diff, wv[e]);
    }
    const uint4 packed = pack8(o);
    if (merged) stg_stream16(merged + r * K + c, packed);
    return packed;
  }
};

// Writes only the merged bf16 weight (no quantised output requested).
template <class F>
__global__ void __launch_bounds__(256) lokr_merge_only_kernel(const MergeLoader<F> load, int64_t N, int64_t K) {
  const int64_t total = N * (K / 8);
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = idx / (K / 8);
    (void)load(r, (idx - r * (K / 8)) * 8);
  }
}

// ---- Kronecker backward ------------------------------------------------------
// Thread (p, q8) walks the up*uq blocks of dW: its dw2 sums are complete (no
// cross-thread reduction); its dw1 contributions are reduced per CTA into scratch.
constexpr int kKronThreads = 128;
constexpr int kMaxFactor = 8;

template <class G, class F>
__global__ void __launch_bounds__(kKronThreads)
kron_backward_kernel(const G* __restrict__ dw, const F* __restrict__ w1, const F* __restrict__ w2,
                     float alpha, int64_t K, int vp, int vq, int up, int uq, float* __restrict__ dw2,
                     float* __restrict__ partial) {
  __shared__ float red[kKronThreads / 32][kMaxFactor * kMaxFactor];
  __shared__ float w1s[kMaxFactor * kMaxFactor];
  if (threadIdx.x < kMaxFactor * kMaxFactor) {
    const int i = threadIdx.x / kMaxFactor, j = threadIdx.x % kMaxFactor;
    w1s[threadIdx.x] = (i < up && j < uq) ? to_f32(w1[i * uq + j]) : 0.f;
  }
  __syncthreads();
  const int vq8 = vq / 8;
  const int64_t item = blockIdx.x * static_cast<int64_t>(kKronThreads) + threadIdx.x;
  const bool active = item < static_cast<int64_t>(vp) * vq8;
  const int p = active ? static_cast<int>(item / vq8) : 0;
  const int q = active ? static_cast<int>(item % vq8) * 8 : 0;

  float w2v[8], acc2[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    w2v[e] = active ? to_f32(w2[static_cast<int64_t>(p) * vq + q + e]) : 0.f;
    acc2[e] = 0.f;
  }
  float t1[kMaxFactor][kMaxFactor];
#pragma unroll
  for (int i = 0; i < kMaxFactor; ++i) {
#pragma unroll
    for (int j = 0; j < kMaxFactor; ++j) {
      float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (active && i < up && j < uq) {
        const G* src = dw + (static_cast<int64_t>(i) * vp + p) * K + static_cast<int64_t>(j) * vq + q;
        if constexpr (sizeof(G) == 2) {
          unpack8(ldg_stream16(src), g);
        } else {
          const float4 a = *reinterpret_cast<const float4*>(src);
          const float4 b = *reinterpret_cast<const float4*>(src + 4);
          g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
          g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
        }
      }
      const float a1 = w1s[i * kMaxFactor + j];
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        s = fmaf(g[e], w2v[e], s);
        acc2[e] = fmaf(g[e], a1, acc2[e]);
      }
      t1[i][j] = s;
    }
  }
  if (active) {
    float* d = dw2 + static_cast<int64_t>(p) * vq + q;
    *reinterpret_cast<float4*>(d) = make_float4(alpha * acc2[0], alpha * acc2[1], alpha * acc2[2], alpha * acc2[3]);
    *reinterpret_cast<float4*>(d + 4) = make_float4(alpha * acc2[4], alpha * acc2[5], alpha * acc2[6], alpha * acc2[7]);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < kMaxFactor; ++i)
#pragma unroll
    for (int j = 0; j < kMaxFactor; ++j) {
      const float s = warp_sum(t1[i][j]);
      if (lane == 0) red[warp][i * kMaxFactor + j] = s;
    }
  __syncthreads();
  if (threadIdx.x < kMaxFactor * kMaxFactor) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kKronThreads / 32; ++w) s += red[w][threadIdx.x];
    partial[blockIdx.x * (kMaxFactor * kMaxFactor) + threadIdx.x] = s;
  }
}

__global__ void kron_backward_finalize_kernel(const float* __restrict__ partial, int blocks, float alpha,
                                              int up, int uq, float* __restrict__ dw1) {
  const float s = sum_partials_64(partial, blocks);
  const int i = threadIdx.x / kMaxFactor, j = threadIdx.x % kMaxFactor;
  if (threadIdx.x < kMaxFactor * kMaxFactor && i < up && j < uq) dw1[i * uq + j] = alpha * s;
}

int check_factors(const char* who, int64_t N, int64_t K, int64_t up, int64_t uq) {
  ANIMA_REQUIRE(N > 0 && K > 0 && up > 0 && uq > 0, ANIMA_E_ARG, "%s: bad sizes", who);
  ANIMA_REQUIRE(N % up == 0 && K % uq == 0, ANIMA_E_SHAPE,
                "%s: N=%lld, K=%lld not divisible by the w1 shape [%lld,%lld]", who, (long long)N,
                (long long)K, (long long)up, (long long)uq);
  ANIMA_REQUIRE((K / uq) % 8 == 0, ANIMA_E_SHAPE, "%s: K/uq=%lld must be a multiple of 8", who,
                (long long)(K / uq));
  return ANIMA_OK;
}

template <class F>
int launch_merge(const void* w, const void* w1, const void* w2, float alpha, int64_t N, int64_t K,
                 int64_t up, int64_t uq, void* merged, uint8_t* codes_row, uint8_t* scales_row,
                 uint8_t* codes_colT, uint8_t* scales_col, int scale_layout, cudaStream_t s) {
  const MergeLoader<F> load{static_cast<const __nv_bfloat16*>(w), static_cast<const F*>(w1),
                            static_cast<const F*>(w2), static_cast<__nv_bfloat16*>(merged), alpha,
                            K, N / up, K / uq, uq, log2_if_pow2(N / up), log2_if_pow2(K / uq)};
  const bool row = codes_row != nullptr, col = codes_colT != nullptr;
  if (!row && !col) {
    const int64_t total = N * (K / 8);
    lokr_merge_only_kernel<F><<<static_cast<unsigned>(std::min<int64_t>(ceil_div(total, 256), 16LL * sm_count())),
                                256, 0, s>>>(load, N, K);
    return ANIMA_OK;
  }
  QuantParams p{N, K, codes_row, scales_row, codes_colT, scales_col, scale_layout == ANIMA_SCALES_TILED};
  const dim3 grid(static_cast<unsigned>(ceil_div(K, kTile)), static_cast<unsigned>(ceil_div(N, kTile)));
  if (row && col)
    mx_quantize_kernel<true, true><<<grid, kThreads, 0, s>>>(p, load);
  else if (row)
    mx_quantize_kernel<true, false><<<grid, kThreads, 0, s>>>(p, load);
  else
    mx_quantize_kernel<false, true><<<grid, kThreads, 0, s>>>(p, load);
  return ANIMA_OK;
}

}  // namespace
}  // namespace anima

using namespace anima;

extern "C" int anima_lokr_merge_quantize(const void* w, const void* w1, const void* w2,
                                         int factors_are_fp32, float alpha, int64_t N, int64_t K,
                                         int64_t up, int64_t uq, void* merged, uint8_t* codes_row,
                                         uint8_t* scales_row, uint8_t* codes_colT, uint8_t* scales_col,
                                         int scale_layout, void* stream) {
  ANIMA_REQUIRE(w && w1 && w2, ANIMA_E_ARG, "lokr_merge_quantize: null pointer");
  if (int rc = check_factors("lokr_merge_quantize", N, K, up, uq)) return rc;
  const bool row = codes_row != nullptr, col = codes_colT != nullptr;
  ANIMA_REQUIRE(merged || row || col, ANIMA_E_ARG, "lokr_merge_quantize: no output requested");
  ANIMA_REQUIRE((codes_row == nullptr) == (scales_row == nullptr) &&
                    (codes_colT == nullptr) == (scales_col == nullptr),
                ANIMA_E_ARG, "lokr_merge_quantize: codes and scales must be given in pairs");
  ANIMA_REQUIRE(scale_layout == ANIMA_SCALES_PLAIN || scale_layout == ANIMA_SCALES_TILED, ANIMA_E_ARG,
                "lokr_merge_quantize: bad scale_layout %d", scale_layout);
  ANIMA_REQUIRE(!row || K % 32 == 0, ANIMA_E_SHAPE, "lokr_merge_quantize: rowwise needs K %% 32 == 0");
  ANIMA_REQUIRE(!col || N % 32 == 0, ANIMA_E_SHAPE, "lokr_merge_quantize: columnwise needs N %% 32 == 0");
  ANIMA_REQUIRE(ceil_div(N, kTile) <= 65535 && K < (1ll << 31), ANIMA_E_TOO_LARGE, "lokr_merge_quantize: N or K too large");
  ANIMA_REQUIRE(aligned16(w) && aligned16(w2) && (!merged || aligned16(merged)) && (!row || aligned16(codes_row)) &&
                    (!col || aligned16(codes_colT)),
                ANIMA_E_ALIGN, "lokr_merge_quantize: W, w2, merged and code buffers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (factors_are_fp32)
    launch_merge<float>(w, w1, w2, alpha, N, K, up, uq, merged, codes_row, scales_row, codes_colT,
                        scales_col, scale_layout, s);
  else
    launch_merge<__nv_bfloat16>(w, w1, w2, alpha, N, K, up, uq, merged, codes_row, scales_row,
                                codes_colT, scales_col, scale_layout, s);
  ANIMA_CHECK_LAUNCH("lokr_merge_quantize");
  return ANIMA_OK;
}

extern "C" int64_t anima_lokr_kron_backward_workspace_bytes(int64_t N, int64_t K, int64_t up,
                                                            int64_t uq) {
  if (N <= 0 || K <= 0 || up <= 0 || uq <= 0 || N % up || K % uq || (K / uq) % 8) return ANIMA_E_SHAPE;
  const int64_t items = (N / up) * (K / uq / 8);
  return ceil_div(items, kKronThreads) * kMaxFactor * kMaxFactor * static_cast<int64_t>(sizeof(float));
}

extern "C" int anima_lokr_kron_backward(const void* dw, int dw_is_fp32, const void* w1, const void* w2,
                                        int factors_are_fp32, float alpha, int64_t N, int64_t K,
                                        int64_t up, int64_t uq, float* dw1, float* dw2, void* workspace,
                                        int64_t workspace_bytes, void* stream) {
  ANIMA_REQUIRE(dw && w1 && w2 && dw1 && dw2, ANIMA_E_ARG, "lokr_kron_backward: null pointer");
  if (int rc = check_factors("lokr_kron_backward", N, K, up, uq)) return rc;
  ANIMA_REQUIRE(up <= kMaxFactor && uq <= kMaxFactor, ANIMA_E_UNSUPPORTED,
                "lokr_kron_backward: w1 larger than %dx%d is not supported", kMaxFactor, kMaxFactor);
  ANIMA_REQUIRE(aligned16(dw) && aligned16(dw2) && (K * (dw_is_fp32 ? 4 : 2)) % 16 == 0, ANIMA_E_ALIGN,
                "lokr_kron_backward: dW and dw2 must be 16-byte aligned");
  const int64_t need = anima_lokr_kron_backward_workspace_bytes(N, K, up, uq);
  ANIMA_REQUIRE(workspace && workspace_bytes >= need, ANIMA_E_WORKSPACE,
                "lokr_kron_backward: workspace of %lld bytes required, got %lld", (long long)need,
                (long long)workspace_bytes);
  const int vp = static_cast<int>(N / up), vq = static_cast<int>(K / uq);
  const int blocks = static_cast<int>(ceil_div(static_cast<int64_t>(vp) * (vq / 8), kKronThreads));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
#define ANIMA_KRON(G, F)                                                                            \
  kron_backward_kernel<G, F><<<blocks, kKronThreads, 0, s>>>(                                       \
      static_cast<const G*>(dw), static_cast<const F*>(w1), static_cast<const F*>(w2), alpha, K, vp, \
      vq, (int)up, (int)uq, dw2, ws)
  if (dw_is_fp32) {
    if (factors_are_fp32) ANIMA_KRON(float, float); else ANIMA_KRON(float, __nv_bfloat16);
  } else {
    if (factors_are_fp32) ANIMA_KRON(__nv_bfloat16, float); else ANIMA_KRON(__nv_bfloat16, __nv_bfloat16);
  }
#undef ANIMA_KRON
  ANIMA_CHECK_LAUNCH("lokr_kron_backward");
  kron_backward_finalize_kernel<<<1, kFinalizeThreads, 0, s>>>(ws, blocks, alpha, (int)up, (int)uq, dw1);
  ANIMA_CHECK_LAUNCH("lokr_kron_backward finalize");
  return ANIMA_OK;
}
