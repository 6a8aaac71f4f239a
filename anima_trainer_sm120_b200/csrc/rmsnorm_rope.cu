// Per-head RMSNorm with optional rotary embedding, forward and backward, for the q / k
// projections of the attention layers (head width 128, bf16).
//
// In anima-trainer these two steps are third-party kernels (Liger RMSNorm, liger_patch.py:31-47, and
// Transformer Engine's fused RoPE, rope_patch.py:28-56); the stand-in DiT of this package would
// otherwise run them as ~10 eager elementwise launches per call. HBM-bound: 4 B/elem forward
// (+ 4 B per vector for rstd), 6 B/elem backward.
//   n   = x * rsqrt(mean(x^2) + eps) * w
//   out = n * cos + rotate_half(n) * sin   (cos / sin: fp32 tables [seq_len, 128], L2-resident)
//           rotate_half(n)[i] = -n[i+64] (i < 64), n[i-64] (i >= 64)
// The norm weight is treated as frozen (no weight gradient), which is the LoKr training setting.
#include "common.cuh"

namespace anima {
namespace {

constexpr int kHeadDim = 128;
constexpr int kThreads = 256;
constexpr int kLanesPerToken = 16;                       // 16 lanes x 8 elements = one 128-wide head vector
constexpr int kTokensPerCta = kThreads / kLanesPerToken;

// A half-warp owns one token and walks its heads: the token's cos / sin row is loaded once into
// registers and reused by every head, so the tables cost 1 KB per token instead of per vector.
// Lane l (0..15) holds elements 8l..8l+7; the rotate-half partner (64 away) is lane l ^ 8.
template <bool ROPE>
__global__ void __launch_bounds__(kThreads)
rmsnorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                        const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, float eps,
                        int64_t tokens, int heads, int64_t seq_len, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ rstd_out) {
  const int l = threadIdx.x & (kLanesPerToken - 1);
  const int64_t token = static_cast<int64_t>(blockIdx.x) * kTokensPerCta + threadIdx.x / kLanesPerToken;
  if (token >= tokens) return;   // whole half-warps leave together; shuffles below stay inside one half
  const unsigned half_mask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
  float wv[8], c[8], sn[8];
  *reinterpret_cast<float4*>(wv) = *reinterpret_cast<const float4*>(w + l * 8);
  *reinterpret_cast<float4*>(wv + 4) = *reinterpret_cast<const float4*>(w + l * 8 + 4);
  if (ROPE) {
    const int64_t pos = token % seq_len;
    const float sign = l < 8 ? -1.f : 1.f;
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cos_tab + pos * kHeadDim + l * 8);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cos_tab + pos * kHeadDim + l * 8 + 4);
    *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sin_tab + pos * kHeadDim + l * 8);
    *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sin_tab + pos * kHeadDim + l * 8 + 4);
#pragma unroll
    for (int k = 0; k < 8; ++k) sn[k] *= sign;
  }
  const __nv_bfloat16* xp = x + token * heads * kHeadDim + l * 8;
  __nv_bfloat16* op = out + token * heads * kHeadDim + l * 8;
#pragma unroll 4
  for (int h = 0; h < heads; ++h) {
    float v[8];
    unpack8(ldg_stream16(xp + h * kHeadDim), v);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
    float tot = ss;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) tot += __shfl_xor_sync(half_mask, tot, o);
    const float rstd = rsqrtf(tot / kHeadDim + eps);
    float o8[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float n = v[k] * rstd * wv[k];
      if (ROPE) {
        const float partner = __shfl_xor_sync(half_mask, n, 8);
        o8[k] = n * c[k] + partner * sn[k];
      } else {
        o8[k] = n;
      }
    }
    stg_stream16(op + h * kHeadDim, pack8(o8));
    if (l == 0) rstd_out[token * heads + h] = rstd;
  }
}

template <bool ROPE>
__global__ void __launch_bounds__(kThreads)
rmsnorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ x,
                        const float* __restrict__ w, const float* __restrict__ cos_tab,
                        const float* __restrict__ sin_tab, const float* __restrict__ rstd_in, int64_t tokens,
                        int heads, int64_t seq_len, __nv_bfloat16* __restrict__ dx) {
  const int l = threadIdx.x & (kLanesPerToken - 1);
  const int64_t token = static_cast<int64_t>(blockIdx.x) * kTokensPerCta + threadIdx.x / kLanesPerToken;
  if (token >= tokens) return;
  const unsigned half_mask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
  float wv[8], c[8], sn[8];
  *reinterpret_cast<float4*>(wv) = *reinterpret_cast<const float4*>(w + l * 8);
  *reinterpret_cast<float4*>(wv + 4) = *reinterpret_cast<const float4*>(w + l * 8 + 4);
  if (ROPE) {
    // out_i = n_i c_i + sign_i n_{p(i)} s_i  =>  dn_j = g_j c_j + sign_{p(j)} g_{p(j)} s_{p(j)}:
    // each lane sends g * (its own signed sin) to its partner.
    const int64_t pos = token % seq_len;
    const float sign = l < 8 ? -1.f : 1.f;
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cos_tab + pos * kHeadDim + l * 8);
    *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cos_tab + pos * kHeadDim + l * 8 + 4);
    *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sin_tab + pos * kHeadDim + l * 8);
    *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sin_tab + pos * kHeadDim + l * 8 + 4);
#pragma unroll
    for (int k = 0; k < 8; ++k) sn[k] *= sign;
  }
  const int64_t base = token * heads * kHeadDim + l * 8;
#pragma unroll 4
  for (int h = 0; h < heads; ++h) {
    float g[8], v[8], dn[8];
    unpack8(ldg_stream16(dout + base + h * kHeadDim), g);
    unpack8(ldg_stream16(x + base + h * kHeadDim), v);
    const float rstd = rstd_in[token * heads + h];
    // n = xhat * w with xhat = x * rstd:  dx = rstd * (gw - xhat * mean(gw * xhat)),  gw = dn * w
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (ROPE) {
        const float from_partner = __shfl_xor_sync(half_mask, g[k] * sn[k], 8);
        dn[k] = (g[k] * c[k] + from_partner) * wv[k];
      } else {
        dn[k] = g[k] * wv[k];
      }
      v[k] *= rstd;
      dot += dn[k] * v[k];
    }
    float tot = dot;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) tot += __shfl_xor_sync(half_mask, tot, o);
    const float m = tot / kHeadDim;
    float o8[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) o8[k] = rstd * (dn[k] - v[k] * m);
    stg_stream16(dx + base + h * kHeadDim, pack8(o8));
  }
}

int check(const char* who, int64_t tokens, int64_t heads, int64_t head_dim, int64_t seq_len, const void* cos_tab, const void* sin_tab) {
  ANIMA_REQUIRE(tokens >= 0 && heads > 0, ANIMA_E_ARG, "%s: bad sizes", who);
  ANIMA_REQUIRE(head_dim == kHeadDim, ANIMA_E_UNSUPPORTED, "%s: head_dim=%lld is not supported (only %d)", who,
                (long long)head_dim, kHeadDim);
  ANIMA_REQUIRE(heads < (1ll << 31) && tokens * heads < (1ll << 40), ANIMA_E_TOO_LARGE, "%s: too many vectors", who);
  ANIMA_REQUIRE((cos_tab == nullptr) == (sin_tab == nullptr), ANIMA_E_ARG, "%s: give both tables or neither", who);
  ANIMA_REQUIRE(!cos_tab || (seq_len > 0 && tokens % seq_len == 0), ANIMA_E_SHAPE,
                "%s: tokens=%lld is not a multiple of seq_len=%lld", who, (long long)tokens, (long long)seq_len);
  return ANIMA_OK;
}

}  // namespace
}  // namespace anima

using namespace anima;

extern "C" int anima_rmsnorm_rope_fwd(const void* x, const float* weight, const float* cos_tab, const float* sin_tab, float eps,
                                      int64_t tokens, int64_t heads, int64_t head_dim, int64_t seq_len,
                                      void* out, float* rstd, void* stream) {
  ANIMA_REQUIRE(x && weight && out && rstd, ANIMA_E_ARG, "rmsnorm_rope_fwd: null pointer");
  if (int rc = check("rmsnorm_rope_fwd", tokens, heads, head_dim, seq_len, cos_tab, sin_tab)) return rc;
  ANIMA_REQUIRE(aligned16(x) && aligned16(out) && aligned16(weight) && (!cos_tab || (aligned16(cos_tab) && aligned16(sin_tab))), ANIMA_E_ALIGN,
                "rmsnorm_rope_fwd: tensors must be 16-byte aligned");
  const int64_t vecs = tokens * heads;
  if (vecs == 0) return ANIMA_OK;
  const unsigned grid = static_cast<unsigned>(ceil_div(tokens, kTokensPerCta));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* op = static_cast<__nv_bfloat16*>(out);
  if (cos_tab)
    rmsnorm_rope_fwd_kernel<true><<<grid, kThreads, 0, s>>>(xp, weight, cos_tab, sin_tab, eps, tokens, (int)heads, seq_len, op, rstd);
  else
    rmsnorm_rope_fwd_kernel<false><<<grid, kThreads, 0, s>>>(xp, weight, nullptr, nullptr, eps, tokens, (int)heads, 1, op, rstd);
  ANIMA_CHECK_LAUNCH("rmsnorm_rope_fwd");
  return ANIMA_OK;
}

extern "C" int anima_rmsnorm_rope_bwd(const void* dout, const void* x, const float* weight, const float* cos_tab,
                                      const float* sin_tab, const float* rstd, int64_t tokens, int64_t heads, int64_t head_dim,
                                      int64_t seq_len, void* dx, void* stream) {
  ANIMA_REQUIRE(dout && x && weight && rstd && dx, ANIMA_E_ARG, "rmsnorm_rope_bwd: null pointer");
  if (int rc = check("rmsnorm_rope_bwd", tokens, heads, head_dim, seq_len, cos_tab, sin_tab)) return rc;
  ANIMA_REQUIRE(aligned16(dout) && aligned16(x) && aligned16(dx) && aligned16(weight) && (!cos_tab || (aligned16(cos_tab) && aligned16(sin_tab))),
                ANIMA_E_ALIGN, "rmsnorm_rope_bwd: tensors must be 16-byte aligned");
  const int64_t vecs = tokens * heads;
  if (vecs == 0) return ANIMA_OK;
  const unsigned grid = static_cast<unsigned>(ceil_div(tokens, kTokensPerCta));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* gp = static_cast<const __nv_bfloat16*>(dout);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* dp = static_cast<__nv_bfloat16*>(dx);
  if (cos_tab)
    rmsnorm_rope_bwd_kernel<true><<<grid, kThreads, 0, s>>>(gp, xp, weight, cos_tab, sin_tab, rstd, tokens, (int)heads, seq_len, dp);
  else
    rmsnorm_rope_bwd_kernel<false><<<grid, kThreads, 0, s>>>(gp, xp, weight, nullptr, nullptr, rstd, tokens, (int)heads, 1, dp);
  ANIMA_CHECK_LAUNCH("rmsnorm_rope_bwd");
  return ANIMA_OK;
}
