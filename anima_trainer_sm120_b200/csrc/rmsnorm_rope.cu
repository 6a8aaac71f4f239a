// Per-head RMSNorm with optional rotary embedding, forward and backward, for the q / k
// projections of the attention layers (head width 128, bf16).
//
// In anima-trainer these two steps are third-party kernels (Liger RMSNorm, liger_patch.py:31-47, and
// Transformer Engine's fused RoPE, rope_patch.py:28-56); the stand-in DiT of this package would
// otherwise run them as ~10 eager elementwise launches per call. One warp owns one (token, head)
// vector: lane l holds elements 4l..4l+3, so the rotate-half partner of an element (64 positions
// away) sits in lane l ^ 16 and is fetched with one shuffle. HBM-bound: 4 B/elem forward
// (+ 4 B per vector for rstd), 6 B/elem backward.
//   n   = x * rsqrt(mean(x^2) + eps) * w
//   out = n * cos + rotate_half(n) * sin   (cos / sin: fp32 tables [seq_len, 128], L2-resident)
//           rotate_half(n)[i] = -n[i+64] (i < 64), n[i-64] (i >= 64)
// The norm weight is treated as frozen (no weight gradient), which is the LoKr training setting.
#include "common.cuh"

namespace anima {
namespace {

constexpr int kHeadDim = 128;
constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ void unpack4(const uint2& raw, float (&f)[4]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint2 pack4(const float (&f)[4]) {
  uint2 raw;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
  p[0] = __floats2bfloat162_rn(f[0], f[1]);
  p[1] = __floats2bfloat162_rn(f[2], f[3]);
  return raw;
}

// vec = (token, head); token = vec / heads; position in the sequence = token % seq_len.
template <bool ROPE>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
rmsnorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                        const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, float eps, int64_t vecs, int heads, int64_t seq_len,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ rstd_out) {
  const int lane = threadIdx.x & 31;
  const int64_t vec = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (vec >= vecs) return;
  float v[4], wv[4];
  unpack4(*reinterpret_cast<const uint2*>(x + vec * kHeadDim + lane * 4), v);
  *reinterpret_cast<float4*>(wv) = *reinterpret_cast<const float4*>(w + lane * 4);
  const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
  const float rstd = rsqrtf(ss / kHeadDim + eps);
  float n[4], o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) n[k] = v[k] * rstd * wv[k];
  if (ROPE) {
    const int64_t pos = (vec / heads) % seq_len;
    float c[4], s[4];
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cos_tab + pos * kHeadDim + lane * 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(sin_tab + pos * kHeadDim + lane * 4);
    const float sign = lane < 16 ? -1.f : 1.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float partner = __shfl_xor_sync(0xffffffffu, n[k], 16);
      o[k] = n[k] * c[k] + sign * partner * s[k];
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = n[k];
  }
  *reinterpret_cast<uint2*>(out + vec * kHeadDim + lane * 4) = pack4(o);
  if (lane == 0) rstd_out[vec] = rstd;
}

template <bool ROPE>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
rmsnorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ x,
                        const float* __restrict__ w, const float* __restrict__ cos_tab,
                        const float* __restrict__ sin_tab, const float* __restrict__ rstd_in, int64_t vecs, int heads, int64_t seq_len,
                        __nv_bfloat16* __restrict__ dx) {
  const int lane = threadIdx.x & 31;
  const int64_t vec = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (vec >= vecs) return;
  float g[4], v[4], wv[4], dn[4];
  unpack4(*reinterpret_cast<const uint2*>(dout + vec * kHeadDim + lane * 4), g);
  unpack4(*reinterpret_cast<const uint2*>(x + vec * kHeadDim + lane * 4), v);
  *reinterpret_cast<float4*>(wv) = *reinterpret_cast<const float4*>(w + lane * 4);
  const float rstd = rstd_in[vec];
  if (ROPE) {
    // out_i = n_i c_i + sign_i n_{p(i)} s_i  =>  dn_j = g_j c_j + sign_{p(j)} g_{p(j)} s_{p(j)}
    const int64_t pos = (vec / heads) % seq_len;
    float c[4], s[4];
    *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cos_tab + pos * kHeadDim + lane * 4);
    *reinterpret_cast<float4*>(s) = *reinterpret_cast<const float4*>(sin_tab + pos * kHeadDim + lane * 4);
    const float partner_sign = lane < 16 ? 1.f : -1.f;  // the partner lane's own sign
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gs_partner = __shfl_xor_sync(0xffffffffu, g[k] * s[k], 16);
      dn[k] = g[k] * c[k] + partner_sign * gs_partner;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) dn[k] = g[k];
  }
  // n = xhat * w with xhat = x * rstd:  dx = rstd * (gw - xhat * mean(gw * xhat)),  gw = dn * w
  float dot = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    dn[k] *= wv[k];
    dot += dn[k] * v[k] * rstd;
  }
  const float m = warp_sum(dot) / kHeadDim;
  float o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) o[k] = rstd * (dn[k] - v[k] * rstd * m);
  *reinterpret_cast<uint2*>(dx + vec * kHeadDim + lane * 4) = pack4(o);
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
  const unsigned grid = static_cast<unsigned>(ceil_div(vecs, kWarpsPerCta));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* op = static_cast<__nv_bfloat16*>(out);
  if (cos_tab)
    rmsnorm_rope_fwd_kernel<true><<<grid, kWarpsPerCta * 32, 0, s>>>(xp, weight, cos_tab, sin_tab, eps, vecs, (int)heads, seq_len, op, rstd);
  else
    rmsnorm_rope_fwd_kernel<false><<<grid, kWarpsPerCta * 32, 0, s>>>(xp, weight, nullptr, nullptr, eps, vecs, (int)heads, 1, op, rstd);
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
  const unsigned grid = static_cast<unsigned>(ceil_div(vecs, kWarpsPerCta));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* gp = static_cast<const __nv_bfloat16*>(dout);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* dp = static_cast<__nv_bfloat16*>(dx);
  if (cos_tab)
    rmsnorm_rope_bwd_kernel<true><<<grid, kWarpsPerCta * 32, 0, s>>>(gp, xp, weight, cos_tab, sin_tab, rstd, vecs, (int)heads, seq_len, dp);
  else
    rmsnorm_rope_bwd_kernel<false><<<grid, kWarpsPerCta * 32, 0, s>>>(gp, xp, weight, nullptr, nullptr, rstd, vecs, (int)heads, 1, dp);
  ANIMA_CHECK_LAUNCH("rmsnorm_rope_bwd");
  return ANIMA_OK;
}
