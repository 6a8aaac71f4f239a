// Fused AdaLN (LayerNorm without affine, then *(1+scale)+shift) and the gated
// residual x + gate*y, forward and backward, for bf16 activations.
//
// Replaces anima-trainer's five Triton kernels in adaln_kernel.py:
//   _fwd_kernel (:34-68), _bwd_dx_kernel (:71-103), _bwd_dsdb_kernel (:106-154),
//   _gated_add_fwd_kernel (:272-295), _gated_add_bwd_dgate_kernel (:298-329).
// All four kernels here are HBM-bound; each tensor is read or written once with
// 16-byte streaming accesses:
//   adaln_fwd      4 B/elem (+ 8 B/row of saved statistics)
//   adaln_bwd      6 B/elem: dx AND the dscale/dshift partial sums come from one
//                  pass over dy and x (the reference makes two passes)
//   gated_add_fwd  6 B/elem
//   gated_add_bwd  6 B/elem: dy and the dgate partial sums from one pass
// The reductions over the hw rows of a sample are two-stage (per-block partials in
// caller-provided scratch, then a fixed-order sum), so results are bit-reproducible;
// the reference uses fp32 atomics.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "mx_quantize_tile.cuh"

namespace anima {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerIter = 4;

// ------------------------------------------------------------------ forward
// One warp per row; lane l owns the 16-byte chunks l, l+32, ... of the row. The row stays packed (bf16)
// in registers and is unpacked in each of the three passes (sum, centred squares, output): that keeps the
// kernel at ~50 registers, so 4 CTAs (32 warps, 128 KB of loads in flight) fit on an SM.
//
// GATED: the row normalised is x_new = x + gate * sub (the gated residual of the PREVIOUS sublayer, same
// arithmetic as gated_add_fwd_kernel: one fp32 fma, rounded once to bf16), which is also written out; the
// two kernels of "residual update, then modulation of the next sublayer" become one pass that reads x and sub
// and writes x_new and y (8 B/elem instead of 6 + 4).
//
// QUANT: the row-wise MXFP8 operand of y (e4m3 codes + one scale byte per 32 columns, the arithmetic of
// mx_quantize on the bf16-rounded y) leaves the same pass: the four lanes that hold 32 consecutive columns
// share their amax with two shuffles, and the scale bytes of 128 columns are gathered into one 32-bit store.
// The linears that consume y then need no quantiser launch of their own (+1.03 B/elem written here against
// 2 B read + 1.03 B written there); y itself may be left unwritten (y == nullptr).
struct RowCodes {
  uint8_t* codes;    // [rows, d]
  uint8_t* scales;   // plain [rows, d/32] or tiled (128 x 4 chunks)
  int tiled;
};

//
// STAGED (hw % 8 == 0: the 8 rows of a CTA belong to one sample; which forms use it is decided where the
// kernel is launched): the CTA converts the sample's modulation row
// once, (1 + scale) and shift as fp32 in shared memory, instead of every warp unpacking and adding them for
// its own row; the output pass then reads two 16-byte pieces per operand (split so that consecutive lanes read
// consecutive 16 bytes) and saves 3 of its ~7.5 instructions per element. Same arithmetic, same bits.
template <int NCH, bool GATED, bool QUANT, bool STAGED>
__global__ void __launch_bounds__(kThreads, NCH > 8 ? 2 : (NCH == 8 && STAGED && !GATED && !QUANT) ? 3 : 4)
adaln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                 const __nv_bfloat16* __restrict__ sub, const __nv_bfloat16* __restrict__ scale,
                 const __nv_bfloat16* __restrict__ shift, float eps, int64_t rows, int64_t hw,
                 int d, __nv_bfloat16* __restrict__ x_new, __nv_bfloat16* __restrict__ y,
                 float* __restrict__ mean_out, float* __restrict__ rstd_out, const RowCodes q) {
  extern __shared__ float4 mod_smem[];   // STAGED: [4][d / 8]: (1 + scale) low / high halves, shift low / high
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
  if (!STAGED && row >= rows) return;    // STAGED: rows % 8 == 0, every warp of every CTA has a row
  const int64_t bt = row / hw;
  const __nv_bfloat16* xr = x + row * d;

  uint4 raw[NCH];
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int col = (i * 32 + lane) * 8;
    raw[i] = make_uint4(0u, 0u, 0u, 0u);
    if (col < d) raw[i] = ldg_stream16(xr + col);
  }
  if (STAGED) {
    const int chunks = d >> 3;
    for (int ch = threadIdx.x; ch < chunks; ch += kThreads) {
      float s[8], b[8];
      unpack8(*reinterpret_cast<const uint4*>(scale + bt * d + ch * 8), s);
      unpack8(*reinterpret_cast<const uint4*>(shift + bt * d + ch * 8), b);
      mod_smem[ch] = make_float4(1.0f + s[0], 1.0f + s[1], 1.0f + s[2], 1.0f + s[3]);
      mod_smem[chunks + ch] = make_float4(1.0f + s[4], 1.0f + s[5], 1.0f + s[6], 1.0f + s[7]);
      mod_smem[2 * chunks + ch] = make_float4(b[0], b[1], b[2], b[3]);
      mod_smem[3 * chunks + ch] = make_float4(b[4], b[5], b[6], b[7]);
    }
    __syncthreads();   // far ahead of the first read: two reductions over the row come first
  }
  if (GATED) {
    // the sublayer output is fetched one chunk ahead of its use (the row of x already fills half the registers)
    uint4 sub_next = make_uint4(0u, 0u, 0u, 0u);
    if (lane * 8 < d) sub_next = ldg_stream16(sub + row * d + lane * 8);
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int col = (i * 32 + lane) * 8;
      const uint4 sub_cur = sub_next;
      if (i + 1 < NCH && col + 256 < d) sub_next = ldg_stream16(sub + row * d + col + 256);
      if (col < d) {
        float xf[8], yf[8], gf[8], o[8];
        unpack8(raw[i], xf);
        unpack8(sub_cur, yf);
        unpack8(*reinterpret_cast<const uint4*>(gate + bt * d + col), gf);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = xf[e] + gf[e] * yf[e];
        raw[i] = pack8(o);
        stg_stream16(x_new + row * d + col, raw[i]);   // the normalisation below sees the rounded values
      }
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    float v[8];
    unpack8(raw[i], v);
#pragma unroll
    for (int k = 0; k < 8; ++k) sum += v[k];
  }
  const float mean = warp_sum(sum) / static_cast<float>(d);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    if ((i * 32 + lane) * 8 < d) {  // padded tail must not add mean^2 (adaln_kernel.py:55-57)
      float v[8];
      unpack8(raw[i], v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float c = v[k] - mean;
        sq += c * c;
      }
    }
  }
  const float var = warp_sum(sq) / static_cast<float>(d);
  const float rstd = 1.0f / sqrtf(var + eps);
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int col = (i * 32 + lane) * 8;
    const bool ok = col < d;
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (ok) {
      float v[8], o[8];
      unpack8(raw[i], v);
      if (STAGED) {
        const int chunks = d >> 3, ch = i * 32 + lane;
        const float4 s0 = mod_smem[ch], s1 = mod_smem[chunks + ch];
        const float4 b0 = mod_smem[2 * chunks + ch], b1 = mod_smem[3 * chunks + ch];
        const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (v[k] - mean) * rstd * s[k] + b[k];
      } else {
        float s[8], b[8];
        unpack8(*reinterpret_cast<const uint4*>(scale + bt * d + col), s);
        unpack8(*reinterpret_cast<const uint4*>(shift + bt * d + col), b);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (v[k] - mean) * rstd * (1.0f + s[k]) + b[k];
      }
      out = pack8(o);
      if (!QUANT || y != nullptr) stg_stream16(y + row * d + col, out);
    }
    if (QUANT) {   // reached by all 32 lanes (d % 32 == 0: the four lanes of a block are in or out together)
      float f[8];
      unpack8(out, f);
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[k]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const int e = mxq::mx_exponent(fmaxf(amax, mxq::kAmaxFloor));
      const float inv = mxq::mx_inv_scale(e);
      uint2 codes;
      codes.x = mxq::e4m3x2(f[0] * inv, f[1] * inv) | (mxq::e4m3x2(f[2] * inv, f[3] * inv) << 16);
      codes.y = mxq::e4m3x2(f[4] * inv, f[5] * inv) | (mxq::e4m3x2(f[6] * inv, f[7] * inv) << 16);
      if (ok) *reinterpret_cast<uint2*>(q.codes + row * d + col) = codes;
      // scale bytes of blocks 8i + lane/4; lanes 0 and 16 collect the four bytes of their 128 columns
      uint32_t sb = ok ? static_cast<uint32_t>(e + 127) : 0u;
      sb |= __shfl_down_sync(0xffffffffu, sb, 4) << 8;
      sb |= __shfl_down_sync(0xffffffffu, sb, 8) << 16;
      if ((lane & 15) == 0 && ok) {
        const int64_t kb4 = d / 128;   // d % 128 == 0 (checked by the host)
        const int64_t c4 = i * 2 + (lane >> 4);
        uint8_t* dst = q.tiled ? q.scales + ((row >> 7) * kb4 + c4) * 512 + mxq::tiled_offset(static_cast<int>(row & 127), 0)
                               : q.scales + (row * kb4 + c4) * 4;
        *reinterpret_cast<uint32_t*>(dst) = sb;
      }
    }
  }
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
}

// ------------------------------------------------------------------ backward
// Work split shared by adaln_bwd and gated_add_bwd: the hw rows of every sample
// are cut into `chunks` contiguous pieces, one CTA each; thread t owns the
// 16-byte column chunks t, t+256, ... and carries their partial sums in registers.
struct RowSplit {
  int chunks;          // CTAs per sample
  int rows_per_chunk;  // multiple of kRowsPerIter
};

RowSplit make_split(int64_t bt, int64_t hw) {
  const int64_t target = 2LL * sm_count();  // two resident CTAs per SM
  int64_t chunks = std::max<int64_t>(1, ceil_div(target, std::max<int64_t>(bt, 1)));
  int64_t rpc = ceil_div(ceil_div(hw, chunks), kRowsPerIter) * kRowsPerIter;
  chunks = ceil_div(hw, rpc);
  return {static_cast<int>(chunks), static_cast<int>(rpc)};
}

// GATED: x is the x_new = x_prev + gate * sub written by the one-pass forward. The gradient that reaches
// x_new is d_res (through the residual stream) plus the LayerNorm gradient computed here; instead of writing
// the latter, adding the two with a separate kernel and reading the sum back for the gated-residual backward,
// the same thread forms dout = d_res + bf16(dx_ln), writes it (it is also the gradient of x_prev), and
// continues with dsub = gate * dout and the dgate partial sums. Every rounding point is that of the three
// separate kernels, so all outputs are bit-identical to them.
// PF (NCH == 1 only): the next group of rows is copied global -> shared with cp.async while the current one is
// worked on, each thread fetching exactly the 16-byte chunks it will read itself, so no barrier is involved
// and no register is spent on the prefetch. Without it the kernel alternates between waiting for its loads and
// computing at 16 resident warps: DRAM half busy, 2.6 long-scoreboard stalls per issue.
// Shared layout: [stage 2][tensor (dy, x[, d_res])][row R][thread] x 16 bytes.
__device__ __forceinline__ uint32_t smem_u32_of(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds16(uint32_t smem_addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_addr));
  return v;
}
constexpr int adaln_bwd_prefetch_bytes(bool gated) { return 2 * (gated ? 3 : 2) * kRowsPerIter * kThreads * 16; }

template <int NCH, bool GATED, bool PF = false>
__global__ void __launch_bounds__(kThreads, NCH == 1 ? 2 : 1)
adaln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                 const __nv_bfloat16* __restrict__ scale, const float* __restrict__ mean,
                 const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ d_res,
                 const __nv_bfloat16* __restrict__ sub, const __nv_bfloat16* __restrict__ gate, int64_t hw, int d,
                 int rows_per_chunk, __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dsub,
                 float* __restrict__ partial) {
  constexpr int R = kRowsPerIter;
  constexpr int NOUT = GATED ? 3 : 2;
  __shared__ float red[2][kThreads / 32][2 * R];

  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int64_t bt = blockIdx.y;
  const int64_t row_begin = bt * hw + static_cast<int64_t>(blockIdx.x) * rows_per_chunk;
  const int64_t row_end = min(bt * hw + hw, row_begin + rows_per_chunk);
  const float inv_d = 1.0f / static_cast<float>(d);

  float one_plus_s[NCH][8], ds[NCH][8], db[NCH][8];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int col = (j * kThreads + t) * 8;
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col < d) unpack8(*reinterpret_cast<const uint4*>(scale + bt * d + col), s);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      one_plus_s[j][k] = 1.0f + s[k];
      ds[j][k] = 0.f;
      db[j][k] = 0.f;
    }
  }
  float gt[GATED ? NCH : 1][8], dg[GATED ? NCH : 1][8];
  if (GATED) {
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int col = (j * kThreads + t) * 8;
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (col < d) unpack8(*reinterpret_cast<const uint4*>(gate + bt * d + col), s);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        gt[j][k] = s[k];
        dg[j][k] = 0.f;
      }
    }
  }

  static_assert(!PF || NCH == 1, "the prefetch form covers one 16-byte chunk per thread and row");
  extern __shared__ uint4 pf_smem[];
  constexpr int kPfTensors = GATED ? 3 : 2;
  const uint32_t pf_base = PF ? smem_u32_of(pf_smem) + t * 16 : 0;
  auto pf_addr = [&](int stage, int tensor, int k) {
    return pf_base + static_cast<uint32_t>(((stage * kPfTensors + tensor) * R + k) * kThreads * 16);
  };
  auto prefetch = [&](int64_t r0n, int stage) {   // this thread's chunks of rows r0n .. r0n + R - 1
    const int col = t * 8;
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int64_t row = r0n + k;
      if (row < row_end && col < d) {
        cp_async16(pf_addr(stage, 0, k), dy + row * d + col);
        cp_async16(pf_addr(stage, 1, k), x + row * d + col);
        if (GATED) cp_async16(pf_addr(stage, 2, k), d_res + row * d + col);
      }
    }
    cp_async_commit();
  };
  if (PF && row_begin < row_end) prefetch(row_begin, 0);

  int buf = 0;
  for (int64_t r0 = row_begin; r0 < row_end; r0 += R) {
    float g[R][NCH][8], xh[R][NCH][8];  // dy then dxhat; x then xhat
    uint4 res_raw[GATED ? R : 1][NCH];
    float mu[R], rs[R];
    if (PF) {
      // start the next group, then wait for this one (a stage is rewritten only after its values were used)
      if (r0 + R < row_end) {
        prefetch(r0 + R, buf ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int64_t row = r0 + k;
      const bool row_ok = row < row_end;
      mu[k] = row_ok ? mean[row] : 0.f;
      rs[k] = row_ok ? rstd[row] : 0.f;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int col = (j * kThreads + t) * 8;
        uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
        if (row_ok && col < d) {
          a = PF ? lds16(pf_addr(buf, 0, k)) : ldg_stream16(dy + row * d + col);
          b = PF ? lds16(pf_addr(buf, 1, k)) : ldg_stream16(x + row * d + col);
        }
        if (GATED) {
          res_raw[k][j] = make_uint4(0u, 0u, 0u, 0u);
          if (row_ok && col < d) res_raw[k][j] = PF ? lds16(pf_addr(buf, 2, k)) : ldg_stream16(d_res + row * d + col);
        }
        unpack8(a, g[k][j]);
        unpack8(b, xh[k][j]);
      }
    }
    float part[2 * R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      float p1 = 0.f, p2 = 0.f;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const bool ok = (j * kThreads + t) * 8 < d;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xhat = ok ? (xh[k][j][e] - mu[k]) * rs[k] : 0.f;
          const float dyv = g[k][j][e];
          ds[j][e] += dyv * xhat;
          db[j][e] += dyv;
          const float dxhat = dyv * one_plus_s[j][e];
          xh[k][j][e] = xhat;
          g[k][j][e] = dxhat;
          p1 += dxhat;
          p2 += dxhat * xhat;
        }
      }
      part[2 * k] = warp_sum(p1);
      part[2 * k + 1] = warp_sum(p2);
    }
    if (lane == 0) {
#pragma unroll
      for (int q = 0; q < 2 * R; ++q) red[buf][warp][q] = part[q];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < R; ++k) {
      float c1 = 0.f, c2 = 0.f;
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) {
        c1 += red[buf][w][2 * k];
        c2 += red[buf][w][2 * k + 1];
      }
      c1 *= inv_d;
      c2 *= inv_d;
      const int64_t row = r0 + k;
      if (row < row_end) {
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          const int col = (j * kThreads + t) * 8;
          if (col < d) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = rs[k] * (g[k][j][e] - c1 - xh[k][j][e] * c2);
            if (!GATED) {
              stg_stream16(dx + row * d + col, pack8(o));
            } else {
              float ln[8], rf[8], df[8], yf[8];
              const uint4 sub_raw = ldg_stream16(sub + row * d + col);   // read late: registers are scarce here
              unpack8(pack8(o), ln);                     // the LayerNorm gradient as its own kernel would store it
              unpack8(res_raw[k][j], rf);
#pragma unroll
              for (int e = 0; e < 8; ++e) df[e] = rf[e] + ln[e];
              const uint4 dout = pack8(df);              // bf16 sum, as the separate add would store it
              stg_stream16(dx + row * d + col, dout);
              unpack8(dout, df);
              unpack8(sub_raw, yf);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                dg[j][e] += df[e] * yf[e];
                o[e] = gt[j][e] * df[e];
              }
              stg_stream16(dsub + row * d + col, pack8(o));
            }
          }
        }
      }
    }
    buf ^= 1;
  }

  // partial[bt][chunk][0] = dscale sums, [1] = dshift sums, ([2] = dgate sums); fp32 [d] each.
  float* out = partial + ((bt * gridDim.x + blockIdx.x) * NOUT) * static_cast<int64_t>(d);
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int col = (j * kThreads + t) * 8;
    if (col < d) {
      *reinterpret_cast<float4*>(out + col) = make_float4(ds[j][0], ds[j][1], ds[j][2], ds[j][3]);
      *reinterpret_cast<float4*>(out + col + 4) = make_float4(ds[j][4], ds[j][5], ds[j][6], ds[j][7]);
      *reinterpret_cast<float4*>(out + d + col) = make_float4(db[j][0], db[j][1], db[j][2], db[j][3]);
      *reinterpret_cast<float4*>(out + d + col + 4) = make_float4(db[j][4], db[j][5], db[j][6], db[j][7]);
      if (GATED) {
        *reinterpret_cast<float4*>(out + 2 * d + col) = make_float4(dg[j][0], dg[j][1], dg[j][2], dg[j][3]);
        *reinterpret_cast<float4*>(out + 2 * d + col + 4) = make_float4(dg[j][4], dg[j][5], dg[j][6], dg[j][7]);
      }
    }
  }
}

// out_k[bt][c] = bf16( sum over chunks (ascending) of partial[bt][chunk][k][c] ), k < nout.
__global__ void finalize_partials_kernel(const float* __restrict__ partial, int64_t bt_count, int chunks,
                                         int nout, int d, __nv_bfloat16* __restrict__ out0,
                                         __nv_bfloat16* __restrict__ out1, __nv_bfloat16* __restrict__ out2 = nullptr) {
  const int64_t total = bt_count * nout * d;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % d);
    const int k = static_cast<int>((i / d) % nout);
    const int64_t bt = i / (static_cast<int64_t>(d) * nout);
    float acc = 0.f;
    for (int ch = 0; ch < chunks; ++ch)
      acc += partial[((bt * chunks + ch) * nout + k) * static_cast<int64_t>(d) + c];
    (k == 0 ? out0 : k == 1 ? out1 : out2)[bt * d + c] = __float2bfloat16_rn(acc);
  }
}

// ------------------------------------------------------------------ gated residual
__global__ void __launch_bounds__(kThreads)
gated_add_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                     const __nv_bfloat16* __restrict__ y, int64_t rows, int64_t hw, int d8,
                     __nv_bfloat16* __restrict__ out) {
  constexpr int U = 4;
  const int64_t total = rows * d8;  // 16-byte chunks
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t base = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; base < total;
       base += stride * U) {
    uint4 xa[U], ya[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + u * stride;
      if (i < total) {
        xa[u] = ldg_stream16(x + i * 8);
        ya[u] = ldg_stream16(y + i * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + u * stride;
      if (i < total) {
        const int64_t row = i / d8;
        const int c8 = static_cast<int>(i - row * d8);
        float xf[8], yf[8], gf[8], o[8];
        unpack8(xa[u], xf);
        unpack8(ya[u], yf);
        unpack8(*reinterpret_cast<const uint4*>(gate + (row / hw) * (d8 * 8LL) + c8 * 8), gf);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = xf[e] + gf[e] * yf[e];
        stg_stream16(out + i * 8, pack8(o));
      }
    }
  }
}

template <int NCH>
__global__ void __launch_bounds__(kThreads)
gated_add_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                     const __nv_bfloat16* __restrict__ gate, int64_t hw, int d, int rows_per_chunk,
                     __nv_bfloat16* __restrict__ dy, float* __restrict__ partial) {
  constexpr int R = kRowsPerIter;
  const int t = threadIdx.x;
  const int64_t bt = blockIdx.y;
  const int64_t row_begin = bt * hw + static_cast<int64_t>(blockIdx.x) * rows_per_chunk;
  const int64_t row_end = min(bt * hw + hw, row_begin + rows_per_chunk);

  float gt[NCH][8], dg[NCH][8];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int col = (j * kThreads + t) * 8;
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col < d) unpack8(*reinterpret_cast<const uint4*>(gate + bt * d + col), s);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      gt[j][k] = s[k];
      dg[j][k] = 0.f;
    }
  }
  for (int64_t r0 = row_begin; r0 < row_end; r0 += R) {
    uint4 a[R][NCH], b[R][NCH];
#pragma unroll
    for (int k = 0; k < R; ++k)
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int col = (j * kThreads + t) * 8;
        a[k][j] = make_uint4(0u, 0u, 0u, 0u);
        b[k][j] = a[k][j];
        if (r0 + k < row_end && col < d) {
          a[k][j] = ldg_stream16(dout + (r0 + k) * d + col);
          b[k][j] = ldg_stream16(y + (r0 + k) * d + col);
        }
      }
#pragma unroll
    for (int k = 0; k < R; ++k)
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int col = (j * kThreads + t) * 8;
        float df[8], yf[8], o[8];
        unpack8(a[k][j], df);
        unpack8(b[k][j], yf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dg[j][e] += df[e] * yf[e];
          o[e] = gt[j][e] * df[e];
        }
        if (r0 + k < row_end && col < d) stg_stream16(dy + (r0 + k) * d + col, pack8(o));
      }
  }
  float* out = partial + (bt * gridDim.x + blockIdx.x) * static_cast<int64_t>(d);
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int col = (j * kThreads + t) * 8;
    if (col < d) {
      *reinterpret_cast<float4*>(out + col) = make_float4(dg[j][0], dg[j][1], dg[j][2], dg[j][3]);
      *reinterpret_cast<float4*>(out + col + 4) = make_float4(dg[j][4], dg[j][5], dg[j][6], dg[j][7]);
    }
  }
}

int check_rows(const char* who, int64_t rows, int64_t hw, int64_t d, int64_t max_d) {
  ANIMA_REQUIRE(rows >= 0 && hw > 0 && d > 0, ANIMA_E_ARG, "%s: bad sizes rows=%lld hw=%lld d=%lld", who,
                (long long)rows, (long long)hw, (long long)d);
  ANIMA_REQUIRE(rows % hw == 0, ANIMA_E_SHAPE, "%s: rows=%lld is not a multiple of hw=%lld", who,
                (long long)rows, (long long)hw);
  ANIMA_REQUIRE(d % 8 == 0, ANIMA_E_SHAPE, "%s: d=%lld must be a multiple of 8", who, (long long)d);
  ANIMA_REQUIRE(d <= max_d, ANIMA_E_TOO_LARGE, "%s: d=%lld exceeds the supported maximum %lld", who,
                (long long)d, (long long)max_d);
  return ANIMA_OK;
}

}  // namespace
}  // namespace anima

using namespace anima;

namespace {

// ANIMA_ADALN_FWD_STAGING=0 keeps the modulation in global memory (read per call; for tests and comparison).
bool adaln_fwd_staging_enabled() {
  const char* v = getenv("ANIMA_ADALN_FWD_STAGING");
  return !(v && v[0] == '0');
}

// One launcher for the four forward forms; the kernel is picked by the row length (256 columns per chunk).
template <bool GATED, bool QUANT>
void launch_adaln_fwd(const void* x, const void* gate, const void* sub, const void* scale, const void* shift, float eps,
                      int64_t rows, int64_t hw, int64_t d, void* x_new, void* y, float* mean, float* rstd,
                      const RowCodes& q, void* stream) {
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  const auto* gp = static_cast<const __nv_bfloat16*>(gate);
  const auto* up = static_cast<const __nv_bfloat16*>(sub);
  const auto* sp = static_cast<const __nv_bfloat16*>(scale);
  const auto* bp = static_cast<const __nv_bfloat16*>(shift);
  auto* xn = static_cast<__nv_bfloat16*>(x_new);
  auto* yp = static_cast<__nv_bfloat16*>(y);
  const unsigned grid = static_cast<unsigned>(ceil_div(rows, kThreads / 32));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int di = static_cast<int>(d);
  // one sample per CTA (8 rows) lets the CTA convert the modulation row once; 8 * d bytes of shared memory
  // Measured at [8, 4096, 2048], 4 CTAs/SM (64 registers): the residual form gains from the staging (119.8 ->
  // 107.5 us, with the operand 137.7 -> 129.5); the plain form spills 168 bytes with it and loses (65.0 -> 85.5).
  // At 3 CTAs/SM (80 registers, no spills) the staged plain form is the fastest of all (58.9 us) while every
  // other form is slower than at 4 (plain + operand 90.1 against 86.5 unstaged, residual 116.7, residual +
  // operand 141.8). Hence: residual forms staged at 4 CTAs/SM, plain form staged at 3, plain + operand unstaged.
  const bool staged = (GATED || !QUANT) && hw % (kThreads / 32) == 0 && adaln_fwd_staging_enabled();
  const size_t smem = staged ? static_cast<size_t>(d) * 8 : 0;
#define ANIMA_LAUNCH_FWD(N)                                                                                      \
  do {                                                                                                           \
    bool launched = false;                                                                                       \
    if constexpr (GATED || (!QUANT && N <= 8)) { /* the plain form of a row longer than 2048 spills when staged */ \
      if (staged) {                                                                                              \
        adaln_fwd_kernel<N, GATED, QUANT, true><<<grid, kThreads, smem, s>>>(xp, gp, up, sp, bp, eps, rows, hw,  \
                                                                             di, xn, yp, mean, rstd, q);         \
        launched = true;                                                                                         \
      }                                                                                                          \
    }                                                                                                            \
    if (!launched)                                                                                               \
      adaln_fwd_kernel<N, GATED, QUANT, false><<<grid, kThreads, 0, s>>>(xp, gp, up, sp, bp, eps, rows, hw, di,  \
                                                                         xn, yp, mean, rstd, q);                 \
  } while (0)
  if (d <= 256) ANIMA_LAUNCH_FWD(1);
  else if (d <= 512) ANIMA_LAUNCH_FWD(2);
  else if (d <= 1024) ANIMA_LAUNCH_FWD(4);
  else if (d <= 2048) ANIMA_LAUNCH_FWD(8);
  else ANIMA_LAUNCH_FWD(16);
#undef ANIMA_LAUNCH_FWD
}

int check_row_codes(const char* who, int64_t rows, int64_t d, const uint8_t* codes_row, const uint8_t* scales_row,
                    int scale_layout) {
  ANIMA_REQUIRE(codes_row && scales_row, ANIMA_E_ARG, "%s: null code or scale buffer", who);
  ANIMA_REQUIRE(scale_layout == ANIMA_SCALES_PLAIN || scale_layout == ANIMA_SCALES_TILED, ANIMA_E_ARG,
                "%s: bad scale_layout %d", who, scale_layout);
  ANIMA_REQUIRE(d % 128 == 0, ANIMA_E_SHAPE, "%s: d=%lld must be a multiple of 128", who, (long long)d);
  ANIMA_REQUIRE(scale_layout == ANIMA_SCALES_PLAIN || rows % 128 == 0, ANIMA_E_SHAPE,
                "%s: tiled scales need rows %% 128 == 0 (rows=%lld)", who, (long long)rows);
  ANIMA_REQUIRE((reinterpret_cast<uintptr_t>(codes_row) & 7) == 0 && (reinterpret_cast<uintptr_t>(scales_row) & 3) == 0,
                ANIMA_E_ALIGN, "%s: codes must be 8-byte and scales 4-byte aligned", who);
  return ANIMA_OK;
}

}  // namespace

extern "C" int anima_adaln_fwd(const void* x, const void* scale, const void* shift, float eps,
                               int64_t rows, int64_t hw, int64_t d, void* y, float* mean, float* rstd,
                               void* stream) {
  ANIMA_REQUIRE(x && scale && shift && y && mean && rstd, ANIMA_E_ARG, "adaln_fwd: null pointer");
  if (int rc = check_rows("adaln_fwd", rows, hw, d, 4096)) return rc;
  ANIMA_REQUIRE(aligned16(x) && aligned16(scale) && aligned16(shift) && aligned16(y), ANIMA_E_ALIGN,
                "adaln_fwd: tensors must be 16-byte aligned");
  if (rows == 0) return ANIMA_OK;
  launch_adaln_fwd<false, false>(x, nullptr, nullptr, scale, shift, eps, rows, hw, d, nullptr, y, mean, rstd,
                                 RowCodes{}, stream);
  ANIMA_CHECK_LAUNCH("adaln_fwd");
  return ANIMA_OK;
}

extern "C" int anima_adaln_fwd_quant(const void* x, const void* scale, const void* shift, float eps, int64_t rows,
                                     int64_t hw, int64_t d, void* y, float* mean, float* rstd, uint8_t* codes_row,
                                     uint8_t* scales_row, int scale_layout, void* stream) {
  ANIMA_REQUIRE(x && scale && shift && mean && rstd, ANIMA_E_ARG, "adaln_fwd_quant: null pointer");
  if (int rc = check_rows("adaln_fwd_quant", rows, hw, d, 4096)) return rc;
  if (int rc = check_row_codes("adaln_fwd_quant", rows, d, codes_row, scales_row, scale_layout)) return rc;
  ANIMA_REQUIRE(aligned16(x) && aligned16(scale) && aligned16(shift) && aligned16(y), ANIMA_E_ALIGN,
                "adaln_fwd_quant: tensors must be 16-byte aligned");
  if (rows == 0) return ANIMA_OK;
  launch_adaln_fwd<false, true>(x, nullptr, nullptr, scale, shift, eps, rows, hw, d, nullptr, y, mean, rstd,
                                RowCodes{codes_row, scales_row, scale_layout == ANIMA_SCALES_TILED}, stream);
  ANIMA_CHECK_LAUNCH("adaln_fwd_quant");
  return ANIMA_OK;
}

extern "C" int anima_gated_add_adaln_fwd(const void* x, const void* gate, const void* sub, const void* scale,
                                         const void* shift, float eps, int64_t rows, int64_t hw, int64_t d,
                                         void* x_new, void* y, float* mean, float* rstd, void* stream) {
  ANIMA_REQUIRE(x && gate && sub && scale && shift && x_new && y && mean && rstd, ANIMA_E_ARG,
                "gated_add_adaln_fwd: null pointer");
  if (int rc = check_rows("gated_add_adaln_fwd", rows, hw, d, 4096)) return rc;
  ANIMA_REQUIRE(aligned16(x) && aligned16(gate) && aligned16(sub) && aligned16(scale) && aligned16(shift) &&
                    aligned16(x_new) && aligned16(y),
                ANIMA_E_ALIGN, "gated_add_adaln_fwd: tensors must be 16-byte aligned");
  if (rows == 0) return ANIMA_OK;
  launch_adaln_fwd<true, false>(x, gate, sub, scale, shift, eps, rows, hw, d, x_new, y, mean, rstd, RowCodes{}, stream);
  ANIMA_CHECK_LAUNCH("gated_add_adaln_fwd");
  return ANIMA_OK;
}

extern "C" int anima_gated_add_adaln_fwd_quant(const void* x, const void* gate, const void* sub, const void* scale,
                                               const void* shift, float eps, int64_t rows, int64_t hw, int64_t d,
                                               void* x_new, void* y, float* mean, float* rstd, uint8_t* codes_row,
                                               uint8_t* scales_row, int scale_layout, void* stream) {
  ANIMA_REQUIRE(x && gate && sub && scale && shift && x_new && mean && rstd, ANIMA_E_ARG,
                "gated_add_adaln_fwd_quant: null pointer");
  if (int rc = check_rows("gated_add_adaln_fwd_quant", rows, hw, d, 4096)) return rc;
  if (int rc = check_row_codes("gated_add_adaln_fwd_quant", rows, d, codes_row, scales_row, scale_layout)) return rc;
  ANIMA_REQUIRE(aligned16(x) && aligned16(gate) && aligned16(sub) && aligned16(scale) && aligned16(shift) &&
                    aligned16(x_new) && aligned16(y),
                ANIMA_E_ALIGN, "gated_add_adaln_fwd_quant: tensors must be 16-byte aligned");
  if (rows == 0) return ANIMA_OK;
  launch_adaln_fwd<true, true>(x, gate, sub, scale, shift, eps, rows, hw, d, x_new, y, mean, rstd,
                               RowCodes{codes_row, scales_row, scale_layout == ANIMA_SCALES_TILED}, stream);
  ANIMA_CHECK_LAUNCH("gated_add_adaln_fwd_quant");
  return ANIMA_OK;
}

namespace anima {
namespace {
// Launch of the AdaLN backward main kernel: the prefetching form for d <= 2048 (ANIMA_ADALN_BWD_PREFETCH=0 keeps
// the plain loads, for comparison; same bits), the two-chunk form above that.
template <bool GATED>
int launch_adaln_bwd_main(dim3 grid, cudaStream_t s, const __nv_bfloat16* dy, const __nv_bfloat16* x,
                          const __nv_bfloat16* scale, const float* mean, const float* rstd, const __nv_bfloat16* d_res,
                          const __nv_bfloat16* sub, const __nv_bfloat16* gate, int64_t hw, int64_t d, int rows_per_chunk,
                          __nv_bfloat16* dx, __nv_bfloat16* dsub, float* ws) {
  if (d > 2048) {
    adaln_bwd_kernel<2, GATED><<<grid, kThreads, 0, s>>>(dy, x, scale, mean, rstd, d_res, sub, gate, hw, (int)d,
                                                         rows_per_chunk, dx, dsub, ws);
    return ANIMA_OK;
  }
  const char* env = getenv("ANIMA_ADALN_BWD_PREFETCH");
  if (env && env[0] == '0') {
    adaln_bwd_kernel<1, GATED><<<grid, kThreads, 0, s>>>(dy, x, scale, mean, rstd, d_res, sub, gate, hw, (int)d,
                                                         rows_per_chunk, dx, dsub, ws);
    return ANIMA_OK;
  }
  constexpr int kBytes = adaln_bwd_prefetch_bytes(GATED);
  static PerDeviceOnce once;
  const cudaError_t rc = per_device_once(once, [] {
    return cudaFuncSetAttribute(adaln_bwd_kernel<1, GATED, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
  });
  ANIMA_REQUIRE(rc == cudaSuccess, ANIMA_E_CUDA, "adaln_bwd: cannot reserve %d bytes of shared memory: %s", kBytes,
                cudaGetErrorString(rc));
  adaln_bwd_kernel<1, GATED, true><<<grid, kThreads, kBytes, s>>>(dy, x, scale, mean, rstd, d_res, sub, gate, hw, (int)d,
                                                                  rows_per_chunk, dx, dsub, ws);
  return ANIMA_OK;
}
}  // namespace
}  // namespace anima

extern "C" int64_t anima_adaln_bwd_workspace_bytes(int64_t rows, int64_t hw, int64_t d) {
  if (rows < 0 || hw <= 0 || d <= 0 || rows % hw) return ANIMA_E_SHAPE;
  const RowSplit sp = make_split(rows / hw, hw);
  return (rows / hw) * sp.chunks * 2 * d * static_cast<int64_t>(sizeof(float));
}

extern "C" int anima_adaln_bwd(const void* dy, const void* x, const void* scale, const float* mean,
                               const float* rstd, int64_t rows, int64_t hw, int64_t d, void* dx,
                               void* dscale, void* dshift, void* workspace, int64_t workspace_bytes,
                               void* stream) {
  ANIMA_REQUIRE(dy && x && scale && mean && rstd && dx && dscale && dshift, ANIMA_E_ARG,
                "adaln_bwd: null pointer");
  if (int rc = check_rows("adaln_bwd", rows, hw, d, 4096)) return rc;
  ANIMA_REQUIRE(aligned16(dy) && aligned16(x) && aligned16(scale) && aligned16(dx), ANIMA_E_ALIGN,
                "adaln_bwd: tensors must be 16-byte aligned");
  if (rows == 0) return ANIMA_OK;
  const int64_t need = anima_adaln_bwd_workspace_bytes(rows, hw, d);
  ANIMA_REQUIRE(workspace && aligned16(workspace) && workspace_bytes >= need, ANIMA_E_WORKSPACE,
                "adaln_bwd: workspace of %lld bytes (16-byte aligned) required, got %lld", (long long)need,
                (long long)workspace_bytes);
  const int64_t bt = rows / hw;
  ANIMA_REQUIRE(bt <= 65535, ANIMA_E_TOO_LARGE, "adaln_bwd: rows/hw=%lld exceeds 65535", (long long)bt);
  const RowSplit sp = make_split(bt, hw);
  const dim3 grid(sp.chunks, static_cast<unsigned>(bt));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  const auto* dyp = static_cast<const __nv_bfloat16*>(dy);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  const auto* scp = static_cast<const __nv_bfloat16*>(scale);
  auto* dxp = static_cast<__nv_bfloat16*>(dx);
  if (int rc = launch_adaln_bwd_main<false>(grid, s, dyp, xp, scp, mean, rstd, nullptr, nullptr, nullptr, hw, d,
                                            sp.rows_per_chunk, dxp, nullptr, ws))
    return rc;
  ANIMA_CHECK_LAUNCH("adaln_bwd");
  const int64_t total = bt * 2 * d;
  finalize_partials_kernel<<<static_cast<unsigned>(std::min<int64_t>(ceil_div(total, 256), 1024)), 256, 0, s>>>(
      ws, bt, sp.chunks, 2, (int)d, static_cast<__nv_bfloat16*>(dscale),
      static_cast<__nv_bfloat16*>(dshift));
  ANIMA_CHECK_LAUNCH("adaln_bwd finalize");
  return ANIMA_OK;
}

extern "C" int64_t anima_gated_add_adaln_bwd_workspace_bytes(int64_t rows, int64_t hw, int64_t d) {
  if (rows < 0 || hw <= 0 || d <= 0 || rows % hw) return ANIMA_E_SHAPE;
  const RowSplit sp = make_split(rows / hw, hw);
  return (rows / hw) * sp.chunks * 3 * d * static_cast<int64_t>(sizeof(float));
}

extern "C" int anima_gated_add_adaln_bwd(const void* d_y, const void* d_xnew, const void* x_new, const void* scale,
                                         const float* mean, const float* rstd, const void* sub, const void* gate,
                                         int64_t rows, int64_t hw, int64_t d, void* dx, void* dsub, void* dscale,
                                         void* dshift, void* dgate, void* workspace, int64_t workspace_bytes,
                                         void* stream) {
  ANIMA_REQUIRE(d_y && d_xnew && x_new && scale && mean && rstd && sub && gate && dx && dsub && dscale && dshift &&
                    dgate,
                ANIMA_E_ARG, "gated_add_adaln_bwd: null pointer");
  if (int rc = check_rows("gated_add_adaln_bwd", rows, hw, d, 4096)) return rc;
  ANIMA_REQUIRE(aligned16(d_y) && aligned16(d_xnew) && aligned16(x_new) && aligned16(scale) && aligned16(sub) &&
                    aligned16(gate) && aligned16(dx) && aligned16(dsub),
                ANIMA_E_ALIGN, "gated_add_adaln_bwd: tensors must be 16-byte aligned");
  if (rows == 0) return ANIMA_OK;
  const int64_t need = anima_gated_add_adaln_bwd_workspace_bytes(rows, hw, d);
  ANIMA_REQUIRE(workspace && aligned16(workspace) && workspace_bytes >= need, ANIMA_E_WORKSPACE,
                "gated_add_adaln_bwd: workspace of %lld bytes (16-byte aligned) required, got %lld", (long long)need,
                (long long)workspace_bytes);
  const int64_t bt = rows / hw;
  ANIMA_REQUIRE(bt <= 65535, ANIMA_E_TOO_LARGE, "gated_add_adaln_bwd: rows/hw=%lld exceeds 65535", (long long)bt);
  const RowSplit sp = make_split(bt, hw);
  const dim3 grid(sp.chunks, static_cast<unsigned>(bt));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  const auto* dyp = static_cast<const __nv_bfloat16*>(d_y);
  const auto* drp = static_cast<const __nv_bfloat16*>(d_xnew);
  const auto* xp = static_cast<const __nv_bfloat16*>(x_new);
  const auto* scp = static_cast<const __nv_bfloat16*>(scale);
  const auto* sbp = static_cast<const __nv_bfloat16*>(sub);
  const auto* gp = static_cast<const __nv_bfloat16*>(gate);
  auto* dxp = static_cast<__nv_bfloat16*>(dx);
  auto* dsp = static_cast<__nv_bfloat16*>(dsub);
  if (int rc = launch_adaln_bwd_main<true>(grid, s, dyp, xp, scp, mean, rstd, drp, sbp, gp, hw, d,
                                           sp.rows_per_chunk, dxp, dsp, ws))
    return rc;
  ANIMA_CHECK_LAUNCH("gated_add_adaln_bwd");
  const int64_t total = bt * 3 * d;
  finalize_partials_kernel<<<static_cast<unsigned>(std::min<int64_t>(ceil_div(total, 256), 1024)), 256, 0, s>>>(
      ws, bt, sp.chunks, 3, (int)d, static_cast<__nv_bfloat16*>(dscale), static_cast<__nv_bfloat16*>(dshift),
      static_cast<__nv_bfloat16*>(dgate));
  ANIMA_CHECK_LAUNCH("gated_add_adaln_bwd finalize");
  return ANIMA_OK;
}

extern "C" int anima_gated_add_fwd(const void* x, const void* gate, const void* y, int64_t rows,
                                   int64_t hw, int64_t d, void* out, void* stream) {
  ANIMA_REQUIRE(x && gate && y && out, ANIMA_E_ARG, "gated_add_fwd: null pointer");
  if (int rc = check_rows("gated_add_fwd", rows, hw, d, INT32_MAX / 2)) return rc;
  ANIMA_REQUIRE(aligned16(x) && aligned16(gate) && aligned16(y) && aligned16(out), ANIMA_E_ALIGN,
                "gated_add_fwd: tensors must be 16-byte aligned");
  if (rows == 0) return ANIMA_OK;
  const int64_t total = rows * (d / 8);
  const unsigned grid =
      static_cast<unsigned>(std::min<int64_t>(ceil_div(total, kThreads * 4), 8LL * sm_count()));
  gated_add_fwd_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gate),
      static_cast<const __nv_bfloat16*>(y), rows, hw, static_cast<int>(d / 8),
      static_cast<__nv_bfloat16*>(out));
  ANIMA_CHECK_LAUNCH("gated_add_fwd");
  return ANIMA_OK;
}

extern "C" int64_t anima_gated_add_bwd_workspace_bytes(int64_t rows, int64_t hw, int64_t d) {
  if (rows < 0 || hw <= 0 || d <= 0 || rows % hw) return ANIMA_E_SHAPE;
  const RowSplit sp = make_split(rows / hw, hw);
  return (rows / hw) * sp.chunks * d * static_cast<int64_t>(sizeof(float));
}

extern "C" int anima_gated_add_bwd(const void* dout, const void* y, const void* gate, int64_t rows,
                                   int64_t hw, int64_t d, void* dy, void* dgate, void* workspace,
                                   int64_t workspace_bytes, void* stream) {
  ANIMA_REQUIRE(dout && y && gate && dy && dgate, ANIMA_E_ARG, "gated_add_bwd: null pointer");
  if (int rc = check_rows("gated_add_bwd", rows, hw, d, 4096)) return rc;
  ANIMA_REQUIRE(aligned16(dout) && aligned16(y) && aligned16(gate) && aligned16(dy), ANIMA_E_ALIGN,
                "gated_add_bwd: tensors must be 16-byte aligned");
  if (rows == 0) return ANIMA_OK;
  const int64_t need = anima_gated_add_bwd_workspace_bytes(rows, hw, d);
  ANIMA_REQUIRE(workspace && aligned16(workspace) && workspace_bytes >= need, ANIMA_E_WORKSPACE,
                "gated_add_bwd: workspace of %lld bytes (16-byte aligned) required, got %lld",
                (long long)need, (long long)workspace_bytes);
  const int64_t bt = rows / hw;
  ANIMA_REQUIRE(bt <= 65535, ANIMA_E_TOO_LARGE, "gated_add_bwd: rows/hw=%lld exceeds 65535", (long long)bt);
  const RowSplit sp = make_split(bt, hw);
  const dim3 grid(sp.chunks, static_cast<unsigned>(bt));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  const auto* dop = static_cast<const __nv_bfloat16*>(dout);
  const auto* yp = static_cast<const __nv_bfloat16*>(y);
  const auto* gp = static_cast<const __nv_bfloat16*>(gate);
  auto* dyp = static_cast<__nv_bfloat16*>(dy);
  if (d <= 2048)
    gated_add_bwd_kernel<1><<<grid, kThreads, 0, s>>>(dop, yp, gp, hw, (int)d, sp.rows_per_chunk, dyp, ws);
  else
    gated_add_bwd_kernel<2><<<grid, kThreads, 0, s>>>(dop, yp, gp, hw, (int)d, sp.rows_per_chunk, dyp, ws);
  ANIMA_CHECK_LAUNCH("gated_add_bwd");
  const int64_t total = bt * d;
  finalize_partials_kernel<<<static_cast<unsigned>(std::min<int64_t>(ceil_div(total, 256), 1024)), 256, 0, s>>>(
      ws, bt, sp.chunks, 1, (int)d, static_cast<__nv_bfloat16*>(dgate), nullptr);
  ANIMA_CHECK_LAUNCH("gated_add_bwd finalize");
  return ANIMA_OK;
}

// ------------------------------------------------------------------ adaln_bwd without caller scratch
// Some hosts of this library may not allocate device memory at the point where they call it: a plugin that
// is handed only its input and output buffers by a framework that owns every other byte of the GPU, or a
// service whose memory plan is frozen after start-up so that a late cudaMalloc could fail or stall. For them
// the partial sums of adaln_bwd live in this fixed array inside the library image instead of a workspace.
namespace {
constexpr int64_t kStaticScratchBytes = ANIMA_ADALN_BWD_NOALLOC_MAX_BYTES;  // resident on every GPU that loads the library
__device__ __align__(256) float g_adaln_bwd_scratch[kStaticScratchBytes / sizeof(float)];

// Device address of the array for the current device. The symbol name is only a host-side handle; the
// address has to be asked for once per device, with that device current.
int static_scratch(float** out) {
  static std::mutex mu;
  static float* cached[64];
  int dev = 0;
  ANIMA_REQUIRE(cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64, ANIMA_E_CUDA,
                "adaln_bwd_noalloc: cannot identify the current device");
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_adaln_bwd_scratch);
    ANIMA_REQUIRE(rc == cudaSuccess && p != nullptr, ANIMA_E_CUDA,
                  "adaln_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(rc));
    cached[dev] = p;
  }
  *out = cached[dev];
  return ANIMA_OK;
}
}  // namespace

extern "C" int anima_adaln_bwd_noalloc(const void* dy, const void* x, const void* scale, const float* mean,
                                       const float* rstd, int64_t rows, int64_t hw, int64_t d, void* dx,
                                       void* dscale, void* dshift, void* stream) {
  const int64_t need = anima_adaln_bwd_workspace_bytes(rows, hw, d);
  ANIMA_REQUIRE(need >= 0, ANIMA_E_SHAPE, "adaln_bwd_noalloc: rows=%lld is not a multiple of hw=%lld (or a size is not positive)",
                (long long)rows, (long long)hw);
  ANIMA_REQUIRE(need <= kStaticScratchBytes, ANIMA_E_TOO_LARGE,
                "adaln_bwd_noalloc: this shape needs %lld bytes of scratch but the built-in array holds %lld; "
                "use anima_adaln_bwd with a caller workspace",
                (long long)need, (long long)kStaticScratchBytes);
  float* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  // Every partial-sum slot that the final pass reads is written earlier in this same call, so nothing in the
  // array has to start at zero and what an earlier call left behind is never read.
  return anima_adaln_bwd(dy, x, scale, mean, rstd, rows, hw, d, dx, dscale, dshift, scratch, kStaticScratchBytes,
                         stream);
}
