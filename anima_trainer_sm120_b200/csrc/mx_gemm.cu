// MXFP8 block-scaled GEMM for sm_100a: C[M,N] = alpha * A[M,K] . B[N,K]^T (+ bias) (+ residual).
//
// Replaces anima-trainer's Triton tl.dot_scaled kernel (mxfp8_gemm.py:254-336) and
// the Transformer-Engine general_gemm calls of fp8_quant.py (:150, :236 forward;
// :504 dgrad; :507 wgrad). Both operands are e4m3 codes contiguous along K with one
// e8m0 scale per 32 K-elements in the 128x4 tiled layout (see anima_b200.h), so the
// forward, dgrad and wgrad GEMMs are all this one "TN" form.
//
// Two kernel families, both persistent and warp-specialised (warp 0 TMA producer, warp 1 MMA issuer, the
// other warps epilogue), accumulating in tensor memory (fp32):
//
//  * mx_gemm2_kernel<BN> — the main one (M > 128 and N > 128): a cluster of two CTAs owns a 256 x 192 (K < 4096)
//    or 256 x 256 tile and issues tcgen05.mma.cta_group::2 (M256 x N192|256 x K32); see the comment above it.
//  * mx_gemm_kernel<BN> — one CTA per 128 x BN tile (BN = 128 or 256) for small or narrow problems:
//      warp 0  per K-block of 128 one 128x128 A box and one BNx128 B box (128-byte swizzle) plus the
//              512-byte scale chunks (bulk copies), all completing on the stage's "full" mbarrier;
//              4-stage shared-memory ring.
//      warp 1  copies the stage's scale chunks shared -> tensor memory (tcgen05.cp 32x128b.warpx4),
//              issues four tcgen05.mma.kind::mxf8f6f4.block_scale per stage, frees the stage and
//              publishes the accumulator with tcgen05.commit.
//      warps 2-5  tcgen05.ld the accumulator in 32-column chunks, add bias, round to bf16 (or keep
//              fp32) and store 64/128 contiguous bytes per thread.
//    Two accumulator buffers let the epilogue of tile i overlap the main loop of tile i+1. For
//    BN = 256 the 512 tensor-memory columns cannot hold two full buffers plus the scale columns, so
//    buffer 1 starts 32 columns before the end of buffer 0 and the epilogue drains those shared
//    columns first, then releases the MMA warp.
//    With caller scratch it also splits the contraction of small outputs (work item = tile x K-range,
//    fp32 partial tiles, fixed-order finalize kernel).
// Every wait is bounded; on a timeout a kernel raises *status, lets copies in flight land, frees its
// tensor memory and returns. Tensor-pipe bound: 2*M*N*K flop. No TMA multicast is used anywhere.
#include <cuda.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "common.cuh"
#include "mx_quantize_tile.cuh"
#include "tma_util.cuh"

namespace anima {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;  // bytes == e4m3 elements per K-block
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kSfChunk = 512;

template <int BN>
struct Cfg {
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = BN * BK;
  static constexpr int kSfbChunks = BN / 128;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfChunk * (1 + kSfbChunks);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int kOverlap = (BN == 256) ? 32 : 0;
  static constexpr int kAcc1Col = BN - kOverlap;
  static constexpr int kSfaCol = kAcc1Col + BN;  // 480 for BN=256, 256 for BN=128
  static constexpr int kSfbCol = kSfaCol + 4;
  static constexpr int kTmemCols = 512;
  static_assert(kSfbCol + 4 * kSfbChunks <= kTmemCols, "tensor memory overflow");
  static constexpr uint32_t kTxBytes = kABytes + kBBytes + kSfChunk * (1 + kSfbChunks);
};

// ------------------------------------------------------------------ tcgen05 wrappers (mbarrier / TMA ones: tma_util.cuh)
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t tmem_addr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}
__device__ __forceinline__ void tc_mma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are 128 B
// apart, 8-row groups 1024 B apart (stride byte offset); descriptor version 1.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t saddr) {
  return static_cast<uint64_t>((saddr >> 4) & 0x3fffu) | (static_cast<uint64_t>(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// Scale chunk for tcgen05.cp: no swizzle, 32 rows x 16 B, 8-row groups 128 B apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  return static_cast<uint64_t>((saddr >> 4) & 0x3fffu) | (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor: e4m3 x e4m3, K-major both, ue8m0 scales, M=128, N=BN.
template <int BN>
__device__ __forceinline__ uint32_t make_idesc(uint32_t sf_id) {
  return (static_cast<uint32_t>(BN >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(BM >> 4) << 24) |
         (sf_id << 29) | (sf_id << 4);
}

struct GemmParams {
  const uint8_t* a_scales;
  const uint8_t* b_scales;
  void* c;
  const __nv_bfloat16* bias;
  int32_t* status;
  int M, N, K;
  int64_t ldc;
  int out_fp32;
  int m_tiles, n_tiles, k_blocks;
  int sfa_rt, sfb_rt;  // number of 128-row scale tiles of A and B
  // Split-K (one-CTA kernel only): work item = (tile, split); split s contracts K-blocks
  // [s * kb_per_split, min(k_blocks, (s + 1) * kb_per_split)) and, when splits > 1, stores its fp32
  // partial tile to partial[s][M][N]; splitk_finalize_kernel then sums the splits in index order.
  int splits, kb_per_split;
  float* partial;
  // Epilogue: C = alpha * (A . B^T) + bias + residual (residual bf16 [M, N], row pitch ldr; may alias C).
  const __nv_bfloat16* residual;
  int64_t ldr;
  float alpha;
  // Work list of the CTA-pair kernel (see PairPlan below): tile columns 0 .. n_wide-1 are pair_bn wide; if
  // `narrow`, one more column of at most 128 valid outputs follows and is computed with N = 128 instructions
  // (n_tiles = n_wide + narrow). Items 0 .. full_items-1 are whole tiles in tile order, dealt round-robin to
  // the pairs (full_items is a multiple of the pair count). The tail_tiles tiles after them are each split along K
  // into tail_splits ranges of tail_kbs K-blocks; those items are dealt round-robin starting at pair tail_shift
  // and leave as fp32 partial tiles in pair_partial [item][256][pair_bn], summed by pair_tail_finalize_kernel.
  int n_wide, narrow;
  int pair_bn;  // width of the wide tile columns, 192 or 256 (the finalize pass reads it; the kernel is compiled per width)
  int full_items, tail_tiles, tail_splits, tail_kbs, tail_shift;
  float* pair_partial;
  int sf_bufs;  // tensor-memory scale buffers the K-blocks rotate through (1, 2 or 4)
  // Mix epilogue of the one-CTA kernel, N = 128 (anima_tlokr_hidden_mix_planes): the accumulator tile is the
  // T-LoKr hidden tensor of 16 tokens (row = token * 8 + j); instead of being stored it is rounded to bf16,
  // mixed over j with the 8 x 8 factor inside each group of eight lanes, masked, rounded, quantised (one MX
  // block per row and 32-column chunk) and written as e4m3 planes (row i of token t at plane row i * items + t).
  const __nv_bfloat16* mix_c;     // [8, 8]
  const __nv_bfloat16* mix_mask;  // [batch, 128] or null
  uint8_t* mix_codes;             // [8 * items, 128]; null = ordinary epilogue
  uint8_t* mix_scales;            // TILED scales of that matrix
  __nv_bfloat16* mix_hidden;      // optional bf16 copy of the hidden tile rows [M, 128]
  int64_t mix_items, mix_n_per_batch;
  int mix_transpose;
  // Low-rank delta folded in as extra K-blocks (anima_mx_gemm_delta): output columns [i * delta_block,
  // (i + 1) * delta_block) also receive planes[i][m, 0:128] . d[p, 0:128]^T. For a tile, every run of its
  // columns inside one block is one more pipeline stage (A slot: 128 rows of plane i; B slot: the factor rows of
  // the run, half per CTA) and one group of MMAs of that width into the run's accumulator columns.
  int delta, delta_block;
  // Measurement aid (anima_mx_gemm_set_clock_probe): if not null, CTA 0 of a pair-kernel launch adds the SM
  // cycles and the nanoseconds it ran, so that the clock the GPU actually held under this kernel's power
  // draw can be read back (the driver's sampled clocks mostly see the idle gaps between launches), and the
  // cycles its producer, MMA-issuing and first epilogue warp spent waiting on their barriers.
  long long* clock_probe;
};


// Tile order of the CTA-pair kernel. The tiles that run at the same time should cover the SHORTER side of
// the tile grid completely, so that the operand of the longer side is streamed once instead of once per
// tile row: with n fastest, the wgrad dW[2048, 8192] (8 x 43 tiles) re-read its 268 MB B operand 8 times and
// ran HBM-bound. The index along the shorter side varies fastest. The narrow last tile column (nt == n_wide)
// stays inside this sweep: run as a phase of its own after the wide tiles it re-read all of A with 16
// K-blocks of work per tile and was HBM-bound (2644 -> 2509 TFLOP/s on 32768 x 2048 x 2048).
__host__ __device__ __forceinline__ void tile_coords_of(int m_tiles, int n_tiles, int tile, int& mt, int& nt) {
  if (m_tiles < n_tiles) {
    nt = tile / m_tiles;
    mt = tile - nt * m_tiles;
  } else {
    mt = tile / n_tiles;
    nt = tile - mt * n_tiles;
  }
}
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& mt, int& nt) {
  tile_coords_of(p.m_tiles, p.n_tiles, tile, mt, nt);
}

// One unit of work of a CTA pair: a whole tile (part < 0) or the K-range [kb0, kb1) of a tail tile, whose fp32
// partial goes to slot `part`. valid == false marks a padding slot of the round robin (nothing to do).
struct PairItem {
  int mt, nt, kb0, kb1, part;
  bool valid;
};
__device__ __forceinline__ int pair_total_slots(const GemmParams& p) {
  const int split_items = p.tail_tiles * p.tail_splits;
  return p.full_items + (split_items ? p.tail_shift + split_items : 0);
}
__device__ __forceinline__ PairItem pair_item(const GemmParams& p, int slot) {
  PairItem it;
  it.kb0 = 0;
  it.kb1 = p.k_blocks;
  it.part = -1;
  it.valid = true;
  int tile = slot;
  if (slot >= p.full_items) {
    const int r = slot - p.full_items - p.tail_shift;
    if (r < 0) {
      it.valid = false;
      it.mt = it.nt = 0;
      return it;
    }
    const int t = r / p.tail_splits, sp = r - t * p.tail_splits;
    tile = p.full_items + t;
    if (p.tail_splits > 1) {
      it.kb0 = sp * p.tail_kbs;
      it.kb1 = min(p.k_blocks, it.kb0 + p.tail_kbs);
      it.part = r;
    }
  }
  tile_coords(p, tile, it.mt, it.nt);
  return it;
}

// First slot >= `slot` of this pair's round robin (stride `stride`) that holds work; `it` receives its item.
// Returns total_slots or more when there is none.
__device__ __forceinline__ int pair_next_item(const GemmParams& p, int slot, int stride, int total_slots, PairItem& it) {
  while (slot < total_slots) {
    it = pair_item(p, slot);
    if (it.valid) break;
    slot += stride;
  }
  return slot;
}

// Epilogue store of one 32-column accumulator chunk of one row: bias, rounding, predicated 16-byte stores.
__device__ __forceinline__ void store_chunk(const GemmParams& p, int row, int col, const uint32_t (&v)[32]) {
  if (row >= p.M || col >= p.N) return;
  float f[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * p.alpha;
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      if (col + j < p.N) {
        float b[8];
        unpack8(*reinterpret_cast<const uint4*>(p.bias + col + j), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[j + e] += b[e];
      }
    }
  }
  if (p.residual) {
    const __nv_bfloat16* res = p.residual + static_cast<int64_t>(row) * p.ldr + col;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      if (col + j < p.N) {
        float b[8];
        unpack8(*reinterpret_cast<const uint4*>(res + j), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[j + e] += b[e];
      }
    }
  }
  if (p.out_fp32) {
    float* dst = static_cast<float*>(p.c) + static_cast<int64_t>(row) * p.ldc + col;
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      if (col + j < p.N) *reinterpret_cast<float4*>(dst + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
  } else {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + static_cast<int64_t>(row) * p.ldc + col;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      if (col + j < p.N) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = f[j + e];
        *reinterpret_cast<uint4*>(dst + j) = pack8(o);
      }
    }
  }
}

// One 32-column chunk of the mix epilogue for the thread that owns accumulator row (token, j = lane % 8) and
// produces output row (token, i = lane % 8). The arithmetic and its order are those of the GEMM's bf16 store
// followed by rank_mix_quant_kernel (fp32 fma over j ascending from 0, mask, bf16 rounding, MX quantisation of
// the rounded values), so codes and scale are bit-identical to running the two kernels.
__device__ __forceinline__ void mix_chunk(const uint32_t (&v)[32], const uint32_t (&cw)[8], int lane,
                                          const __nv_bfloat16* mask_chunk, __nv_bfloat16* hidden_chunk,
                                          uint4 (&codes)[2], uint32_t& scale_byte) {
  uint32_t pk[16];  // the chunk rounded to bf16, two columns per word
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
    pk[k] = *reinterpret_cast<const uint32_t*>(&h);
  }
  if (hidden_chunk != nullptr) {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      stg_stream16(hidden_chunk + 8 * q, make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]));
  }
  float acc[32];
#pragma unroll
  for (int k = 0; k < 32; ++k) acc[k] = 0.f;
  const int base = lane & 24;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    // fma.rn.f32.bf16: bf16 x bf16 + fp32 with one rounding, i.e. fmaf(float(h), float(w), acc) without the two
    // instructions that widen the halves of the shuffled word (a third of this loop's instruction count)
    const uint32_t w = cw[j];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t other = __shfl_sync(0xffffffffu, pk[k], base + j);
      asm("{\n\t.reg .b16 lo, hi, wl, wh;\n\t"
          "mov.b32 {lo, hi}, %2;\n\t"
          "mov.b32 {wl, wh}, %3;\n\t"
          "fma.rn.f32.bf16 %0, lo, wl, %0;\n\t"
          "fma.rn.f32.bf16 %1, hi, wl, %1;\n\t}"
          : "+f"(acc[2 * k]), "+f"(acc[2 * k + 1])
          : "r"(other), "r"(w));
    }
  }
  if (mask_chunk != nullptr) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float m[8];
      unpack8(*reinterpret_cast<const uint4*>(mask_chunk + 8 * q), m);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[8 * q + e] *= m[e];
    }
  }
  float f[32];
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const float2 r = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]));
    f[2 * k] = r.x;
    f[2 * k + 1] = r.y;
    amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
  }
  const int ex = mxq::mx_exponent(fmaxf(amax, mxq::kAmaxFloor));
  const float inv = mxq::mx_inv_scale(ex);
  uint32_t w8[8];
#pragma unroll
  for (int q = 0; q < 8; ++q)
    w8[q] = mxq::e4m3x2(f[4 * q] * inv, f[4 * q + 1] * inv) | (mxq::e4m3x2(f[4 * q + 2] * inv, f[4 * q + 3] * inv) << 16);
  codes[0] = make_uint4(w8[0], w8[1], w8[2], w8[3]);
  codes[1] = make_uint4(w8[4], w8[5], w8[6], w8[7]);
  scale_byte = static_cast<uint32_t>(ex + 127);
}

// EPI = number of epilogue warps: 4 (one per tensor-memory lane quadrant) for the ordinary epilogue; 8 for the mix
// epilogue, whose shuffles and conversions are bound by instruction latency with a single warp per scheduler
// (two warps per quadrant then take two of the four 32-column chunks each).
template <int BN, int EPI = 4>
__global__ void __launch_bounds__(64 + 32 * EPI, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_flag;
  __shared__ uint32_t tmem_base_slot;

  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // 128B-swizzled TMA boxes need 1024-byte alignment
  // Operand tiles first (each a multiple of 1024 bytes), then the scale chunks, then the barriers.
  const uint32_t sf_base = base + kStages * (C::kABytes + C::kBBytes);
  const uint32_t bar_base = base + kStages * C::kStageBytes;
  auto a_smem = [&](int s) { return base + s * (C::kABytes + C::kBBytes); };
  auto b_smem = [&](int s) { return base + s * (C::kABytes + C::kBBytes) + C::kABytes; };
  auto sfa_smem = [&](int s) { return sf_base + s * kSfChunk * (1 + C::kSfbChunks); };
  auto sfb_smem = [&](int s, int i) { return sfa_smem(s) + kSfChunk * (1 + i); };
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (kStages + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8 * (2 * kStages + s); };
  const uint32_t acc_free_bar = bar_base + 8 * (2 * kStages + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full_bar(0), 1);
    mbar_init(acc_full_bar(1), 1);
    mbar_init(acc_free_bar, EPI);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(C::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const int total_items = p.m_tiles * p.n_tiles * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t kiter = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int tile = item / p.splits, split = item - tile * p.splits;
        const int kb0 = split * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        const int mt = tile / p.n_tiles, nt = tile - mt * p.n_tiles;
        for (int kb = kb0; kb < kb1; ++kb, ++kiter) {
          const int s = kiter % kStages;
          const uint32_t ph = (kiter / kStages) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), C::kTxBytes);
          tma_load_2d(a_smem(s), &map_a, full_bar(s), kb * BK, mt * BM);
          tma_load_2d(b_smem(s), &map_b, full_bar(s), kb * BK, nt * BN);
          const int64_t kb4 = p.k_blocks;  // one 512-byte chunk per (row tile, K-block)
          bulk_load(sfa_smem(s), p.a_scales + (static_cast<int64_t>(mt) * kb4 + kb) * kSfChunk, kSfChunk, full_bar(s));
#pragma unroll
          for (int i = 0; i < C::kSfbChunks; ++i) {
            const int rt = min(nt * C::kSfbChunks + i, p.sfb_rt - 1);  // clamp: tail chunk rows are never stored
            bulk_load(sfb_smem(s, i), p.b_scales + (static_cast<int64_t>(rt) * kb4 + kb) * kSfChunk, kSfChunk,
                      full_bar(s));
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t kiter = 0;
      bool ok = true;
      int it = 0;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
        const int split = item % p.splits;
        const int kb0 = split * p.kb_per_split, kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        const int as = it & 1;
        if (it > 0) {
          // The previous tile's epilogue must have drained the columns shared by the two buffers
          // (and, by program order, finished the tile before it, which used this buffer).
          if (!mbar_wait(acc_free_bar, (it - 1) & 1u, &abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        const uint32_t d_tmem = tmem_base + (as ? C::kAcc1Col : 0);
        for (int kb = kb0; kb < kb1; ++kb, ++kiter) {
          const int s = kiter % kStages;
          const uint32_t ph = (kiter / kStages) & 1u;
          if (!mbar_wait(full_bar(s), ph, &abort_flag)) { ok = false; break; }
          tc_fence_after();
          tc_cp_sf(tmem_base + C::kSfaCol, make_sf_desc(sfa_smem(s)));
#pragma unroll
          for (int i = 0; i < C::kSfbChunks; ++i)
            tc_cp_sf(tmem_base + C::kSfbCol + 4 * i, make_sf_desc(sfb_smem(s, i)));
          const uint64_t a_desc = make_sw128_desc(a_smem(s));
          const uint64_t b_desc = make_sw128_desc(b_smem(s));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            // +32 bytes along K inside the 128-byte swizzle atom = +2 in the 16-byte address field.
            tc_mma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, make_idesc<BN>(k), tmem_base + C::kSfaCol,
                        tmem_base + C::kSfbCol, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(s));  // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(acc_full_bar(as));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // tensor-memory lane quadrant this warp may access
    bool ok = true;
    int it = 0;
    if (BN == 128 && p.mix_codes != nullptr) {
      // mix epilogue: see GemmParams. splits == 1 here, so an item is a tile.
      uint32_t cw[8];   // this row's mix weights as raw bf16 bits (low half)
      {
        const int i = lane & 7;
#pragma unroll
        for (int j = 0; j < 8; ++j) cw[j] = __bfloat16_as_ushort(p.mix_transpose ? p.mix_c[j * 8 + i] : p.mix_c[i * 8 + j]);
      }
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
        const int mt = item;  // n_tiles == 1
        const int as = it & 1;
        if (!mbar_wait(acc_full_bar(as), (it >> 1) & 1u, &abort_flag)) { ok = false; break; }
        tc_fence_after();
        const int64_t row = static_cast<int64_t>(mt) * BM + quad * 32 + lane;   // accumulator row (token * 8 + j)
        const int64_t token = row >> 3;
        const int64_t prow = static_cast<int64_t>(lane & 7) * p.mix_items + token;   // plane row this thread writes
        const __nv_bfloat16* mask_row = p.mix_mask ? p.mix_mask + (token / p.mix_n_per_batch) * 128 : nullptr;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + (as ? C::kAcc1Col : 0);
        constexpr int kChunks = 16 / EPI;                 // chunks per warp: 4, or 2 with two warps per quadrant
        const int c0 = ((warp - 2) >> 2) * kChunks;
        uint32_t scale_word = 0;
#pragma unroll 1
        for (int c = c0; c < c0 + kChunks; ++c) {
          uint32_t v[32];
          tc_ld32(t_row + c * 32, v);
          tc_wait_ld();
          if (c == c0) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_free_bar);
          }
          uint4 codes[2];
          uint32_t sb;
          mix_chunk(v, cw, lane, mask_row ? mask_row + c * 32 : nullptr,
                    p.mix_hidden ? p.mix_hidden + row * 128 + c * 32 : nullptr, codes, sb);
          uint8_t* dst = p.mix_codes + prow * 128 + c * 32;
          stg_stream16(dst, codes[0]);
          stg_stream16(dst + 16, codes[1]);
          scale_word |= sb << (8 * (c - c0));
        }
        // the row's scale bytes are adjacent in the tiled layout (one 128-column chunk per row tile)
        uint8_t* sdst = p.mix_scales + (prow >> 7) * 512 + mxq::tiled_offset(static_cast<int>(prow & 127), c0);
        if (kChunks == 4) *reinterpret_cast<uint32_t*>(sdst) = scale_word;
        else *reinterpret_cast<uint16_t*>(sdst) = static_cast<uint16_t>(scale_word);
      }
    } else {
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
      const int tile = item / p.splits, split = item - tile * p.splits;
      const int mt = tile / p.n_tiles, nt = tile - mt * p.n_tiles;
      const int as = it & 1;
      GemmParams dst = p;
      if (p.splits > 1) {  // this split's fp32 partial; bias and rounding happen in the finalize pass
        dst.c = p.partial + static_cast<int64_t>(split) * p.M * p.N;
        dst.ldc = p.N;
        dst.out_fp32 = 1;
        dst.bias = nullptr;
        dst.residual = nullptr;
        dst.alpha = 1.f;
      }
      if (!mbar_wait(acc_full_bar(as), (it >> 1) & 1u, &abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = mt * BM + quad * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + (as ? C::kAcc1Col : 0);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        // Buffer 0 shares its LAST 32 columns with buffer 1, buffer 1 its FIRST 32: drain those first.
        const int chunk = (C::kOverlap && as == 0) ? (BN / 32 - 1 - c) : c;
        uint32_t v[32];
        tc_ld32(t_row + chunk * 32, v);
        tc_wait_ld();
        if (c == 0) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_free_bar);
        }
        store_chunk(dst, row, nt * BN + chunk * 32, v);
      }
    }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (abort_flag) {
    // Give copies that are still in flight time to land before shared memory is released.
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
  }
}

// C = sum over splits (in index order, so the result is reproducible) of partial[s] (+ bias), 4 columns per thread.
__global__ void __launch_bounds__(256) splitk_finalize_kernel(const GemmParams p) {
  const int64_t n4 = p.N / 4, total = static_cast<int64_t>(p.M) * n4, plane = static_cast<int64_t>(p.M) * p.N;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / n4, col = (i - row * n4) * 4;
    const float* src = p.partial + row * p.N + col;
    float4 acc = *reinterpret_cast<const float4*>(src);
    // The loads of eight splits are issued together and then added in index order: the sum keeps its fixed
    // association, and a thread no longer waits one memory latency per split (a [256, 128] factor gradient is
    // summed over up to 74 splits by 8192 threads).
    int s = 1;
    for (; s + 8 <= p.splits; s += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const float4*>(src + (s + u) * plane);
#pragma unroll
      for (int u = 0; u < 8; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
    }
    for (; s < p.splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + s * plane);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= p.alpha; acc.y *= p.alpha; acc.z *= p.alpha; acc.w *= p.alpha;
    if (p.bias) {
      acc.x += __bfloat162float(p.bias[col]);
      acc.y += __bfloat162float(p.bias[col + 1]);
      acc.z += __bfloat162float(p.bias[col + 2]);
      acc.w += __bfloat162float(p.bias[col + 3]);
    }
    if (p.residual) {
      const __nv_bfloat16* res = p.residual + row * p.ldr + col;
      acc.x += __bfloat162float(res[0]);
      acc.y += __bfloat162float(res[1]);
      acc.z += __bfloat162float(res[2]);
      acc.w += __bfloat162float(res[3]);
    }
    if (p.out_fp32) {
      *reinterpret_cast<float4*>(static_cast<float*>(p.c) + row * p.ldc + col) = acc;
    } else {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(acc.x, acc.y);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.c) + row * p.ldc + col) = o;
    }
  }
}

// ================================================================== 2-CTA variant
// A cluster of two CTAs (two SMs) owns one 256 x BN output tile, BN = 192 or 256. CTA r stages rows
// [128 r, 128 r + 128) of the A tile and its half of the B tile's rows, so every tcgen05.mma (cta_group::2,
// M256 x N192 x K32) is fed by 7 KB of shared-memory fill per SM (the one-CTA kernel needs 12 KB per
// M128 x N256 x K32), and 5 or 6 stages are in flight.
// Only the leader CTA (cluster rank 0) issues scale copies, MMAs and commits; the commits
// are delivered to the mbarriers of both CTAs, and both CTAs' TMA loads complete on the
// leader's "full" barrier. Each CTA drains its own 128 accumulator rows. The loads carry no
// multicast: each CTA fetches its own boxes.
// Tile widths are multiples of 64: tiles start at multiples of 64 columns, so a tile touches two 128-column scale
// chunks of B and its scales start 0 or 2 tensor-memory columns into the first. A 224-wide variant (tiles at
// multiples of 32, odd scale-column offsets) raised a misaligned-address fault on its first tile with an odd
// offset; such widths are therefore not used.
// What limits it (cycle counters of anima_mx_gemm_set_clock_probe, and builds with parts of the epilogue left
// out): at BN = 192 a K-block costs 404 - 516 cycles depending on K and on the box, against the tensor pipe's
// 384: operand delivery (57 KB written to and read from shared memory per CTA and K-block) is the limit, and each
// tile adds about 1200 cycles, of which ~350 are the epilogue's st.shared into the staging buffers and ~200 its
// TMA stores. At BN = 256 a K-block costs the tensor pipe's 512 cycles (64 KB), and each tile adds about 2800
// because it also waits for the previous tile's shared columns to be read. The SM clock sits at the
// board's power limit throughout, so energy per flop (operand traffic per flop: 7/8 at BN = 256) decides as much
// as idle cycles do.
// Epilogue warps per CTA: 4 * kEpiHalves. With two halves, two warps share each 32-lane quadrant of tensor memory
// and drain different column ranges of the accumulator at the same time.
#ifndef ANIMA_PAIR_EPI_HALVES
#define ANIMA_PAIR_EPI_HALVES 2
#endif
constexpr int kEpiHalves = ANIMA_PAIR_EPI_HALVES;
constexpr int kThreads2 = 64 + 128 * kEpiHalves;
constexpr int kSfbChunks2 = 2;  // 128-column scale chunks of B a tile can touch
static_assert(kEpiHalves == 1 || kEpiHalves == 2, "one or two epilogue warps per tensor-memory quadrant");

// Two tile widths. 256 x 192: two disjoint accumulator buffers, so a tile's MMAs follow the previous tile's
// without a gap; per K-block the tensor pipe works 384 cycles on 28 KB of operands. 256 x 256: 512 cycles on
// 32 KB, i.e. less shared-memory and L2 traffic (and energy) per flop, but the two buffers must share 32 columns
// of tensor memory and every tile starts only after the epilogue has read those columns of the tile before it
// (about 2000 idle cycles per tile, measured). The wide form wins once a tile holds enough K-blocks to pay for
// that gap (K >= 4096 on a power-capped B200), the narrow form below.
template <int BN>
struct Cfg2 {
  static_assert(BN == 192 || BN == 256, "tile widths whose scale columns start at even tensor-memory offsets");
  static constexpr int kStages = BN == 256 ? 5 : 6;
  static constexpr int kABytes = 128 * BK;
  static constexpr int kBBytes = (BN / 2) * BK;  // this CTA's half of the B rows
  // At N = 192 the accumulator buffers are disjoint. At N = 256 buffer 0 = columns 0..255 and buffer 1 =
  // 224..479: the epilogue reads the shared columns first (buffer 0: its last chunk, buffer 1: its first).
  static constexpr int kOverlap = (BN == 256) ? 32 : 0;
  static constexpr int kAcc1Col = BN - kOverlap;  // second accumulator buffer
  static constexpr int kSfaCol = 2 * BN - kOverlap;  // scale buffers: 16 columns each (SFA 4, SFB 2 x 4)
  static constexpr int kTmemCols = 512;
  static constexpr int kMaxSfBufs = (kTmemCols - kSfaCol) / 16 >= 4 ? 4 : 2;
  static_assert(kSfaCol + 16 * kMaxSfBufs <= kTmemCols, "accumulators and scale buffers must fit tensor memory");
  static constexpr int kSfBytes = kSfChunk * (1 + kSfbChunks2);  // SFA chunk + the SFB chunks
  static constexpr int kStageBytes = kABytes + kBBytes + kSfBytes;
  // Output staging, per epilogue half: two buffers of one 128-row x 32-column bf16 chunk each, alternating; an
  // fp32 chunk takes both (single-buffered: fp32 outputs are the long-K products, whose epilogue is idle most of
  // the time).
  static constexpr int kStoreBytes = 128 * 64;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiHalves * 2 * kStoreBytes + 1024 + 256;
  static_assert(kSmemBytes <= 227 * 1024, "pair kernel exceeds the shared memory of one CTA");
  static constexpr uint32_t kTxBytes = 2u * kStageBytes;  // both CTAs land on the leader's barrier
};

// True in exactly one (converged) lane of the warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1,
                                             int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tc2_commit_both(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(static_cast<uint16_t>(3))
               : "memory");
}
// One K-block of the pair kernel as straight-line PTX: scale chunks shared -> tensor memory, four
// M256 x N192 x K32 block-scaled MMAs (scale-factor id k selects the k-th byte of each scale word;
// +32 bytes along K = +2 in the descriptor's 16-byte address field), then the commit that frees the
// stage in both CTAs. Descriptor high words: stride 1024 B (operands, 128-byte swizzle) / 128 B (scales).
// Instruction descriptor of the pair kernel without the scale-factor ids: e4m3 x e4m3, K-major, ue8m0 scales,
// M = 256, N = n (192, or 128 for the narrow last tile column).
__device__ __forceinline__ uint32_t pair_idesc(int n) {
  return (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(256 >> 4) << 24);
}
__device__ __forceinline__ void tc2_kblock(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t sf_lo, uint32_t sfa_t,
                                           uint32_t sfb_t, uint32_t sfb_use, uint32_t accumulate, uint32_t empty_bar,
                                           uint32_t kI) {
  constexpr uint32_t kOpHi = (1024u >> 4) | (1u << 14) | (2u << 29);
  constexpr uint32_t kSfHi = (128u >> 4) | (1u << 14);
  asm volatile(
      "{\n\t"
      ".reg .pred p, pt;\n\t"
      ".reg .b32 t;\n\t"
      ".reg .b64 da, db, ds;\n\t"
      ".reg .b16 m;\n\t"
      "mov.b16 m, 3;\n\t"
      "setp.ne.b32 p, %7, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "mov.b64 ds, {%3, %10};\n\t"
      "tcgen05.cp.cta_group::2.32x128b.warpx4 [%4], ds;\n\t"
      "add.u32 t, %3, 32;\n\t"
      "mov.b64 ds, {t, %10};\n\t"
      "tcgen05.cp.cta_group::2.32x128b.warpx4 [%5], ds;\n\t"
      "add.u32 t, %3, 64;\n\t"
      "mov.b64 ds, {t, %10};\n\t"
      "add.u32 t, %5, 4;\n\t"
      "tcgen05.cp.cta_group::2.32x128b.warpx4 [t], ds;\n\t"
      "mov.b64 da, {%1, %9};\n\t"
      "mov.b64 db, {%2, %9};\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %11, [%4], [%6], p;\n\t"
      "add.u32 t, %1, 2;\n\t"
      "mov.b64 da, {t, %9};\n\t"
      "add.u32 t, %2, 2;\n\t"
      "mov.b64 db, {t, %9};\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %12, [%4], [%6], pt;\n\t"
      "add.u32 t, %1, 4;\n\t"
      "mov.b64 da, {t, %9};\n\t"
      "add.u32 t, %2, 4;\n\t"
      "mov.b64 db, {t, %9};\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %13, [%4], [%6], pt;\n\t"
      "add.u32 t, %1, 6;\n\t"
      "mov.b64 da, {t, %9};\n\t"
      "add.u32 t, %2, 6;\n\t"
      "mov.b64 db, {t, %9};\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %14, [%4], [%6], pt;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%8], m;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(sf_lo), "r"(sfa_t), "r"(sfb_t), "r"(sfb_use), "r"(accumulate),
        "r"(empty_bar), "r"(kOpHi), "r"(kSfHi), "r"(kI), "r"(kI | (1u << 29) | (1u << 4)),
        "r"(kI | (2u << 29) | (2u << 4)), "r"(kI | (3u << 29) | (3u << 4))
      : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kThreads2, 1)
mx_gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_part,
                const __grid_constant__ CUtensorMap map_pl, const __grid_constant__ CUtensorMap map_d,
                const __grid_constant__ CUtensorMap map_plsf, const __grid_constant__ CUtensorMap map_dsf,
                const GemmParams p) {
  using C = Cfg2<BN>;
  constexpr int kStages2 = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ volatile int abort_flag;
  __shared__ uint32_t tmem_base_slot;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t store_base = base + kStages2 * (C::kABytes + C::kBBytes);  // 1024-aligned staging for C
  const uint32_t sf_base = store_base + kEpiHalves * 2 * C::kStoreBytes;
  const uint32_t bar_base = sf_base + kStages2 * C::kSfBytes;
  auto a_smem = [&](int s) { return base + s * (C::kABytes + C::kBBytes); };
  auto b_smem = [&](int s) { return a_smem(s) + C::kABytes; };
  auto sfa_smem = [&](int s) { return sf_base + s * C::kSfBytes; };
  auto sfb_smem = [&](int s) { return sfa_smem(s) + kSfChunk; };
  auto full_bar = [&](int s) { return bar_base + 8 * s; };
  auto empty_bar = [&](int s) { return bar_base + 8 * (kStages2 + s); };
  auto acc_full_bar = [&](int s) { return bar_base + 8 * (2 * kStages2 + s); };
  auto acc_empty_bar = [&](int s) { return bar_base + 8 * (2 * kStages2 + 2 + s); };
  auto ovl_free_bar = [&](int s) { return bar_base + 8 * (2 * kStages2 + 4 + s); };  // N = 256 only

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool probe = p.clock_probe != nullptr;
  const long long probe_cycles0 = clock64();
  const uint64_t probe_ns0 = global_timer_ns();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(full_bar(s), 1);   // the leader producer's arrive.expect_tx; bytes come from both CTAs
      mbar_init(empty_bar(s), 1);  // one multicast commit
    }
    mbar_init(acc_full_bar(0), 1);
    mbar_init(acc_full_bar(1), 1);
    mbar_init(acc_empty_bar(0), 8 * kEpiHalves);  // every epilogue warp of both CTAs arrives on the leader's barriers
    mbar_init(acc_empty_bar(1), 8 * kEpiHalves);
    mbar_init(ovl_free_bar(0), 8);  // the four warps of the half that owns the shared columns, in both CTAs
    mbar_init(ovl_free_bar(1), 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfa) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_sfb) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
    if (p.tail_splits > 1) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_part) : "memory");
  }
  if (warp == 1) {  // the same warp of both CTAs performs the pair allocation
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(C::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrive or TMA completion
  tc_fence_after();
  // The kernel owns all 512 columns, so the allocation can only start at column 0; using the constant keeps
  // every tensor-memory address warp-uniform. Anything else is reported through *status and nothing runs.
  const uint32_t tmem_alloc = tmem_base_slot;
  constexpr uint32_t tmem_base = 0;
  const int total_slots = (tmem_alloc == 0) ? pair_total_slots(p) : 0;
  if (tmem_alloc != 0 && threadIdx.x == 0 && p.status) atomicExch(p.status, 2);

  // Warps 0 and 1 run their loops with all 32 lanes so that every loop variable is warp-uniform (the
  // compiler then keeps descriptors and addresses in uniform registers); only the asynchronous
  // instructions themselves are issued by one elected lane.
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint32_t leader_full0 = map_to_cta(full_bar(0), 0);
      long long w_empty = 0;
      PairItem it = {}, next_it = {};
      for (int slot = pair_next_item(p, pair, num_pairs, total_slots, it), next_slot; slot < total_slots && ok;
           slot = next_slot, it = next_it) {
        // the next item is worked out before this item's K loop: the divisions of its tile index stay off the
        // path between the last instruction of one tile and the first of the next
        next_slot = pair_next_item(p, slot + num_pairs, num_pairs, total_slots, next_it);
        const bool narrow = it.nt >= p.n_wide;  // N = 128 instruction: each CTA supplies 64 rows of B
        const int row_a = it.mt * 256 + static_cast<int>(rank) * 128;
        const int row_b = it.nt * BN + static_cast<int>(rank) * (narrow ? 64 : BN / 2);
        const int sfa_rt = it.mt * 2 + static_cast<int>(rank), sfb_rt = (it.nt * BN) >> 7;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          // (try_wait itself blocks for a while before it gives up, so the wait is timed around both)
          const long long t0 = probe ? clock64() : 0;
          if (!mbar_try_wait(empty_bar(s), ph ^ 1u)) ok = mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag);
          if (probe) w_empty += clock64() - t0;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (elect_one()) {
            if (rank == 0) mbar_expect_tx(full_bar(s), C::kTxBytes);
            const uint32_t leader_full = leader_full0 + 8 * s;
            tma2_load_2d(a_smem(s), &map_a, leader_full, kb * BK, row_a);
            tma2_load_2d(b_smem(s), &map_b, leader_full, kb * BK, row_b);  // 96-row box; rows past N read as 0
            tma2_load_3d(sfa_smem(s), &map_sfa, leader_full, 0, kb, sfa_rt);
            tma2_load_3d(sfb_smem(s), &map_sfb, leader_full, 0, kb, sfb_rt);  // the two 128-column chunks it spans
          }
          __syncwarp();
          if (++s == kStages2) { s = 0; ph ^= 1u; }
        }
        if (p.delta && it.kb1 == p.k_blocks) {
          // one stage per run of this tile's columns inside one delta block
          int c = it.nt * BN;
          const int c_end = min(c + (narrow ? 128 : BN), p.N);
          while (c < c_end) {
            const int blk = c / p.delta_block, p0 = c - blk * p.delta_block;
            const int n = min(c_end - c, p.delta_block - p0);
            if (!mbar_try_wait(empty_bar(s), ph ^ 1u)) ok = mbar_wait(empty_bar(s), ph ^ 1u, &abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (elect_one()) {
              if (rank == 0) mbar_expect_tx(full_bar(s), C::kTxBytes);
              const uint32_t leader_full = leader_full0 + 8 * s;
              const int prow = blk * p.M + row_a;  // row of the plane matrix [8 * M, 128]
              tma2_load_2d(a_smem(s), &map_pl, leader_full, 0, prow);
              tma2_load_2d(b_smem(s), &map_d, leader_full, 0, p0 + static_cast<int>(rank) * (n >> 1));
              tma2_load_3d(sfa_smem(s), &map_plsf, leader_full, 0, 0, prow >> 7);
              tma2_load_3d(sfb_smem(s), &map_dsf, leader_full, 0, 0, p0 >> 7);
            }
            __syncwarp();
            if (++s == kStages2) { s = 0; ph ^= 1u; }
            c += n;
          }
        }
      }
      if (probe && blockIdx.x == 0 && lane == 0) p.clock_probe[3] += w_empty;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0) {
      const uint32_t a_lo0 = (a_smem(0) >> 4) & 0x3fffu;
      const uint32_t sf_lo0 = (sfa_smem(0) >> 4) & 0x3fffu;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it_n = 0;
      uint32_t sf_rot = 0;  // scale buffer of the next K-block
      const uint32_t sf_mask = static_cast<uint32_t>(p.sf_bufs - 1);
      long long w_full = 0, w_acc = 0;
      PairItem it = {}, next_it = {};
      for (int slot = pair_next_item(p, pair, num_pairs, total_slots, it), next_slot; slot < total_slots && ok;
           slot = next_slot, it = next_it) {
        // the next item is worked out before this item's K loop: the divisions of its tile index stay off the
        // path between the last instruction of one tile and the first of the next
        next_slot = pair_next_item(p, slot + num_pairs, num_pairs, total_slots, next_it);
        const int as = it_n & 1;
        // the epilogues of both CTAs must have drained this buffer (used by item it_n - 2)
        const long long ta = probe ? clock64() : 0;
        ok = __all_sync(0xffffffffu, mbar_wait(acc_empty_bar(as), ((it_n >> 1) & 1u) ^ 1u, &abort_flag));
        if (C::kOverlap && ok && it_n > 0)  // the tile before this one has read the columns its buffer shares with ours
          ok = __all_sync(0xffffffffu, mbar_wait(ovl_free_bar(as ^ 1), ((it_n - 1) >> 1) & 1u, &abort_flag));
        if (probe) w_acc += clock64() - ta;
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (as ? C::kAcc1Col : 0);
        const uint32_t idesc = pair_idesc(it.nt >= p.n_wide ? 128 : BN);
        // a tile starts 0 or 64 columns into its first 128-column scale chunk: 32 columns per TMEM column
        const uint32_t sfb_off = ((it.nt * BN) & 127) >> 5;
        uint32_t acc = 0;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          const long long t0 = probe ? clock64() : 0;
          if (!mbar_try_wait(full_bar(s), ph)) ok = mbar_wait(full_bar(s), ph, &abort_flag);
          if (probe) w_full += clock64() - t0;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * ((C::kABytes + C::kBBytes) >> 4);
          const uint32_t sf_lo = sf_lo0 + s * (C::kSfBytes >> 4);
          // The scale columns rotate so that the copy for this K-block need not wait for the MMAs of the
          // previous one to have read theirs.
          const uint32_t sfa_t = tmem_base + C::kSfaCol + 16u * sf_rot, sfb_t = sfa_t + 4;
          if (elect_one())
            tc2_kblock(d_tmem, a_lo, a_lo + (C::kABytes >> 4), sf_lo, sfa_t, sfb_t, sfb_t + sfb_off, acc, empty_bar(s),
                       idesc);
          __syncwarp();
          acc = 1;
          sf_rot = (sf_rot + 1) & sf_mask;
          if (++s == kStages2) { s = 0; ph ^= 1u; }
        }
        if (ok && p.delta && it.kb1 == p.k_blocks) {
          const int col0 = it.nt * BN;
          int c = col0;
          const int c_end = min(c + (it.nt >= p.n_wide ? 128 : BN), p.N);
          while (c < c_end) {
            const int blk = c / p.delta_block, p0 = c - blk * p.delta_block;
            const int n = min(c_end - c, p.delta_block - p0);
            if (!mbar_try_wait(full_bar(s), ph)) ok = mbar_wait(full_bar(s), ph, &abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + s * ((C::kABytes + C::kBBytes) >> 4);
            const uint32_t sf_lo = sf_lo0 + s * (C::kSfBytes >> 4);
            const uint32_t sfa_t = tmem_base + C::kSfaCol + 16u * sf_rot, sfb_t = sfa_t + 4;
            if (elect_one())
              tc2_kblock(d_tmem + static_cast<uint32_t>(c - col0), a_lo, a_lo + (C::kABytes >> 4), sf_lo, sfa_t, sfb_t,
                         sfb_t + static_cast<uint32_t>((p0 & 127) >> 5), acc, empty_bar(s), pair_idesc(n));
            __syncwarp();
            acc = 1;
            sf_rot = (sf_rot + 1) & sf_mask;
            if (++s == kStages2) { s = 0; ph ^= 1u; }
            c += n;
          }
        }
        if (ok && elect_one()) tc2_commit_both(acc_full_bar(as));
        __syncwarp();
        ++it_n;
      }
      if (probe && blockIdx.x == 0 && lane == 0) {
        p.clock_probe[4] += w_full;
        p.clock_probe[5] += w_acc;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    // Each 128-row x 32-column chunk goes tensor memory -> registers -> (bias, rounding) -> a swizzled
    // shared-memory staging buffer -> one TMA store, which writes full lines and clips rows / columns that
    // lie outside C. Two staging buffers alternate; named barrier 1 joins the 128 epilogue threads.
    const int quad = warp & 3;          // the 32-lane quadrant of tensor memory this warp may read
    const int half = (warp - 2) >> 2;   // which share of the tile's column chunks this warp drains
    const int r_in = quad * 32 + lane;  // row inside this CTA's 128 accumulator rows
    // residual == C (bf16, same pitch): the tile is ADDED to C by the TMA store (bf16 add at the memory side)
    // instead of being loaded by the epilogue threads, whose per-chunk loads would serialise on latency.
    const bool reduce_add = p.residual && static_cast<const void*>(p.residual) == p.c && !p.out_fp32 && p.ldr == p.ldc;
    const bool issuer = threadIdx.x == 64 + 128 * half;  // one thread per half issues and tracks its TMA stores
    const uint32_t my_store = store_base + half * (2 * C::kStoreBytes);
    const int bar_id = 1 + half;  // named barrier of this half's 128 threads
    const uint32_t leader_empty0 = map_to_cta(acc_empty_bar(0), 0), leader_empty1 = map_to_cta(acc_empty_bar(1), 0);
    const uint32_t leader_ovl0 = map_to_cta(ovl_free_bar(0), 0), leader_ovl1 = map_to_cta(ovl_free_bar(1), 0);
    bool ok = true;
    int it_n = 0;
    uint32_t buf = 0;
    bool last_fp32 = false;
    long long w_idle = 0;
    PairItem it = {}, next_it = {};
    for (int slot = pair_next_item(p, pair, num_pairs, total_slots, it), next_slot; slot < total_slots && ok;
         slot = next_slot, it = next_it) {
      next_slot = pair_next_item(p, slot + num_pairs, num_pairs, total_slots, next_it);
      const int as = it_n & 1;
      const long long te = probe ? clock64() : 0;
      // the half that owns the columns shared with the other buffer is on the path to the next tile's first MMA:
      // it polls without backing off
      const bool ovl_owner = C::kOverlap && half == (as == 0 ? kEpiHalves - 1 : 0);
      if (!mbar_wait(acc_full_bar(as), (it_n >> 1) & 1u, &abort_flag, ovl_owner ? 0 : 200)) { ok = false; break; }
      if (probe) w_idle += clock64() - te;
      ++it_n;
      tc_fence_after();
      const bool partial = it.part >= 0;  // a K-range of a tail tile: raw fp32 accumulators to the scratch tile
      const int row0 = partial ? it.part * 256 + static_cast<int>(rank) * 128 : it.mt * 256 + static_cast<int>(rank) * 128;
      const int col_base = partial ? 0 : it.nt * BN;
      // 32-column chunks per half: the narrow column accumulates 128 columns only
      const int chunks = (it.nt >= p.n_wide ? 4 : BN / 32) / kEpiHalves;
      const bool fp32_stage = partial || p.out_fp32;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + (as ? C::kAcc1Col : 0);
      // Shared columns first: buffer 0 is drained from its last chunk down, buffer 1 from its first chunk up.
      const bool reverse = C::kOverlap && as == 0;
#pragma unroll 1
      for (int ci = 0; ci < chunks; ++ci, buf ^= 1u) {
        const int chunk = half * chunks + (reverse ? chunks - 1 - ci : ci);
        uint32_t v[32];
        tc_ld32(t_row + chunk * 32, v);
        tc_wait_ld();
        if (ovl_owner && ci == 0) {  // the next tile's MMAs may overwrite the shared columns
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(as ? leader_ovl1 : leader_ovl0);
        }
        if (ci == chunks - 1) {  // this warp's share is read: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(as ? leader_empty1 : leader_empty0);
        }
        const int col0 = col_base + chunk * 32;
        float f[32];
        if (partial) {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * p.alpha;
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                float bv[8];
                unpack8(*reinterpret_cast<const uint4*>(p.bias + col0 + j), bv);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[j + e] += bv[e];
              }
            }
          }
          if (p.residual && !reduce_add && row0 + r_in < p.M) {
            const __nv_bfloat16* res = p.residual + static_cast<int64_t>(row0 + r_in) * p.ldr + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                float bv[8];
                unpack8(*reinterpret_cast<const uint4*>(res + j), bv);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[j + e] += bv[e];
              }
            }
          }
        }
        const uint32_t stage = my_store + (fp32_stage ? 0u : buf * C::kStoreBytes);
        // The stores that last read the staging bytes about to be written must have finished reading them: all
        // earlier ones when this chunk or the previous one is fp32 (both buffers), else all but the latest.
        if (issuer) {
          if (fp32_stage || last_fp32)
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          else
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        }
        last_fp32 = fp32_stage;
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        if (fp32_stage) {  // 128-byte rows, 128-byte swizzle: 16-byte piece j of row r sits at piece j ^ (r & 7)
          const uint32_t rb = stage + r_in * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(rb + (((j ^ (r_in & 7))) << 4)), "f"(f[4 * j]),
                         "f"(f[4 * j + 1]), "f"(f[4 * j + 2]), "f"(f[4 * j + 3])
                         : "memory");
          }
        } else {  // 64-byte rows, 64-byte swizzle: piece j of row r sits at piece j ^ ((r >> 1) & 3)
          const uint32_t rb = stage + r_in * 64;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = f[8 * j + e];
            const uint4 w = pack8(o);
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(rb + ((j ^ ((r_in >> 1) & 3)) << 4)), "r"(w.x),
                         "r"(w.y), "r"(w.z), "r"(w.w)
                         : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the TMA engine
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        if (issuer) {
          if (partial)
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&map_part),
                         "r"(stage), "r"(col0), "r"(row0)
                         : "memory");
          else if (reduce_add)
            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             &map_c),
                         "r"(stage), "r"(col0), "r"(row0)
                         : "memory");
          else
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&map_c),
                         "r"(stage), "r"(col0), "r"(row0)
                         : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (probe && blockIdx.x == 0 && threadIdx.x == 64) p.clock_probe[6] += w_idle;
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  if (abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, 1);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA releases shared or tensor memory while its peer may still use it
  if (probe && blockIdx.x == 0 && threadIdx.x == 0) {
    p.clock_probe[0] += clock64() - probe_cycles0;
    p.clock_probe[1] += static_cast<long long>(global_timer_ns() - probe_ns0);
    p.clock_probe[2] += 1;  // launches seen
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_alloc), "r"(C::kTmemCols) : "memory");
  }
}

// C tile = sum over the K-range partials of a tail tile, in index order (reproducible), then the epilogue
// (alpha, bias, residual, rounding). One thread per 4 columns of a 256 x pair_bn tile.
__global__ void __launch_bounds__(256) pair_tail_finalize_kernel(const GemmParams p) {
  const int kBN2 = p.pair_bn;
  const int kPerRow = kBN2 / 4, kPerTile = 256 * kPerRow, kTileElems = 256 * kBN2;
  const int64_t total = static_cast<int64_t>(p.tail_tiles) * kPerTile;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / kPerTile), r = static_cast<int>(i - static_cast<int64_t>(t) * kPerTile);
    const int row_in = r / kPerRow, c4 = (r - row_in * kPerRow) * 4;
    int mt, nt;
    tile_coords(p, p.full_items + t, mt, nt);
    const int row = mt * 256 + row_in, col = nt * kBN2 + c4;
    if (row >= p.M || col >= p.N) continue;
    const float* src = p.pair_partial + static_cast<int64_t>(t) * p.tail_splits * kTileElems + row_in * kBN2 + c4;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int sp = 1; sp < p.tail_splits; ++sp) {
      const float4 v = *reinterpret_cast<const float4*>(src + static_cast<int64_t>(sp) * kTileElems);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= p.alpha; acc.y *= p.alpha; acc.z *= p.alpha; acc.w *= p.alpha;
    if (p.bias) {
      acc.x += __bfloat162float(p.bias[col]);
      acc.y += __bfloat162float(p.bias[col + 1]);
      acc.z += __bfloat162float(p.bias[col + 2]);
      acc.w += __bfloat162float(p.bias[col + 3]);
    }
    if (p.residual) {
      const __nv_bfloat16* res = p.residual + static_cast<int64_t>(row) * p.ldr + col;
      acc.x += __bfloat162float(res[0]);
      acc.y += __bfloat162float(res[1]);
      acc.z += __bfloat162float(res[2]);
      acc.w += __bfloat162float(res[3]);
    }
    if (p.out_fp32) {
      *reinterpret_cast<float4*>(static_cast<float*>(p.c) + static_cast<int64_t>(row) * p.ldc + col) = acc;
    } else {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(acc.x, acc.y);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.c) + static_cast<int64_t>(row) * p.ldc + col) = o;
    }
  }
}

// ------------------------------------------------------------------ host side
// u8 matrix [rows, k] row-major; box = 128 bytes along k x box_rows rows; 128-byte swizzle; OOB reads give 0.
bool make_map(CUtensorMap* map, const uint8_t* ptr, int64_t rows, int64_t k, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// TILED scale tensor viewed as u32 [row_tiles][k_blocks][128]: one 512-byte chunk per (row tile, K-block);
// box = box_rt chunks of consecutive row tiles at one K-block. Row tiles past the end read as 0.
bool make_sf_map(CUtensorMap* map, const uint8_t* ptr, int64_t row_tiles, int64_t k_blocks, int box_rt) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(k_blocks), static_cast<cuuint64_t>(row_tiles)};
  const cuuint64_t strides[2] = {512, static_cast<cuuint64_t>(512 * k_blocks)};
  const cuuint32_t box[3] = {128, 1, static_cast<cuuint32_t>(box_rt)};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<uint8_t*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// C [M, N] (bf16 or fp32, row pitch ldc) for the epilogue's TMA stores: box = 32 columns x 128 rows, swizzled
// like the staging buffer (64-byte rows for bf16, 128-byte rows for fp32). Stores outside [M, N] are dropped.
bool make_c_map(CUtensorMap* map, const GemmParams& p) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const int elt = p.out_fp32 ? 4 : 2;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.N), static_cast<cuuint64_t>(p.M)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ldc) * elt};
  const cuuint32_t box[2] = {32, 128};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, p.out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.c, dims, strides,
            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, p.out_fp32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The scratch of the K-split tail tiles viewed as fp32 [items * 256, tile width] for the epilogue's TMA stores.
bool make_part_map(CUtensorMap* map, float* ptr, int64_t items, int kBN2) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kBN2), static_cast<cuuint64_t>(std::max<int64_t>(items, 1) * 256)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kBN2) * 4};
  const cuuint32_t box[2] = {32, 128};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Device buffer of the clock probe per device (null = off).
long long* g_clock_probe[64] = {};

int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  return v ? atoi(v) : fallback;
}

// Work list of the CTA-pair kernel for one problem. A launch holds `pairs` CTA pairs; whole tiles are dealt
// round-robin in tile order, and what does not fill a last round, or
// the whole problem when it has fewer tiles than pairs, may be split along K so that every pair ends at about
// the same time instead of a few pairs running one more tile while the rest idle: the weight gradient
// dW[2048, 2048] over K = 32768 is 88 tiles on 74 pairs, i.e. two rounds for 1.19 rounds of work.
// The choice minimises the modelled finish time (unit: one K-block of a wide tile; a narrow tile costs 128 / width,
// every item a constant, a split item a larger constant for its fp32 partial store, the finalize pass a
// constant) over the number of splits; it depends on the shape and the SM count only, so results are
// reproducible from call to call.
struct PairPlan {
  int pairs, n_wide, narrow, full_items, tail_tiles, tail_splits, tail_kbs, tail_shift, bn;
  int64_t ws_bytes;
};

PairPlan plan_pair_uncached(int64_t M, int64_t N, int64_t K, bool allow_split, int sms, int kBN2) {
  PairPlan pl{};
  pl.bn = kBN2;
  const int m_tiles = static_cast<int>(ceil_div(M, 256));
  pl.n_wide = static_cast<int>(N / kBN2);
  const int rem_cols = static_cast<int>(N - static_cast<int64_t>(pl.n_wide) * kBN2);
  pl.narrow = (rem_cols > 0 && rem_cols <= 128 && env_int("ANIMA_MX_GEMM_NARROW", 1)) ? 1 : 0;
  if (rem_cols > 0 && !pl.narrow) pl.n_wide += 1;
  const int n_tiles = pl.n_wide + pl.narrow, tiles = m_tiles * n_tiles;
  const int kb = static_cast<int>(ceil_div(K, BK));
  const int max_pairs = std::max(1, sms / 2);
  const double kItem = 1.0, kSplitItem = 8.0, kFinalize = 36.0;   // the finalize launch measures 5 - 10 us, a K-block 0.27 us
  auto tile_cost = [&](int tile, double frac) {
    int mt, nt;
    tile_coords_of(m_tiles, n_tiles, tile, mt, nt);
    return (nt < pl.n_wide ? 1.0 : 128.0 / kBN2) * kb * frac;
  };

  double best = 1e300;
  std::vector<double> load;
  auto consider = [&](int pairs, int full_items, int splits) {
    const int tail = tiles - full_items;
    const int kbs = static_cast<int>(ceil_div(kb, splits));
    if (static_cast<int>(ceil_div(kb, kbs)) != splits) return;   // would leave an empty K-range
    load.assign(pairs, 0.0);
    for (int i = 0; i < full_items; ++i) load[i % pairs] += tile_cost(i, 1.0) + kItem;
    int shift = 0;
    for (int q = 1; q < pairs; ++q)
      if (load[q] < load[shift]) shift = q;                       // the round robin resumes at the least loaded pair
    for (int t = 0; t < tail; ++t)
      for (int sp = 0; sp < splits; ++sp) {
        const int kbn = std::min(kb, (sp + 1) * kbs) - sp * kbs;
        load[(shift + t * splits + sp) % pairs] +=
            tile_cost(full_items + t, static_cast<double>(kbn) / kb) + (splits > 1 ? kSplitItem : kItem);
      }
    double finish = 0.0;
    for (double l : load) finish = std::max(finish, l);
    if (splits > 1) finish += kFinalize;
    if (finish < best - 1e-9) {
      best = finish;
      pl.pairs = pairs;
      pl.full_items = full_items;
      pl.tail_tiles = tail;
      pl.tail_splits = splits;
      pl.tail_kbs = kbs;
      pl.tail_shift = tail ? shift : 0;
    }
  };
  const int base_pairs = std::min(tiles, max_pairs);
  const int base_full = tiles / base_pairs * base_pairs;
  consider(base_pairs, base_full, 1);
  if (allow_split && kb >= 2 && env_int("ANIMA_MX_GEMM_TAIL", 1)) {
    const int max_splits = std::min(kb, 32);
    if (base_full < tiles)
      for (int sp = 2; sp <= max_splits; ++sp) consider(base_pairs, base_full, sp);
    if (tiles < max_pairs)                                          // fewer tiles than pairs: split all of them
      for (int sp = 2; sp <= max_splits; ++sp) consider(max_pairs, 0, sp);
  }
  pl.ws_bytes = pl.tail_splits > 1 ? static_cast<int64_t>(pl.tail_tiles) * pl.tail_splits * 256 * kBN2 * 4 : 0;
  return pl;
}

// Tile width for a problem: 256 when a tile holds at least 32 K-blocks (its start-up gap is then under a
// tenth of the tile), else 192. ANIMA_MX_GEMM_BN = 192 / 256 forces one (read per call; for tests and tuning).
int pair_tile_width(int64_t K) {
  const int forced = env_int("ANIMA_MX_GEMM_BN", 0);
  if (forced == 192 || forced == 256) return forced;
  return K >= 4096 ? 256 : 192;
}

PairPlan plan_pair(int64_t M, int64_t N, int64_t K, bool allow_split) {
  const int sms = sm_count();
  const int bn = pair_tile_width(K);
  const int narrow = env_int("ANIMA_MX_GEMM_NARROW", 1), tail = env_int("ANIMA_MX_GEMM_TAIL", 1);
  using Key = std::tuple<int64_t, int64_t, int64_t, int, int>;
  static std::mutex mu;
  static std::map<Key, PairPlan> cache;
  const Key key{M, N, K, sms, (allow_split ? 1 : 0) | (narrow ? 2 : 0) | (tail ? 4 : 0) | (bn == 256 ? 8 : 0)};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (cache.size() > 4096) cache.clear();
  const PairPlan pl = plan_pair_uncached(M, N, K, allow_split, sms, bn);
  cache.emplace(key, pl);
  return pl;
}

// Operands of the low-rank delta (all null = none): the eight activation planes [8 * M, 128] and the factor
// [block, 128] whose rows are the output columns inside one block, both K-major e4m3 with TILED scales.
struct DeltaOperands {
  const uint8_t* planes_codes;
  const uint8_t* planes_scales;
  const uint8_t* d_codes;
  const uint8_t* d_scales;
  int64_t block;
};

template <int BN>
int launch_pair_width(const uint8_t* a_codes, const uint8_t* b_codes, GemmParams p, const PairPlan& pl, void* workspace,
                      const DeltaOperands& delta, cudaStream_t s);

int launch_pair(const uint8_t* a_codes, const uint8_t* b_codes, GemmParams p, void* workspace, int64_t workspace_bytes,
                const DeltaOperands& delta, cudaStream_t s) {
  const PairPlan pl = plan_pair(p.M, p.N, p.K, workspace != nullptr);
  ANIMA_REQUIRE(workspace_bytes >= pl.ws_bytes, ANIMA_E_WORKSPACE,
                "mx_gemm: workspace of %lld bytes is too small (need %lld)", (long long)workspace_bytes,
                (long long)pl.ws_bytes);
  return pl.bn == 256 ? launch_pair_width<256>(a_codes, b_codes, p, pl, workspace, delta, s)
                      : launch_pair_width<192>(a_codes, b_codes, p, pl, workspace, delta, s);
}

template <int kBN2>
int launch_pair_width(const uint8_t* a_codes, const uint8_t* b_codes, GemmParams p, const PairPlan& pl, void* workspace,
                      const DeltaOperands& delta, cudaStream_t s) {
  using C2 = Cfg2<kBN2>;
  static PerDeviceOnce once;
  const cudaError_t attr_rc = per_device_once(once, [] {
    return cudaFuncSetAttribute(mx_gemm2_kernel<kBN2>, cudaFuncAttributeMaxDynamicSharedMemorySize, C2::kSmemBytes);
  });
  ANIMA_REQUIRE(attr_rc == cudaSuccess, ANIMA_E_CUDA, "mx_gemm: cannot reserve %d bytes of shared memory: %s",
                C2::kSmemBytes, cudaGetErrorString(attr_rc));
  p.m_tiles = static_cast<int>(ceil_div(p.M, 256));
  p.n_wide = pl.n_wide;
  p.narrow = pl.narrow;
  p.n_tiles = pl.n_wide + pl.narrow;
  p.pair_bn = kBN2;
  p.full_items = pl.full_items;
  p.tail_tiles = pl.tail_tiles;
  p.tail_splits = pl.tail_splits;
  p.tail_kbs = pl.tail_kbs;
  p.tail_shift = pl.tail_shift;
  p.pair_partial = pl.ws_bytes ? static_cast<float*>(workspace) : nullptr;
  {
    int dev = 0;
    p.clock_probe = (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) ? g_clock_probe[dev] : nullptr;
  }
  const int sf_bufs = env_int("ANIMA_MX_GEMM_SFBUFS", C2::kMaxSfBufs);
  p.sf_bufs = (sf_bufs == 1 || sf_bufs == 2) ? sf_bufs : C2::kMaxSfBufs;
  CUtensorMap ma, mb, msa, msb, mc, mp;
  ANIMA_REQUIRE(make_map(&ma, a_codes, p.M, p.K, 128) && make_map(&mb, b_codes, p.N, p.K, kBN2 / 2) &&
                    make_sf_map(&msa, p.a_scales, p.sfa_rt, p.k_blocks, 1) &&
                    make_sf_map(&msb, p.b_scales, p.sfb_rt, p.k_blocks, kSfbChunks2) && make_c_map(&mc, p) &&
                    (pl.ws_bytes ? make_part_map(&mp, p.pair_partial, static_cast<int64_t>(pl.tail_tiles) * pl.tail_splits, kBN2)
                                 : make_c_map(&mp, p)),
                ANIMA_E_CUDA, "mx_gemm: cuTensorMapEncodeTiled failed (driver entry point missing or bad operand)");
  CUtensorMap mpl = ma, md = mb, mplsf = msa, mdsf = msb;   // placeholders when there is no delta
  p.delta = delta.planes_codes ? 1 : 0;
  p.delta_block = static_cast<int>(delta.block);
  if (p.delta) {
    const int64_t plane_rows = 8 * static_cast<int64_t>(p.M);
    ANIMA_REQUIRE(make_map(&mpl, delta.planes_codes, plane_rows, 128, 128) &&
                      make_map(&md, delta.d_codes, delta.block, 128, kBN2 / 2) &&
                      make_sf_map(&mplsf, delta.planes_scales, plane_rows / 128, 1, 1) &&
                      make_sf_map(&mdsf, delta.d_scales, ceil_div(delta.block, 128), 1, kSfbChunks2),
                  ANIMA_E_CUDA, "mx_gemm_delta: cuTensorMapEncodeTiled failed (driver entry point missing or bad operand)");
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pl.pairs);
  cfg.blockDim = dim3(kThreads2);
  cfg.dynamicSmemBytes = C2::kSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t rc = cudaLaunchKernelEx(&cfg, mx_gemm2_kernel<kBN2>, ma, mb, msa, msb, mc, mp, mpl, md, mplsf, mdsf, p);
  ANIMA_REQUIRE(rc == cudaSuccess, ANIMA_E_CUDA, "mx_gemm: cluster launch failed: %s", cudaGetErrorString(rc));
  if (pl.ws_bytes) {
    const int64_t threads = static_cast<int64_t>(pl.tail_tiles) * 256 * (kBN2 / 4);
    pair_tail_finalize_kernel<<<static_cast<unsigned>(std::min<int64_t>(ceil_div(threads, 256), 8LL * sm_count())), 256, 0,
                                s>>>(p);
    ANIMA_CHECK_LAUNCH("mx_gemm K-split tail finalize");
  }
  return ANIMA_OK;
}

// 0 = choose by shape, 1 = one CTA per tile, 2 = CTA pairs (ANIMA_MX_GEMM_VARIANT, read per call; for tests).
int forced_variant() {
  const char* v = getenv("ANIMA_MX_GEMM_VARIANT");
  return v ? atoi(v) : 0;
}

template <int BN, int EPI = 4>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams p, cudaStream_t s) {
  static PerDeviceOnce once;
  const cudaError_t attr_rc = per_device_once(once, [] {
    return cudaFuncSetAttribute(mx_gemm_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Cfg<BN>::kSmemBytes);
  });
  ANIMA_REQUIRE(attr_rc == cudaSuccess, ANIMA_E_CUDA, "mx_gemm: cannot reserve %d bytes of shared memory: %s",
                Cfg<BN>::kSmemBytes, cudaGetErrorString(attr_rc));
  p.n_tiles = static_cast<int>(ceil_div(p.N, BN));
  const int items = p.m_tiles * p.n_tiles * p.splits;
  const int grid = std::min(items, sm_count());
  mx_gemm_kernel<BN, EPI><<<grid, 64 + 32 * EPI, Cfg<BN>::kSmemBytes, s>>>(ma, mb, p);
  ANIMA_CHECK_LAUNCH("mx_gemm");
  if (p.splits > 1) {
    const int64_t groups = static_cast<int64_t>(p.M) * (p.N / 4);
    splitk_finalize_kernel<<<static_cast<unsigned>(std::min<int64_t>(ceil_div(groups, 256), 4LL * sm_count())), 256, 0,
                             s>>>(p);
    ANIMA_CHECK_LAUNCH("mx_gemm split-K finalize");
  }
  return ANIMA_OK;
}

// Does the shape go to the CTA-pair kernel?
bool use_pair(int64_t M, int64_t N) {
  const int variant = forced_variant();
  // CTA pairs pay off once a 256 x 256 tile is mostly full; small or narrow problems keep one CTA per tile.
  return variant == 2 || (variant == 0 && N > 128 && M > 128);
}

// Split-K plan of the one-CTA kernel: a small output with a long contraction (the T-LoKr factor
// gradients are [128..1024, 128..1024] over K = rows * 8 = 262144) would otherwise occupy 1 - 8 SMs.
// Splits are sized to fill the GPU once, with at least 8 K-blocks (1024 elements of K) per split.
void plan_splits(int64_t M, int64_t N, int64_t K, int* splits, int* kb_per_split) {
  const int kb = static_cast<int>(ceil_div(K, BK));
  *splits = 1;
  *kb_per_split = kb;
  if (use_pair(M, N) || N % 4 != 0) return;
  const int64_t tiles = ceil_div(M, BM) * ceil_div(N, N > 128 ? 256 : 128);
  const int sms = sm_count();
  if (tiles * 2 > sms || kb < 32) return;
  const int want = static_cast<int>(std::min<int64_t>(sms / tiles, kb / 8));
  if (want < 2) return;
  *kb_per_split = static_cast<int>(ceil_div(kb, want));
  *splits = static_cast<int>(ceil_div(kb, *kb_per_split));
}

}  // namespace
}  // namespace anima

using namespace anima;

static int mx_gemm_impl(const uint8_t* a_codes, const uint8_t* a_scales, const uint8_t* b_codes,
                        const uint8_t* b_scales, void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                        const void* bias, const void* residual, int64_t ldr, float alpha, int out_dtype,
                        void* workspace, int64_t workspace_bytes, int32_t* status, void* stream,
                        const DeltaOperands& delta = DeltaOperands{}) {
  ANIMA_REQUIRE(!residual || (aligned16(residual) && ldr >= N && ldr % 8 == 0), ANIMA_E_ALIGN,
                "mx_gemm: residual must be 16-byte aligned with a row pitch that is a multiple of 8 elements");
  ANIMA_REQUIRE(a_codes && a_scales && b_codes && b_scales && c, ANIMA_E_ARG, "mx_gemm: null pointer");
  ANIMA_REQUIRE(M > 0 && N > 0 && K > 0 && ldc >= N, ANIMA_E_ARG, "mx_gemm: bad sizes M=%lld N=%lld K=%lld ldc=%lld",
                (long long)M, (long long)N, (long long)K, (long long)ldc);
  ANIMA_REQUIRE(M < (1ll << 31) - 256 && N < (1ll << 31) - 256 && K < (1ll << 31) - 256, ANIMA_E_TOO_LARGE,
                "mx_gemm: a dimension exceeds 2^31");
  ANIMA_REQUIRE(K % 32 == 0, ANIMA_E_SHAPE, "mx_gemm: K=%lld must be a multiple of 32", (long long)K);
  ANIMA_REQUIRE(out_dtype == 0 || out_dtype == 1, ANIMA_E_ARG, "mx_gemm: out_dtype must be 0 (bf16) or 1 (fp32)");
  const int celt = out_dtype ? 4 : 2;
  ANIMA_REQUIRE(N % 8 == 0 && (ldc * celt) % 16 == 0, ANIMA_E_SHAPE,
                "mx_gemm: N must be a multiple of 8 and the row pitch of C a multiple of 16 bytes");
  ANIMA_REQUIRE(aligned16(a_codes) && aligned16(b_codes) && aligned16(a_scales) && aligned16(b_scales) &&
                    aligned16(c) && (!bias || aligned16(bias)),
                ANIMA_E_ALIGN, "mx_gemm: all buffers must be 16-byte aligned");
  GemmParams p{};
  p.a_scales = a_scales;
  p.b_scales = b_scales;
  p.c = c;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.ldc = ldc;
  p.out_fp32 = out_dtype;
  p.m_tiles = static_cast<int>(ceil_div(M, BM));
  p.k_blocks = static_cast<int>(ceil_div(K, BK));
  p.sfa_rt = static_cast<int>(ceil_div(M, 128));
  p.sfb_rt = static_cast<int>(ceil_div(N, 128));
  p.splits = 1;
  p.kb_per_split = p.k_blocks;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.alpha = alpha;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ANIMA_REQUIRE(!workspace || aligned16(workspace), ANIMA_E_ALIGN, "mx_gemm: workspace must be 16-byte aligned");
  if (use_pair(M, N)) return launch_pair(a_codes, b_codes, p, workspace, workspace_bytes, delta, s);
  ANIMA_REQUIRE(!delta.planes_codes, ANIMA_E_UNSUPPORTED,
                "mx_gemm_delta: M=%lld N=%lld runs on the one-CTA kernel, which has no delta K-blocks", (long long)M,
                (long long)N);
  if (workspace) {
    int splits, kb_per;
    plan_splits(M, N, K, &splits, &kb_per);
    if (splits > 1) {
      ANIMA_REQUIRE(workspace_bytes >= static_cast<int64_t>(splits) * M * N * 4, ANIMA_E_WORKSPACE,
                    "mx_gemm: workspace of %lld bytes is too small (need %lld)", (long long)workspace_bytes,
                    (long long)(static_cast<int64_t>(splits) * M * N * 4));
      p.splits = splits;
      p.kb_per_split = kb_per;
      p.partial = static_cast<float*>(workspace);
    }
  }
  const bool wide = N > 128;
  CUtensorMap ma, mb;
  ANIMA_REQUIRE(make_map(&ma, a_codes, M, K, BM) && make_map(&mb, b_codes, N, K, wide ? 256 : 128), ANIMA_E_CUDA,
                "mx_gemm: cuTensorMapEncodeTiled failed (driver entry point missing or bad operand)");
  return wide ? launch<256>(ma, mb, p, s) : launch<128>(ma, mb, p, s);
}

extern "C" int anima_mx_gemm(const uint8_t* a_codes, const uint8_t* a_scales, const uint8_t* b_codes,
                             const uint8_t* b_scales, void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                             const void* bias, int out_dtype, int32_t* status, void* stream) {
  return mx_gemm_impl(a_codes, a_scales, b_codes, b_scales, c, M, N, K, ldc, bias, nullptr, 0, 1.f, out_dtype, nullptr,
                      0, status, stream);
}

extern "C" int64_t anima_mx_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return ANIMA_E_ARG;
  if (M >= (1ll << 31) - 256 || N >= (1ll << 31) - 256 || K >= (1ll << 31) - 256) return ANIMA_E_TOO_LARGE;
  if (use_pair(M, N)) return plan_pair(M, N, K, true).ws_bytes;
  int splits, kb_per;
  plan_splits(M, N, K, &splits, &kb_per);
  return splits > 1 ? static_cast<int64_t>(splits) * M * N * 4 : 0;
}

extern "C" int anima_mx_gemm_ex(const uint8_t* a_codes, const uint8_t* a_scales, const uint8_t* b_codes,
                                const uint8_t* b_scales, void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                                const void* bias, const void* residual, int64_t ldr, float alpha, int out_dtype,
                                void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  return mx_gemm_impl(a_codes, a_scales, b_codes, b_scales, c, M, N, K, ldc, bias, residual, ldr, alpha, out_dtype,
                      workspace, workspace_bytes, status, stream);
}

extern "C" int anima_mx_gemm_pair_plan(int64_t M, int64_t N, int64_t K, int with_workspace, int32_t* out9) {
  ANIMA_REQUIRE(out9 != nullptr, ANIMA_E_ARG, "mx_gemm_pair_plan: null pointer");
  ANIMA_REQUIRE(M > 0 && N > 0 && K > 0, ANIMA_E_ARG, "mx_gemm_pair_plan: bad sizes");
  ANIMA_REQUIRE(M < (1ll << 31) - 256 && N < (1ll << 31) - 256 && K < (1ll << 31) - 256, ANIMA_E_TOO_LARGE,
                "mx_gemm_pair_plan: a dimension exceeds 2^31");
  if (!use_pair(M, N)) return 1;
  const PairPlan pl = plan_pair(M, N, K, with_workspace != 0);
  const int32_t v[9] = {pl.pairs, pl.n_wide, pl.narrow, pl.full_items, pl.tail_tiles, pl.tail_splits, pl.tail_kbs,
                        pl.tail_shift, pl.bn};
  for (int i = 0; i < 9; ++i) out9[i] = v[i];
  return ANIMA_OK;
}

extern "C" int anima_mx_gemm_set_clock_probe(void* device_buffer_8xint64) {
  int dev = 0;
  const cudaError_t rc = cudaGetDevice(&dev);
  ANIMA_REQUIRE(rc == cudaSuccess && dev >= 0 && dev < 64, ANIMA_E_CUDA, "mx_gemm_set_clock_probe: no current device");
  ANIMA_REQUIRE(!device_buffer_8xint64 || (reinterpret_cast<uintptr_t>(device_buffer_8xint64) & 7) == 0, ANIMA_E_ALIGN,
                "mx_gemm_set_clock_probe: buffer must be 8-byte aligned");
  g_clock_probe[dev] = static_cast<long long*>(device_buffer_8xint64);
  return ANIMA_OK;
}

extern "C" int anima_mx_gemm_delta(const uint8_t* a_codes, const uint8_t* a_scales, const uint8_t* b_codes,
                                   const uint8_t* b_scales, void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                                   const void* bias, int out_dtype, const uint8_t* planes_codes,
                                   const uint8_t* planes_scales, const uint8_t* d_codes, const uint8_t* d_scales,
                                   void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  ANIMA_REQUIRE(planes_codes && planes_scales && d_codes && d_scales, ANIMA_E_ARG, "mx_gemm_delta: null delta operand");
  ANIMA_REQUIRE(aligned16(planes_codes) && aligned16(planes_scales) && aligned16(d_codes) && aligned16(d_scales),
                ANIMA_E_ALIGN, "mx_gemm_delta: delta operands must be 16-byte aligned");
  ANIMA_REQUIRE(M > 0 && N > 0 && M % 128 == 0 && N % 8 == 0 && (N / 8) % 64 == 0, ANIMA_E_SHAPE,
                "mx_gemm_delta: needs M %% 128 == 0 and N / 8 a multiple of 64 (M=%lld N=%lld)", (long long)M,
                (long long)N);
  DeltaOperands delta{planes_codes, planes_scales, d_codes, d_scales, N / 8};
  return mx_gemm_impl(a_codes, a_scales, b_codes, b_scales, c, M, N, K, ldc, bias, nullptr, 0, 1.f, out_dtype, workspace,
                      workspace_bytes, status, stream, delta);
}

extern "C" int anima_tlokr_hidden_mix_planes(const uint8_t* g_codes, const uint8_t* g_scales, const uint8_t* f_codes,
                                             const uint8_t* f_scales, const void* c, const void* mask, int64_t batch,
                                             int64_t n_per_batch, int64_t k, int transpose, void* hidden_out,
                                             uint8_t* planes_codes, uint8_t* planes_scales, int32_t* status,
                                             void* stream) {
  ANIMA_REQUIRE(g_codes && g_scales && f_codes && f_scales && c && planes_codes && planes_scales, ANIMA_E_ARG,
                "tlokr_hidden_mix_planes: null pointer");
  ANIMA_REQUIRE(batch > 0 && n_per_batch > 0 && k > 0, ANIMA_E_ARG, "tlokr_hidden_mix_planes: bad sizes");
  const int64_t items = batch * n_per_batch, M = items * 8;
  ANIMA_REQUIRE(items % 128 == 0 && k % 32 == 0, ANIMA_E_SHAPE,
                "tlokr_hidden_mix_planes: batch * n = %lld must be a multiple of 128 and k = %lld of 32", (long long)items,
                (long long)k);
  ANIMA_REQUIRE(M < (1ll << 31) - 256 && k < (1ll << 31) - 256, ANIMA_E_TOO_LARGE, "tlokr_hidden_mix_planes: too large");
  ANIMA_REQUIRE(aligned16(g_codes) && aligned16(g_scales) && aligned16(f_codes) && aligned16(f_scales) &&
                    aligned16(planes_codes) && aligned16(planes_scales) && (!mask || aligned16(mask)) &&
                    (!hidden_out || aligned16(hidden_out)),
                ANIMA_E_ALIGN, "tlokr_hidden_mix_planes: buffers must be 16-byte aligned");
  GemmParams p{};
  p.a_scales = g_scales;
  p.b_scales = f_scales;
  p.c = planes_codes;   // not written through the ordinary epilogue
  p.status = status;
  p.M = static_cast<int>(M);
  p.N = 128;
  p.K = static_cast<int>(k);
  p.ldc = 128;
  p.m_tiles = static_cast<int>(M / BM);
  p.k_blocks = static_cast<int>(ceil_div(k, BK));
  p.sfa_rt = p.m_tiles;
  p.sfb_rt = 1;
  p.splits = 1;
  p.kb_per_split = p.k_blocks;
  p.alpha = 1.f;
  p.mix_c = static_cast<const __nv_bfloat16*>(c);
  p.mix_mask = static_cast<const __nv_bfloat16*>(mask);
  p.mix_codes = planes_codes;
  p.mix_scales = planes_scales;
  p.mix_hidden = static_cast<__nv_bfloat16*>(hidden_out);
  p.mix_items = items;
  p.mix_n_per_batch = n_per_batch;
  p.mix_transpose = transpose ? 1 : 0;
  CUtensorMap ma, mb;
  ANIMA_REQUIRE(make_map(&ma, g_codes, M, k, BM) && make_map(&mb, f_codes, 128, k, 128), ANIMA_E_CUDA,
                "tlokr_hidden_mix_planes: cuTensorMapEncodeTiled failed (driver entry point missing or bad operand)");
  return launch<128, 8>(ma, mb, p, static_cast<cudaStream_t>(stream));
}
