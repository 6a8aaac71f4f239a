// MXFP8 block-scaled GEMM for sm_100a: C[M,N] = A[M,K] . B[N,K]^T (+ bias).
//
// Replaces anima-trainer's Triton tl.dot_scaled kernel (mxfp8_gemm.py:254-336) and
// the Transformer-Engine general_gemm calls of fp8_quant.py (:150, :236 forward;
// :504 dgrad; :507 wgrad). Both operands are e4m3 codes contiguous along K with one
// e8m0 scale per 32 K-elements in the 128x4 tiled layout (see anima_b200.h), so the
// forward, dgrad and wgrad GEMMs are all this one "TN" form.
//
// Design (one persistent CTA per SM, 192 threads, warp-specialised):
//   warp 0  TMA producer: per K-block of 128 one 128x128 A box and one BNx128 B box
//           (128-byte swizzle) plus the 512-byte scale chunks (bulk copies), all
//           completing on the stage's "full" mbarrier; 4-stage shared-memory ring.
//   warp 1  MMA issuer: copies the stage's scale chunks shared -> tensor memory
//           (tcgen05.cp 32x128b.warpx4), issues four
//           tcgen05.mma.kind::mxf8f6f4.block_scale (M128 x N{128,256} x K32) per
//           stage, and frees the stage / publishes the accumulator with
//           tcgen05.commit. Accumulators live in tensor memory (fp32).
//   warps 2-5 epilogue: tcgen05.ld the 128 x BN accumulator in 32-column chunks,
//           add bias, round to bf16 (or keep fp32) and store 64/128 contiguous bytes
//           per thread.
// Two accumulator buffers let the epilogue of tile i overlap the main loop of tile
// i+1. For BN = 256 the 512 tensor-memory columns cannot hold two full buffers plus
// the scale columns, so buffer 1 starts 32 columns before the end of buffer 0 and
// the epilogue always drains those shared 32 columns first, then releases the MMA
// warp. Every wait is bounded; on a timeout the kernel raises *status, lets copies
// in flight land, frees its tensor memory and returns.
// Tensor-pipe bound: 2*M*N*K flop; no TMA multicast is used anywhere.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace anima {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;  // bytes == e4m3 elements per K-block
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kSfChunk = 512;
constexpr uint64_t kWaitLimitNs = 2000000000ull;

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

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false if another role already aborted or ~2 s passed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t spins = 0;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63u) == 63u) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
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
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
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
    mbar_init(acc_free_bar, 4);
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

  const int total_tiles = p.m_tiles * p.n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t kiter = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mt = tile / p.n_tiles, nt = tile - mt * p.n_tiles;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++kiter) {
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
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const int as = it & 1;
        if (it > 0) {
          // The previous tile's epilogue must have drained the columns shared by the two buffers
          // (and, by program order, finished the tile before it, which used this buffer).
          if (!mbar_wait(acc_free_bar, (it - 1) & 1u, &abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        const uint32_t d_tmem = tmem_base + (as ? C::kAcc1Col : 0);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++kiter) {
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
                        tmem_base + C::kSfbCol, (kb | k) != 0 ? 1u : 0u);
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
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const int mt = tile / p.n_tiles, nt = tile - mt * p.n_tiles;
      const int as = it & 1;
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
        const int col = nt * BN + chunk * 32;
        if (row < p.M && col < p.N) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
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

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

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

template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams p, cudaStream_t s) {
  static std::once_flag once;
  static cudaError_t attr_rc = cudaSuccess;
  std::call_once(once, [] {
    attr_rc = cudaFuncSetAttribute(mx_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   Cfg<BN>::kSmemBytes);
  });
  ANIMA_REQUIRE(attr_rc == cudaSuccess, ANIMA_E_CUDA, "mx_gemm: cannot reserve %d bytes of shared memory: %s",
                Cfg<BN>::kSmemBytes, cudaGetErrorString(attr_rc));
  p.n_tiles = static_cast<int>(ceil_div(p.N, BN));
  const int tiles = p.m_tiles * p.n_tiles;
  const int grid = std::min(tiles, sm_count());
  mx_gemm_kernel<BN><<<grid, kThreads, Cfg<BN>::kSmemBytes, s>>>(ma, mb, p);
  ANIMA_CHECK_LAUNCH("mx_gemm");
  return ANIMA_OK;
}

}  // namespace
}  // namespace anima

using namespace anima;

extern "C" int anima_mx_gemm(const uint8_t* a_codes, const uint8_t* a_scales, const uint8_t* b_codes,
                             const uint8_t* b_scales, void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                             const void* bias, int out_dtype, int32_t* status, void* stream) {
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
  CUtensorMap ma, mb;
  const bool wide = N > 128;
  ANIMA_REQUIRE(make_map(&ma, a_codes, M, K, BM) && make_map(&mb, b_codes, N, K, wide ? 256 : 128), ANIMA_E_CUDA,
                "mx_gemm: cuTensorMapEncodeTiled failed (driver entry point missing or bad operand)");
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
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return wide ? launch<256>(ma, mb, p, s) : launch<128>(ma, mb, p, s);
}
