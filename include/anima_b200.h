/*
 * anima_b200.h — C ABI of libanima_b200.so: hand-written sm_100a CUDA for the
 * quantised-linear hot path of anima-trainer (MXFP8 quantise, block-scaled
 * GEMM fwd/dgrad/wgrad with the LoKr delta, fused AdaLN + gated residual,
 * T-LoKr rank mix and its weight gradient).
 *
 * Citations "ref: <file>:<lines>" name the anima-trainer interface (paths
 * relative to that project's root) that an entry point replaces.
 *
 * Conventions for every function below
 *   - all pointers are DEVICE pointers unless the name says otherwise;
 *   - tensors are dense row-major; "bf16" means 16-bit bfloat words;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - nothing allocates, frees or synchronises; scratch memory is passed in by
 *     the caller and its size is given by the matching *_workspace_bytes();
 *   - the return value is ANIMA_OK or a negative ANIMA_E_* code; the text for
 *     the last failure on the calling thread is anima_last_error();
 *   - there is no CPU fallback: with no usable GPU the call fails.
 */
#ifndef ANIMA_B200_H_
#define ANIMA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ANIMA_ABI_VERSION 1

enum {
  ANIMA_OK = 0,
  ANIMA_E_ARG = -1,         /* null pointer, negative size, bad enum             */
  ANIMA_E_ALIGN = -2,       /* pointer or leading dimension not 16-byte aligned  */
  ANIMA_E_SHAPE = -3,       /* size not divisible as the kernel requires         */
  ANIMA_E_CUDA = -4,        /* a CUDA runtime/driver call failed                 */
  ANIMA_E_UNSUPPORTED = -5, /* valid request this build has no kernel for        */
  ANIMA_E_WORKSPACE = -6,   /* workspace pointer null or too small               */
  ANIMA_E_TOO_LARGE = -7    /* exceeds a fixed capacity of the entry point       */
};

/* Layout of an e8m0 scale tensor that belongs to a code matrix [rows, k]
 * quantised along k in blocks of 32 (kb = k/32 scale bytes per row).
 *   PLAIN  : [rows, kb] row-major — the layout of ref: mxfp8_gemm.py:51-65.
 *   TILED  : the tensor-core operand layout. Rows are padded to 128 and kb to 4;
 *            tile (rt, kt) = 128 rows x 4 scale bytes is a contiguous 512-byte
 *            chunk at ((rt * ceil(kb/4)) + kt) * 512, and inside a chunk the
 *            byte of (r, j) sits at (r % 32) * 16 + (r / 32) * 4 + j.
 *            Padding bytes are written as 0. */
enum { ANIMA_SCALES_PLAIN = 0, ANIMA_SCALES_TILED = 1 };

int anima_abi_version(void);
const char* anima_last_error(void);

/* ---------------------------------------------------------------- MXFP8 quantise
 * ref: mxfp8_gemm.py:68-183 (quantize_rowwise + _quantize_rowwise_kernel),
 *      mxfp8_gemm.py:186-222 (quantize_weight_for_lhs / quantize_weight_for_dgrad).
 *
 * x is bf16 [rows, cols] with row pitch ld_x elements. Per group of 32 elements:
 *   amax = max(max|x|, 1e-30); e = ceil(log2(amax / 448)) clamped to [-127, 127];
 *   code = e4m3(x * 2^-e) round-to-nearest-even, saturating at +-448; scale byte = e + 127.
 * Two optional outputs, produced from ONE read of x:
 *   rowwise   : groups run along cols. codes_row u8 [rows, cols], scales_row for
 *               matrix [rows, k=cols].                      needs cols % 32 == 0
 *   columnwise: groups run along rows; written TRANSPOSED so it is again K-major:
 *               codes_colT u8 [cols, rows], scales_col for matrix [cols, k=rows].
 *               This is quantize_rowwise(x.t().contiguous()).  needs rows % 32 == 0
 * Pass NULL for the pair that is not wanted. */
int anima_mx_quantize(const void* x_bf16, int64_t rows, int64_t cols, int64_t ld_x,
                      uint8_t* codes_row, uint8_t* scales_row,
                      uint8_t* codes_colT, uint8_t* scales_col,
                      int scale_layout, void* stream);

/* 0, or 1 if a bounded wait inside the copy-engine-fed quantiser kernel gave up on the current device since the
 * last call that returned 1 (the outputs of that launch are undefined; the flag is cleared when it is reported);
 * negative on a CUDA error. Synchronises: call it where the host waits anyway (after a step's loss is read). */
int anima_mx_quantize_status(void);

/* Test aid (ref: mxfp8_gemm.py:118-120): for n fp32 block maxima, the scale exponent by the integer rule this
 * library uses (E - 8 + (mantissa > 1.75) for amax = m * 2^E) and by the reference's literal expression
 * ceil(log2(amax) - log2(448)) evaluated with lg2.approx.f32, the instruction its kernel runs on a GPU; both
 * after the 1e-30 floor and the clamp to [-127, 127]. int32 outputs. Used to show on hardware where, if anywhere,
 * the two differ (a block maximum with mantissa exactly 1.75 sits on the ceiling's edge). */
int anima_mx_exponent_probe(const float* amax, int64_t n, int32_t* by_rule, int32_t* by_lg2_approx, void* stream);

/* Quantise an MLP activation without materialising it (no reference counterpart: the reference
 * runs GELU as a separate eager kernel between mlp.layer1 and mlp.layer2 and quantises its output).
 * h bf16 [rows, cols] is the pre-activation.
 *   grad_act == NULL : quantises bf16(gelu(h)), exact erf form, bit-identical to an eager fp32-math bf16 GELU.
 *   grad_act != NULL : quantises bf16(grad_act * gelu'(h)), the gradient w.r.t. h; grad_act has h's
 *                      shape and leading dimension.
 * act_bf16 (optional, [rows, cols] contiguous) also receives the bf16 tensor that is being quantised.
 * Outputs, scale layout and size rules are those of anima_mx_quantize. The first call on each device
 * fills two small lookup tables and waits for that fill (one host synchronisation, once per device);
 * make it outside stream capture. */
int anima_mx_quantize_gelu(const void* h, const void* grad_act, int64_t rows, int64_t cols,
                           int64_t ld, void* act_bf16, uint8_t* codes_row, uint8_t* scales_row,
                           uint8_t* codes_colT, uint8_t* scales_col, int scale_layout,
                           void* stream);

/* Bytes of the scale tensor of a code matrix [rows, k] in the given layout. */
int64_t anima_mx_scales_bytes(int64_t rows, int64_t k, int scale_layout);

/* ref: mxfp8_gemm.py:225-232 (dequantize_rowwise). out bf16 [rows, k]. */
int anima_mx_dequantize(const uint8_t* codes, const uint8_t* scales, int64_t rows, int64_t k,
                        int scale_layout, void* out_bf16, void* stream);

/* PLAIN -> TILED re-layout of a scale tensor (for callers holding reference-layout blocks). */
int anima_mx_scales_retile(const uint8_t* plain, int64_t rows, int64_t k, uint8_t* tiled,
                           void* stream);

/* TILED scales of a code matrix [rows_in, k_in] -> TILED scales of the same code buffer viewed as
 * [rows_out, k_out] (equal element counts, both k multiples of 32). T-LoKr contracts the grouped
 * view x.reshape(rows * uq, K / uq) of the tensor its base projection contracts as [rows, K]
 * (ref: tlokr.py:472-476, :743): the row-wise codes are the same bytes, so one quantisation serves
 * both GEMMs once its scales are re-tiled for the second shape. */
int anima_mx_scales_regroup(const uint8_t* tiled_in, int64_t rows_in, int64_t k_in,
                            uint8_t* tiled_out, int64_t rows_out, int64_t k_out, void* stream);

/* ---------------------------------------------------------------- MXFP8 GEMM
 * ref: mxfp8_gemm.py:254-336 (_mxfp8_gemm_kernel, mxfp8_matmul);
 *      fp8_quant.py:146-150 (general_gemm 'TN'), :503-507 ('NN' dgrad, 'NT' wgrad).
 *
 * C[M,N] = A[M,K] . B[N,K]^T  (+ bias[N]) with A, B e4m3 codes, both K-major, and
 * TILED e8m0 scales of [M,K] and [N,K]; fp32 accumulation in tensor memory.
 * The three training GEMMs map onto this one form through the quantiser outputs:
 *   fwd   y  = x . W^T        : A = rowwise(x),     B = rowwise(W)
 *   dgrad dx = dy . W         : A = rowwise(dy),    B = columnwise(W)   (codes_colT [K_in, N_out])
 *   wgrad dW = dy^T . x       : A = columnwise(dy), B = columnwise(x)   (contraction over rows)
 * out_dtype 0: C bf16; 1: C fp32. ldc in elements. M, N, K > 0, K % 32 == 0.
 * status (device int32, may be NULL): set non-zero if a bounded wait inside the
 * kernel gave up; the kernel then returns early and C is undefined. */
int anima_mx_gemm(const uint8_t* a_codes, const uint8_t* a_scales,
                  const uint8_t* b_codes, const uint8_t* b_scales,
                  void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                  const void* bias_bf16, int out_dtype, int32_t* status, void* stream);

/* The same GEMM with a fused epilogue and caller scratch for split-K:
 *   C = alpha * (A . B^T) + bias + residual
 * residual (may be NULL) is bf16 [M, N] with row pitch ldr elements and MAY ALIAS C (every element
 * is read before it is written, by the thread that writes it): T-LoKr's
 * torch.add(base, delta, alpha=alpha) (ref: tlokr.py:757-759) becomes the epilogue of the last
 * delta GEMM, written over base.
 * Split-K: a small output with a long contraction (the T-LoKr factor gradients, ref:
 * tlokr.py:619-667: [r, vq] and [vp, r] outputs contracted over rows * uq = 262144) has only
 * 1 - 8 output tiles; with a workspace the contraction is split over the SMs into fp32 partial
 * tiles that a second kernel sums in a fixed order (bit-reproducible, no atomics).
 * Large outputs (M > 128 and N > 128, the CTA-pair kernel) use the workspace for their LAST tiles only: when
 * the tile count does not fill a whole number of rounds over the CTA pairs (the weight gradient
 * dW[2048,2048] over K = 32768 is 88 tiles on 74 pairs), the tiles of the last, partial round are split
 * along K over all pairs, again as fp32 partial tiles summed in a fixed order; without a workspace they run
 * unsplit.
 * anima_mx_gemm_workspace_bytes returns the scratch such a shape uses, or 0 when the shape is not
 * split (workspace may then be NULL).
 * residual == C (same pitch, bf16 C) on the CTA-pair kernel: whole tiles are rounded to bf16
 * (alpha * acc + bias) and ADDED to C by the store itself, i.e. two roundings; the one-CTA kernel, the split
 * paths and a residual that is another buffer add in fp32 and round once. Both stay within bf16 rounding of
 * the exact sum; bit patterns can differ between the two forms. */
int64_t anima_mx_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int anima_mx_gemm_ex(const uint8_t* a_codes, const uint8_t* a_scales,
                     const uint8_t* b_codes, const uint8_t* b_scales,
                     void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                     const void* bias_bf16, const void* residual_bf16, int64_t ldr, float alpha,
                     int out_dtype, void* workspace, int64_t workspace_bytes,
                     int32_t* status, void* stream);

/* A T-LoKr linear as ONE GEMM: the low-rank delta enters as extra K-blocks of the base product.
 * ref: tlokr.py:738-759 (base = fp8_frozen_linear(x); delta = _FP8StructuredLoKr(x); torch.add(base, delta,
 * alpha=)) and, for the input gradient, :531-532 (grad_hidden @ B) added to the base dgrad.
 *   C[m, i * (N/8) + p] = sum_k A[m,k] B[i*(N/8)+p, k]  +  sum_r planes[i*M + m, r] * d[p, r]   (+ bias)
 * planes: e4m3 [8 * M, 128] + TILED scales of that matrix, plane i = rows [i*M, (i+1)*M): the mixed hidden
 * tensor (forward) or the mixed gradient (backward) as written by anima_tlokr_rank_mix_quant_planes.
 * d: e4m3 [N/8, 128] + TILED scales: the factor whose rows are the output columns inside a block (alpha * A for
 * the forward, the column-wise form of B for the input gradient); a scalar alpha is folded into d by the caller.
 * The accumulator holds base + delta in fp32 and is rounded once. The rank is 128 (one K-block). Needs
 * M % 128 == 0, N/8 % 64 == 0 and a shape of the CTA-pair kernel (M > 128, N > 128), else ANIMA_E_SHAPE /
 * ANIMA_E_UNSUPPORTED. workspace as for anima_mx_gemm_ex (anima_mx_gemm_workspace_bytes). */
int anima_mx_gemm_delta(const uint8_t* a_codes, const uint8_t* a_scales,
                        const uint8_t* b_codes, const uint8_t* b_scales,
                        void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                        const void* bias_bf16, int out_dtype,
                        const uint8_t* planes_codes, const uint8_t* planes_scales,
                        const uint8_t* d_codes, const uint8_t* d_scales,
                        void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);

/* The work list the CTA-pair kernel uses for a problem on the current device (no reference counterpart; for
 * tests and tuning, nothing is launched): out9 = { CTA pairs launched, wide tile columns, 1 if a narrow
 * last column (<= 128 outputs, computed with N = 128 instructions) follows them, whole-tile items dealt
 * round-robin, tail tiles after those, K-ranges per tail tile, K-blocks (of 128) per range, pair at which the
 * tail's round robin starts, width of the wide tile columns (256 for K >= 4096, else 192; the environment
 * variable ANIMA_MX_GEMM_BN = 192 / 256 forces one) }. with_workspace == 0 gives the plan of a call without
 * scratch (no K-split). Returns 0, 1 if the shape runs on the one-CTA kernel instead (out9 untouched), or a
 * negative status. */
int anima_mx_gemm_pair_plan(int64_t M, int64_t N, int64_t K, int with_workspace, int32_t* out9);

/* Measurement aid (no reference counterpart). With a device buffer of eight int64 registered for the current
 * device (zeroed by the caller), CTA 0 of every later CTA-pair GEMM launch on that device ADDS to it
 *   [0] SM cycles it ran, [1] nanoseconds it ran, [2] 1,
 *   [3] cycles its TMA producer waited for a free pipeline stage,
 *   [4] cycles its MMA-issuing warp waited for operands to land, [5] ... for an accumulator buffer to be drained,
 *   [6] cycles its first epilogue warp waited for a finished accumulator ([7] unused).
 * [0] / [1] is the SM clock the GPU held under the kernel's own power draw, which sampling nvidia-smi between
 * launches does not show. NULL switches it off. The buffer must outlive every launch made while it is
 * registered; launches that overlap on several streams race on it. */
int anima_mx_gemm_set_clock_probe(void* device_buffer_8xint64);

/* ---------------------------------------------------------------- LoKr merged weight
 * ref: lokr_patch.py:76-84 (merged = W + alpha * kron(w1, w2)) followed by the two
 *      weight quantisations of fp8_quant.py:234-235 / :501.
 *
 * W bf16 [N,K]; w1 [up,uq], w2 [vp,vq] = [N/up, K/uq], both fp32 (factors_are_fp32 != 0)
 * or both bf16. With n = i*vp + p and k = j*vq + q:
 *   diff   = bf16(w1[i,j] * w2[p,q])                  (torch.kron in the weight dtype)
 *   merged = bf16(W[n,k] + alpha * diff)              (fp32 sum, rounded once)
 * Emits (each optional) the bf16 merged weight and its rowwise / columnwise MXFP8
 * forms exactly as anima_mx_quantize(merged) would. vq % 8 == 0. */
int anima_lokr_merge_quantize(const void* w_bf16, const void* w1, const void* w2,
                              int factors_are_fp32, float alpha, int64_t N, int64_t K,
                              int64_t up, int64_t uq,
                              void* merged_bf16,
                              uint8_t* codes_row, uint8_t* scales_row,
                              uint8_t* codes_colT, uint8_t* scales_col,
                              int scale_layout, void* stream);

/* ref: autograd of lokr_patch.py:76-84 through torch.kron (docstring :19-21).
 * dW [N,K] (bf16 if dw_is_fp32 == 0 else fp32):
 *   dw1[i,j] = alpha * sum_{p,q} dW[i*vp+p, j*vq+q] * w2[p,q]
 *   dw2[p,q] = alpha * sum_{i,j} dW[i*vp+p, j*vq+q] * w1[i,j]
 * dw1 fp32 [up,uq], dw2 fp32 [vp,vq]; up, uq <= 8; deterministic two-stage reduction. */
int64_t anima_lokr_kron_backward_workspace_bytes(int64_t N, int64_t K, int64_t up, int64_t uq);
int anima_lokr_kron_backward(const void* dw, int dw_is_fp32, const void* w1, const void* w2,
                             int factors_are_fp32, float alpha, int64_t N, int64_t K, int64_t up,
                             int64_t uq, float* dw1, float* dw2, void* workspace,
                             int64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------- fused AdaLN
 * ref: adaln_kernel.py:34-68 (_fwd_kernel), :157-207 (FusedAdaLN.forward).
 * x, y bf16 [rows, d]; scale, shift bf16 [rows / hw, d]; row r uses modulation row r / hw.
 *   mean = sum(x)/d; var = sum((x-mean)^2)/d; rstd = 1/sqrt(var+eps);
 *   y = (x-mean)*rstd*(1+scale) + shift;  mean, rstd fp32 [rows] are saved. */
int anima_adaln_fwd(const void* x, const void* scale, const void* shift, float eps,
                    int64_t rows, int64_t hw, int64_t d, void* y, float* mean, float* rstd,
                    void* stream);

/* ref: adaln_kernel.py:71-154 (_bwd_dx_kernel, _bwd_dsdb_kernel), :209-255.
 * One pass over dy and x yields dx bf16 [rows,d] and, through per-block partial
 * sums in the workspace plus a fixed-order final sum, dscale / dshift bf16 [rows/hw, d]
 * (bit-reproducible; the reference accumulates these with fp32 atomics). */
int64_t anima_adaln_bwd_workspace_bytes(int64_t rows, int64_t hw, int64_t d);
int anima_adaln_bwd(const void* dy, const void* x, const void* scale, const float* mean,
                    const float* rstd, int64_t rows, int64_t hw, int64_t d, void* dx,
                    void* dscale, void* dshift, void* workspace, int64_t workspace_bytes,
                    void* stream);

/* anima_adaln_bwd for callers that cannot hand over scratch memory (no counterpart in anima-trainer).
 *
 * Who needs it: code that runs where allocating device memory is not an option — an operator plugged
 * into a framework that passes it input and output buffers and nothing else, or a long-running service
 * whose GPU memory is fully planned at start-up, where a later cudaMalloc may fail, fragment the plan or
 * stall the device. Same arguments and results as anima_adaln_bwd minus the workspace: the per-block
 * partial sums go to a fixed array compiled into the library (ANIMA_ADALN_BWD_NOALLOC_MAX_BYTES bytes of
 * global memory on every GPU that loads it, held until the process exits). The call itself performs no
 * cudaMalloc / cudaFree and calls no allocating routine.
 *   - Limit: shapes whose anima_adaln_bwd_workspace_bytes(rows, hw, d) exceeds the array are refused with
 *     ANIMA_E_TOO_LARGE (config 3, x [8, 4096, 2048], needs 4.6 MiB and fits).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current); make that first call outside any stream capture.
 *   - All calls on a device share the one array. Calls that may overlap on the GPU (different streams
 *     without ordering between them) race on it; stream-ordered calls are safe, and nothing in the array
 *     needs clearing between calls because every slot that is read was written earlier in the same call. */
#define ANIMA_ADALN_BWD_NOALLOC_MAX_BYTES (8ll << 20)
int anima_adaln_bwd_noalloc(const void* dy, const void* x, const void* scale, const float* mean,
                            const float* rstd, int64_t rows, int64_t hw, int64_t d, void* dx,
                            void* dscale, void* dshift, void* stream);

/* ---------------------------------------------------------------- gated residual
 * ref: adaln_kernel.py:272-295 (_gated_add_fwd_kernel), :332-380.
 * out = x + gate[r / hw] * y, all bf16, evaluated in fp32 and rounded once. */
int anima_gated_add_fwd(const void* x, const void* gate, const void* y, int64_t rows,
                        int64_t hw, int64_t d, void* out, void* stream);

/* ref: adaln_kernel.py:298-329 (_gated_add_bwd_dgate_kernel), :382-419.
 * dy = gate * dout (bf16), dgate[bt] = sum over the hw rows of dout * y (fp32 sum,
 * fixed order, stored bf16). dx is dout itself and is not written. */
int64_t anima_gated_add_bwd_workspace_bytes(int64_t rows, int64_t hw, int64_t d);
int anima_gated_add_bwd(const void* dout, const void* y, const void* gate, int64_t rows,
                        int64_t hw, int64_t d, void* dy, void* dgate, void* workspace,
                        int64_t workspace_bytes, void* stream);

/* The gated residual of one sublayer and the AdaLN modulation of the next in one pass (no single
 * reference counterpart: adaln_patch.py:42-153 calls FusedGatedAdd, then FusedAdaLN, on the same tensor):
 *   x_new = x + gate * sub                      (as anima_gated_add_fwd)
 *   y     = LayerNorm(x_new) * (1 + scale) + shift, mean / rstd of x_new   (as anima_adaln_fwd)
 * Both outputs are bit-identical to the two separate calls. gate, scale, shift bf16 [rows/hw, d]. */
int anima_gated_add_adaln_fwd(const void* x, const void* gate, const void* sub, const void* scale,
                              const void* shift, float eps, int64_t rows, int64_t hw, int64_t d,
                              void* x_new, void* y, float* mean, float* rstd, void* stream);

/* AdaLN forward that also emits the row-wise MXFP8 operand of y (no reference counterpart: the reference
 * writes y in adaln_kernel.py:34-68 and quantises it again inside each consuming linear, fp8_quant.py:149-150,
 * 483-485; its audit lists "quantise in the producer" as the open item). codes_row u8 [rows, d] and scales_row
 * (PLAIN [rows, d/32] or TILED) are bit-identical to anima_mx_quantize of the bf16 y. y may be NULL (then only
 * the operand and the statistics are written). d % 128 == 0; TILED needs rows % 128 == 0. The _gated_add_ form
 * is anima_gated_add_adaln_fwd with the same extra outputs. */
int anima_adaln_fwd_quant(const void* x, const void* scale, const void* shift, float eps, int64_t rows,
                          int64_t hw, int64_t d, void* y, float* mean, float* rstd, uint8_t* codes_row,
                          uint8_t* scales_row, int scale_layout, void* stream);
int anima_gated_add_adaln_fwd_quant(const void* x, const void* gate, const void* sub, const void* scale,
                                    const void* shift, float eps, int64_t rows, int64_t hw, int64_t d,
                                    void* x_new, void* y, float* mean, float* rstd, uint8_t* codes_row,
                                    uint8_t* scales_row, int scale_layout, void* stream);

/* Backward of the pair in one pass. d_y is the gradient of y, d_xnew the gradient reaching x_new through
 * the residual stream. With dx_ln the AdaLN input gradient (as anima_adaln_bwd):
 *   dx   = d_xnew + dx_ln        (gradient of x, bf16)        dsub  = gate * dx
 *   dscale, dshift as anima_adaln_bwd;                        dgate as anima_gated_add_bwd (of dx and sub)
 * All five outputs are bit-identical to anima_adaln_bwd, a bf16 add and anima_gated_add_bwd run in turn. */
int64_t anima_gated_add_adaln_bwd_workspace_bytes(int64_t rows, int64_t hw, int64_t d);
int anima_gated_add_adaln_bwd(const void* d_y, const void* d_xnew, const void* x_new, const void* scale,
                              const float* mean, const float* rstd, const void* sub, const void* gate,
                              int64_t rows, int64_t hw, int64_t d, void* dx, void* dsub, void* dscale,
                              void* dshift, void* dgate, void* workspace, int64_t workspace_bytes,
                              void* stream);

/* ---------------------------------------------------------------- T-LoKr rank mix
 * ref: tlokr_kernels.py:15-82, :125-166 (rank_mix).
 * hidden, out bf16 [batch, n, 8, rank]; c bf16 [8,8]; mask bf16 [batch, rank] or NULL.
 *   out[b,n,i,r] = (sum_j (transpose ? c[j,i] : c[i,j]) * hidden[b,n,j,r]) * mask[b,r]
 * fp32 accumulation in j order. rank % 8 == 0. */
int anima_tlokr_rank_mix(const void* hidden, const void* c, const void* mask, int64_t batch,
                         int64_t n_per_batch, int64_t rank, int transpose, void* out,
                         void* stream);

/* The same mix with its output leaving as MXFP8 operands for the factor GEMMs (no reference counterpart:
 * _FP8StructuredLoKr, tlokr.py:589-667, writes the mixed tensor in bf16 and quantises it in a second pass).
 * Row form: codes_row u8 [R, rank] + TILED scales, R = batch * n_per_batch * 8; column form, transposed:
 * codes_colT u8 [rank, R] + TILED scales. Either pair may be NULL; out (bf16, as anima_tlokr_rank_mix) may be
 * NULL too. Codes and scales are bit-identical to anima_mx_quantize of the bf16 output.
 * rank in {128, 256, 512}; batch * n_per_batch % 16 == 0. */
int anima_tlokr_rank_mix_quant(const void* hidden, const void* c, const void* mask, int64_t batch,
                               int64_t n_per_batch, int64_t rank, int transpose, void* out,
                               uint8_t* codes_row, uint8_t* scales_row, uint8_t* codes_colT,
                               uint8_t* scales_col, void* stream);

/* The same, with the row form written as EIGHT PLANES: row i of item t (t = b * n_per_batch + n) becomes row
 * i * items + t of a u8 [8 * items, rank] matrix (TILED scales of that matrix), so that plane i is a K-major
 * [items, rank] GEMM operand over the items: what the delta K-blocks of anima_mx_gemm_delta consume. The
 * codes of a row equal those of anima_tlokr_rank_mix_quant. items = batch * n_per_batch must be a multiple of
 * 128 (whole scale row tiles per plane). The column form (may be NULL) is unchanged. No reference counterpart. */
int anima_tlokr_rank_mix_quant_planes(const void* hidden, const void* c, const void* mask, int64_t batch,
                                      int64_t n_per_batch, int64_t rank, int transpose,
                                      uint8_t* codes_planes, uint8_t* scales_planes,
                                      uint8_t* codes_colT, uint8_t* scales_col, void* stream);

/* First half of the T-LoKr delta in one kernel: hidden = g . f^T (block-scaled GEMM over k), then the 8x8 mix,
 * the mask and the MXFP8 quantisation of the mixed tensor, written as eight planes. The hidden tensor stays in
 * tensor memory and registers; it is written (bf16 [batch * n * 8, 128]) only if hidden_out is given.
 * ref: tlokr.py:476-483 (hidden = grouped @ B.T; mixed = rank_mix(hidden, C, mask)) followed by the
 * quantisation of `mixed` in _FP8StructuredLoKr (:589-590).
 * g: e4m3 [batch * n * 8, k] + TILED scales (the grouped view of the layer input, row = token * 8 + j);
 * f: e4m3 [128, k] + TILED scales (B, rank 128). c bf16 [8, 8], mask bf16 [batch, 128] or NULL.
 * planes_codes / planes_scales as anima_tlokr_rank_mix_quant_planes writes them; values are bit-identical to
 * anima_mx_gemm (bf16 output) followed by that call. batch * n % 128 == 0, k % 32 == 0. */
int anima_tlokr_hidden_mix_planes(const uint8_t* g_codes, const uint8_t* g_scales,
                                  const uint8_t* f_codes, const uint8_t* f_scales,
                                  const void* c, const void* mask, int64_t batch, int64_t n_per_batch, int64_t k,
                                  int transpose, void* hidden_out, uint8_t* planes_codes, uint8_t* planes_scales,
                                  int32_t* status, void* stream);

/* ref: tlokr_kernels.py:85-122, :168-204 (rank_mix_wgrad).
 *   dc[i,j] = sum_{b,n,r} grad_mixed[b,n,i,r] * hidden[b,n,j,r] * mask[b,r]   (fp32 [8,8])
 * Reads both tensors once (the reference reads them once per (i,j) pair). */
int64_t anima_tlokr_rank_mix_wgrad_workspace_bytes(int64_t batch, int64_t n_per_batch,
                                                   int64_t rank);
int anima_tlokr_rank_mix_wgrad(const void* grad_mixed, const void* hidden, const void* mask,
                               int64_t batch, int64_t n_per_batch, int64_t rank, float* dc,
                               void* workspace, int64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------- q / k preparation
 * Per-head RMSNorm followed by rotary embedding in one pass (head_dim must be 128).
 * ref: the two third-party kernels the trainer patches in at this point — Liger RMSNorm
 * (liger_patch.py:31-47, rms_norm casting mode "llama") and Transformer Engine's fused RoPE,
 * rotate-half / non-interleaved (rope_patch.py:28-56).
 * x, out bf16 [tokens, heads, 128]; weight fp32 [128]; cos_tab, sin_tab fp32 [seq_len, 128] or
 * both NULL (norm only; cross-attention q / k); position of a token = token index % seq_len.
 *   n = x * rsqrt(mean(x^2) + eps) * weight;  out = n * cos + rotate_half(n) * sin   (fp32 math)
 * rstd fp32 [tokens, heads] is written by fwd and read by bwd. bwd gives dx only: the norm
 * weight is frozen in adapter training. */
int anima_rmsnorm_rope_fwd(const void* x, const float* weight, const float* cos_tab,
                           const float* sin_tab, float eps, int64_t tokens, int64_t heads,
                           int64_t head_dim, int64_t seq_len, void* out, float* rstd,
                           void* stream);
int anima_rmsnorm_rope_bwd(const void* dout, const void* x, const float* weight,
                           const float* cos_tab, const float* sin_tab, const float* rstd,
                           int64_t tokens, int64_t heads, int64_t head_dim, int64_t seq_len,
                           void* dx, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ANIMA_B200_H_ */
