/*
 * C ABI of the B200-native block-scaled quantize -> dense GEMM path.
 *
 * Plain pointers and sizes only: every entry point takes device pointers that
 * the caller owns, the CUDA device ordinal they live on and the stream to
 * launch on, never synchronises, and returns 0 on success or a non-zero
 * HQ_ERR_* code with a NUL-terminated message in `err` (when `err` is not
 * NULL and `errlen` > 0).  The message texts follow the reference's
 * TORCH_CHECK texts so that a binding can raise them unchanged.
 *
 * Each declaration cites the reference interface it replaces (paths relative
 * to the reference project).
 */
#ifndef HALOPS_B200_H_
#define HALOPS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Quantisation recipe; same order as the reference's QuantMode
 * (csrc/kernel/gemm/group_wise_quant.cu:36-40). */
enum {
    HQ_MODE_W8A8_MXFP8 = 0, /* e4m3 values, UE8M0 scale per 32 */
    HQ_MODE_W4A4_MXFP4 = 1, /* packed e2m1 values, UE8M0 scale per 32 */
    HQ_MODE_W4A4_NVFP4 = 2, /* packed e2m1 values, UE4M3 scale per 16 */
    /* GEMM-only mode of hq_group_masked_gemm / hq_group_contiguous_gemm: e4m3 activations
     * (quantised as W8A8_MXFP8) x packed e2m1 weights (quantised as W4A4_MXFP4), UE8M0 scales
     * per 32 on both (csrc/kernel/gemm/group_masked_gemm.cu:96-121); not a quantizer mode. */
    HQ_MODE_W4A8_MXFP4 = 3
};

/* Input element type of the quantizer. */
enum { HQ_DTYPE_BF16 = 0, HQ_DTYPE_FP16 = 1 };

/* Epilogue selector; values of the reference's EpilogueOp
 * (csrc/kernel/gemm/epilogue_op.h:21-28).  hq_dense_gemm takes Identity and Sigmoid,
 * hq_dense_gemm_situ_quant is SituQuant, hq_batch_gemm takes Identity and
 * hq_batch_gemm_quant the three Quant forms: the same split as in the reference, whose
 * dense entry has no Quant forms and whose batch entry has no Sigmoid / SituQuant. */
enum {
    HQ_EPILOGUE_IDENTITY = 0,
    HQ_EPILOGUE_QUANT = 1,
    HQ_EPILOGUE_GATE_MUL_QUANT = 2,
    HQ_EPILOGUE_SIGMOID = 3,
    HQ_EPILOGUE_SITU_QUANT = 4,
    HQ_EPILOGUE_SIGMOID_GATE_MUL_QUANT = 5
};

enum {
    HQ_OK = 0,
    HQ_ERR_INVALID = 1,     /* argument rejected; nothing was launched */
    HQ_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed */
    HQ_ERR_UNSUPPORTED = 3, /* legal in the reference, not built here */
    HQ_ERR_DEVICE = 4       /* a kernel gave up on a bounded wait (see hq_device_status) */
};

/* Maps "w8a8-mxfp8" / "w4a4-mxfp4" / "w4a4-nvfp4" to HQ_MODE_*, -1 otherwise.
 * Replaces ParseQuantMode (csrc/kernel/gemm/group_wise_quant.cu:49-61) and the
 * mode check of DenseGemm (csrc/kernel/gemm/dense_gemm.cu:33-36). */
int hq_parse_mode(const char* mode);

/* Group size (32 or 16) of a mode, 0 for an unknown mode.
 * Replaces GroupSize (csrc/kernel/gemm/group_wise_quant.cu:44-46). */
int hq_group_size(int mode);

/* Rows of a swizzled scale tensor: m rounded up to whole 128-row SfAtoms.
 * Replaces AlignSfM (csrc/kernel/gemm/gemm_utils.h:56-60). */
int64_t hq_sf_rows(int64_t m);

/*
 * Group-wise quantisation of a row-major [m, k] bf16/fp16 matrix along k.
 * Replaces halops::GroupWiseQuant (csrc/kernel/gemm/group_wise_quant.cu:297-375,
 * bound at csrc/common/cpp_extensions.cc:300-303) minus the tensor allocation,
 * which stays with the caller:
 *   input   row-major, `ld_elems` elements between rows, rows 16-byte aligned
 *   out_q   [m, k] e4m3 bytes (mxfp8) or [m, k/2] packed e2m1 (even index in
 *           the low nibble), contiguous
 *   out_sf  swizzle != 0: hq_sf_rows(m) * k/g bytes in SfAtom order (128 rows
 *           x 4 K-blocks per 512-byte atom; padding rows written as zero);
 *           swizzle == 0: [m, k/g] row-major bytes
 * use_pdl != 0 launches with programmatic stream serialisation.
 */
int hq_group_wise_quant(const void* input, int64_t ld_elems, int in_dtype,
                        int64_t m, int64_t k, int mode, int use_swizzle,
                        int use_pdl, void* out_q, void* out_sf, int device,
                        void* stream, char* err, size_t errlen);

/*
 * RMSNorm fused with the MXFP8 quantizer: y = bf16(x * rsqrt(mean(x^2) + eps) *
 * weight), quantised as hq_group_wise_quant(y, HQ_MODE_W8A8_MXFP8) would.
 * Replaces halops::RmsNormQuant (csrc/kernel/gemm/rms_norm_quant.cu:111-155,
 * bound at csrc/common/cpp_extensions.cc) minus the tensor allocation:
 *   input   [m, k] bf16, `ld_elems` between rows, rows 16-byte aligned;
 *           k a multiple of 128 and at most 8192
 *   weight  [k] bf16 (gamma)
 *   out_q   [m, k] e4m3 bytes; out_sf as for hq_group_wise_quant
 */
int hq_rms_norm_quant(const void* input, int64_t ld_elems, const void* weight,
                      float eps, int64_t m, int64_t k, int use_swizzle,
                      int use_pdl, void* out_q, void* out_sf, int device,
                      void* stream, char* err, size_t errlen);

/*
 * out[M, N] = bf16(alpha * (A . B^T)) with block-scaled operands.
 * Replaces halops::DenseGemm (csrc/kernel/gemm/dense_gemm.cu:23-189, bound at
 * csrc/common/cpp_extensions.cc:280-286) for EpilogueOp::Identity and
 * EpilogueOp::Sigmoid (out = bf16(sigmoid(alpha * A.B^T + bias))):
 *   a     [M, K] e4m3 or [M, K/2] packed e2m1, row-major contiguous
 *   b     [N, K] / [N, K/2], same encoding
 *   sfa   SfAtom-swizzled scales of A, at least hq_sf_rows(M) * K/g bytes
 *   sfb   SfAtom-swizzled scales of B, at least hq_sf_rows(N) * K/g bytes
 *   out   [M, N] bf16, `ldo` elements between rows (ldo % 8 == 0)
 *   bias  NULL or [N] bf16, 16-byte aligned; w8a8-mxfp8 only and, as in the
 *         reference, only with M % 256 == 0 (csrc/kernel/gemm/dense_gemm.cu:96-99)
 *   alpha device pointer to one float: required for nvfp4, must be NULL for
 *         mxfp4, ignored for mxfp8 (csrc/kernel/gemm/dense_gemm.cu:126-164)
 *   sm_count <= 0 uses every SM of the device
 *   use_pdl  0: plain launch.  1: programmatic stream serialisation, as the
 *         reference's use_pdl: the kernel's set-up overlaps the tail of the
 *         preceding kernel and nothing is read before that kernel is complete.
 *         2 (no counterpart in the reference): the same, and the caller
 *         vouches that `b` and `sfb` are not written by the preceding kernel
 *         (a weight that was quantised at load time); the small-M kernel (MXFP8,
 *         M <= 64) then asks for the weight of its first stages before it
 *         waits for the preceding kernel, so a chain of decode GEMMs streams
 *         its weights back to back.  Other kernels treat 2 as 1.
 * Rows of A past M are never read into the result and rows of out past M are
 * never written.
 */
int hq_dense_gemm(const void* a, const void* b, const void* sfa,
                  const void* sfb, void* out, const void* bias,
                  const float* alpha, int64_t m,
                  int64_t n, int64_t k, int64_t sfa_bytes, int64_t sfb_bytes,
                  int64_t ldo, int mode, int epilogue, int sm_count,
                  int use_pdl, int device, void* stream, char* err,
                  size_t errlen);

/*
 * SiTU-GLU quantising GEMM: with y = A . B^T + bias and the rows of B (and bias)
 * ordered [16 gate rows, 16 up rows, ...] (the reference's interleave_gate_up),
 *   out_q[M, N/2] = e4m3( situ_beta tanh(gate / situ_beta) sigmoid(gate)
 *                         * situ_linear_beta tanh(up / situ_linear_beta) )   (times up
 * itself when situ_linear_beta == 0), rounded to bf16 and then quantised per 32
 * output columns with UE8M0 scales written to out_sf in SfAtom order
 * (hq_sf_rows(M) x N/64 bytes; padding rows are left untouched).
 * Replaces halops::DenseGemm with EpilogueOp::SituQuant
 * (csrc/kernel/gemm/dense_gemm.cu:100-125, csrc/kernel/gemm/epilogue.cuh:867-905,990-1051).
 * MXFP8 operands only; N % 256 == 0 (the output's N/64 scale columns fill whole atoms).
 */
int hq_dense_gemm_situ_quant(const void* a, const void* b, const void* sfa,
                             const void* sfb, void* out_q, void* out_sf,
                             const void* bias, int64_t m, int64_t n, int64_t k,
                             int64_t sfa_bytes, int64_t sfb_bytes,
                             int64_t out_sf_bytes, float situ_beta,
                             float situ_linear_beta, int sm_count, int use_pdl,
                             int device, void* stream, char* err, size_t errlen);

/*
 * Batch GEMM: out[:, b*N:(b+1)*N] = alpha[b] * (A[b] . B[b]^T) + bias[b] for b < batches.
 * Replaces halops::BatchGemm with EpilogueOp::Identity
 * (csrc/kernel/gemm/batch_gemm.cu:22-188, bound at csrc/common/cpp_extensions.cc
 * "batch_gemm"; Python face halops/gemm/batch_gemm.py:27-117).
 *   a     [batches, M, K] e4m3 bytes or [batches, M, K/2] packed e2m1, contiguous
 *   b     [batches, N, K] / [batches, N, K/2], contiguous
 *   sfa   SfAtom-swizzled scales over the STACKED rows [batches * M]: at least
 *         hq_sf_rows(batches * M) * K/g bytes (what hq_group_wise_quant returns for
 *         the [batches * M, K] view)
 *   sfb   per batch its own atoms: batches * hq_sf_rows(N) * K/g bytes
 *   out   [M, batches * N] bf16, `ldo` elements between rows (ldo % 8 == 0)
 *   bias  NULL or [batches, N] bf16 (w8a8-mxfp8 only); any M
 *   alpha NULL or [batches] float on the device: required for nvfp4, must be NULL
 *         for mxfp4, ignored for mxfp8
 * A 128-row tile of the stacked rows that straddles two batches is worked once per
 * batch (csrc/kernel/gemm/gemm_dispatch.cuh:90-93); every output element is written
 * exactly once.  The quantising epilogues of the reference (Quant, GateMulQuant,
 * SigmoidGateMulQuant) have their own entry, hq_batch_gemm_quant.
 */
int hq_batch_gemm(const void* a, const void* b, const void* sfa, const void* sfb,
                  void* out, const void* bias, const float* alpha,
                  int64_t batches, int64_t m, int64_t n, int64_t k,
                  int64_t sfa_bytes, int64_t sfb_bytes, int64_t ldo, int mode,
                  int epilogue, int sm_count, int use_pdl, int device,
                  void* stream, char* err, size_t errlen);

/*
 * Masked grouped GEMM (MoE, padded slots): expert e owns rows
 * [e * max_m, (e + 1) * max_m) of A and of out, of which the first masked_m[e] are valid:
 *   out[e * max_m + i, :] = alpha[e] * (A[e * max_m + i, :] . B[e]^T) + bias[e],  i < masked_m[e].
 * Rows past masked_m[e] are neither computed nor written.
 * Replaces halops::GroupMaskedGemm (csrc/kernel/gemm/group_masked_gemm.cu:22-186; Python face
 * halops/gemm/group_masked_gemm.py:25-116; scheduler csrc/kernel/gemm/tile_scheduler.cuh:393-460).
 *   a [num_experts * max_m, K or K/2], b [num_experts, N, K or K/2], contiguous
 *   sfa SfAtom scales over all rows of a; sfb per expert its own atoms (as hq_batch_gemm)
 *   masked_m [num_experts] int32 on the device, read by the kernel (values are clamped to [0, max_m])
 *   out [num_experts * max_m, N] bf16, `ldo` elements between rows
 *   bias NULL or [num_experts, N] bf16 (w8a8-mxfp8 only); alpha NULL or [num_experts] float
 * max_m must be a multiple of 64.  mode may also be HQ_MODE_W4A8_MXFP4 (a [.., K] e4m3, b
 * [num_experts, N, K/2] packed e2m1, no bias, no alpha).
 */
int hq_group_masked_gemm(const void* a, const void* b, const void* sfa,
                         const void* sfb, const int32_t* masked_m, void* out,
                         const void* bias, const float* alpha,
                         int64_t num_experts, int64_t max_m_per_expert,
                         int64_t n, int64_t k, int64_t sfa_bytes,
                         int64_t sfb_bytes, int64_t ldo, int mode, int sm_count,
                         int use_pdl, int device, void* stream, char* err,
                         size_t errlen);

/*
 * Contiguous grouped GEMM (MoE, packed rows): row r of A uses weight expert_ids[r]:
 *   out[r, :] = alpha[e] * (A[r, :] . B[e]^T) + bias[e],  e = expert_ids[r].
 * Replaces halops::GroupContiguousGemm (csrc/kernel/gemm/group_contiguous_gemm.cu:22-176;
 * Python face halops/gemm/group_contiguous_gemm.py:25-105; scheduler
 * csrc/kernel/gemm/tile_scheduler.cuh:575-670, which reads expert_ids at the first row of
 * each tile).
 *   expert_ids [M] int32 on the device, non-decreasing; every run of equal ids must
 *   start on a multiple of 64 rows (the reference wants runs aligned to the tile it
 *   picks: 64, 128 or 256 rows); ids are clamped to [0, num_experts).  M % 64 == 0.
 * Other operands as hq_group_masked_gemm with out [M, N].
 */
int hq_group_contiguous_gemm(const void* a, const void* b, const void* sfa,
                             const void* sfb, const int32_t* expert_ids,
                             void* out, const void* bias, const float* alpha,
                             int64_t num_experts, int64_t m, int64_t n,
                             int64_t k, int64_t sfa_bytes, int64_t sfb_bytes,
                             int64_t ldo, int mode, int sm_count, int use_pdl,
                             int device, void* stream, char* err, size_t errlen);

/*
 * Decode-sized MXFP8 GEMM (M <= 16) on scales in the PLAIN row-major layout
 * ([rows, K / 32] bytes, row stride a multiple of 16 bytes: what hq_group_wise_quant writes
 * with use_swizzle = 0), with two fused forms:
 *   concat-K     (a2, b2, sfa2, sfb2 given, out2 NULL):  out = A . B^T + A2 . B2^T
 *   dual output  (b2, sfb2, out2 given, a2 / sfa2 NULL): out = A . B^T and out2 = A . B2^T
 * Replaces halops::LowLatencyMmaGemm (csrc/kernel/gemm/low_latency_mma_gemm.cu:23-76, checks
 * of csrc/kernel/gemm/low_latency_utils.cuh:222-273; Python face
 * halops/gemm/low_latency_mma_gemm.py:25-109).
 *   a [M, K1] e4m3, b [N, K1] e4m3, contiguous, 16-byte aligned; N % 8 == 0; K1 + K2 a multiple
 *   of 256 (each a multiple of 128); concat-K wants K1 % 512 == 0 as the reference does
 *   sfa [M, K1/32], sfb [N, K1/32] UE8M0 bytes with the row strides given in bytes
 *   out [M, N] bf16 (ldo elements between rows, ldo % 8 == 0); out2 [M, N2] likewise
 *   use_sigmoid: write sigmoid(bf16(result)) instead (not with a2 / out2)
 * K is not bounded by shared memory here (the reference keeps A resident and rejects large K).
 */
int hq_low_latency_gemm(const void* a, const void* b, const void* sfa, const void* sfb,
                        void* out, const void* a2, const void* b2, const void* sfa2,
                        const void* sfb2, void* out2, int64_t m, int64_t n, int64_t n2,
                        int64_t k1, int64_t k2, int64_t sfa_stride, int64_t sfb_stride,
                        int64_t sfa2_stride, int64_t sfb2_stride, int64_t ldo, int64_t ldo2,
                        int use_sigmoid, int sm_count, int use_pdl, int device, void* stream,
                        char* err, size_t errlen);

/* Grouped kinds for hq_describe_group_tile. */
enum { HQ_GROUP_BATCH = 1, HQ_GROUP_MASKED = 2, HQ_GROUP_CONTIGUOUS = 3 };

/*
 * Batch GEMM with a quantising epilogue (MXFP8 operands): with y = bf16(A[b] . B[b]^T + bias[b]),
 *   HQ_EPILOGUE_QUANT                   v = y
 *   HQ_EPILOGUE_GATE_MUL_QUANT          v = y * gate                 (bf16 product)
 *   HQ_EPILOGUE_SIGMOID_GATE_MUL_QUANT  v = y * bf16(sigmoid(gate))
 * out_q[M, batches * N] = e4m3(v * 2^(127 - e)) per 32 columns, e = UE8M0 exponent of the group's
 * bf16 amax (the exact-integer recipe of csrc/common/mx_quant.cuh:60-71), written to out_sf in
 * SfAtom order over [M, batches * N / 32] (hq_sf_rows(M) * batches * N / 32 bytes; padding rows
 * are left untouched).  Replaces halops::BatchGemm with those epilogues
 * (csrc/kernel/gemm/batch_gemm.cu:60-133, csrc/kernel/gemm/epilogue.cuh:990-1051).
 *   N % 128 == 0; ldq = bytes between rows of out_q (multiple of 16)
 *   gate [M, batches * N] bf16, gate_ld elements between rows, rows 32-byte aligned; NULL for QUANT
 */
int hq_batch_gemm_quant(const void* a, const void* b, const void* sfa, const void* sfb,
                        void* out_q, void* out_sf, const void* gate, int64_t gate_ld,
                        const void* bias, int64_t batches, int64_t m, int64_t n, int64_t k,
                        int64_t sfa_bytes, int64_t sfb_bytes, int64_t ldq,
                        int64_t out_sf_bytes, int epilogue, int sm_count, int use_pdl,
                        int device, void* stream, char* err, size_t errlen);

/* hq_describe_tile for the grouped GEMMs: the tile picked for `count` weights with
 * `rows` rows each (batch, masked: the slot; contiguous: M / num_experts) and `total_m`
 * rows of A in all, or the reference's "No <batch|masked|contiguous> <mode> tile for
 * M=.. (grid M=..), N=.., K=.." text (csrc/kernel/gemm/gemm_dispatch.cuh:65-100) with
 * HQ_ERR_INVALID.  Needs no device. */
int hq_describe_group_tile(int kind, int64_t count, int64_t rows, int64_t total_m,
                           int64_t n, int64_t k, int mode, int sm_count, int device,
                           char* buf, size_t buflen);

/* Number of SMs of `device`, cached per device.
 * Replaces GetSmCount (csrc/kernel/gemm/gemm_utils.h:29-37), whose cache is
 * keyed by nothing and so returns the first device's count on every device. */
int hq_sm_count(int device);

/*
 * Reads (and clears) the device-side status word of `device` after
 * synchronising `stream`: 0 when no kernel of this library gave up on a
 * bounded wait since the last call, else a code whose low byte names the
 * role that timed out.  The reference's waits are unbounded
 * (csrc/common/ptx.cuh:131-139); it has no counterpart of this call.
 */
int hq_device_status(int device, void* stream, uint32_t* status, char* err,
                     size_t errlen);

/*
 * Launches a one-CTA kernel whose bounded wait runs out after `limit_us`
 * microseconds (1..100000): a thread waits on an mbarrier that nothing arrives
 * on, gives up, records the "MMA role" code 0x02 in the status word and raises
 * the CTA's abort flag, on which a second waiting thread leaves.  The next
 * hq_device_status on the same stream therefore returns HQ_ERR_DEVICE with
 * status 0x02, and the one after it 0.  This exercises, with nothing in
 * flight, the code every GEMM role runs when a wait times out.  The reference
 * has no counterpart (its waits are unbounded, csrc/common/ptx.cuh:131-139).
 */
int hq_selftest_bounded_wait(uint32_t limit_us, int device, void* stream,
                             char* err, size_t errlen);

/*
 * Column-parallel MXFP8 dense GEMM with the all-gather of the output fused into
 * its epilogue.  The reference has no multi-GPU dense GEMM (its tensor-parallel
 * tests combine single-GPU calls with framework collectives,
 * tests/test_fused_all_reduce_mhc.py:181-218); this is the N-sharded mode of the
 * benchmark's largest configuration in one kernel.
 *   a, sfa          the replicated activation [m, k] e4m3 and its SfAtom scales
 *   b, sfb          this rank's weight shard [n_local, k] and its scales
 *   outs[world]     one [m, ldo] bf16 matrix per rank, ldo >= world * n_local;
 *                   outs[rank] lives on this device, the others are the peers'
 *                   matrices mapped into this process (symmetric memory)
 * The kernel (2-CTA 256 x 256 tile) writes columns [rank * n_local, (rank + 1) *
 * n_local) of EVERY matrix: each staged 32 x 64 piece of a finished tile goes
 * out by one TMA store per matrix (rows of 128 bytes; the peers' over NVLink),
 * tile by tile, so the transfer overlaps the math.  Every load of the kernel
 * (operands, scales) is from this GPU's memory.
 * The caller fences across ranks: nobody may still read a matrix
 * when the first rank starts, and a rank may read its matrix once every rank's
 * kernel has completed.  HQ_ERR_UNSUPPORTED unless n_local % 256 == 0,
 * k % 128 == 0 and m > 128; world <= 8.
 */
int hq_dense_gemm_allgather(const void* a, const void* b, const void* sfa,
                            const void* sfb, void* const* outs, int world,
                            int rank, int64_t m, int64_t n_local, int64_t k,
                            int64_t sfa_bytes, int64_t sfb_bytes, int64_t ldo,
                            int sm_count, int use_pdl, int device, void* stream,
                            char* err, size_t errlen);

/*
 * MXFP8 dense GEMM for at most 32 activation rows that allocates nothing: no
 * cudaMalloc, no cudaFree, no allocating library call, on any call.  It has no
 * counterpart in the reference.  It is for callers that cannot have a library
 * allocate device memory under them: code between the begin and the end of a
 * stream capture, servers that give all device memory to their own pool at
 * start-up, paths that must not take the allocator's locks.  hq_dense_gemm
 * gets the scratch memory of its small-M kernel (float32 partial tiles and one
 * counter per 128 weight rows, used when one tile of the weight is dealt to
 * several CTAs) from cudaMalloc on first use; this entry point keeps it in a
 * fixed array of 5 MiB + 16 KiB inside the library, which every GPU that loads
 * the library holds until the process ends.
 *
 *   out[m, n] = bf16(a[m, k] . b[n, k]^T), or its sigmoid (epilogue = Identity / Sigmoid);
 *   operands, scales, strides and alignment as for hq_dense_gemm in "w8a8-mxfp8" mode,
 *   no bias, no alpha.  Same kernel and same deal of the work as hq_dense_gemm makes for
 *   the shape, hence the same bits.
 *
 * Rejected with HQ_ERR_INVALID and a message: m > 32, n > 524288 (4096 tiles
 * of 128 rows), a launch of more than 160 CTAs (pass a smaller sm_count).
 * The first call on a device looks the array's device address up
 * (cudaGetSymbolAddress) and opts the kernel in to its shared memory; make it
 * before any stream capture.  All calls on a device share the one array, and
 * it keeps the last call's contents: the entry point clears the tile counters
 * it is going to use with a cudaMemsetAsync on `stream` before the launch, and
 * the partial tiles are written before they are read.  Two calls whose kernels
 * may overlap on the GPU (different streams, or programmatic launches that run
 * ahead) race on the array: serialise them.
 */
int hq_dense_gemm_small_m_noalloc(const void* a, const void* b, const void* sfa,
                                  const void* sfb, void* out, int64_t m,
                                  int64_t n, int64_t k, int64_t sfa_bytes,
                                  int64_t sfb_bytes, int64_t ldo, int epilogue,
                                  int sm_count, int use_pdl, int device,
                                  void* stream, char* err, size_t errlen);

/*
 * Host-only check of how the small-M kernel deals its (128 weight rows) x (256
 * bytes of K) units out to `sm_count` CTAs for an [n, k] MXFP8 weight: every
 * unit worked exactly once, the runs contiguous, and the scratch slots of the
 * CTAs that share a tile distinct.  `force_split` = 1 checks the split deal
 * (every tile to a power-of-two number of CTAs) also where the dispatch would
 * keep whole tiles per CTA, 2 the general even deal of one contiguous run of
 * units per CTA.  Needs no GPU.  The
 * reference has no counterpart (its small-M tiles are never split over K).
 */
int hq_selftest_decode_plan(int64_t n, int64_t k, int sm_count, int force_split,
                            char* err, size_t errlen);

/* Human-readable description of the tile the GEMM dispatch picks for a shape
 * (what the reference prints under IR_GEMM_TRACE,
 * csrc/kernel/gemm/gemm_dispatch.cuh:389-416).  Returns 0 and fills `buf`, or
 * HQ_ERR_INVALID with the reference's "No dense ... tile" message. */
int hq_describe_tile(int64_t m, int64_t n, int64_t k, int mode, int sm_count,
                     int device, char* buf, size_t buflen);

const char* hq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HALOPS_B200_H_ */
